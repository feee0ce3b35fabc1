/*
 * frontend.c -- the `nncp-metal` command line and container (include/nncp_metal_frontend.h).
 *
 * Verbs, flags and messages follow src/metal/nncp_metal.c:41-122 and :1229-1330 of the
 * reference; the 24-byte header is its NNCPHeader (:174-185) with the checksum of :307-311.
 * Where the reference hands the bytes to its Metal integration layer
 * (compression_integration_compress, :262-290) this build hands them to the Transformer-XL
 * compressor on the GPU (nch_compress: the block loop of nncp.c over libnncu.so), and the
 * payload is the nncp.c stream.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "nncp_metal_frontend.h"

static __thread char g_err[256] = "";

static void set_err(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

const char *nncpm_last_error(void) { return g_err; }

uint32_t nncpm_checksum(const uint8_t *data, size_t n)
{
    uint32_t c = 0;
    for (size_t i = 0; i < n; i++)
        c = c * 31u + data[i];
    return c;
}

int nncpm_route(const nncpm_header *h)
{
    if (h->compression_level & 0x8000)
        return NNCPM_ROUTE_NEURAL_ENGINE;
    if (h->quantization_bits == 8) {
        if (h->compression_level == 6)
            return NNCPM_ROUTE_LSTM;
        if (h->compression_level == 8)
            return NNCPM_ROUTE_TRANSFORMER;
        if (h->compression_level <= 9)
            return NNCPM_ROUTE_CPU_ORIGINAL;
    }
    return NNCPM_ROUTE_UNKNOWN;
}

int nncpm_level_params(int level, nch_file_params *fp)
{
    if (!fp)
        return NCH_ERR_INVALID;
    if (level < 1)
        level = 1;
    if (level > 9)
        level = 9;
    memset(fp, 0, sizeof(*fp));
    nncu_params *m = &fp->model;
    /* the "default" profile of nncp.c:2471-2513 ... */
    m->n_layer = 4; m->d_model = 256; m->n_head = 8; m->d_key = 32; m->d_value = 32;
    m->d_inner = 512; m->d_pos = 32; m->mem_len = 32; m->seg_len = 32; m->n_streams = 16;
    m->n_symbols = 256; m->use_bias = 1; m->use_w_r = 1; m->tied_w_r = 1; m->tied_b_r = 1;
    m->ln_flags = NNCU_LN_POST; m->ff_act = NNCU_FF_GELU; m->embed_mult = 1.0f;
    m->init_range = 1.0f; m->init_kind = NNCU_INIT_UNIFORM; m->seed = 123;
    m->lr = 3e-4f; m->beta2 = 0.9999f; m->eps = 1e-8f; m->gradient_clip = 0.1f;
    m->device = -1;
    fp->lr.n_steps = 1;
    fp->lr.val[0] = 3e-4f; fp->lr.val[1] = 1e-4f; fp->lr.pos[0] = 5000000 / 32;
    fp->block_len.n_steps = 0;
    fp->block_len.val[0] = 500000.0f;
    /* ... narrower below level 4, wider (and bf16 on the tensor cores) above level 6 */
    if (level <= 3) {
        m->n_layer = 2; m->d_model = 128; m->n_head = 4; m->d_inner = 256;
    } else if (level >= 7) {
        m->n_layer = 6; m->d_model = 512; m->n_head = 8; m->d_key = 64; m->d_value = 64;
        m->d_inner = 1024; m->d_pos = 64; m->mem_len = 64; m->seg_len = 64; m->n_streams = 16;
        m->use_bf16 = 1;
        fp->lr.val[0] = 2e-4f;
    }
    return NCH_OK;
}

size_t nncpm_estimate_output_size(size_t n)
{
    /* the coder spends at most 15 bits of redundancy per binary decision in the worst case;
       incompressible input costs a little over 8 bits per byte */
    return NNCPM_HEADER_BYTES + 256 + n + n / 8 + 64;
}

/* directory of this shared object, for the default libnncu.so path */
static const char *default_libnncu(char *buf, size_t cap)
{
    Dl_info info;
    if (dladdr((void *)&nncpm_checksum, &info) && info.dli_fname) {
        const char *slash = strrchr(info.dli_fname, '/');
        if (slash) {
            snprintf(buf, cap, "%.*s/libnncu.so", (int)(slash - info.dli_fname), info.dli_fname);
            return buf;
        }
    }
    return "libnncu.so";
}

size_t nncpm_lossless_compress(const uint8_t *in, size_t n, uint8_t *out, size_t cap, int level,
                               const char *libnncu_path)
{
    g_err[0] = 0;
    if ((!in && n) || !out) {
        set_err("null buffer");
        return 0;
    }
    if (n > 0xFFFFFFFFu - 4096) {
        set_err("input of %zu bytes exceeds the container's 32-bit size fields", n);
        return 0;
    }
    char path[1024];
    if (!libnncu_path)
        libnncu_path = default_libnncu(path, sizeof(path));
    nch_file_params fp;
    nncpm_level_params(level, &fp);
    nch_model_ops ops;
    if (nch_bind_cuda(libnncu_path, &fp.model, &ops) != NCH_OK) {
        set_err("cannot start the GPU model (%s): no usable B200, or the library is missing", libnncu_path);
        return 0;
    }
    uint16_t *sym = (uint16_t *)malloc(sizeof(uint16_t) * (n ? n : 1));
    uint8_t *payload = NULL;
    size_t plen = 0, total = 0;
    if (!sym) {
        set_err("out of memory");
    } else {
        for (size_t i = 0; i < n; i++)
            sym[i] = in[i];
        int rc = nch_compress(&ops, &fp, sym, n, NCH_EVAL_SEGMENT, NCH_OUT_CODER_READY, &payload, &plen, NULL);
        if (rc != NCH_OK) {
            set_err("compression failed (status %d)", rc);
        } else if (NNCPM_HEADER_BYTES + plen > cap) {
            set_err("output buffer of %zu bytes is too small for %zu", cap, NNCPM_HEADER_BYTES + plen);
        } else {
            nncpm_header h;
            h.magic = NNCPM_MAGIC;
            h.version = NNCPM_VERSION;
            h.original_size = (uint32_t)n;
            h.compressed_size = (uint32_t)(plen + NNCPM_HEADER_BYTES);
            h.compression_level = 8; /* the Transformer route (nncp_metal.c:324-326) */
            h.quantization_bits = 8;
            h.checksum = nncpm_checksum(in, n);
            memcpy(out, &h, NNCPM_HEADER_BYTES);
            memcpy(out + NNCPM_HEADER_BYTES, payload, plen);
            total = NNCPM_HEADER_BYTES + plen;
        }
    }
    nch_free(payload);
    free(sym);
    nch_unbind_cuda(&ops);
    return total;
}

size_t nncpm_lossless_decompress(const uint8_t *in, size_t n, uint8_t *out, size_t cap, const char *libnncu_path)
{
    g_err[0] = 0;
    if (!in || n < NNCPM_HEADER_BYTES || (!out && cap)) {
        set_err("input shorter than the %d-byte header", NNCPM_HEADER_BYTES);
        return 0;
    }
    nncpm_header h;
    memcpy(&h, in, NNCPM_HEADER_BYTES);
    if (h.magic != NNCPM_MAGIC || h.version != NNCPM_VERSION) {
        set_err("not an nncp-metal file (magic %08x, version %u)", h.magic, h.version);
        return 0;
    }
    if (nncpm_route(&h) != NNCPM_ROUTE_TRANSFORMER) {
        set_err("header routes to another codec (level %u, %u bits); only the Transformer route is built",
                h.compression_level, h.quantization_bits);
        return 0;
    }
    if (h.compressed_size < NNCPM_HEADER_BYTES || h.compressed_size > n) {
        set_err("truncated file: header says %u bytes, %zu present", h.compressed_size, n);
        return 0;
    }
    if (h.original_size > cap) {
        set_err("output buffer of %zu bytes is too small for %u", cap, h.original_size);
        return 0;
    }
    if (h.original_size == 0) {
        set_err("the file holds no data (a header alone): nothing to decode");
        return 0;
    }
    const uint8_t *stream = in + NNCPM_HEADER_BYTES;
    const size_t slen = h.compressed_size - NNCPM_HEADER_BYTES;
    nch_file_params fp;
    uint32_t nsym = 0;
    size_t used = 0;
    if (nch_read_header(stream, slen, &fp, &nsym, &used) != NCH_OK || nsym != h.original_size ||
        fp.model.n_symbols != 256 || fp.dict_len != 0) { /* this container holds bytes, never tokenised text */
        set_err("bad inner stream header");
        return 0;
    }
    char path[1024];
    if (!libnncu_path)
        libnncu_path = default_libnncu(path, sizeof(path));
    nch_model_ops ops;
    if (nch_bind_cuda(libnncu_path, &fp.model, &ops) != NCH_OK) {
        set_err("cannot start the GPU model (%s): no usable B200, or the library is missing", libnncu_path);
        return 0;
    }
    uint16_t *sym = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)nsym);
    size_t total = 0;
    if (!sym) {
        set_err("out of memory");
    } else {
        int rc = nch_decompress(&ops, &fp, stream + used, slen - used, nsym, NCH_OUT_DEVICE, sym);
        if (rc != NCH_OK) {
            set_err("decompression failed (status %d)", rc);
        } else {
            for (size_t i = 0; i < nsym; i++)
                out[i] = (uint8_t)sym[i];
            if (nncpm_checksum(out, nsym) != h.checksum)
                set_err("checksum mismatch: the file is damaged or was written by another build");
            else
                total = nsym;
        }
    }
    free(sym);
    nch_unbind_cuda(&ops);
    return total;
}

static uint8_t *read_file(const char *path, size_t *n)
{
    FILE *f = fopen(path, "rb");
    if (!f)
        return NULL;
    fseek(f, 0, SEEK_END);
    long sz = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (sz < 0) {
        fclose(f);
        return NULL;
    }
    uint8_t *buf = (uint8_t *)malloc((size_t)sz + 1);
    if (buf && fread(buf, 1, (size_t)sz, f) != (size_t)sz) {
        free(buf);
        buf = NULL;
    }
    fclose(f);
    *n = (size_t)sz;
    return buf;
}

int nncpm_compress_file(const char *input_file, const char *output_file, int level, int verbose,
                        const char *libnncu_path)
{
    size_t n = 0;
    uint8_t *in = read_file(input_file, &n);
    if (!in) {
        printf("ERROR: Cannot open input file '%s'\n", input_file);
        return -1;
    }
    if (verbose)
        printf("Compressing '%s' to '%s' (level %d, %zu bytes)\n", input_file, output_file, level, n);
    size_t cap = nncpm_estimate_output_size(n), len = 0;
    uint8_t *out = (uint8_t *)malloc(cap);
    int rc = -1;
    if (!out) {
        printf("ERROR: out of memory\n");
    } else if (n == 0) {
        /* an empty file is a header alone */
        nncpm_header h = {NNCPM_MAGIC, NNCPM_VERSION, 0, NNCPM_HEADER_BYTES, 8, 8, 0};
        memcpy(out, &h, NNCPM_HEADER_BYTES);
        len = NNCPM_HEADER_BYTES;
    } else {
        len = nncpm_lossless_compress(in, n, out, cap, level, libnncu_path);
        if (!len)
            printf("ERROR: %s\n", nncpm_last_error());
    }
    if (len) {
        FILE *f = fopen(output_file, "wb");
        if (!f) {
            printf("ERROR: Cannot create output file '%s'\n", output_file);
        } else {
            rc = fwrite(out, 1, len, f) == len ? 0 : -1;
            fclose(f);
            if (verbose && rc == 0)
                printf("Compressed %zu bytes to %zu bytes (%.2f%%)\n", n, len, n ? 100.0 * len / n : 0.0);
        }
    }
    free(out);
    free(in);
    return rc;
}

int nncpm_decompress_file(const char *input_file, const char *output_file, int verbose, const char *libnncu_path)
{
    size_t n = 0;
    uint8_t *in = read_file(input_file, &n);
    if (!in) {
        printf("ERROR: Cannot open input file '%s'\n", input_file);
        return -1;
    }
    if (n < NNCPM_HEADER_BYTES) {
        printf("ERROR: Cannot read file header for format detection\n");
        free(in);
        return -1;
    }
    nncpm_header h;
    memcpy(&h, in, NNCPM_HEADER_BYTES);
    if (verbose) {
        static const char *names[] = {"", "Neural Engine", "LSTM", "Transformer", "CPU NNCP Original", "Unknown"};
        printf("Auto-detected compression format: %s\n", names[nncpm_route(&h)]);
    }
    int rc = -1;
    uint8_t *out = (uint8_t *)malloc((size_t)h.original_size + 1);
    if (!out) {
        printf("ERROR: out of memory\n");
    } else {
        size_t len = 0;
        int ok = 1;
        if (h.magic == NNCPM_MAGIC && h.version == NNCPM_VERSION && h.original_size == 0 &&
            h.compressed_size == NNCPM_HEADER_BYTES) {
            len = 0;
        } else {
            len = nncpm_lossless_decompress(in, n, out, h.original_size, libnncu_path);
            if (!len) {
                printf("ERROR: %s\n", nncpm_last_error());
                ok = 0;
            }
        }
        if (ok) {
            FILE *f = fopen(output_file, "wb");
            if (!f) {
                printf("ERROR: Cannot create output file '%s'\n", output_file);
            } else {
                rc = fwrite(out, 1, len, f) == len ? 0 : -1;
                fclose(f);
                if (verbose && rc == 0)
                    printf("Decompressed %zu bytes to %zu bytes\n", n, len);
            }
        }
    }
    free(out);
    free(in);
    return rc;
}

static void show_usage(void)
{
    printf("nncp-metal (B200 backend) - Transformer-XL lossless compression\n\n");
    printf("Usage: nncp-metal <command> [options] <input> <output>\n\n");
    printf("Commands:\n");
    printf("  c, compress    Compress input file to output file\n");
    printf("  d, decompress  Decompress input file to output file\n");
    printf("  test           Check that the GPU library loads\n");
    printf("Options:\n");
    printf("  -v, --verbose       Enable verbose output\n");
    printf("  -l, --level <1-9>   Set compression level (default: 6)\n");
    printf("  --cpu               Refused: this build has no CPU model\n");
    printf("  -h, --help          Show this help message\n");
}

int nncpm_main(int argc, char **argv)
{
    if (argc < 2) {
        printf("Error: Invalid arguments\n\n");
        show_usage();
        return 1;
    }
    const char *cmd = argv[1], *in = NULL, *out = NULL;
    int verbose = 0, level = 6, cpu = 0;
    const int is_c = !strcmp(cmd, "c") || !strcmp(cmd, "compress");
    const int is_d = !strcmp(cmd, "d") || !strcmp(cmd, "decompress");
    if (!strcmp(cmd, "-h") || !strcmp(cmd, "--help")) {
        show_usage();
        return 0;
    }
    if (!strcmp(cmd, "neural")) {
        printf("Error: the 'neural' command (lossy Neural Engine demo) is not part of this build\n");
        return 1;
    }
    if (!is_c && !is_d && strcmp(cmd, "test")) {
        printf("Error: Unknown command '%s'\n", cmd);
        printf("Error: Invalid arguments\n\n");
        show_usage();
        return 1;
    }
    if (is_c || is_d) {
        if (argc < 4) {
            printf("Error: %s command requires input and output file arguments\n", is_c ? "compress" : "decompress");
            printf("Error: Invalid arguments\n\n");
            show_usage();
            return 1;
        }
        in = argv[2];
        out = argv[3];
    }
    /* options may stand anywhere after the command, as in the reference's loop over argv */
    for (int i = 2; i < argc; i++) {
        if (!strcmp(argv[i], "-v") || !strcmp(argv[i], "--verbose")) {
            verbose = 1;
        } else if (!strcmp(argv[i], "--cpu")) {
            cpu = 1;
        } else if ((!strcmp(argv[i], "-l") || !strcmp(argv[i], "--level")) && i + 1 < argc) {
            level = atoi(argv[i + 1]);
            if (level < 1) level = 1;
            if (level > 9) level = 9;
            i++;
        }
    }
    if (cpu) {
        printf("ERROR: --cpu: this build has no CPU model; the Transformer runs on the GPU only\n");
        return 1;
    }
    const char *lib = getenv("NNCP_LIBNNCU"); /* NULL: libnncu.so next to the host library */
    if (!strcmp(cmd, "test")) {
        char path[1024];
        const char *p = lib ? lib : default_libnncu(path, sizeof(path));
        void *dl = dlopen(p, RTLD_NOW);
        if (!dl) {
            printf("ERROR: cannot load %s\n", p);
            return 1;
        }
        int (*ver)(void) = (int (*)(void))dlsym(dl, "nncu_abi_version");
        printf("GPU library %s loaded (ABI version %d)\n", p, ver ? ver() : -1);
        return 0;
    }
    int rc = is_c ? nncpm_compress_file(in, out, level, verbose, lib) : nncpm_decompress_file(in, out, verbose, lib);
    return rc == 0 ? 0 : 1;
}
