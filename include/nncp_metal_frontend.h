/*
 * nncp_metal_frontend.h -- the `nncp-metal` command-line surface and container on top of the
 * B200 Transformer-XL compressor (nncp_host.h / nncu.h).
 *
 * What each part replaces in the reference (paths relative to the reference project):
 *   nncpm_header, NNCPM_MAGIC        NNCPHeader, NNCP_MAGIC, NNCP_VERSION   src/metal/nncp_metal.c:174-185
 *   nncpm_checksum                   the checksum fold of the compressor    src/metal/nncp_metal.c:307-311
 *   nncpm_route                      format sniffing of `decompress`         src/metal/nncp_metal.c:1272-1300
 *   nncpm_lossless_compress /        neural_bridge_cuda_lossless_compress /  src/metal/compression_integration.c:6-10,
 *   nncpm_lossless_decompress        _decompress (0 = failure)               src/neural/integration/neural_bridge.h:206-236
 *   nncpm_estimate_output_size       compression_integration_estimate_output_size
 *                                                                            src/metal/compression_integration.h:176-179
 *   nncpm_compress_file /            compress_file_metal_integrated /        src/metal/nncp_metal.c:187-353, 740-900
 *   nncpm_decompress_file            decompress_file_metal_integrated
 *   nncpm_main                       parse_args + main: verbs c, compress,   src/metal/nncp_metal.c:41-122, 1229-1330
 *                                    d, decompress, test; -v, -l, --cpu, -h
 *
 * The container is the reference's: a 24-byte native-endian header followed by the payload.
 * The payload is the nncp.c stream (its own self-describing big-endian header, nncp.c:2662-2690,
 * then the range coder's bytes), so a file decodes without knowing the level it was made with.
 * Files written here carry compression_level 8 and quantization_bits 8, the values the
 * reference writes for its Transformer route (nncp_metal.c:324-326, 338).
 *
 * There is no CPU model: `--cpu`, the `neural` verb (the reference's lossy Neural Engine demo)
 * and files whose header routes to another codec are refused with a message and a non-zero
 * exit status.
 */
#ifndef NNCP_METAL_FRONTEND_H
#define NNCP_METAL_FRONTEND_H

#include <stddef.h>
#include <stdint.h>

#include "nncp_host.h"

#ifdef __cplusplus
extern "C" {
#endif

#define NNCPM_MAGIC 0x4E4E4350u /* "NNCP" */
#define NNCPM_VERSION 1u
#define NNCPM_HEADER_BYTES 24

typedef struct nncpm_header {
    uint32_t magic;
    uint32_t version;
    uint32_t original_size;
    uint32_t compressed_size; /* payload bytes + NNCPM_HEADER_BYTES */
    uint16_t compression_level;
    uint16_t quantization_bits;
    uint32_t checksum; /* nncpm_checksum of the original bytes */
} nncpm_header;

/* routes of the reference's decoder (nncp_metal.c:1277-1300) */
#define NNCPM_ROUTE_NEURAL_ENGINE 1 /* level bit 15 set: lossy demo, not decodable here */
#define NNCPM_ROUTE_LSTM 2          /* level 6, 8 bits */
#define NNCPM_ROUTE_TRANSFORMER 3   /* level 8, 8 bits: the route this build writes and reads */
#define NNCPM_ROUTE_CPU_ORIGINAL 4  /* other levels <= 9, 8 bits */
#define NNCPM_ROUTE_UNKNOWN 5

/* checksum = fold over the bytes of c * 31 + byte, starting from 0 (mod 2^32) */
uint32_t nncpm_checksum(const uint8_t *data, size_t n);
int nncpm_route(const nncpm_header *h);

/* The model a compression level selects (levels 1..9, clamped as the reference does,
   nncp_metal.c:111-113): fills *fp with the hyper-parameters, learning-rate schedule and block
   length.  Levels 1-3: 2 layers x 128; 4-6: the "default" profile of nncp.c:2471-2513 (4 layers x
   256); 7-9: 6 layers x 512, bf16.  All are byte-level (256 symbols). */
int nncpm_level_params(int level, nch_file_params *fp);

/* Upper bound of the container size for n input bytes. */
size_t nncpm_estimate_output_size(size_t n);

/*
 * Memory to memory, container included.  Returns the number of bytes written to out, 0 on
 * failure (buffer too small, no usable GPU, model error: see nncpm_last_error).
 * libnncu_path: the CUDA library to bind (NULL = "libnncu.so" next to this library).
 */
size_t nncpm_lossless_compress(const uint8_t *in, size_t n, uint8_t *out, size_t cap, int level,
                               const char *libnncu_path);
size_t nncpm_lossless_decompress(const uint8_t *in, size_t n, uint8_t *out, size_t cap,
                                 const char *libnncu_path);
const char *nncpm_last_error(void);

/* File to file; 0 on success, -1 on failure (message on stdout, as the reference prints). */
int nncpm_compress_file(const char *input_file, const char *output_file, int level, int verbose,
                        const char *libnncu_path);
int nncpm_decompress_file(const char *input_file, const char *output_file, int verbose,
                          const char *libnncu_path);

/* The command line: nncp-metal <command> [options] <input> <output>. */
int nncpm_main(int argc, char **argv);

#ifdef __cplusplus
}
#endif
#endif /* NNCP_METAL_FRONTEND_H */
