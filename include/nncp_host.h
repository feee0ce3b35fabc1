/*
 * nncp_host.h -- host-side C code around the train step: range coder, symbol coder,
 * stream layout, learning-rate schedule, container header and the block loop that drives
 * a model through the plugin verbs.  Plain C, no CUDA: the model is reached through a
 * table of function pointers (nch_model_ops) exactly as process_block reaches it through
 * NNCPModelClass (nncp.c:49-69).  nch_bind_cuda() fills that table from libnncu.so.
 *
 * What each part restates (paths relative to the reference project):
 *   nch_enc_* / nch_dec_*         put_bit, get_bit, renormalisation, flush   arith.c:43-310
 *   nch_write_sym / nch_read_sym  write_sym, read_sym                        cp_utils.c:299-349
 *   nch_vec_sum_f32               vec_sum_f32 (LibNC symbol, libnc.h:600)
 *   nch_interp                    get_interp_param                           cp_utils.c:380-410
 *   nch_get_symb / nch_put_symb   get_symb, put_symb                         nncp.c:2945-2965
 *   nch_process_block             process_block                              nncp.c:2968-3147
 *   nch_write_header/read_header  nncp_write_file_header, trf_write_params   nncp.c:2665-2760, 1333-1445
 *   nch_compress / nch_decompress encode_file, decode_file (memory to memory) nncp.c:3307-3677
 *   nch_words_encode / _decode    word_encode, word_decode (text tokenizer)  preprocess.c:1093-1323
 *   nch_read_dict, fp->dict       write/read_compressed_file (zlib)          nncp.c:3222-3305, 3407-3413
 */
#ifndef NNCP_HOST_H
#define NNCP_HOST_H

#include <stddef.h>
#include <stdint.h>

#include "nncu.h"

#ifdef __cplusplus
extern "C" {
#endif

#define NCH_OK 0
#define NCH_ERR_INVALID 1
#define NCH_ERR_NOMEM 3
#define NCH_ERR_FORMAT 7   /* bad magic, version or truncated header */
#define NCH_ERR_MODEL 8    /* a model call failed; see nncu_last_error */
#define NCH_ERR_RANKS 9    /* the file was coded by a different number of ranks than is decoding it */

/* ---- range coder (arith.c) ---- */
typedef struct nch_enc nch_enc;
typedef struct nch_dec nch_dec;
nch_enc *nch_enc_new(void);
void nch_enc_put_bit(nch_enc *e, int prob0, int bit);          /* 0 < prob0 < 32768 */
/* put_bit_flush: ends the stream; *out stays owned by e.  Returns the byte count. */
size_t nch_enc_finish(nch_enc *e, const uint8_t **out);
size_t nch_enc_bytes(const nch_enc *e);                        /* bytes emitted so far */
void nch_enc_free(nch_enc *e);
nch_dec *nch_dec_new(const uint8_t *buf, size_t len);          /* reads past the end are zeros */
int nch_dec_get_bit(nch_dec *d, int prob0);
void nch_dec_free(nch_dec *d);

/* ---- symbol coder (cp_utils.c:299-349) ---- */
float nch_vec_sum_f32(const float *tab, size_t n);
void nch_write_sym(nch_enc *e, const float *prob, int n_symb, int sym);
int nch_read_sym(nch_dec *d, const float *prob, int n_symb);
/* the same walk fed by coder-ready device output (nncu_coder_paths / nncu_coder_trees).
   nch_write_sym_path takes the decisions from the bits of sym: alphabets that are a power of two.
   nch_write_sym_path_any and nch_read_sym_tree repeat write_sym's splitting (n >> 1 symbols to the
   left) and serve any alphabet; a tree row has 1 << nch_tree_depth(n_symb) entries in heap order,
   a path row nch_tree_depth(n_symb) = ceil(log2 n_symb). */
void nch_write_sym_path(nch_enc *e, const uint16_t *prob0, int n_bits, int sym);
void nch_write_sym_path_any(nch_enc *e, const uint16_t *prob0, int n_symb, int sym);
int nch_read_sym_tree(nch_dec *d, const uint16_t *tree, int n_symb);
int nch_tree_depth(int n_symb);
/* n symbols in a row: prob0 [n][n_bits] / [n][depth], trees [n][1 << depth] (the coding rank of a sharded job) */
void nch_write_sym_paths(nch_enc *e, const uint16_t *prob0, int n_bits, const int32_t *sym, size_t n);
void nch_write_sym_paths_any(nch_enc *e, const uint16_t *prob0, int n_symb, const int32_t *sym, size_t n);
void nch_read_sym_trees(nch_dec *d, const uint16_t *trees, int n_symb, size_t n, int32_t *sym_out);

/* ---- schedule (cp_utils.h:60-71, cp_utils.c:380-410) ---- */
#define NCH_INTERP_MAX_STEPS 8
typedef struct nch_interp_params {
    int32_t n_steps;
    float val[NCH_INTERP_MAX_STEPS + 1];
    int64_t pos[NCH_INTERP_MAX_STEPS];
    float decay_power;
} nch_interp_params;
float nch_interp(const nch_interp_params *p, int64_t pos);

/* ---- stream layout (nncp.c:2945-2965): stream s owns a contiguous slice ---- */
int nch_get_symb(const uint16_t *buf, int stride, int rem, int stream_idx, int pos);
int nch_put_symb(uint16_t *buf, int stride, int rem, int stream_idx, int pos, int c);

/* ---- model plugin as the block loop sees it ---- */
typedef struct nch_model_ops {
    void *ctx;
    int n_streams, seg_len, n_symbols;
    int (*reset)(void *ctx);
    int (*set_lr)(void *ctx, float lr);
    int (*eval)(void *ctx, int output_index, const int32_t *input);
    int (*read_probs)(void *ctx, int t0, int nt, float *probs);
    int (*coder_paths)(void *ctx, int t0, int nt, const int32_t *sym, uint16_t *prob0, int *n_bits); /* may be NULL */
    int (*coder_trees)(void *ctx, int t0, int nt, uint16_t *tree);                                   /* may be NULL */
    int (*eval_end)(void *ctx);
    int (*eval_gradient)(void *ctx, const int32_t *expected, float *loss);
    int (*update)(void *ctx);
    /* range decoder on the device (nncu_decoder_begin / nncu_decode_steps / nncu_decoder_end);
       all three NULL for a model without one */
    /* encoder order (nncu_coder_paths_begin / _end, nncu_eval_gradient without its loss, nncu_read_loss):
       lets nch_process_block queue the backward pass and the next forward pass before it range-codes a
       segment; all four NULL for a model without them */
    int (*coder_paths_begin)(void *ctx, int t0, int nt, const int32_t *sym);
    int (*coder_paths_end)(void *ctx, uint16_t *prob0, int *n_bits);
    int (*eval_gradient_queue)(void *ctx, const int32_t *expected);
    int (*read_loss)(void *ctx, float *loss);
    int (*decoder_begin)(void *ctx, const uint8_t *payload, size_t len);
    int (*decode_steps)(void *ctx, int t0, int nt, const int32_t *ids_t0, int limit_t, int limit_b, int32_t *symbols);
    int (*decoder_end)(void *ctx, size_t *bytes_consumed);
} nch_model_ops;

/* Loads libnncu.so (dlopen), creates a model and fills *ops.  nch_unbind_cuda destroys it. */
int nch_bind_cuda(const char *libnncu_path, const nncu_params *p, nch_model_ops *ops);
void nch_unbind_cuda(nch_model_ops *ops);

/* ---- block loop ---- */
#define NCH_EVAL_STEP 0     /* one symbol per stream per model_eval: the reference's default, and
                               the only way to decode (nncp.c:2996-3022) */
#define NCH_EVAL_SEGMENT 1  /* one model_eval per segment: --encode_only (nncp.c:3023-3046) */
#define NCH_OUT_FLOAT 0     /* float tables to the host, write_sym/read_sym on them */
#define NCH_OUT_CODER_READY 1 /* prob0 paths (encode) / trees (decode) from the device */
#define NCH_OUT_DEVICE 2      /* decode: the range decoder runs on the device too (encode: as CODER_READY).
                                 Falls back to CODER_READY when the model has no device decoder or
                                 refuses the geometry. */

typedef struct nch_block_stats {
    int64_t n_symbols, train_steps;
    double sum_log2; /* -sum log2 p[target] over the trained segments (from the returned loss) */
} nch_block_stats;

/* process_block: codes block_len symbols split in n_streams streams; exactly one of enc/dec is
   set.  *train_step is the running step counter the learning-rate schedule reads. */
int nch_process_block(const nch_model_ops *m, nch_enc *enc, nch_dec *dec, uint16_t *block_buf,
                      int block_len, const nch_interp_params *lr, int64_t *train_step, int eval_mode,
                      int out_mode, nch_block_stats *stats);

/* ---- container (nncp.c:2662-2690, 1333-1365) ---- */
typedef struct nch_file_params {
    nncu_params model;            /* n_streams is batch_size; d_model = d_key * n_head on read */
    nch_interp_params lr, block_len;
    int32_t n_ranks;              /* ranks the streams were sharded over; 0 or 1: one process (header version 3 otherwise) */
    const uint8_t *dict;          /* write: the word dictionary to carry (text of nch_words_encode), NULL: none.
                                     read: always NULL; fetch the text with nch_read_dict */
    uint32_t dict_len;            /* its size in bytes; on read, the size recorded in the file (0: no dictionary) */
    /* the retrain pass between blocks (retrain_block, nncp.c:2821-2941): every retrain_period coded
       symbols the model is reset and trained again over the last retrain_len symbols, laid out in
       n_streams contiguous runs.  0: no retrain.  The reference also switches dropout on for that
       pass; dropout is not built, so the header's two dropout probabilities are written as 0 and a
       file that holds others is refused (NCH_ERR_FORMAT). */
    uint32_t retrain_period, retrain_len;
    int32_t has_retrain_lr;       /* the pass has a schedule of its own, read with its own step counter */
    nch_interp_params retrain_lr;
} nch_file_params;
int nch_write_header(const nch_file_params *fp, uint32_t n_symbols_in_file, uint8_t *out, size_t cap,
                     size_t *len);
int nch_read_header(const uint8_t *in, size_t n, nch_file_params *fp, uint32_t *n_symbols_in_file,
                    size_t *consumed);

/* The dictionary a file carries (nncp.c:3264-3305): inflates it into *dict (malloc'ed, free with
   nch_free).  *dict = NULL and *dict_len = 0 when the file has none. */
int nch_read_dict(const uint8_t *in, size_t n, uint8_t **dict, size_t *dict_len);

/* length of the block that starts at symbol file_pos (schedule value rounded down to whole
   segments of all streams, at least one, at most what remains; nncp.c:3428-3441) */
int nch_next_block_len(const nch_file_params *fp, size_t file_pos, size_t remaining);

/* encode_file / decode_file, memory to memory.  *out is malloc'ed (free with nch_free).
   NCH_ERR_RANKS when fp->n_ranks > 1: a file of a sharded job is coded and decoded by that many
   processes together. */
int nch_compress(const nch_model_ops *m, const nch_file_params *fp, const uint16_t *symbols, size_t n,
                 int eval_mode, int out_mode, uint8_t **out, size_t *out_len, nch_block_stats *stats);
int nch_decompress(const nch_model_ops *m, const nch_file_params *fp, const uint8_t *payload, size_t n,
                   uint32_t n_symbols_in_file, int out_mode, uint16_t *symbols_out);
void nch_free(void *p);

/* ---- word tokenizer (preprocess.c) ----
   nch_words_encode folds case and spaces, builds a dictionary of at most about n_words entries
   (256 bytes + words seen at least min_word_freq times) and writes the text as 16-bit indices
   into it: word_encode (preprocess.c:1093-1226), same dictionary text and same symbols.  *dict,
   *symbols are malloc'ed (nch_free); texts above 1 GiB and n_words above 65535 are refused
   (NCH_ERR_INVALID); *n_entries is the number of dictionary entries, and the
   model's alphabet is that rounded up to a multiple of 8 (nncp.c:3382).
   nch_words_decode is word_decode (preprocess.c:1270-1323): NCH_ERR_FORMAT for a symbol past
   the dictionary or an escape other than backslash-n or backslash-backslash (an entry above 4096
   bytes, which the reference's encoder can make and its decoder refuses, decodes here).
   nch_words_count returns the number of entries of a dictionary text (negative: -error). */
int nch_words_encode(const uint8_t *text, size_t n, int n_words, int min_word_freq, uint8_t **dict,
                     size_t *dict_len, uint16_t **symbols, size_t *n_symbols, int *n_entries);
int nch_words_decode(const uint8_t *dict, size_t dict_len, const uint16_t *symbols, size_t n_symbols,
                     uint8_t **text, size_t *text_len);
int nch_words_count(const uint8_t *dict, size_t dict_len);

#ifdef __cplusplus
}
#endif
#endif /* NNCP_HOST_H */
