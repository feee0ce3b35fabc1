/*
 * nncu.h -- C ABI of the B200 (sm_100a) backend for NNCP's Transformer-XL
 * model plugin.
 *
 * Every entry point takes plain pointers and sizes, returns a status code
 * (0 = NNCU_OK) and never throws or aborts.  The library needs only the CUDA
 * runtime; it has no CPU fallback: every compute entry point fails with
 * NNCU_ERR_CUDA when no sm_100 device is usable.
 *
 * What each group replaces in the reference (paths are relative to the
 * reference project):
 *
 *   nncu_create / nncu_destroy      trf_init / trf_end            nncp.c:304-550
 *   nncu_eval / nncu_eval_dev       trf_eval (model_eval)         nncp.c:581-1029
 *   nncu_eval_end                   trf_eval_end                  nncp.c:1032-1060
 *   nncu_eval_gradient[_dev]        trf_eval_gradient             nncp.c:1099-1193
 *   nncu_update                     trf_update + mem_update       nncp.c:1205-1235
 *   nncu_reset                      trf_reset                     nncp.c:1195-1203
 *   nncu_set_lr                     trf_set_lr                    nncp.c:1243-1247
 *   nncu_read_probs                 nc_tensor_to_cpu_device +
 *                                   nc_tensor_get_ptr on the
 *                                   tensor model_eval returns     nncp.c:3003-3011, 3031-3040
 *   nncu_coder_*                    write_sym / read_sym walk     cp_utils.c:299-349
 *   nncu_param_* / nncu_grad_*      NCParamList iteration         libnc.h:499-536
 *   nncu_attention_*                the attention sub-graph of
 *                                   trf_eval and its autograd     nncp.c:722-800
 *
 * Layout conventions (all row-major, "row" = one (time, stream) position):
 *   - token ids, targets:  int32 [T][B]  (index t*B + b), exactly the
 *     (B, T) LibNC tensor process_block fills with nc_set1_i32_2d
 *     (nncp.c:2984-3001; dim 0 = stream is the contiguous one).
 *   - probabilities:       fp32 [T][B][V], the (V, B, T) tensor model_eval
 *     returns (nncp.c:1007-1008); the caller's per-symbol table is
 *     probs + (t*B + b)*V  (nncp.c:3011, 3040).
 *   - parameters are exchanged as fp32, row-major, matrices as [out][in]
 *     (contraction axis contiguous): w_q [H*dk][D], w_kv [2*H*dk][D] (K rows
 *     first, nncp.c:663-664), w_o [D][H*dv], ff1 [F'][D], ff2 [D][F],
 *     embed [V][D], embed_out [V][D], w_r [H][P][dk], b_r [H][L].  For the
 *     2-d matrices this is the transpose of LibNC's storage (dim 0
 *     contiguous, libnc.h:183-185); tables and embed have LibNC's order.
 */
#ifndef NNCU_H
#define NNCU_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NNCU_ABI_VERSION 1

/* status codes */
#define NNCU_OK 0
#define NNCU_ERR_INVALID 1   /* bad argument or unsupported option          */
#define NNCU_ERR_CUDA 2      /* CUDA runtime/driver error, or no device     */
#define NNCU_ERR_NOMEM 3     /* host or device allocation failed            */
#define NNCU_ERR_STATE 4     /* call order violated (e.g. gradient w/o eval)*/
#define NNCU_ERR_TIMEOUT 5   /* a bounded device-side wait gave up          */
#define NNCU_ERR_RANGE 6     /* size beyond a stated maximum                */

/* ln_flags, same bit values as nncp.c:74-78 */
#define NNCU_LN_POST (1 << 0)
#define NNCU_LN_PRE (1 << 1)
#define NNCU_LN_FINAL (1 << 2)
#define NNCU_LN_COEF (1 << 3) /* per-layer scalar alpha (starts at 0) on both sub-layer outputs before the residual */
#define NNCU_LN_RMSNORM (1 << 4)

/* ff_act, same values as FFActivationEnum nncp.c:82-87 */
#define NNCU_FF_RELU 0
#define NNCU_FF_GELU 1
#define NNCU_FF_GEGLU 2
#define NNCU_FF_GATED_SILU 3 /* ff1 has 2 * d_inner rows: silu(first half) * second half */

#define NNCU_N_LAYER_MAX 32 /* N_LAYER_MAX nncp.c:80 */

/* init_kind */
#define NNCU_INIT_UNIFORM 0 /* U(-a, a), a = init_range / sqrt(d_model); nncp.c:263-266, 341 */
#define NNCU_INIT_NORMAL 1  /* approx. N(0, init_range^2) (sum of 12 uniforms) */

/* gemm_backend */
#define NNCU_GEMM_AUTO 0    /* tcgen05 for bf16 models, SIMT fp32 for fp32 models */
#define NNCU_GEMM_SIMT 1    /* CUDA-core fp32-accumulate GEMM for every contraction */
#define NNCU_GEMM_TCGEN05 2 /* tcgen05/TMEM GEMM (bf16 models only) */

/*
 * Hyper-parameters: the union of NNCPModelParams (nncp.c:141-163) and
 * TransformerModelParams (nncp.c:89-115) fields the train step reads, plus
 * the optimizer constants of SGDOptParams (libnc.h:547-561).
 */
typedef struct nncu_params {
    int32_t n_layer;
    int32_t d_model;
    int32_t n_head;
    int32_t d_key;
    int32_t d_value;   /* must equal d_key (w_o is always present) */
    int32_t d_inner;
    int32_t d_pos;     /* P <= mem_len + seg_len */
    int32_t mem_len;   /* M */
    int32_t seg_len;   /* T */
    int32_t n_streams; /* B held by THIS model instance (this GPU) */
    int32_t n_streams_total; /* B of the whole job; the loss is scaled by
                                -1/(T * n_streams_total) (nncp.c:1175).
                                0 means n_streams. */
    int32_t n_symbols; /* V */
    int32_t attn_len[NNCU_N_LAYER_MAX]; /* 0 means mem_len + seg_len */
    uint8_t use_bias;
    uint8_t use_w_r;
    uint8_t tied_w_r;
    uint8_t tied_b_r;
    uint8_t query_bias;
    uint8_t ln_flags;
    uint8_t ff_act;
    uint8_t use_bf16; /* bf16 weights/activations, fp32 master + optimizer state */
    float embed_mult;
    float init_range;
    int32_t init_kind;
    uint32_t seed;
    /* optimizer: v = beta2*v + (1-beta2)*g*g ; w -= lr * g / (sqrt(v) + eps).
       bias_correction != 0 divides v by (1 - beta2^step) first.
       gradient_clip != 0 clamps every gradient element to [-clip, clip]. */
    float lr;
    float beta2;
    float eps;
    float gradient_clip;
    int32_t bias_correction;
    int32_t gemm_backend;
    int32_t device; /* CUDA device ordinal; -1 = the current device */
} nncu_params;

typedef struct nncu_model nncu_model;

/* Fills *p with the "default" profile of nncp.c:2471-2513 except for the
   optimizer, which is plain RMSProp (beta2 0.99, eps 1e-8, no clip). */
void nncu_default_params(nncu_params *p);

int nncu_abi_version(void);
/* Message of the last failing call on this thread ("" if none). */
const char *nncu_last_error(void);

/* ---- model lifetime (trf_init / trf_end, nncp.c:304-550) ---- */
int nncu_create(const nncu_params *p, nncu_model **out);
int nncu_destroy(nncu_model *m);
/* All later launches go to this cudaStream_t (default: the legacy stream 0).  On any other
   stream the whole-segment forward and the backward pass are captured into CUDA graphs on
   their second use and replayed afterwards (same results, fewer launch gaps). */
int nncu_set_stream(nncu_model *m, void *cuda_stream);

/* ---- the 13-pointer plugin surface (nncp.c:49-69) ---- */
/* model_reset: zero the memory of every layer (nncp.c:1195-1203). */
int nncu_reset(nncu_model *m);
/* model_set_lr (nncp.c:1243-1247). */
int nncu_set_lr(nncu_model *m, float lr);
/*
 * model_eval (nncp.c:581-1029).  input_host is int32 [T][B].
 * output_index < 0: forward over the whole segment (the --encode_only path,
 * nncp.c:3031).  0 <= output_index < T: forward of time step output_index
 * only, reading column output_index of input (nncp.c:616-620); steps must be
 * issued in increasing order starting at 0, as process_block does.
 * Probabilities stay on the device; fetch them with nncu_read_probs.
 * Every row of the result is bit-identical between the two modes.
 */
int nncu_eval(nncu_model *m, int output_index, const int32_t *input_host);
/* Same with the ids already on the device (int32 [T][B]). */
int nncu_eval_dev(nncu_model *m, int output_index, const int32_t *input_dev);
/* model_eval_end (nncp.c:1032-1060): forget a forward that gets no gradient. */
int nncu_eval_end(nncu_model *m);
/* Copies probability rows [t0*B, (t0+nt)*B) x V to host memory and waits for
   them (nc_tensor_to_cpu_device, nncp.c:3004, 3033). */
int nncu_read_probs(nncu_model *m, int t0, int nt, float *probs_host);
/* Device address of the fp32 [T][B][V] probabilities. */
int nncu_probs_dev(nncu_model *m, float **probs_dev);
/*
 * model_eval_gradient (nncp.c:1099-1193): loss = sum ln p[target] over the
 * segment (returned un-averaged in *loss_out, may be NULL), backward pass of
 * -loss / (T * n_streams_total).  expected_host is int32 [T][B].
 */
int nncu_eval_gradient(nncu_model *m, const int32_t *expected_host, float *loss_out);
int nncu_eval_gradient_dev(nncu_model *m, const int32_t *expected_dev);
/*
 * model_eval_gradient and the optimizer half of model_update in one call (no counterpart in the
 * reference, whose process_block always calls the two in turn, nncp.c:3052-3053): the RMSProp
 * update of each layer's parameters is queued as soon as that layer's gradients are final
 * (behind their all-reduce when a communicator is attached), beside the rest of the backward
 * pass, instead of after it.  Same arithmetic, same bits as nncu_eval_gradient followed by
 * nncu_optimizer_step.  Follow with nncu_memory_shift, not nncu_update.  The gradients stay
 * readable (nncu_grad_get); the loss is collected with nncu_read_loss.
 */
int nncu_eval_gradient_update(nncu_model *m, const int32_t *expected_host, float *loss_out);
int nncu_eval_gradient_update_dev(nncu_model *m, const int32_t *expected_dev);
/* Reads the loss of the last nncu_eval_gradient / _dev.  The loss is copied to the host right
   behind the backward pass, and this call waits for that copy only: work the host has queued
   since (nncu_update, the next nncu_eval) keeps running. */
int nncu_read_loss(nncu_model *m, float *loss_out);
/* model_update (nncp.c:1224-1235): optimizer step, then the memory shift. */
int nncu_update(nncu_model *m);
/* The two halves of nncu_update, for hosts that reduce gradients between
   ranks first: nncu_update == nncu_optimizer_step + nncu_memory_shift. */
int nncu_optimizer_step(nncu_model *m);
int nncu_memory_shift(nncu_model *m);
/* Blocks until everything queued on the model's stream has finished and
   reports a device-side error flag if one was raised. */
int nncu_synchronize(nncu_model *m);
/* Queues a one-thread kernel whose bounded wait (the mbar_wait of the GEMM and
   attention kernels, with a limit of 256 tries) runs out on a barrier nothing
   completes: the next nncu_synchronize returns NNCU_ERR_TIMEOUT, the one after
   NNCU_OK, and the model keeps working.  For tests of the error path; it has
   no counterpart in the reference, whose device waits are unbounded. */
int nncu_selftest_expired_wait(nncu_model *m);

/* ---- parameters (NCParamList, libnc.h:499-536) ---- */
int nncu_param_count(const nncu_model *m);
/* name_out (>= 32 bytes) gets the nncp.c parameter name ("w_q_0", "embed"...);
   offset is the element offset inside the flat fp32 buffers. */
int nncu_param_info(const nncu_model *m, int index, char *name_out, size_t name_cap,
                    size_t *numel_out, size_t *offset_out);
int nncu_param_get(nncu_model *m, int index, float *host_out, size_t numel);
int nncu_param_set(nncu_model *m, int index, const float *host_in, size_t numel);
int nncu_grad_get(nncu_model *m, int index, float *host_out, size_t numel);
/* Device addresses of the flat fp32 master-weight, gradient and second-moment
   buffers (n_floats each, same offsets).  A multi-GPU host all-reduces the
   gradient buffer between nncu_eval_gradient and nncu_optimizer_step. */
int nncu_flat_buffers(nncu_model *m, float **master_dev, float **grad_dev,
                      float **moment_dev, size_t *n_floats);
/*
 * Gradient exchange inside the library -- no counterpart in the reference, which is
 * single-device (the stream sharding of this build is described in nncp-metal_b200/dist.py).
 * With a communicator attached, nncu_eval_gradient* sums each layer's gradient slots over
 * the ranks (ncclAllReduce, fp32, on a stream of its own) as soon as that layer's backward
 * is complete, so the exchange overlaps the rest of the backward pass; on return the
 * gradient buffer holds the global sum and no separate all-reduce is needed.
 * Rank 0 makes the 128-byte id (nncu_comm_unique_id) and passes it to the other ranks by
 * any means (torch.distributed broadcast in bench.py); every rank then calls nncu_comm_init.
 * NCCL is loaded with dlopen("libnccl.so.2") on first use.
 */
int nncu_comm_unique_id(void *id_out_128_bytes);
int nncu_comm_init(nncu_model *m, int n_ranks, int rank, const void *id_128_bytes);
/*
 * With NNCU_SHARDED_UPDATE=1 in the environment, nncu_eval_gradient_update[_dev]
 * under a communicator shards the optimizer: each layer's matrices are
 * reduce-scattered, every rank updates its 1/N of them and the updated bf16
 * weights (fp32 in an fp32 model) are all-gathered; small parameters are
 * all-reduced and updated whole; the embedding gradient is rebuilt on every
 * rank from the gathered input ids and input gradients (that part alone is
 * the default; NNCU_SPARSE_EMBED=0 returns to the dense all-reduce).  Second moments and fp32 master weights of the
 * matrices are then current on the owning rank only.
 * nncu_comm_gather_master -- a collective: every rank calls it -- completes
 * them everywhere; nncu_param_get / _set, nncu_weights_hash,
 * nncu_eval_gradient and nncu_optimizer_step return NNCU_ERR_STATE until it
 * has run.  The default is one all-reduce per layer and the whole update on
 * every rank, which measured faster at 2 and 4 GPUs on the 55 M-parameter
 * model (csrc/model.cu, shard_enabled).
 */
int nncu_comm_gather_master(nncu_model *m);

/* 64-bit order-independent digest (sum of mixed (index, bit pattern) words) of the fp32
   master weights (DUMP_HASH-style check that
   ranks / runs hold identical weights, nncp.c:1062-1071). */
int nncu_weights_hash(nncu_model *m, uint64_t *hash_out);

/* ---- coder-ready output (write_sym / read_sym, cp_utils.c:299-349) ---- */
/*
 * For every row r in [t0*B, (t0+nt)*B) and its symbol sym[r - t0*B]
 * (int32, host), writes the 15-bit prob0 values that write_sym would pass
 * to put_bit, root first, to prob0_host [nt*B][n_bits] (uint16), n_bits =
 * ceil(log2 V).  V may be any size from 2 up (16384; 25600 when a power of
 * two): write_sym sends n >> 1 of a node's n symbols left, so for a V that
 * is not a power of two some leaves sit at depth n_bits - 1; such a row
 * uses n_bits - 1 values and its last entry is 0.  The partial sums use the
 * pairing vec_sum_f32(tab, n) = vec_sum_f32(tab, n/2) +
 * vec_sum_f32(tab + n/2, n - n/2), which is that same tree.
 */
int nncu_coder_paths(nncu_model *m, int t0, int nt, const int32_t *sym_host,
                     uint16_t *prob0_host, int *n_bits_out);
/*
 * The same in two halves, for an encoder: _begin queues the work behind the
 * forward pass and returns without waiting; _end waits for it and hands the
 * values over.  Between the two the host may call nncu_eval_gradient for
 * the segment (an encoder knows the targets already), so that the backward
 * pass is queued before the host starts range-coding and the GPU never
 * idles on the host.  No counterpart in the reference, whose process_block
 * (nncp.c:3003-3053) runs eval, coder and gradient strictly in turn; a
 * decoder, which learns the symbols only from the coder, keeps that order.
 * One _begin may be outstanding; NNCU_ERR_STATE otherwise.
 */
int nncu_coder_paths_begin(nncu_model *m, int t0, int nt, const int32_t *sym_host);
int nncu_coder_paths_end(nncu_model *m, uint16_t *prob0_host, int *n_bits_out);
/*
 * For the same rows writes the whole implicit tree: prob0 of node k
 * (heap order: root = 1, children 2k and 2k+1) at tree_host[row][k],
 * [nt*B][2^ceil(log2 V)] uint16, which is [nt*B][V] for a power of two
 * (entry 0 and the slots of one-symbol nodes hold 0).  read_sym then needs
 * no float math.
 */
int nncu_coder_trees(nncu_model *m, int t0, int nt, uint16_t *tree_host);
/*
 * The range decoder itself on the device (get_bit and read_sym, arith.c:241-310,
 * cp_utils.c:326-349): decoding needs the symbol of step t before step t+1 can
 * run, and the reference's decode loop (nncp.c:2996-3022) pays a device-to-host
 * round trip of the whole probability table for every symbol.  Here the coded
 * bytes are uploaded once, and each step runs forward, trees and the tree walk
 * back to back on the device, the decoded symbols feeding the next step's
 * input there; the host only collects the symbols of the steps it asked for.
 *
 * nncu_decoder_begin   uploads payload_host[0, len) and initialises low/range
 *                      as get_bit_init does.  NNCU_ERR_RANGE when the trees of
 *                      this n_symbols / n_streams do not fit shared memory (the
 *                      caller then decodes through nncu_coder_trees).
 * nncu_decode_steps    steps t0 .. t0+nt-1 of the current segment, t0 == the
 *                      number of steps done so far.  ids_t0_host [B] are the
 *                      inputs of step t0 (required when t0 == 0, else optional:
 *                      NULL keeps the symbols decoded at t0-1).  Streams past
 *                      the end of a block are skipped and yield 0: at step
 *                      t == limit_t those with index >= limit_b, and every
 *                      stream at t > limit_t (limit_t >= seg_len: none).
 *                      symbols_host [nt][B] receives the symbols; they are also
 *                      left in place as the targets of the gradient pass, which
 *                      nncu_eval_gradient overwrites with the same values.
 * nncu_decoder_end     reports how many payload bytes were consumed.
 */
int nncu_decoder_begin(nncu_model *m, const uint8_t *payload_host, size_t len);
int nncu_decode_steps(nncu_model *m, int t0, int nt, const int32_t *ids_t0_host,
                      int limit_t, int limit_b, int32_t *symbols_host);
int nncu_decoder_end(nncu_model *m, size_t *bytes_consumed);

/* ---- isolated attention op (the sub-graph nncp.c:722-800 and its autograd) ----
 * All pointers are device memory.  dtype_bf16 selects bf16 or fp32 for
 * q, kv, out and their gradients; w_r, b_r and their gradients are fp32.
 *   q    [T*B][H*dk]          row t*B+b
 *   kv   [L*B][2*H*dk]        row j*B+b; K in columns [0,H*dk), V after
 *   w_r  [H][P][dk]   (may be NULL: no position product)
 *   b_r  [H][L]
 *   out  [T*B][H*dk]
 *   lse  [B*H][T]  fp32 log-sum-exp of every score row (saved for backward)
 * score(i,j) = (q_i.k_j + q_i.w_r[max(r-(L-P),0)] + br_scale*b_r[r]) / sqrt(dk),
 * r = j + T-1-i, visible iff 0 <= i+M-j < attn_len.
 */
typedef struct nncu_attn_shape {
    int32_t n_streams, n_head, d_key, seg_len, mem_len, d_pos, attn_len;
    int32_t t0, t1; /* query time range [t0, t1) */
    float br_scale; /* sqrt(d_key * d_model) in the model (nncp.c:751-752) */
    int32_t dtype_bf16;
} nncu_attn_shape;

int nncu_attention_forward(const nncu_attn_shape *s, const void *q, const void *kv,
                           const float *w_r, const float *b_r, void *out, float *lse,
                           void *cuda_stream);
/*
 * Backward: dq [T*B][H*dk], dkv [L*B][2*H*dk] (same dtype as q), and the
 * per-(stream, head) partial table gradients dwr_part [B][H][P][dk],
 * dbr_part [B][H][L] (fp32), which the caller sums over streams in stream
 * order (nncu_attention_reduce_tables does exactly that).
 */
int nncu_attention_backward(const nncu_attn_shape *s, const void *q, const void *kv,
                            const float *w_r, const float *b_r, const void *out,
                            const float *lse, const void *dout, void *dq, void *dkv,
                            float *dwr_part, float *dbr_part, void *cuda_stream);
int nncu_attention_reduce_tables(const nncu_attn_shape *s, const float *dwr_part,
                                 const float *dbr_part, float *dw_r, float *db_r,
                                 int accumulate, void *cuda_stream);

/*
 * nncu_attention_backward_noalloc -- no counterpart in the reference.
 *
 * Same result as nncu_attention_backward followed by nncu_attention_reduce_tables
 * (accumulate = 0), for callers that cannot give the op a scratch buffer: a host that
 * has handed all of its device memory to its own pool at start-up, or a per-segment
 * loop that must not pay the device-wide synchronisation cudaMalloc and cudaFree imply.
 * The per-(stream, head) partial table gradients, which the plain entry point takes from
 * the caller, live here in one fixed array of NNCU_NOALLOC_SCRATCH_FLOATS floats (16 MiB)
 * that is part of the library image: every GPU that loads the library holds it until the
 * process exits.  The call allocates nothing and frees nothing.
 *
 *   - Needs n_streams * n_head * (d_pos * d_key + mem_len + seg_len) <= NNCU_NOALLOC_SCRATCH_FLOATS
 *     (the d_pos * d_key term only when w_r is given); larger shapes are refused with
 *     NNCU_ERR_RANGE and nothing is launched.
 *   - The first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress, with that device current).  Make that first call before
 *     starting any stream capture.
 *   - All calls share the one array.  Nothing in it has to start at zero (every partial the
 *     reduction reads is written first by the same call), and it keeps the last call's
 *     contents.  Two calls that overlap on the GPU (different streams, or different host
 *     threads) race on it: serialise them.
 * dw_r [H][P][dk] (may be NULL when w_r is NULL) and db_r [H][L] receive the table gradients
 * summed over streams in stream order.
 */
#define NNCU_NOALLOC_SCRATCH_FLOATS (4u << 20)
int nncu_attention_backward_noalloc(const nncu_attn_shape *s, const void *q, const void *kv,
                                    const float *w_r, const float *b_r, const void *out,
                                    const float *lse, const void *dout, void *dq, void *dkv,
                                    float *dw_r, float *db_r, void *cuda_stream);

/* ---- dense contraction used by every projection (nc_matmul, libnc.h:270-276) ----
 * C[M][N] = A[M][K] * B[N][K]^T (+ bias[N]), bf16 operands, fp32 accumulate,
 * C bf16 (c_is_f32 == 0) or fp32.  Exposed so that the tcgen05 kernel can be
 * checked against the SIMT one on the same inputs.  backend as gemm_backend.
 */
int nncu_gemm_bf16_nt(int backend, int M, int N, int K, const void *A, int lda,
                      const void *B, int ldb, void *C, int ldc, int c_is_f32,
                      const float *bias, void *cuda_stream);
/* The three operand arrangements of the train step (mode 0, 1, 2):
 *   0  C[m][n] = sum_k A[m][k] B[n][k]     y  = x W^T      (A [M][K], B [N][K])
 *   1  C[m][n] = sum_k A[m][k] B[k][n]     dx = dy W       (A [M][K], B [K][N])
 *   2  C[m][n] = sum_k A[k][m] B[k][n]     dW = dy^T x     (A [K][M], B [K][N])
 * The tensor-core engine reads the second and third arrangement in place (MN-major
 * operands); no transposed copies are made. */
int nncu_gemm_bf16(int backend, int mode, int M, int N, int K, const void *A, int lda,
                   const void *B, int ldb, void *C, int ldc, int c_is_f32, void *cuda_stream);

/* ---- measurement hooks (PROF_* buckets of libnc.h:16-65 count cycles per phase; here the
 * library counts its own kernel launches and, on request, times every launch of the
 * tensor-core GEMM with CUDA events on the launching stream) ---- */
typedef struct nncu_profile {
    uint64_t launches;      /* kernels launched by this library since nncu_profile_begin */
    uint64_t gemm_launches; /* timed tcgen05 GEMM launches */
    double gemm_ms;         /* sum of their device durations */
    double gemm_flops;      /* sum of 2*M*N*K over them */
} nncu_profile;
int nncu_profile_begin(int time_gemms);
int nncu_profile_end(nncu_profile *out);

#ifdef __cplusplus
}
#endif
#endif /* NNCU_H */
