// model.cu -- the Transformer-XL train step behind the C ABI of include/nncu.h.
//
// Host-side orchestration only; every number is produced by the kernels in
// gemm_simt.cuh, gemm_tc.cuh, attention.cuh, kernels.cuh and coder.cuh.
//
//   forward_range    trf_eval            nncp.c:581-1029
//   backward         trf_eval_gradient   nncp.c:1099-1193 (hand-derived adjoint)
//   optimizer_step   nc_sgd_opt_update   nncp.c:1229
//   memory_shift     mem_update          nncp.c:1205-1221
//
// Data layout in HBM.  A "row" is one (time, stream) position, row = time*B +
// stream, so the rows of one time step are contiguous: a one-symbol step is the
// batched forward restricted to a row range.  Per layer, hcat = [memory ; segment]
// rows (memory first) is the input of the K/V projection; the segment part is
// also the query input and what becomes memory after the step.  All layers'
// hcat live in one allocation with a twin: the memory shift copies rows
// [T*B, L*B) of every layer into rows [0, M*B) of the twin and swaps.
// Parameters, gradients and second moments are three flat fp32 buffers with
// identical offsets (512-byte aligned slots); bf16 models add a bf16 shadow
// and a transposed bf16 shadow of the matrices, refreshed by the optimizer.
#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <string.h>

#include <algorithm>
#include <initializer_list>
#include <string>
#include <vector>

#include "attention_mma.cuh"
#include "coder.cuh"

// ceil(log2 V): the depth of the coder's tree for any alphabet (its heap has 1 << depth slots per row)
static int coder_depth(int V)
{
    int n = 0;
    while ((1 << n) < V)
        n++;
    return n;
}
#include "common.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "kernels.cuh"
#include "decoder.cuh"

thread_local char g_nncu_err[512] = "";
unsigned long long g_nncu_launches = 0;
GemmProfiler *g_nncu_prof = nullptr;

int nncu_fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_nncu_err, sizeof(g_nncu_err), fmt, ap);
    va_end(ap);
    return code;
}

#define NONE ((size_t)-1)

// ------------------------------------------------------------------ NCCL (loaded at run time)
// Only what the gradient exchange needs, resolved with dlopen so that single-GPU hosts carry no
// NCCL dependency.  Types as in nccl.h: ncclComm_t is an opaque pointer, ncclUniqueId 128 bytes,
// ncclFloat32 = 7, ncclSum = 0.
typedef struct { char b[128]; } nccl_id_t;
struct NcclApi {
    void *dl;
    int (*GetUniqueId)(void *id);
    int (*CommInitRank)(void **comm, int nranks, nccl_id_t id, int rank);
    int (*AllReduce)(const void *send, void *recv, size_t count, int dtype, int op, void *comm, cudaStream_t st);
    int (*ReduceScatter)(const void *send, void *recv, size_t recvcount, int dtype, int op, void *comm, cudaStream_t st);
    int (*AllGather)(const void *send, void *recv, size_t sendcount, int dtype, void *comm, cudaStream_t st);
    int (*CommDestroy)(void *comm);
    const char *(*GetErrorString)(int);
};

static NcclApi *nccl_api()
{
    static NcclApi api;
    static int state = 0; // 0 untried, 1 ok, -1 unavailable
    if (state == 0) {
        void *dl = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL); // torch's copy, if loaded
        if (!dl)
            dl = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!dl)
            dl = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        state = -1;
        if (dl) {
            api.dl = dl;
            *(void **)&api.GetUniqueId = dlsym(dl, "ncclGetUniqueId");
            *(void **)&api.CommInitRank = dlsym(dl, "ncclCommInitRank");
            *(void **)&api.AllReduce = dlsym(dl, "ncclAllReduce");
            *(void **)&api.ReduceScatter = dlsym(dl, "ncclReduceScatter");
            *(void **)&api.AllGather = dlsym(dl, "ncclAllGather");
            *(void **)&api.CommDestroy = dlsym(dl, "ncclCommDestroy");
            *(void **)&api.GetErrorString = dlsym(dl, "ncclGetErrorString");
            if (api.GetUniqueId && api.CommInitRank && api.AllReduce && api.ReduceScatter && api.AllGather && api.CommDestroy &&
                api.GetErrorString)
                state = 1;
        }
    }
    return state == 1 ? &api : nullptr;
}

struct ParamInfo {
    char name[32];
    size_t numel, off;
    int rows, cols; // matrices that get a transposed shadow: rows x cols, else rows = 0
};

struct LayerOff {
    size_t w_q, w_kv, b_q, w_o, ff1, ff_bias1, ff2, ff_bias2, w_r, b_r, ln_g1, ln_b1, ln_g2, ln_b2;
    size_t alpha; // LN_COEF: the scalar both sub-layer outputs are multiplied by (NONE without the flag)
    size_t small; // the layer's slots are [w_q, small): the four matrices, then [small, next layer): everything else
};

struct LayerAct {
    void *xin, *qkv, *o, *s1, *y, *u, *hpre, *hact, *s2; // qkv: [L*B][q | k | v], q unused in memory rows
    void *ao = nullptr, *aff = nullptr;                  // LN_COEF: the sub-layer outputs before the multiplication
    float *lse, *st_pre1, *st_1, *st_pre2, *st_2;
};

struct TransposeJob {
    unsigned long long src_off, dst_off;
    int rows, cols, tile0, tiles_x;
};

constexpr int SPLITK = 4, SPLITK_MIN_K = 8192; // split-K of the output head's dX GEMM

struct nncu_model {
    nncu_params p;
    int D, H, dk, HD, F, F1, T, B, M, L, V, TB, LB, Bt, nl;
    bool bf;      // bf16 model
    bool use_tc;  // tcgen05 GEMMs
    size_t esz;   // bytes per activation element
    int device;
    cudaStream_t st;
    cudaStream_t st2;            // weight-gradient GEMMs run here, beside the dX chain
    cudaEvent_t ev_fork, ev_join;
    bool overlap;
    // CUDA graphs of the whole-segment forward and of the backward pass, one per memory twin
    struct StepGraph {
        cudaGraphExec_t exec;
        unsigned long long launches;
        int calls;
    } graphs[3][2]; // [forward, backward, backward with the optimizer step][memory twin]
    bool graphs_on;
    std::vector<StepGraph> step_graphs; // device decoder: one-symbol step + trees + decode, [t][memory twin]
    uint8_t *dec_payload = nullptr;     // the coded bytes on the device (nncu_decoder_begin)
    size_t dec_cap = 0;
    dec::State *dec_state = nullptr;
    int dec_ring = 0;
    bool dec_open = false;
    // gradient exchange between ranks (nncu_comm_init): per-layer all-reduces on a third stream,
    // issued as soon as a layer's gradients are complete, so they overlap the rest of backward
    void *comm;
    int comm_ranks, comm_rank = 0;
    bool shard_update = false;  // fused step under a communicator: reduce-scatter, update of the own shard, all-gather
    bool sparse_embed = false;  // ... and the embedding gradient rebuilt from gathered ids and rows
    bool master_stale = false;  // second moments (and, in a bf16 model, fp32 master weights) of the matrices are
                                // current only on the rank that owns the shard
    int32_t *ids_all = nullptr; // every rank's input ids and embedding-input gradients, gathered for the
    void *dx_all = nullptr;     // embedding gradient (nncu_comm_init)
    cudaStream_t st3;
    cudaEvent_t ev_bucket, ev_comm;
    size_t tail_begin; // first parameter slot after the last layer
    std::vector<ParamInfo> pinfo;
    std::vector<LayerOff> lo;
    size_t ln_g, ln_b, embed, embed_out, out_bias, n_floats;
    // device memory (one arena)
    char *arena;
    size_t arena_bytes;
    float *W, *G, *Vm;
    bf16 *Wb, *WbT;
    char *hcat[2];
    int cur;
    std::vector<LayerAct> act;
    void *xlast, *xf, *pool[4], *dz, *dh, *dhp, *dof, *dqkv, *tA, *tB;
    float *st_f, *probs, *dwr_part, *dbr_part, *part, *logp, *loss_dev;
    size_t part_floats = 0; // floats per region of `part`
    float *skw = nullptr;   // split-K workspace [SPLITK][TB][D] (models with n_symbols >= SPLITK_MIN_K)
    size_t skw_floats = 0;
    int part_idx = 0;       // regions handed out since the last join
    ReduceJobs rjobs;       // column / stream reductions queued since the last flush (one launch per layer)
    int rjob_blocks = 0;
    bool fuse_update = false; // this backward pass applies the optimizer to each bucket as it completes
    float *hyper_dev = nullptr; // {lr, bias correction} of the fused optimizer step
    int32_t *ids_dev, *tgt_dev;
    void *dt_ff = nullptr, *dt_at = nullptr; // LN_COEF: alpha * d(residual sum) of the two sub-layers, [TB][D]
    float *alpha_part = nullptr;             // LN_COEF: per-row shares of d alpha, [2][TB]
    int32_t *sym_dev;   // [TB] symbols whose coder paths are wanted (nncu_coder_paths*)
    int32_t *tgt_fixed; // the targets whose entries of dz carry the (p - 1) correction
    int *dz_fixed;      // device flag: dz has been corrected since the last forward pass
    int *first_dev;     // [V] smallest row carrying each symbol (embedding gradient)
    int *err_flag;
    unsigned long long *hash_dev;
    TransposeJob *jobs_dev;
    int n_jobs, n_job_tiles;
    uint16_t *coder_dev;
    size_t coder_bytes;
    // host staging (pinned)
    int32_t *ids_pin, *tgt_pin, *sym_pin; // pinned staging of ids, targets, coder symbols
    uint16_t *coder_pin;                  // pinned landing area of nncu_coder_paths_begin
    float *loss_pin;
    // recorded after the copy that reads (ids, tgt, sym) or writes (coder) the staging area;
    // the next user of the area waits for the event instead of draining the stream
    cudaEvent_t ev_ids = nullptr, ev_tgt = nullptr, ev_sym = nullptr, ev_coder = nullptr, ev_loss = nullptr;
    int loss_pending = 0; // the loss of the last backward pass is on its way to loss_pin
    int coder_rows = 0, coder_nb = 0; // what nncu_coder_paths_begin has in flight
    float lr;
    long step;
    int steps_done;
    bool have_forward;
};

// ------------------------------------------------------------------ helpers

template <typename AT> static inline AT *at(void *base, size_t elem) { return reinterpret_cast<AT *>(base) + elem; }
template <typename AT> static inline const AT *atc(const void *base, size_t elem) { return reinterpret_cast<const AT *>(base) + elem; }

static inline char *hcat_layer(nncu_model *m, int which, int l)
{
    return m->hcat[which] + (size_t)l * m->LB * m->D * m->esz;
}

// compute copy of a parameter: the fp32 master for fp32 models, the bf16 shadow otherwise
template <typename AT> static inline const AT *wptr(nncu_model *m, size_t off);
template <> inline const float *wptr<float>(nncu_model *m, size_t off) { return m->W + off; }
template <> inline const bf16 *wptr<bf16>(nncu_model *m, size_t off) { return m->Wb + off; }

static inline const float *wf(nncu_model *m, size_t off) { return off == NONE ? nullptr : m->W + off; }
static inline float *gf(nncu_model *m, size_t off) { return m->G + off; }

static int check_err_flag(nncu_model *m)
{
    int flag = 0;
    CUDA_TRY(cudaMemcpyAsync(&flag, m->err_flag, sizeof(int), cudaMemcpyDeviceToHost, m->st));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    if (flag != 0) {
        cudaMemsetAsync(m->err_flag, 0, sizeof(int), m->st);
        return nncu_fail(NNCU_ERR_TIMEOUT, "a bounded device-side wait expired (code %d)", flag);
    }
    return NNCU_OK;
}

// y = x W^T (+bias): C[M][N] = A[M][K] . Wt[N][K]^T
template <typename AT, typename TC>
static int mm_nt(nncu_model *m, int M, int N, int K, const AT *A, long lda, size_t w_off, TC *C,
                 long ldc, const float *bias, int bias_n = 1 << 30);

template <typename TC>
static int mm_nt_impl(nncu_model *m, int M, int N, int K, const float *A, long lda, size_t w_off,
                      TC *C, long ldc, const float *bias, int bias_n)
{
    return gemm_simt<float, float, TC>(m->st, GEMM_NT, M, N, K, A, lda, m->W + w_off, K, C, ldc, bias, 0,
                                       bias_n);
}
template <typename TC>
static int mm_nt_impl(nncu_model *m, int M, int N, int K, const bf16 *A, long lda, size_t w_off,
                      TC *C, long ldc, const float *bias, int bias_n)
{
    const bf16 *Wt = m->Wb + w_off;
    if (m->use_tc && tc::usable(A, lda, Wt, K, K))
        return tc::gemm_nt<TC>(m->st, M, N, K, A, lda, Wt, K, C, ldc, bias, nullptr, m->err_flag, bias_n);
    return gemm_simt<bf16, bf16, TC>(m->st, GEMM_NT, M, N, K, A, lda, Wt, K, C, ldc, bias, 0, bias_n);
}
// bias (if any) is added to output columns n < bias_n only
template <typename AT, typename TC>
static int mm_nt(nncu_model *m, int M, int N, int K, const AT *A, long lda, size_t w_off, TC *C,
                 long ldc, const float *bias, int bias_n)
{
    return mm_nt_impl<TC>(m, M, N, K, A, lda, w_off, C, ldc, bias, bias_n);
}

// MN-major tensor-core operands (default) or explicit transposes (NNCU_TC_TRANSPOSE=1)
static bool tc_mn_major()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("NNCU_TC_TRANSPOSE");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

// dx = dy W (+ addsrc): C[M][Kin] = dY[M][Nout] . W[Nout][Kin]
static int mm_nn(nncu_model *m, int M, int Kin, int Nout, const float *dY, long ldy, size_t w_off,
                 float *C, long ldc, const float *addsrc)
{
    if (addsrc && addsrc != C)
        CUDA_TRY(cudaMemcpy2DAsync(C, ldc * 4, addsrc, ldc * 4, (size_t)Kin * 4, M,
                                   cudaMemcpyDeviceToDevice, m->st));
    return gemm_simt<float, float, float>(m->st, GEMM_NN, M, Kin, Nout, dY, ldy, m->W + w_off, Kin,
                                          C, ldc, nullptr, addsrc ? 1 : 0);
}
static int mm_nn(nncu_model *m, int M, int Kin, int Nout, const bf16 *dY, long ldy, size_t w_off,
                 bf16 *C, long ldc, const bf16 *addsrc)
{
    if (m->use_tc && tc_mn_major() && tc::usable(dY, ldy, m->Wb + w_off, Kin, Nout)) {
        // W is [Nout][Kin] = [k][n]: read in place as an MN-major operand
        if (Nout >= SPLITK_MIN_K && !addsrc && m->skw && M % 128 == 0 && ldc == Kin && Kin % 4 == 0 &&
            (size_t)SPLITK * M * Kin <= m->skw_floats) {
            // a long contraction into few tiles (the output head's dX): four CTAs per tile
            NNCU_TRY((tc::gemm_splitk<false, true>(m->st, M, Kin, Nout, dY, ldy, m->Wb + w_off, Kin, m->skw, SPLITK,
                                                   m->err_flag)));
            const size_t n = (size_t)M * Kin;
            launch_k(splitk_reduce_kernel<bf16>, dim3((unsigned)ceil_div((long long)(n / 4), 256)), dim3(256), 0, m->st,
                     m->skw, SPLITK, n, C);
            KERNEL_CHECK();
            return NNCU_OK;
        }
        return tc::gemm<bf16, false, true>(m->st, M, Kin, Nout, dY, ldy, m->Wb + w_off, Kin, C, ldc, nullptr,
                                           addsrc, m->err_flag);
    }
    const bf16 *WT = m->WbT + w_off; // [Kin][Nout]
    if (m->use_tc && tc::usable(dY, ldy, WT, Nout, Nout))
        return tc::gemm_nt<bf16>(m->st, M, Kin, Nout, dY, ldy, WT, Nout, C, ldc, nullptr, addsrc,
                                 m->err_flag);
    if (addsrc && addsrc != C)
        CUDA_TRY(cudaMemcpy2DAsync(C, ldc * 2, addsrc, ldc * 2, (size_t)Kin * 2, M,
                                   cudaMemcpyDeviceToDevice, m->st));
    return gemm_simt<bf16, bf16, bf16>(m->st, GEMM_NN, M, Kin, Nout, dY, ldy, m->Wb + w_off, Kin, C,
                                       ldc, nullptr, addsrc ? 1 : 0);
}

// dW = dY^T X: G[Nout][Kin] = sum over R rows of dY[r][Nout] X[r][Kin]   (fp32 result)
// The weight gradients are off the critical path of the backward pass (nothing downstream
// reads them before the optimizer), so they go to a second stream: fork after the operands
// exist, join once per layer before any operand buffer is reused.
static cudaStream_t side_fork(nncu_model *m)
{
    if (!m->overlap || g_nncu_prof)
        return m->st;
    cudaEventRecord(m->ev_fork, m->st);
    cudaStreamWaitEvent(m->st2, m->ev_fork, 0);
    return m->st2;
}
static void side_join(nncu_model *m)
{
    m->part_idx = 0;
    if (!m->overlap || g_nncu_prof)
        return;
    cudaEventRecord(m->ev_join, m->st2);
    cudaStreamWaitEvent(m->st, m->ev_join, 0);
}
// Partial column sums go to one of PART_SLOTS scratch regions, so that the kernel that reduces
// them can run on the side stream while the main stream's next kernel fills another region.
// At most nine regions are taken between two joins (output bias, final norm, four norms, the
// activation, two bias sums); a join makes all of them free again.
constexpr int PART_SLOTS = 10;
static float *part_slot(nncu_model *m)
{
    float *p = m->part + (size_t)(m->part_idx % PART_SLOTS) * m->part_floats;
    m->part_idx++;
    return p;
}

static int mm_tn(nncu_model *m, int Nout, int Kin, int R, const float *dY, long ldy, const float *X,
                 long ldx, float *Gout)
{
    return gemm_simt<float, float, float>(side_fork(m), GEMM_TN, Nout, Kin, R, dY, ldy, X, ldx, Gout, Kin,
                                          nullptr, 0);
}
static int mm_tn(nncu_model *m, int Nout, int Kin, int R, const bf16 *dY, long ldy, const bf16 *X,
                 long ldx, float *Gout)
{
    if (m->use_tc && tc_mn_major() && tc::usable(dY, ldy, X, ldx, R))
        // dY is [R][Nout] = [k][m], X is [R][Kin] = [k][n]: both MN-major, read in place
        return tc::gemm<float, true, true>(side_fork(m), Nout, Kin, R, dY, ldy, X, ldx, Gout, Kin, nullptr,
                                           nullptr, m->err_flag);
    if (m->use_tc && (R % 8) == 0) {
        // both operands become K-major by an explicit transpose (the contraction runs over rows)
        bf16 *tA = reinterpret_cast<bf16 *>(m->tA), *tB = reinterpret_cast<bf16 *>(m->tB);
        transpose_bf16_kernel<<<dim3(ceil_div(Nout, 32), ceil_div(R, 32)), 256, 0, m->st>>>(
            dY, ldy, tA, R, R, Nout);
        KERNEL_CHECK();
        transpose_bf16_kernel<<<dim3(ceil_div(Kin, 32), ceil_div(R, 32)), 256, 0, m->st>>>(
            X, ldx, tB, R, R, Kin);
        KERNEL_CHECK();
        return tc::gemm_nt<float>(m->st, Nout, Kin, R, tA, R, tB, R, Gout, Kin, nullptr, nullptr,
                                  m->err_flag);
    }
    return gemm_simt<bf16, bf16, float>(side_fork(m), GEMM_TN, Nout, Kin, R, dY, ldy, X, ldx, Gout, Kin,
                                        nullptr, 0);
}

// The column and stream reductions of the backward pass only write gradient buffers, which nobody
// reads before the optimizer: they are queued and run as ONE launch per layer on the side stream
// (flush_reductions, in front of the layer's join), instead of a 5 us launch each.
static int flush_reductions(nncu_model *m)
{
    if (m->rjobs.n_jobs == 0)
        return NNCU_OK;
    launch_k(reduce_jobs_kernel, dim3(m->rjob_blocks), dim3(256), 0, side_fork(m), m->rjobs);
    m->rjobs.n_jobs = 0;
    m->rjob_blocks = 0;
    KERNEL_CHECK();
    return NNCU_OK;
}
static int queue_reduction(nncu_model *m, int kind, const float *part, int n_parts, int stride, int n, int off, float *out,
                           int accumulate)
{
    if (m->rjobs.n_jobs == MAX_REDUCE_JOBS)
        NNCU_TRY(flush_reductions(m));
    ReduceJob &j = m->rjobs.job[m->rjobs.n_jobs++];
    j.part = part; j.out = out; j.n_parts = n_parts; j.stride = stride; j.n = n; j.off = off; j.kind = kind;
    j.accumulate = accumulate; j.blk0 = m->rjob_blocks;
    m->rjob_blocks += kind == 1 ? ceil_div(n, 256) : ceil_div(n, 32);
    return NNCU_OK;
}
// out_k[c] = sum over parts of part[p*stride + off_k + c], up to three outputs
static int reduce_cols(nncu_model *m, const float *part, int n_parts, int stride, int n, float *o0, int off0,
                       float *o1 = nullptr, int off1 = 0, float *o2 = nullptr, int off2 = 0)
{
    NNCU_TRY(queue_reduction(m, 0, part, n_parts, stride, n, off0, o0, 0));
    if (o1)
        NNCU_TRY(queue_reduction(m, 0, part, n_parts, stride, n, off1, o1, 0));
    if (o2)
        NNCU_TRY(queue_reduction(m, 0, part, n_parts, stride, n, off2, o2, 0));
    return NNCU_OK;
}

template <typename AT>
static int colsum(nncu_model *m, const AT *A, long lda, int R, int N, float *out)
{
    const int rows_per = 64;
    int chunks = ceil_div(R, rows_per);
    float *part = part_slot(m);
    launch_k(colsum_part_kernel<AT>, dim3(ceil_div(N, 128), chunks), dim3(128), 0, side_fork(m), A, lda, R, N, rows_per, part);
    KERNEL_CHECK();
    return reduce_cols(m, part, chunks, N, N, out, 0);
}

template <typename AT>
static int norm_fwd(nncu_model *m, const AT *a, const AT *res, AT *s_out, AT *y, size_t g_off,
                    size_t b_off, float *stats, int rows, bool do_norm)
{
    int mode = !do_norm ? 0 : ((m->p.ln_flags & NNCU_LN_RMSNORM) ? 2 : 1);
    const float *g = do_norm ? m->W + g_off : nullptr, *b = do_norm ? m->W + b_off : nullptr;
    if (sizeof(AT) == 2 && (m->D == 256 || m->D == 512 || m->D == 1024 || m->D == 2048)) {
        // rows that fit in a warp's registers: one pass, 16-byte accesses
        const bf16 *a16 = (const bf16 *)a, *r16 = (const bf16 *)res;
        bf16 *s16 = (bf16 *)s_out, *y16 = (bf16 *)y;
        const dim3 grid(ceil_div(rows, 4)), block(128);
        switch (m->D / 256) {
        case 1: launch_k(residual_norm_vec_kernel<1>, grid, block, 0, m->st, a16, r16, s16, y16, g, b, stats, rows, mode); break;
        case 2: launch_k(residual_norm_vec_kernel<2>, grid, block, 0, m->st, a16, r16, s16, y16, g, b, stats, rows, mode); break;
        case 4: launch_k(residual_norm_vec_kernel<4>, grid, block, 0, m->st, a16, r16, s16, y16, g, b, stats, rows, mode); break;
        default: launch_k(residual_norm_vec_kernel<8>, grid, block, 0, m->st, a16, r16, s16, y16, g, b, stats, rows, mode); break;
        }
        KERNEL_CHECK();
        return NNCU_OK;
    }
    launch_k(residual_norm_kernel<AT>, dim3(ceil_div(rows, 4)), dim3(128), 0, m->st, a, res, s_out, y, g, b, stats,
             rows, m->D, mode);
    KERNEL_CHECK();
    return NNCU_OK;
}

template <typename AT>
static int norm_bwd(nncu_model *m, const AT *dy, const AT *x, size_t g_off, size_t b_off,
                    const float *stats, const AT *base, AT *dx, int rows, float *dxsum = nullptr)
{
    const int rpb = 8;
    int blocks = ceil_div(rows, rpb);
    int mode = (m->p.ln_flags & NNCU_LN_RMSNORM) ? 2 : 1;
    size_t smem = (size_t)8 * 3 * m->D * sizeof(float);
    float *part = part_slot(m);
    if (sizeof(AT) == 2 && (m->D == 256 || m->D == 512 || m->D == 1024)) {
        const bf16 *dy16 = (const bf16 *)dy, *x16 = (const bf16 *)x, *b16 = (const bf16 *)base;
        bf16 *dx16 = (bf16 *)dx;
        const float *g = m->W + g_off;
        const int ws = dxsum ? 1 : 0;
        switch (m->D / 256) {
        case 1: launch_k(norm_bwd_vec_kernel<1>, dim3(blocks), dim3(256), smem, m->st, dy16, x16, g, stats, b16, dx16, part, rows, mode, ws); break;
        case 2: launch_k(norm_bwd_vec_kernel<2>, dim3(blocks), dim3(256), smem, m->st, dy16, x16, g, stats, b16, dx16, part, rows, mode, ws); break;
        default: launch_k(norm_bwd_vec_kernel<4>, dim3(blocks), dim3(256), smem, m->st, dy16, x16, g, stats, b16, dx16, part, rows, mode, ws); break;
        }
    } else {
        launch_k(norm_bwd_kernel<AT>, dim3(blocks), dim3(256), smem, m->st, dy, x, m->W + g_off, stats, base, dx, part,
                 rows, m->D, mode, rpb, dxsum ? 1 : 0);
    }
    KERNEL_CHECK();
    return reduce_cols(m, part, blocks, 3 * m->D, m->D, gf(m, g_off), 0, gf(m, b_off), m->D, dxsum, 2 * m->D);
}

static nncu_attn_shape attn_shape(nncu_model *m, int l, int t0, int t1)
{
    nncu_attn_shape s;
    s.n_streams = m->B; s.n_head = m->H; s.d_key = m->dk; s.seg_len = m->T; s.mem_len = m->M;
    s.d_pos = m->p.d_pos; s.attn_len = m->p.attn_len[l] ? m->p.attn_len[l] : m->L;
    s.t0 = t0; s.t1 = t1;
    s.br_scale = sqrtf((float)m->dk * (float)m->D);
    s.dtype_bf16 = m->bf ? 1 : 0;
    return s;
}

// ------------------------------------------------------------------ CUDA graphs
//
// A train step is some 370 launches of 5-20 us kernels: launch gaps are a tenth of it.  When
// the model runs on a capturable stream (anything but the legacy default stream), the second
// whole-segment forward / backward issued for a memory twin is captured (side stream and
// all) and later ones replay the graph.  Operand addresses never change: ids and targets are
// copied into fixed staging buffers before the graph runs, and the two memory twins have
// a graph each.  One-symbol steps, the optimizer (its learning rate is a launch argument) and
// the timed-GEMM profiling pass stay eager.
enum { GRAPH_FWD = 0, GRAPH_BWD = 1, GRAPH_BWD_UPD = 2, N_GRAPH_KINDS = 3 };

template <typename F>
static int run_graphed(nncu_model *m, nncu_model::StepGraph &g, F body)
{
    const bool can = m->graphs_on && m->st != nullptr && m->st != cudaStreamLegacy && !g_nncu_prof;
    if (!can)
        return body();
    if (g.exec) {
        CUDA_TRY(cudaGraphLaunch(g.exec, m->st));
        g_nncu_launches += g.launches;
        return NNCU_OK;
    }
    if (g.calls++ < 1)
        return body(); // first call eager: kernel attributes and tensor maps get set up
    const unsigned long long before = g_nncu_launches;
    if (cudaStreamBeginCapture(m->st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        m->graphs_on = false;
        return body();
    }
    int rc = body();
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(m->st, &graph);
    if (rc == NNCU_OK && e == cudaSuccess && graph)
        e = cudaGraphInstantiate(&g.exec, graph, 0);
    if (graph)
        cudaGraphDestroy(graph);
    if (rc != NNCU_OK || e != cudaSuccess || !g.exec) {
        // nothing was executed during the capture: give up on graphs and run it for real
        cudaGetLastError();
        g.exec = nullptr;
        m->graphs_on = false;
        g_nncu_launches = before;
        return rc != NNCU_OK ? rc : body();
    }
    g.launches = g_nncu_launches - before;
    g_nncu_launches = before;
    CUDA_TRY(cudaGraphLaunch(g.exec, m->st));
    g_nncu_launches += g.launches;
    return NNCU_OK;
}

template <typename F>
static int run_graphed(nncu_model *m, int kind, F body)
{
    return run_graphed(m, m->graphs[kind][m->cur], body);
}

// ------------------------------------------------------------------ forward

template <typename AT>
static int forward_range(nncu_model *m, int t0, int t1)
{
    const nncu_params &p = m->p;
    const int D = m->D, HD = m->HD, F = m->F, F1 = m->F1, B = m->B, M = m->M, V = m->V;
    const int r0 = t0 * B, nr = (t1 - t0) * B;
    const bool pre = p.ln_flags & NNCU_LN_PRE, post = p.ln_flags & NNCU_LN_POST;
    const float emul = sqrtf((float)D) * p.embed_mult;
    AT *tmp = reinterpret_cast<AT *>(m->pool[0]); // [TB][D] scratch

    launch_k(embed_kernel<AT>, dim3(nr), dim3(128), 0, m->st, m->ids_dev + r0, m->W + m->embed,
                                            at<AT>(m->act[0].xin, (size_t)r0 * D), nr, D, emul, V);
    KERNEL_CHECK();
    for (int l = 0; l < m->nl; l++) {
        const LayerOff &o = m->lo[l];
        LayerAct &a = m->act[l];
        AT *hc = reinterpret_cast<AT *>(hcat_layer(m, m->cur, l));
        AT *x1 = hc + ((size_t)M * B + r0) * D;   // attention input of these rows (train_h)
        AT *xin = at<AT>(a.xin, (size_t)r0 * D);  // residual-stream input
        if (pre)
            NNCU_TRY(norm_fwd<AT>(m, xin, nullptr, nullptr, x1, o.ln_g1, o.ln_b1, a.st_pre1 + 2 * r0, nr, true));
        // fused projections over [memory ; segment]: Q for the segment rows, K|V for the
        // memory rows (once per segment) and the segment rows (nncp.c:659-695)
        // one GEMM against [w_q ; w_kv] (adjacent in the flat buffers): rows of the memory get
        // a q they never use, which costs less than a second launch
        // one GEMM over [memory ; segment] rows.  Measured alternative: the memory rows' K|V projections of
        // all layers on the side stream at the start of the pass, the main chain projecting the segment
        // rows only -- 2.686 against 2.594 ms per step: twelve more launches competing for SMs cost the
        // latency-bound main chain more than the shorter projection saves.
        if (t0 == 0 && M > 0)
            NNCU_TRY((mm_nt<AT, AT>(m, M * B + nr, 3 * HD, D, hc, D, o.w_q, at<AT>(a.qkv, 0), 3 * HD,
                                    wf(m, o.b_q), HD)));
        else
            NNCU_TRY((mm_nt<AT, AT>(m, nr, 3 * HD, D, x1, D, o.w_q,
                                    at<AT>(a.qkv, ((size_t)M * B + r0) * 3 * HD), 3 * HD, wf(m, o.b_q), HD)));
        nncu_attn_shape s = attn_shape(m, l, t0, t1);
        const AttnPitch pt = {3 * HD, 3 * HD, 3 * HD, 3 * HD};
        NNCU_TRY(attn_forward_any<AT>(&s, at<AT>(a.qkv, (size_t)M * B * 3 * HD), at<AT>(a.qkv, HD),
                                      wf(m, o.w_r), m->W + o.b_r, a.o, a.lse, m->st, &pt,
                                      (m->bf && o.w_r != NONE) ? m->Wb + o.w_r : nullptr, m->err_flag));
        // output projection, residual, post-LN (nncp.c:865-920)
        if (o.alpha != NONE) { // LN_COEF: the projection is kept as it is for the backward pass, tmp = alpha * it
            AT *ao = at<AT>(a.ao, (size_t)r0 * D);
            NNCU_TRY((mm_nt<AT, AT>(m, nr, D, HD, at<AT>(a.o, (size_t)r0 * HD), HD, o.w_o, ao, D, nullptr)));
            launch_k(scale_rows_kernel<AT>, dim3(ceil_div((long long)nr * D, 256)), dim3(256), 0, m->st, (const AT *)ao,
                     (const float *)(m->W + o.alpha), tmp, (size_t)nr * D);
            KERNEL_CHECK();
        } else {
            NNCU_TRY((mm_nt<AT, AT>(m, nr, D, HD, at<AT>(a.o, (size_t)r0 * HD), HD, o.w_o, tmp, D, nullptr)));
        }
        AT *yy = at<AT>(a.y, (size_t)r0 * D);
        NNCU_TRY(norm_fwd<AT>(m, tmp, xin, post ? at<AT>(a.s1, (size_t)r0 * D) : nullptr, yy, o.ln_g1,
                              o.ln_b1, a.st_1 + 2 * r0, nr, post));
        // feed-forward (nncp.c:925-986)
        AT *u = yy;
        if (pre) {
            u = at<AT>(a.u, (size_t)r0 * D);
            NNCU_TRY(norm_fwd<AT>(m, yy, nullptr, nullptr, u, o.ln_g2, o.ln_b2, a.st_pre2 + 2 * r0, nr, true));
        }
        AT *hpre = at<AT>(a.hpre, (size_t)r0 * F1), *hact = at<AT>(a.hact, (size_t)r0 * F);
        NNCU_TRY((mm_nt<AT, AT>(m, nr, F1, D, u, D, o.ff1, hpre, F1, wf(m, o.ff_bias1))));
        if (sizeof(AT) == 2 && F % 8 == 0 && F1 % 8 == 0)
            launch_k(act_fwd_vec_kernel, dim3(ceil_div((long long)nr * (F / 8), 256)), dim3(256), 0, m->st,
                     (const bf16 *)hpre, (bf16 *)hact, nr, F, F1, p.ff_act);
        else
            act_fwd_kernel<AT><<<ceil_div((long long)nr * F, 256), 256, 0, m->st>>>(hpre, hact, nr, F, F1, p.ff_act);
        KERNEL_CHECK();
        if (o.alpha != NONE) {
            AT *aff = at<AT>(a.aff, (size_t)r0 * D);
            NNCU_TRY((mm_nt<AT, AT>(m, nr, D, F, hact, F, o.ff2, aff, D, wf(m, o.ff_bias2))));
            launch_k(scale_rows_kernel<AT>, dim3(ceil_div((long long)nr * D, 256)), dim3(256), 0, m->st, (const AT *)aff,
                     (const float *)(m->W + o.alpha), tmp, (size_t)nr * D);
            KERNEL_CHECK();
        } else {
            NNCU_TRY((mm_nt<AT, AT>(m, nr, D, F, hact, F, o.ff2, tmp, D, wf(m, o.ff_bias2))));
        }
        AT *xout = (l + 1 < m->nl) ? at<AT>(m->act[l + 1].xin, (size_t)r0 * D)
                                   : at<AT>(m->xlast, (size_t)r0 * D);
        NNCU_TRY(norm_fwd<AT>(m, tmp, yy, post ? at<AT>(a.s2, (size_t)r0 * D) : nullptr, xout, o.ln_g2,
                              o.ln_b2, a.st_2 + 2 * r0, nr, post));
    }
    AT *xf = at<AT>(m->xlast, (size_t)r0 * D);
    if (p.ln_flags & NNCU_LN_FINAL) {
        xf = at<AT>(m->xf, (size_t)r0 * D);
        NNCU_TRY(norm_fwd<AT>(m, at<AT>(m->xlast, (size_t)r0 * D), nullptr, nullptr, xf, m->ln_g, m->ln_b,
                              m->st_f + 2 * r0, nr, true));
    }
    float *pr = m->probs + (size_t)r0 * V;
    NNCU_TRY((mm_nt<AT, float>(m, nr, V, D, xf, D, m->embed_out, pr, V, wf(m, m->out_bias))));
    // the output kernel: probabilities for the coder, and p / (T * B) for the backward pass
    AT *dzr = reinterpret_cast<AT *>(m->dz) + (size_t)r0 * V;
    const float sc = 1.0f / ((float)m->T * (float)m->Bt);
    if (V % 1024 == 0 && V <= 16384)
        launch_k(softmax_rows_reg_kernel<AT>, dim3(nr), dim3(256), 0, m->st, pr, nr, V, dzr, sc, m->dz_fixed);
    else
        launch_k(softmax_rows_kernel<AT>, dim3(nr), dim3(256), 0, m->st, pr, nr, V, dzr, sc, m->dz_fixed);
    KERNEL_CHECK();
    return NNCU_OK;
}

// sum G[begin, end) over the ranks on the communication stream, after everything queued on
// the main stream so far
static int exchange_bucket(nncu_model *m, size_t begin, size_t end)
{
    if (!m->comm || end <= begin)
        return NNCU_OK;
    NcclApi *nc = nccl_api();
    CUDA_TRY(cudaEventRecord(m->ev_bucket, m->st));
    CUDA_TRY(cudaStreamWaitEvent(m->st3, m->ev_bucket, 0));
    int r = nc->AllReduce(m->G + begin, m->G + begin, end - begin, 7 /* ncclFloat32 */, 0 /* ncclSum */, m->comm, m->st3);
    if (r != 0)
        return nncu_fail(NNCU_ERR_CUDA, "ncclAllReduce: %s", nc->GetErrorString(r));
    return NNCU_OK;
}
static int exchange_finish(nncu_model *m)
{
    if (!m->comm)
        return NNCU_OK;
    CUDA_TRY(cudaEventRecord(m->ev_comm, m->st3));
    CUDA_TRY(cudaStreamWaitEvent(m->st, m->ev_comm, 0));
    return NNCU_OK;
}

// Fused optimizer step: the RMSProp update of the gradient slots [begin, end), queued as soon as
// they are final -- behind the bucket's all-reduce on the exchange stream, or on the side stream.
// The update streams 22 bytes per parameter while the rest of the backward pass is latency-bound,
// so the two overlap well.  lr and the bias correction come from device memory (the launch is
// part of a captured graph).
static int opt_range(nncu_model *m, size_t begin, size_t end, bool last)
{
    if (!m->fuse_update || end <= begin)
        return NNCU_OK;
    // Measured on the c2 step of one process: the same update throttled to 48 / 96 / 192 blocks on a
    // third stream, so that it would trickle along under the latency-bound kernels of the remaining
    // layers, gave 2.94 / 2.82 / 2.76 ms per step against 2.61 for the separate full-width pass: a
    // block of 256 threads keeps too few loads in flight, and the pass outlasts the backward pass.
    cudaStream_t st = m->comm ? m->st3 : (last ? m->st : side_fork(m));
    const size_t n4 = (end - begin) / 4;
    const unsigned blocks = (unsigned)ceil_div((long long)n4, 256);
    launch_k(rmsprop_kernel, dim3(blocks), dim3(256), 0, st, m->W + begin, m->G + begin,
             m->Vm + begin, m->Wb ? m->Wb + begin : (bf16 *)nullptr, n4, 0.0f, m->p.beta2, m->p.eps, m->p.gradient_clip,
             1.0f, (const float *)m->hyper_dev);
    KERNEL_CHECK();
    return NNCU_OK;
}

// A bucket of gradient slots whose exchange and update are queued together: [begin, mid) are
// matrices, [mid, end) the small parameters behind them.  One process, or a caller that wants the
// summed gradients whole (nncu_eval_gradient): all-reduce, then the update of the whole range on
// every rank.  The fused step under a communicator: the matrices are reduce-scattered, each rank
// applies RMSProp to its 1/N of them and the updated bf16 shadows (fp32 weights of an fp32 model)
// are all-gathered, so the optimizer streams 22 bytes per parameter over 1/N of the matrices and
// the exchange moves 6 bytes per parameter instead of 8; the small parameters, which forward and
// backward read in fp32, stay whole on every rank (all-reduce, replicated update).  The fp32
// master copy of a matrix is then current only on the rank that owns its shard
// (nncu_comm_gather_master).  Every NCCL call of a bucket is queued on the exchange stream in the
// same order on every rank.
static int nccl_ok(int r, const char *what)
{
    if (r != 0)
        return nncu_fail(NNCU_ERR_CUDA, "%s: %s", what, nccl_api()->GetErrorString(r));
    return NNCU_OK;
}
enum { NCCL_F32 = 7, NCCL_BF16 = 9, NCCL_I32 = 2, NCCL_SUM = 0 };

static int exchange_update(nncu_model *m, size_t begin, size_t mid, size_t end)
{
    if (!m->comm || !m->shard_update) {
        NNCU_TRY(exchange_bucket(m, begin, end));
        return opt_range(m, begin, end, false);
    }
    NcclApi *nc = nccl_api();
    const size_t N = (size_t)m->comm_ranks, nbig = mid - begin;
    CUDA_TRY(cudaEventRecord(m->ev_bucket, m->st));
    CUDA_TRY(cudaStreamWaitEvent(m->st3, m->ev_bucket, 0));
    if (nbig && nbig % (4 * N) == 0) {
        const size_t chunk = nbig / N, mine = begin + chunk * (size_t)m->comm_rank;
        NNCU_TRY(nccl_ok(nc->ReduceScatter(m->G + begin, m->G + mine, chunk, NCCL_F32, NCCL_SUM, m->comm, m->st3), "ncclReduceScatter"));
        NNCU_TRY(opt_range(m, mine, mine + chunk, false));
        if (m->Wb) {
            NNCU_TRY(nccl_ok(nc->AllGather(m->Wb + mine, m->Wb + begin, chunk, NCCL_BF16, m->comm, m->st3), "ncclAllGather"));
        } else {
            NNCU_TRY(nccl_ok(nc->AllGather(m->W + mine, m->W + begin, chunk, NCCL_F32, m->comm, m->st3), "ncclAllGather"));
        }
    } else if (nbig) {
        NNCU_TRY(nccl_ok(nc->AllReduce(m->G + begin, m->G + begin, nbig, NCCL_F32, NCCL_SUM, m->comm, m->st3), "ncclAllReduce"));
        NNCU_TRY(opt_range(m, begin, mid, false));
    }
    if (end > mid) {
        NNCU_TRY(nccl_ok(nc->AllReduce(m->G + mid, m->G + mid, end - mid, NCCL_F32, NCCL_SUM, m->comm, m->st3), "ncclAllReduce"));
        NNCU_TRY(opt_range(m, mid, end, false));
    }
    return NNCU_OK;
}

// Layers per gradient exchange.  One all-reduce per layer overlaps best, but each NCCL operation has
// a fixed cost that grows with the number of ranks (a ring all-reduce is 2(N-1) hops), so at 8
// ranks several layers share one.  NNCU_BUCKET_LAYERS overrides.  The sharded update keeps one.
static int bucket_layers(nncu_model *m)
{
    if (!m->comm || m->shard_update)
        return 1;
    static int env = -1;
    if (env < 0) {
        const char *e = getenv("NNCU_BUCKET_LAYERS");
        env = e ? std::max(1, atoi(e)) : 0;
    }
    if (env)
        return env;
    return m->comm_ranks >= 8 ? 2 : 1; // measured at 8 GPUs (symbols/s): 1 layer 907 k, 2 layers 979 k, 4 layers 973 k, 12 layers 845 k
}

// ------------------------------------------------------------------ backward

template <typename AT>
static AT *pick(nncu_model *m, std::initializer_list<const void *> used)
{
    for (int i = 0; i < 4; i++) {
        bool taken = false;
        for (const void *u : used)
            if (u == m->pool[i])
                taken = true;
        if (!taken)
            return reinterpret_cast<AT *>(m->pool[i]);
    }
    return nullptr;
}

template <typename AT>
static int backward(nncu_model *m)
{
    const nncu_params &p = m->p;
    const int D = m->D, HD = m->HD, F = m->F, F1 = m->F1, B = m->B, M = m->M, V = m->V;
    const int TB = m->TB, LB = m->LB;
    const bool pre = p.ln_flags & NNCU_LN_PRE, post = p.ln_flags & NNCU_LN_POST;
    AT *dz = reinterpret_cast<AT *>(m->dz);
    AT *dh = reinterpret_cast<AT *>(m->dh), *dhp = reinterpret_cast<AT *>(m->dhp);
    AT *dof = reinterpret_cast<AT *>(m->dof);
    // [L*B][dq | dk | dv]; the dq columns of the memory rows are never written and stay zero
    AT *dqkv = reinterpret_cast<AT *>(m->dqkv);
    AT *dq = dqkv + (size_t)M * B * 3 * HD, *dkv = dqkv + HD;
    const AttnPitch pt = {3 * HD, 3 * HD, 3 * HD, 3 * HD};

    // loss and d logits (nncp.c:1170-1175)
    const float sc = 1.0f / ((float)m->T * (float)m->Bt);
    if (!(m->comm && m->sparse_embed)) {
        // which row carries each symbol first: needed only by the embedding gradient at the very end
        cudaStream_t s2 = side_fork(m);
        CUDA_TRY(cudaMemsetAsync(m->first_dev, 0x7f, sizeof(int) * (size_t)V, s2));
        launch_k(first_rows_kernel, dim3(ceil_div(TB, 256)), dim3(256), 0, s2, (const int32_t *)m->ids_dev, TB, V, m->first_dev);
        KERNEL_CHECK();
    }
    launch_k(loss_fix_kernel<AT>, dim3(ceil_div(TB, 256)), dim3(256), 0, m->st, (const float *)m->probs, (const int32_t *)m->tgt_dev,
             m->tgt_fixed, (const int *)m->dz_fixed, dz, m->logp, TB, V, sc);
    KERNEL_CHECK();
    launch_k(loss_sum_kernel, dim3(1), dim3(256), 0, m->st, (const float *)m->logp, TB, m->loss_dev, m->dz_fixed);
    KERNEL_CHECK();
    const AT *xf = (p.ln_flags & NNCU_LN_FINAL) ? atc<AT>(m->xf, 0) : atc<AT>(m->xlast, 0);
    if (m->out_bias != NONE)
        NNCU_TRY(colsum<AT>(m, dz, V, TB, V, gf(m, m->out_bias)));
    NNCU_TRY(mm_tn(m, V, D, TB, dz, V, xf, D, gf(m, m->embed_out)));
    AT *dx = pick<AT>(m, {});
    NNCU_TRY(mm_nn(m, TB, D, V, dz, V, m->embed_out, dx, D, (const AT *)nullptr));
    if (p.ln_flags & NNCU_LN_FINAL) {
        AT *t = pick<AT>(m, {dx});
        NNCU_TRY(norm_bwd<AT>(m, dx, atc<AT>(m->xlast, 0), m->ln_g, m->ln_b, m->st_f, nullptr, t, TB));
        dx = t;
    }
    // tied tables collect the contributions of every layer
    if (p.tied_b_r)
        CUDA_TRY(cudaMemsetAsync(gf(m, m->lo[0].b_r), 0, sizeof(float) * (size_t)m->H * m->L, m->st));
    if (p.use_w_r && p.tied_w_r)
        CUDA_TRY(cudaMemsetAsync(gf(m, m->lo[0].w_r), 0, sizeof(float) * (size_t)m->H * p.d_pos * m->dk, m->st));

    for (int l = m->nl - 1; l >= 0; l--) {
        const LayerOff &o = m->lo[l];
        LayerAct &a = m->act[l];
        const AT *hc = reinterpret_cast<const AT *>(hcat_layer(m, m->cur, l));
        // ---- feed-forward block
        AT *ds2 = dx;
        const bool coef = o.alpha != NONE;
        if (post) {
            ds2 = pick<AT>(m, {dx});
            // the column sums of ds2 are the ff_bias2 gradient: taken in the same pass
            NNCU_TRY(norm_bwd<AT>(m, dx, atc<AT>(a.s2, 0), o.ln_g2, o.ln_b2, a.st_2, nullptr, ds2, TB,
                                  (o.ff_bias2 != NONE && !coef) ? gf(m, o.ff_bias2) : nullptr));
        } else if (o.ff_bias2 != NONE && !coef) {
            NNCU_TRY(colsum<AT>(m, ds2, D, TB, D, gf(m, o.ff_bias2)));
        }
        // LN_COEF: the branch sees alpha * ds2 (its own buffer: the weight-gradient GEMMs read it until the
        // layer's join), the residual keeps ds2; the rows' shares of d alpha wait for the layer's reduction launch
        AT *dt2 = ds2;
        if (coef) {
            dt2 = reinterpret_cast<AT *>(m->dt_ff);
            launch_k(scale_dot_kernel<AT>, dim3(TB), dim3(128), 0, m->st, (const AT *)ds2, atc<AT>(a.aff, 0),
                     (const float *)(m->W + o.alpha), dt2, m->alpha_part, TB, D);
            KERNEL_CHECK();
            if (o.ff_bias2 != NONE)
                NNCU_TRY(colsum<AT>(m, dt2, D, TB, D, gf(m, o.ff_bias2)));
        }
        NNCU_TRY(mm_tn(m, D, F, TB, dt2, D, atc<AT>(a.hact, 0), F, gf(m, o.ff2)));
        NNCU_TRY(mm_nn(m, TB, F, D, dt2, D, o.ff2, dh, F, (const AT *)nullptr));
        float *apart = o.ff_bias1 != NONE ? part_slot(m) : nullptr;
        const bool act_vec = sizeof(AT) == 2 && F % 2 == 0;
        const int act_rows = act_vec ? ACT_BWD_ROWS : 32;
        if (act_vec)
            launch_k(act_bwd_vec_kernel, dim3(ceil_div(F, 256), ceil_div(TB, act_rows)), dim3(128), 0, m->st,
                     (const bf16 *)atc<AT>(a.hpre, 0), (const bf16 *)dh, (bf16 *)dhp, apart, TB, F, F1, p.ff_act);
        else
            act_bwd_kernel<AT><<<dim3(ceil_div(F, 128), ceil_div(TB, act_rows)), 128, 0, m->st>>>(
                atc<AT>(a.hpre, 0), dh, dhp, apart, TB, F, F1, p.ff_act);
        KERNEL_CHECK();
        if (apart)
            NNCU_TRY(reduce_cols(m, apart, ceil_div(TB, act_rows), F1, F1, gf(m, o.ff_bias1), 0));
        const AT *u = pre ? atc<AT>(a.u, 0) : atc<AT>(a.y, 0);
        NNCU_TRY(mm_tn(m, F1, D, TB, dhp, F1, u, D, gf(m, o.ff1)));
        AT *dy = pick<AT>(m, {ds2});
        if (pre) {
            AT *du = pick<AT>(m, {ds2, dy});
            NNCU_TRY(mm_nn(m, TB, D, F1, dhp, F1, o.ff1, du, D, (const AT *)nullptr));
            NNCU_TRY(norm_bwd<AT>(m, du, atc<AT>(a.y, 0), o.ln_g2, o.ln_b2, a.st_pre2, ds2, dy, TB));
        } else {
            NNCU_TRY(mm_nn(m, TB, D, F1, dhp, F1, o.ff1, dy, D, (const AT *)ds2));
        }
        // ---- attention block
        AT *ds1 = dy;
        if (post) {
            ds1 = pick<AT>(m, {dy, ds2});
            NNCU_TRY(norm_bwd<AT>(m, dy, atc<AT>(a.s1, 0), o.ln_g1, o.ln_b1, a.st_1, nullptr, ds1, TB));
        }
        AT *dt1 = ds1;
        if (coef) {
            dt1 = reinterpret_cast<AT *>(m->dt_at);
            launch_k(scale_dot_kernel<AT>, dim3(TB), dim3(128), 0, m->st, (const AT *)ds1, atc<AT>(a.ao, 0),
                     (const float *)(m->W + o.alpha), dt1, m->alpha_part + TB, TB, D);
            KERNEL_CHECK();
            // d alpha = sum over the rows of both sub-layers, one ordered job
            NNCU_TRY(queue_reduction(m, 1, m->alpha_part, 2 * TB, 1, 1, 0, gf(m, o.alpha), 0));
        }
        NNCU_TRY(mm_tn(m, D, HD, TB, dt1, D, atc<AT>(a.o, 0), HD, gf(m, o.w_o)));
        NNCU_TRY(mm_nn(m, TB, HD, D, dt1, D, o.w_o, dof, HD, (const AT *)nullptr));
        nncu_attn_shape s = attn_shape(m, l, 0, m->T);
        NNCU_TRY(attn_backward_any<AT>(&s, at<AT>(a.qkv, (size_t)M * B * 3 * HD), at<AT>(a.qkv, HD), wf(m, o.w_r),
                                       m->W + o.b_r, a.o, a.lse, dof, dq, dkv, m->dwr_part, m->dbr_part, m->st,
                                       &pt, (m->bf && o.w_r != NONE) ? m->Wb + o.w_r : nullptr, m->err_flag));
        {
            // the partials are next written after the join at the layer's end
            size_t nb = (size_t)m->H * m->L;
            NNCU_TRY(queue_reduction(m, 1, m->dbr_part, B, (int)nb, (int)nb, 0, gf(m, o.b_r), p.tied_b_r ? 1 : 0));
            if (o.w_r != NONE) {
                size_t nw = (size_t)m->H * p.d_pos * m->dk;
                NNCU_TRY(queue_reduction(m, 1, m->dwr_part, B, (int)nw, (int)nw, 0, gf(m, o.w_r), p.tied_w_r ? 1 : 0));
            }
        }
        // d[w_q ; w_kv] = [dq | dk | dv]^T [memory ; segment] in one contraction over all L*B rows
        NNCU_TRY(mm_tn(m, 3 * HD, D, LB, dqkv, 3 * HD, hc, D, gf(m, o.w_q)));
        if (o.b_q != NONE)
            NNCU_TRY(colsum<AT>(m, dq, 3 * HD, TB, HD, gf(m, o.b_q)));
        // d(attention input) = [dq | dk | dv](segment rows) [w_q ; w_kv]; the memory rows get no gradient
        AT *dxn = pick<AT>(m, {ds1, ds2}); // ds1, ds2 are still read by weight-gradient GEMMs
        if (pre) {
            AT *dx1 = pick<AT>(m, {ds1, ds2, dxn});
            NNCU_TRY(mm_nn(m, TB, D, 3 * HD, dq, 3 * HD, o.w_q, dx1, D, (const AT *)nullptr));
            NNCU_TRY(norm_bwd<AT>(m, dx1, atc<AT>(a.xin, 0), o.ln_g1, o.ln_b1, a.st_pre1, ds1, dxn, TB));
        } else {
            NNCU_TRY(mm_nn(m, TB, D, 3 * HD, dq, 3 * HD, o.w_q, dxn, D, (const AT *)ds1));
        }
        NNCU_TRY(flush_reductions(m));
        side_join(m); // this layer's weight gradients are done before dhp, dqkv, ds1, ds2 are rewritten
        const int G = bucket_layers(m);
        if (G > 1) {
            // several layers per exchange: their slots are contiguous, and the group is complete when its
            // lowest layer is (the pass runs from the last layer down)
            if (l % G == 0) {
                const int l1 = std::min(l + G, m->nl);
                const size_t lb = o.w_q, le = l1 < m->nl ? m->lo[l1].w_q : m->tail_begin;
                NNCU_TRY(exchange_bucket(m, lb, le));
                NNCU_TRY(opt_range(m, lb, le, false));
            }
            if (l == m->nl - 1)
                NNCU_TRY(exchange_update(m, m->embed_out, m->out_bias != NONE ? m->out_bias : m->n_floats, m->n_floats));
        } else {
            // layer l's slots are contiguous; tied tables live in layer 0, which is exchanged last
            const size_t lb = o.w_q, le = l + 1 < m->nl ? m->lo[l + 1].w_q : m->tail_begin;
            NNCU_TRY(exchange_update(m, lb, o.small, le));
            if (l == m->nl - 1) // the output head's gradients have been complete since the first join
                NNCU_TRY(exchange_update(m, m->embed_out, m->out_bias != NONE ? m->out_bias : m->n_floats, m->n_floats));
        }
        dx = dxn;
    }
    const float emul = sqrtf((float)D) * p.embed_mult;
    if (m->comm && m->sparse_embed) {
        // The embedding gradient has at most T * B_total non-zero rows: instead of summing the dense
        // table over the ranks, every rank gathers all ranks' ids and input gradients (rank order)
        // and builds the same table from them, rows of one symbol summed in ascending gathered order.
        NNCU_TRY(flush_reductions(m));
        side_join(m);
        NNCU_TRY(exchange_update(m, m->tail_begin, m->tail_begin, m->embed)); // final norm: small parameters
        NcclApi *nc = nccl_api();
        const int rows = TB * m->comm_ranks;
        NNCU_TRY(nccl_ok(nc->AllGather(m->ids_dev, m->ids_all, (size_t)TB, NCCL_I32, m->comm, m->st3), "ncclAllGather"));
        NNCU_TRY(nccl_ok(nc->AllGather(dx, m->dx_all, (size_t)TB * D, sizeof(AT) == 2 ? NCCL_BF16 : NCCL_F32, m->comm, m->st3),
                         "ncclAllGather"));
        CUDA_TRY(cudaMemsetAsync(gf(m, m->embed), 0, sizeof(float) * (size_t)V * D, m->st3));
        CUDA_TRY(cudaMemsetAsync(m->first_dev, 0x7f, sizeof(int) * (size_t)V, m->st3));
        launch_k(first_rows_kernel, dim3(ceil_div(rows, 256)), dim3(256), 0, m->st3, (const int32_t *)m->ids_all, rows, V, m->first_dev);
        KERNEL_CHECK();
        launch_k(embed_grad_kernel<AT>, dim3(rows), dim3(128), 0, m->st3, (const int32_t *)m->ids_all, (const AT *)m->dx_all,
                 gf(m, m->embed), (const int *)m->first_dev, rows, D, emul, V);
        KERNEL_CHECK();
        NNCU_TRY(opt_range(m, m->embed, m->embed_out, false));
    } else {
        CUDA_TRY(cudaMemsetAsync(gf(m, m->embed), 0, sizeof(float) * (size_t)V * D, m->st));
        launch_k(embed_grad_kernel<AT>, dim3(TB), dim3(128), 0, m->st, (const int32_t *)m->ids_dev, (const AT *)dx, gf(m, m->embed),
                 (const int *)m->first_dev, TB, D, emul, V);
        KERNEL_CHECK();
        NNCU_TRY(flush_reductions(m));
        side_join(m);
        NNCU_TRY(exchange_bucket(m, m->tail_begin, m->embed_out)); // final norm and the embedding
        NNCU_TRY(opt_range(m, m->tail_begin, m->embed_out, true));
    }
    NNCU_TRY(opt_range(m, 0, m->lo[0].w_q, true)); // (empty: layer 0 opens the parameter table)
    NNCU_TRY(exchange_finish(m));
    return NNCU_OK;
}

// ------------------------------------------------------------------ shadows

__global__ void __launch_bounds__(256)
transpose_jobs_kernel(const bf16 *__restrict__ src, bf16 *__restrict__ dst,
                      const TransposeJob *__restrict__ jobs, int n_jobs)
{
    __shared__ bf16 tile[32][33];
    int j = 0;
    while (j + 1 < n_jobs && (int)blockIdx.x >= jobs[j + 1].tile0)
        j++;
    const TransposeJob jb = jobs[j];
    int t = blockIdx.x - jb.tile0;
    int c0 = (t % jb.tiles_x) * 32, r0 = (t / jb.tiles_x) * 32;
    int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const bf16 *s = src + jb.src_off;
    bf16 *d = dst + jb.dst_off;
    for (int k = ty; k < 32; k += 8) {
        int r = r0 + k, c = c0 + tx;
        if (r < jb.rows && c < jb.cols)
            tile[k][tx] = s[(size_t)r * jb.cols + c];
    }
    __syncthreads();
    for (int k = ty; k < 32; k += 8) {
        int c = c0 + k, r = r0 + tx;
        if (r < jb.rows && c < jb.cols)
            d[(size_t)c * jb.rows + r] = tile[tx][k];
    }
}

static int refresh_transposed(nncu_model *m)
{
    if (m->bf && m->use_tc && !tc_mn_major() && m->n_jobs > 0) {
        transpose_jobs_kernel<<<m->n_job_tiles, 256, 0, m->st>>>(m->Wb, m->WbT, m->jobs_dev, m->n_jobs);
        KERNEL_CHECK();
    }
    return NNCU_OK;
}

static int refresh_shadows(nncu_model *m)
{
    if (!m->bf)
        return NNCU_OK;
    f32_to_bf16_kernel<<<ceil_div(m->n_floats, 256), 256, 0, m->st>>>(m->W, m->Wb, m->n_floats);
    KERNEL_CHECK();
    return refresh_transposed(m);
}

// ------------------------------------------------------------------ parameter table

static uint64_t splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
static uint64_t name_hash(const char *s)
{
    uint64_t h = 0xcbf29ce484222325ull;
    while (*s) {
        h ^= (uint8_t)*s++;
        h *= 0x100000001b3ull;
    }
    return h;
}
static inline float u01(uint64_t key, uint64_t idx, uint32_t k)
{
    uint64_t r = splitmix64(key ^ splitmix64(idx * 16 + k));
    return (float)(r >> 40) * (1.0f / 16777216.0f);
}
// Counter-based initial values: element i of parameter `name` depends only on
// (seed, name, i).  Integer hashing plus exactly-rounded float adds/multiplies,
// so encoder and decoder hosts produce the same bits (trf_init draws from
// nc_tensor_set_rnd_unif in creation order, nncp.c:263-266, whose generator is
// not part of the reference tree).
static void init_values(float *dst, size_t n, const char *name, uint32_t seed, int kind, float scale)
{
    uint64_t key = splitmix64(name_hash(name) ^ ((uint64_t)seed << 32));
    for (size_t i = 0; i < n; i++) {
        if (kind == NNCU_INIT_NORMAL) {
            float s = 0.0f;
            for (uint32_t k = 0; k < 12; k++)
                s += u01(key, i, k);
            dst[i] = (s - 6.0f) * scale;
        } else {
            dst[i] = (2.0f * u01(key, i, 0) - 1.0f) * scale;
        }
    }
}

static size_t add_param(nncu_model *m, const char *base, int idx, size_t numel, int rows = 0, int cols = 0,
                        bool pad = true)
{
    ParamInfo pi;
    memset(&pi, 0, sizeof(pi));
    if (idx >= 0)
        snprintf(pi.name, sizeof(pi.name), "%s_%d", base, idx);
    else
        snprintf(pi.name, sizeof(pi.name), "%s", base);
    pi.numel = numel;
    pi.off = m->n_floats;
    pi.rows = rows;
    pi.cols = cols;
    m->n_floats += numel;
    if (pad)
        m->n_floats = (m->n_floats + 127) & ~(size_t)127; // the next slot starts 512-byte aligned
    m->pinfo.push_back(pi);
    return pi.off;
}

static int validate(const nncu_params *p)
{
    if (!p)
        return nncu_fail(NNCU_ERR_INVALID, "null parameters");
    if (p->n_layer < 1 || p->n_layer > NNCU_N_LAYER_MAX || p->d_model < 1 || p->n_head < 1 ||
        p->d_key < 1 || p->d_inner < 1 || p->seg_len < 1 || p->mem_len < 0 || p->n_streams < 1 ||
        p->n_symbols < 2)
        return nncu_fail(NNCU_ERR_INVALID, "a size is out of range");
    if (p->d_value != p->d_key)
        return nncu_fail(NNCU_ERR_INVALID, "d_value must equal d_key");
    if (p->d_pos < 1 || p->d_pos > p->mem_len + p->seg_len)
        return nncu_fail(NNCU_ERR_INVALID, "d_pos must be in [1, mem_len + seg_len]");
    if ((p->ln_flags & NNCU_LN_PRE) && (p->ln_flags & NNCU_LN_POST))
        return nncu_fail(NNCU_ERR_INVALID, "LN_PRE and LN_POST together are not supported");
    if (p->ff_act > NNCU_FF_GATED_SILU)
        return nncu_fail(NNCU_ERR_INVALID, "ff_act %d is not supported", p->ff_act);
    if (p->use_bf16 && (p->d_key & 1))
        return nncu_fail(NNCU_ERR_INVALID, "bf16 models need an even d_key");
    if (((long)p->n_head * p->d_key * p->d_model) % 8)
        return nncu_fail(NNCU_ERR_INVALID, "n_head * d_key * d_model must be a multiple of 8");
    if (p->gemm_backend == NNCU_GEMM_TCGEN05 && !p->use_bf16)
        return nncu_fail(NNCU_ERR_INVALID, "the tcgen05 backend needs a bf16 model");
    for (int l = 0; l < p->n_layer; l++)
        if (p->attn_len[l] < 0 || p->attn_len[l] > p->mem_len + p->seg_len)
            return nncu_fail(NNCU_ERR_INVALID, "attn_len[%d] out of range", l);
    return NNCU_OK;
}

// ------------------------------------------------------------------ C ABI

extern "C" {

void nncu_default_params(nncu_params *p)
{
    memset(p, 0, sizeof(*p));
    p->n_layer = 4; p->d_model = 256; p->n_head = 8; p->d_key = 32; p->d_value = 32;
    p->d_inner = 512; p->d_pos = 32; p->mem_len = 32; p->seg_len = 32; p->n_streams = 16;
    p->n_symbols = 256; p->use_bias = 1; p->use_w_r = 1; p->tied_w_r = 1; p->tied_b_r = 1;
    p->ln_flags = NNCU_LN_POST; p->ff_act = NNCU_FF_GELU; p->embed_mult = 1.0f;
    p->init_range = 1.0f; p->init_kind = NNCU_INIT_UNIFORM; p->seed = 123;
    p->lr = 3e-4f; p->beta2 = 0.99f; p->eps = 1e-8f; p->device = -1;
}

int nncu_abi_version(void) { return NNCU_ABI_VERSION; }
const char *nncu_last_error(void) { return g_nncu_err; }

int nncu_destroy(nncu_model *m)
{
    if (!m)
        return NNCU_OK;
    cudaSetDevice(m->device);
    cudaStreamSynchronize(m->st);
    // graphs first: a captured ncclAllReduce keeps its communicator busy until the graph is gone
    for (int k = 0; k < 3; k++)
        for (int c = 0; c < 2; c++)
            if (m->graphs[k][c].exec)
                cudaGraphExecDestroy(m->graphs[k][c].exec);
    for (auto &g : m->step_graphs)
        if (g.exec)
            cudaGraphExecDestroy(g.exec);
    if (m->ids_all) cudaFree(m->ids_all);
    if (m->dx_all) cudaFree(m->dx_all);
    if (m->dec_payload) cudaFree(m->dec_payload);
    if (m->dec_state) cudaFree(m->dec_state);
    if (m->st3) cudaStreamSynchronize(m->st3);
    if (m->comm && nccl_api())
        nccl_api()->CommDestroy(m->comm);
    if (m->st3) cudaStreamDestroy(m->st3);
    if (m->ev_bucket) cudaEventDestroy(m->ev_bucket);
    if (m->ev_comm) cudaEventDestroy(m->ev_comm);
    if (m->st2) { cudaStreamSynchronize(m->st2); cudaStreamDestroy(m->st2); }
    if (m->ev_fork) cudaEventDestroy(m->ev_fork);
    if (m->ev_join) cudaEventDestroy(m->ev_join);
    if (m->arena) cudaFree(m->arena);
    if (m->ids_pin) cudaFreeHost(m->ids_pin);
    if (m->tgt_pin) cudaFreeHost(m->tgt_pin);
    if (m->sym_pin) cudaFreeHost(m->sym_pin);
    if (m->coder_pin) cudaFreeHost(m->coder_pin);
    if (m->ev_ids) cudaEventDestroy(m->ev_ids);
    if (m->ev_tgt) cudaEventDestroy(m->ev_tgt);
    if (m->ev_sym) cudaEventDestroy(m->ev_sym);
    if (m->ev_coder) cudaEventDestroy(m->ev_coder);
    if (m->ev_loss) cudaEventDestroy(m->ev_loss);
    if (m->loss_pin) cudaFreeHost(m->loss_pin);
    delete m;
    return NNCU_OK;
}

int nncu_create(const nncu_params *p, nncu_model **out)
{
    if (!out)
        return nncu_fail(NNCU_ERR_INVALID, "null output pointer");
    *out = nullptr;
    NNCU_TRY(validate(p));
    {
        // shapes no attention kernel pair can run are refused here, not at the first segment
        nncu_attn_shape s;
        s.n_streams = p->n_streams; s.n_head = p->n_head; s.d_key = p->d_key; s.seg_len = p->seg_len;
        s.mem_len = p->mem_len; s.d_pos = p->d_pos; s.attn_len = 0; s.t0 = 0; s.t1 = p->seg_len;
        s.br_scale = 1.0f; s.dtype_bf16 = p->use_bf16 ? 1 : 0;
        NNCU_TRY(p->use_bf16 ? attn_shape_supported<bf16>(&s, p->use_w_r != 0)
                             : attn_shape_supported<float>(&s, p->use_w_r != 0));
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        return nncu_fail(NNCU_ERR_CUDA, "no CUDA device: this library has no CPU path");
    int dev = p->device;
    if (dev < 0)
        CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaSetDevice(dev));
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
        return nncu_fail(NNCU_ERR_CUDA, "device %d is sm_%d%d; this library is built for sm_100a only",
                         dev, prop.major, prop.minor);

    nncu_model *m = new nncu_model();
    m->p = *p;
    m->device = dev;
    m->st = 0;
    m->st2 = nullptr;
    m->ev_fork = m->ev_join = nullptr;
    m->overlap = false;
    memset(m->graphs, 0, sizeof(m->graphs));
    m->comm = nullptr;
    m->comm_ranks = 1;
    m->st3 = nullptr;
    m->ev_bucket = m->ev_comm = nullptr;
    {
        const char *e = getenv("NNCU_NO_GRAPH");
        m->graphs_on = !(e && e[0] == '1');
    }
    m->D = p->d_model; m->H = p->n_head; m->dk = p->d_key; m->HD = m->H * m->dk; m->F = p->d_inner;
    m->F1 = (p->ff_act == NNCU_FF_GEGLU || p->ff_act == NNCU_FF_GATED_SILU) ? 2 * m->F : m->F;
    m->T = p->seg_len; m->B = p->n_streams; m->M = p->mem_len; m->L = m->M + m->T; m->V = p->n_symbols;
    m->TB = m->T * m->B; m->LB = m->L * m->B; m->nl = p->n_layer;
    m->Bt = p->n_streams_total > 0 ? p->n_streams_total : m->B;
    m->bf = p->use_bf16 != 0;
    m->use_tc = m->bf && p->gemm_backend != NNCU_GEMM_SIMT;
    m->esz = m->bf ? 2 : 4;
    m->lr = p->lr;
    m->step = 0;
    m->steps_done = 0;
    m->have_forward = false;
    m->cur = 0;
    m->n_floats = 0;
    const int D = m->D, HD = m->HD, F = m->F, F1 = m->F1, V = m->V, TB = m->TB, LB = m->LB;

    const bool has_ln = (p->ln_flags & (NNCU_LN_POST | NNCU_LN_PRE)) != 0;
    m->lo.resize(m->nl);
    for (int l = 0; l < m->nl; l++) {
        LayerOff &o = m->lo[l];
        // w_q and w_kv are contiguous: together they are the [3*H*dk][D] matrix of the fused projection.
        // The matrices come first and everything small after them, so that a sharded optimizer can
        // split the first range over the ranks and keep the second whole on each
        o.w_q = add_param(m, "w_q", l, (size_t)HD * D, HD, D, false);
        o.w_kv = add_param(m, "w_kv", l, (size_t)2 * HD * D, 2 * HD, D);
        o.w_o = add_param(m, "w_o", l, (size_t)D * HD, D, HD);
        o.ff1 = add_param(m, "ff1", l, (size_t)F1 * D, F1, D);
        o.ff2 = add_param(m, "ff2", l, (size_t)D * F, D, F);
        o.small = m->n_floats;
        o.b_q = p->query_bias ? add_param(m, "b_q", l, HD) : NONE;
        o.ff_bias1 = p->use_bias ? add_param(m, "ff_bias1", l, F1) : NONE;
        o.ff_bias2 = p->use_bias ? add_param(m, "ff_bias2", l, D) : NONE;
        if (p->use_w_r)
            o.w_r = (l == 0 || !p->tied_w_r) ? add_param(m, "w_r", l, (size_t)m->H * p->d_pos * m->dk)
                                             : m->lo[0].w_r;
        else
            o.w_r = NONE;
        o.b_r = (l == 0 || !p->tied_b_r) ? add_param(m, "b_r", l, (size_t)m->H * m->L) : m->lo[0].b_r;
        if (has_ln) {
            o.ln_g1 = add_param(m, "ln_g", 2 * l, D);
            o.ln_b1 = add_param(m, "ln_b", 2 * l, D);
            o.ln_g2 = add_param(m, "ln_g", 2 * l + 1, D);
            o.ln_b2 = add_param(m, "ln_b", 2 * l + 1, D);
        } else {
            o.ln_g1 = o.ln_b1 = o.ln_g2 = o.ln_b2 = NONE;
        }
        o.alpha = (p->ln_flags & NNCU_LN_COEF) ? add_param(m, "alpha", l, 1) : NONE; // starts at 0 (nncp.c:437)
    }
    if (p->ln_flags & NNCU_LN_FINAL) {
        m->ln_g = add_param(m, "ln_g", 2 * m->nl, D);
        m->ln_b = add_param(m, "ln_b", 2 * m->nl, D);
    } else {
        m->ln_g = m->ln_b = NONE;
    }
    m->tail_begin = m->ln_g != NONE ? m->ln_g : m->n_floats;
    m->embed = add_param(m, "embed", -1, (size_t)V * D);
    m->embed_out = add_param(m, "embed_out", -1, (size_t)V * D, V, D);
    m->out_bias = p->use_bias ? add_param(m, "out_bias", -1, V) : NONE;

    // ---- arena layout
    size_t total = 0;
    auto take = [&](size_t bytes) {
        size_t o = total;
        total += (bytes + 255) & ~(size_t)255;
        return o;
    };
    const size_t e = m->esz;
    const bool pre = p->ln_flags & NNCU_LN_PRE, post = p->ln_flags & NNCU_LN_POST;
    size_t oW = take(m->n_floats * 4), oG = take(m->n_floats * 4), oV = take(m->n_floats * 4);
    size_t oWb = m->bf ? take(m->n_floats * 2) : 0, oWbT = m->bf ? take(m->n_floats * 2) : 0;
    size_t oH0 = take((size_t)m->nl * LB * D * e), oH1 = take((size_t)m->nl * LB * D * e);
    struct LOff { size_t xin, qkv, o, s1, y, u, hpre, hact, s2, lse, sp1, s_1, sp2, s_2, ao, aff; };
    const bool coef = (p->ln_flags & NNCU_LN_COEF) != 0;
    std::vector<LOff> lofs(m->nl);
    for (int l = 0; l < m->nl; l++) {
        LOff &x = lofs[l];
        x.xin = pre ? take((size_t)TB * D * e) : NONE;
        x.qkv = take((size_t)LB * 3 * HD * e);
        x.o = take((size_t)TB * HD * e);
        x.s1 = post ? take((size_t)TB * D * e) : NONE;
        x.y = take((size_t)TB * D * e);
        x.u = pre ? take((size_t)TB * D * e) : NONE;
        x.hpre = take((size_t)TB * F1 * e);
        x.hact = take((size_t)TB * F * e);
        x.s2 = post ? take((size_t)TB * D * e) : NONE;
        x.lse = take((size_t)m->B * m->H * m->T * 4);
        x.sp1 = take((size_t)TB * 2 * 4);
        x.s_1 = take((size_t)TB * 2 * 4);
        x.sp2 = take((size_t)TB * 2 * 4);
        x.s_2 = take((size_t)TB * 2 * 4);
        x.ao = coef ? take((size_t)TB * D * e) : NONE;
        x.aff = coef ? take((size_t)TB * D * e) : NONE;
    }
    size_t oDtFf = coef ? take((size_t)TB * D * e) : 0, oDtAt = coef ? take((size_t)TB * D * e) : 0;
    size_t oAlphaPart = coef ? take((size_t)2 * TB * 4) : 0;
    size_t oXlast = take((size_t)TB * D * e), oXf = take((size_t)TB * D * e), oStf = take((size_t)TB * 8);
    size_t oProbs = take((size_t)TB * V * 4);
    size_t oPool[4];
    for (int i = 0; i < 4; i++)
        oPool[i] = take((size_t)TB * D * e);
    size_t oDz = take((size_t)TB * V * e), oDh = take((size_t)TB * F * e), oDhp = take((size_t)TB * F1 * e);
    size_t oDof = take((size_t)TB * HD * e);
    size_t oDqkv = take((size_t)LB * 3 * HD * e);
    size_t max_n = (size_t)std::max(std::max(V, F1), std::max(3 * HD, D));
    size_t max_k = (size_t)std::max(std::max(F, D), HD);
    size_t oTA = m->use_tc ? take(max_n * LB * 2) : 0, oTB = m->use_tc ? take(max_k * LB * 2) : 0;
    size_t oWr = take((size_t)m->B * m->H * p->d_pos * m->dk * 4), oBr = take((size_t)m->B * m->H * m->L * 4);
    size_t part_floats = std::max((size_t)ceil_div(LB, 32) * max_n, (size_t)ceil_div(TB, 8) * 3 * D);
    part_floats = std::max(part_floats, (size_t)ceil_div(TB, ACT_BWD_ROWS) * F1);
    size_t oPart = take(part_floats * 4 * PART_SLOTS);
    m->part_floats = part_floats;
    const size_t skw_floats = (m->use_tc && V >= SPLITK_MIN_K) ? (size_t)SPLITK * TB * D : 0;
    size_t oSkw = take(skw_floats * 4 + 256);
    size_t oLogp = take((size_t)TB * 4), oLoss = take(256);
    size_t oIds = take((size_t)TB * 4), oTgt = take((size_t)TB * 4), oErr = take(256), oHash = take(256);
    size_t oTgtFixed = take((size_t)TB * 4), oFirst = take((size_t)V * 4), oSym = take((size_t)TB * 4);
    // transposed-shadow jobs
    std::vector<TransposeJob> jobs;
    int tiles = 0;
    if (m->bf)
        for (const ParamInfo &pi : m->pinfo)
            if (pi.rows > 0) {
                TransposeJob j;
                j.src_off = pi.off; j.dst_off = pi.off; j.rows = pi.rows; j.cols = pi.cols;
                j.tile0 = tiles; j.tiles_x = ceil_div(pi.cols, 32);
                tiles += j.tiles_x * ceil_div(pi.rows, 32);
                jobs.push_back(j);
            }
    size_t oJobs = take(sizeof(TransposeJob) * (jobs.size() + 1));
    m->coder_bytes = (size_t)TB * ((size_t)1 << coder_depth(V)) * 2; // a tree per row: 2^ceil(log2 V) entries
    size_t oCoder = take(m->coder_bytes);

    m->arena_bytes = total;
    cudaError_t ce = cudaMalloc(&m->arena, total);
    if (ce != cudaSuccess) {
        delete m;
        return nncu_fail(NNCU_ERR_NOMEM, "cudaMalloc of %zu bytes failed: %s", total, cudaGetErrorString(ce));
    }
    auto fail_cleanup = [&](int rc) {
        nncu_destroy(m);
        return rc;
    };
    if (cudaMemset(m->arena, 0, total) != cudaSuccess)
        return fail_cleanup(nncu_fail(NNCU_ERR_CUDA, "cudaMemset failed"));
    char *A = m->arena;
    m->W = (float *)(A + oW); m->G = (float *)(A + oG); m->Vm = (float *)(A + oV);
    m->Wb = m->bf ? (bf16 *)(A + oWb) : nullptr;
    m->WbT = m->bf ? (bf16 *)(A + oWbT) : nullptr;
    m->hcat[0] = A + oH0; m->hcat[1] = A + oH1;
    m->act.resize(m->nl);
    m->xlast = A + oXlast; m->xf = A + oXf; m->st_f = (float *)(A + oStf); m->probs = (float *)(A + oProbs);
    for (int i = 0; i < 4; i++)
        m->pool[i] = A + oPool[i];
    m->dz = A + oDz; m->dh = A + oDh; m->dhp = A + oDhp; m->dof = A + oDof; m->dqkv = A + oDqkv;
    m->tA = m->use_tc ? A + oTA : nullptr; m->tB = m->use_tc ? A + oTB : nullptr;
    m->dwr_part = (float *)(A + oWr); m->dbr_part = (float *)(A + oBr); m->part = (float *)(A + oPart);
    m->skw = skw_floats ? (float *)(A + oSkw) : nullptr;
    m->skw_floats = skw_floats;
    m->logp = (float *)(A + oLogp); m->loss_dev = (float *)(A + oLoss);
    m->hyper_dev = m->loss_dev + 8;
    m->ids_dev = (int32_t *)(A + oIds); m->tgt_dev = (int32_t *)(A + oTgt);
    m->err_flag = (int *)(A + oErr); m->hash_dev = (unsigned long long *)(A + oHash);
    m->dz_fixed = m->err_flag + 16; // same 256-byte slot, zeroed with the arena
    m->tgt_fixed = (int32_t *)(A + oTgtFixed);
    m->first_dev = (int *)(A + oFirst);
    m->sym_dev = (int32_t *)(A + oSym);
    m->jobs_dev = (TransposeJob *)(A + oJobs);
    m->n_jobs = (int)jobs.size(); m->n_job_tiles = tiles;
    m->coder_dev = (uint16_t *)(A + oCoder);
    for (int l = 0; l < m->nl; l++) {
        LOff &x = lofs[l];
        LayerAct &a = m->act[l];
        a.qkv = A + x.qkv; a.o = A + x.o; a.y = A + x.y; a.hpre = A + x.hpre; a.hact = A + x.hact;
        a.s1 = post ? A + x.s1 : nullptr; a.s2 = post ? A + x.s2 : nullptr; a.u = pre ? A + x.u : nullptr;
        a.lse = (float *)(A + x.lse); a.st_pre1 = (float *)(A + x.sp1); a.st_1 = (float *)(A + x.s_1);
        a.st_pre2 = (float *)(A + x.sp2); a.st_2 = (float *)(A + x.s_2);
        a.xin = pre ? A + x.xin : nullptr; // without pre-LN the residual input IS the hcat segment part
        a.ao = coef ? A + x.ao : nullptr; a.aff = coef ? A + x.aff : nullptr;
    }
    if (coef) {
        m->dt_ff = A + oDtFf; m->dt_at = A + oDtAt;
        m->alpha_part = (float *)(A + oAlphaPart);
    }
    if (cudaStreamCreateWithFlags(&m->st2, cudaStreamNonBlocking) == cudaSuccess &&
        cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming) == cudaSuccess &&
        cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming) == cudaSuccess) {
        const char *e = getenv("NNCU_NO_OVERLAP");
        m->overlap = !(e && e[0] == '1');
    }
    if (cudaMallocHost(&m->ids_pin, sizeof(int32_t) * TB) != cudaSuccess ||
        cudaMallocHost(&m->tgt_pin, sizeof(int32_t) * TB) != cudaSuccess ||
        cudaMallocHost(&m->sym_pin, sizeof(int32_t) * TB) != cudaSuccess ||
        cudaMallocHost(&m->coder_pin, sizeof(uint16_t) * TB * 16) != cudaSuccess ||
        cudaMallocHost(&m->loss_pin, 64) != cudaSuccess)
        return fail_cleanup(nncu_fail(NNCU_ERR_NOMEM, "pinned host allocation failed"));
    if (cudaEventCreateWithFlags(&m->ev_ids, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->ev_tgt, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->ev_sym, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->ev_coder, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->ev_loss, cudaEventDisableTiming) != cudaSuccess)
        return fail_cleanup(nncu_fail(NNCU_ERR_CUDA, "event creation failed"));
    if (!jobs.empty() &&
        cudaMemcpy(m->jobs_dev, jobs.data(), sizeof(TransposeJob) * jobs.size(), cudaMemcpyHostToDevice) != cudaSuccess)
        return fail_cleanup(nncu_fail(NNCU_ERR_CUDA, "job table upload failed"));
    if ((size_t)8 * 3 * D * 4 > 48 * 1024) {
        cudaFuncSetAttribute(norm_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * D * 4);
        cudaFuncSetAttribute(norm_bwd_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * D * 4);
        if (D == 1024)
            cudaFuncSetAttribute(norm_bwd_vec_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * D * 4);
    }
    if ((size_t)2 * V * 4 > 48 * 1024 && (size_t)2 * V * 4 <= 200 * 1024) {
        cudaFuncSetAttribute(coder_paths_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * V * 4);
        cudaFuncSetAttribute(coder_trees_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * V * 4);
    }
    {
        const size_t heap_bytes = ((size_t)2 << coder_depth(V)) * 4; // the any-alphabet kernels: 2 * 2^ceil(log2 V) floats
        if (heap_bytes > 48 * 1024 && heap_bytes <= 200 * 1024) {
            cudaFuncSetAttribute(coder_paths_any_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)heap_bytes);
            cudaFuncSetAttribute(coder_trees_any_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)heap_bytes);
        }
    }

    // ---- initial values (trf_init, nncp.c:341-497), computed on the host
    {
        std::vector<float> host(m->n_floats, 0.0f);
        float a0 = p->init_kind == NNCU_INIT_NORMAL ? p->init_range : p->init_range / sqrtf((float)D);
        for (const ParamInfo &pi : m->pinfo) {
            float *dst = host.data() + pi.off;
            if (!strncmp(pi.name, "ln_g", 4)) {
                for (size_t k = 0; k < pi.numel; k++)
                    dst[k] = 1.0f;
            } else if (!strncmp(pi.name, "w_", 2) || !strncmp(pi.name, "ff1", 3) || !strncmp(pi.name, "embed", 5)) {
                init_values(dst, pi.numel, pi.name, p->seed, p->init_kind, a0);
            } else if (!strncmp(pi.name, "ff2", 3)) {
                init_values(dst, pi.numel, pi.name, p->seed, p->init_kind, a0 * sqrtf((float)D / (float)F));
            }
        }
        if (cudaMemcpy(m->W, host.data(), m->n_floats * 4, cudaMemcpyHostToDevice) != cudaSuccess)
            return fail_cleanup(nncu_fail(NNCU_ERR_CUDA, "weight upload failed"));
    }
    int rc = refresh_shadows(m);
    if (rc == NNCU_OK && cudaStreamSynchronize(m->st) != cudaSuccess)
        rc = nncu_fail(NNCU_ERR_CUDA, "initialisation kernels failed: %s", cudaGetErrorString(cudaGetLastError()));
    if (rc != NNCU_OK)
        return fail_cleanup(rc);
    // without pre-LN, xin aliases the hcat segment rows of the CURRENT twin; resolved per call
    *out = m;
    return NNCU_OK;
}

int nncu_set_stream(nncu_model *m, void *cuda_stream)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    CUDA_TRY(cudaStreamSynchronize(m->st));
    m->st = (cudaStream_t)cuda_stream;
    return NNCU_OK;
}

int nncu_reset(nncu_model *m)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    CUDA_TRY(cudaSetDevice(m->device));
    if (m->M > 0)
        CUDA_TRY(cudaMemset2DAsync(m->hcat[m->cur], (size_t)m->LB * m->D * m->esz, 0,
                                   (size_t)m->M * m->B * m->D * m->esz, m->nl, m->st));
    m->steps_done = 0;
    m->have_forward = false;
    return NNCU_OK;
}

int nncu_set_lr(nncu_model *m, float lr)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    m->lr = lr;
    return NNCU_OK;
}

static void bind_xin(nncu_model *m)
{
    if (m->p.ln_flags & NNCU_LN_PRE)
        return;
    for (int l = 0; l < m->nl; l++)
        m->act[l].xin = hcat_layer(m, m->cur, l) + (size_t)m->M * m->B * m->D * m->esz;
}

static int eval_common(nncu_model *m, int output_index)
{
    if (output_index >= m->T)
        return nncu_fail(NNCU_ERR_INVALID, "output_index %d >= seg_len %d", output_index, m->T);
    if (output_index > 0 && output_index != m->steps_done)
        return nncu_fail(NNCU_ERR_STATE, "step %d issued after %d steps", output_index, m->steps_done);
    bind_xin(m);
    if (m->coder_rows) // coder values of the pass before are still being produced from its probabilities
        CUDA_TRY(cudaStreamWaitEvent(m->st, m->ev_coder, 0));
    int t0 = output_index < 0 ? 0 : output_index, t1 = output_index < 0 ? m->T : output_index + 1;
    auto body = [&]() { return m->bf ? forward_range<bf16>(m, t0, t1) : forward_range<float>(m, t0, t1); };
    int rc = output_index < 0 ? run_graphed(m, GRAPH_FWD, body) : body();
    if (rc != NNCU_OK)
        return rc;
    m->steps_done = t1;
    m->have_forward = (t1 == m->T);
    return NNCU_OK;
}

int nncu_eval(nncu_model *m, int output_index, const int32_t *input_host)
{
    if (!m || !input_host)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(m->device));
    if (output_index >= m->T)
        return nncu_fail(NNCU_ERR_INVALID, "output_index %d >= seg_len %d", output_index, m->T);
    int t0 = output_index < 0 ? 0 : output_index, n = output_index < 0 ? m->TB : m->B;
    // the staging buffer may still feed the copy of the call before (an unrecorded event is complete)
    CUDA_TRY(cudaEventSynchronize(m->ev_ids));
    memcpy(m->ids_pin + (size_t)t0 * m->B, input_host + (size_t)t0 * m->B, sizeof(int32_t) * n);
    CUDA_TRY(cudaMemcpyAsync(m->ids_dev + (size_t)t0 * m->B, m->ids_pin + (size_t)t0 * m->B,
                             sizeof(int32_t) * n, cudaMemcpyHostToDevice, m->st));
    CUDA_TRY(cudaEventRecord(m->ev_ids, m->st));
    return eval_common(m, output_index);
}

int nncu_eval_dev(nncu_model *m, int output_index, const int32_t *input_dev)
{
    if (!m || !input_dev)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(m->device));
    if (output_index >= m->T)
        return nncu_fail(NNCU_ERR_INVALID, "output_index %d >= seg_len %d", output_index, m->T);
    int t0 = output_index < 0 ? 0 : output_index, n = output_index < 0 ? m->TB : m->B;
    CUDA_TRY(cudaMemcpyAsync(m->ids_dev + (size_t)t0 * m->B, input_dev + (size_t)t0 * m->B,
                             sizeof(int32_t) * n, cudaMemcpyDeviceToDevice, m->st));
    return eval_common(m, output_index);
}

int nncu_eval_end(nncu_model *m)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    m->steps_done = 0;
    m->have_forward = false;
    return NNCU_OK;
}

int nncu_read_probs(nncu_model *m, int t0, int nt, float *probs_host)
{
    if (!m || !probs_host || t0 < 0 || nt < 0 || t0 + nt > m->T)
        return nncu_fail(NNCU_ERR_INVALID, "bad probability range");
    CUDA_TRY(cudaSetDevice(m->device));
    CUDA_TRY(cudaMemcpyAsync(probs_host, m->probs + (size_t)t0 * m->B * m->V,
                             sizeof(float) * (size_t)nt * m->B * m->V, cudaMemcpyDeviceToHost, m->st));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    return NNCU_OK;
}

int nncu_probs_dev(nncu_model *m, float **probs_dev)
{
    if (!m || !probs_dev)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    *probs_dev = m->probs;
    return NNCU_OK;
}

// The sharded optimizer is off unless asked for: on the 32-stream step of the 55 M-parameter model it
// measured slower than per-layer all-reduce + whole update (symbols/s, sharded against all-reduce:
// 785 k / 845 k at 2 GPUs, 807 k / 948 k at 4).  The exchange stream then carries five operations per
// layer (reduce-scatter, shard update, all-gather, small all-reduce, small update) instead of two,
// and at 13 MB per layer the fixed cost of each NCCL operation outweighs the bytes and the optimizer
// traffic it saves.  The embedding gradient from gathered ids and rows, which replaces the 33.5 MB
// dense all-reduce at the tail of the step, is on: 964 k against 951 k at 4 GPUs.
//   NNCU_SHARDED_UPDATE=1  reduce-scatter, RMSProp on the own shard, all-gather of the weights
//   NNCU_SPARSE_EMBED=0    back to the dense all-reduce of the embedding gradient
static bool env_on(const char *name)
{
    const char *e = getenv(name);
    return e && e[0] == '1';
}
static bool shard_enabled()
{
    static int on = -1;
    if (on < 0)
        on = env_on("NNCU_SHARDED_UPDATE") ? 1 : 0;
    return on != 0;
}
static bool sparse_embed_enabled()
{
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("NNCU_SPARSE_EMBED");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

static int gradient_common(nncu_model *m, bool fused = false)
{
    if (!fused && m->master_stale)
        return nncu_fail(NNCU_ERR_STATE, "the optimizer state is sharded over the ranks: nncu_comm_gather_master first");
    if (!m->have_forward)
        return nncu_fail(NNCU_ERR_STATE, "eval_gradient needs a complete forward pass first");
    bind_xin(m);
    if (fused) {
        // this step's learning rate and bias correction, read by the captured optimizer launches
        m->step++;
        const float hyper[2] = {m->lr, m->p.bias_correction ? 1.0f / (1.0f - powf(m->p.beta2, (float)m->step)) : 1.0f};
        CUDA_TRY(cudaMemcpyAsync(m->hyper_dev, hyper, sizeof(hyper), cudaMemcpyHostToDevice, m->st));
    }
    m->fuse_update = fused;
    m->shard_update = fused && m->comm && m->comm_ranks > 1 && shard_enabled();
    m->sparse_embed = fused && m->comm && m->comm_ranks > 1 && (m->shard_update || sparse_embed_enabled());
    int rc = run_graphed(m, fused ? GRAPH_BWD_UPD : GRAPH_BWD,
                         [&]() { return m->bf ? backward<bf16>(m) : backward<float>(m); });
    if (m->shard_update)
        m->master_stale = true;
    m->fuse_update = false;
    m->shard_update = m->sparse_embed = false;
    if (rc == NNCU_OK && fused)
        rc = refresh_transposed(m);
    return rc;
}

int nncu_read_loss(nncu_model *m, float *loss_out)
{
    if (!m || !loss_out)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(m->device));
    if (m->loss_pending) {
        // queued right behind the backward pass: wait for that copy, not for what the host has
        // queued since (the optimizer step, the next segment's forward pass)
        CUDA_TRY(cudaEventSynchronize(m->ev_loss));
        m->loss_pending = 0;
    } else {
        CUDA_TRY(cudaMemcpyAsync(m->loss_pin, m->loss_dev, sizeof(float), cudaMemcpyDeviceToHost, m->st));
        CUDA_TRY(cudaStreamSynchronize(m->st));
    }
    *loss_out = *m->loss_pin;
    return NNCU_OK;
}

// the loss follows the backward pass to the host; nncu_read_loss collects it
static int queue_loss(nncu_model *m)
{
    CUDA_TRY(cudaMemcpyAsync(m->loss_pin, m->loss_dev, sizeof(float), cudaMemcpyDeviceToHost, m->st));
    CUDA_TRY(cudaEventRecord(m->ev_loss, m->st));
    m->loss_pending = 1;
    return NNCU_OK;
}

int nncu_eval_gradient(nncu_model *m, const int32_t *expected_host, float *loss_out)
{
    if (!m || !expected_host)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(m->device));
    CUDA_TRY(cudaEventSynchronize(m->ev_tgt));
    memcpy(m->tgt_pin, expected_host, sizeof(int32_t) * m->TB);
    CUDA_TRY(cudaMemcpyAsync(m->tgt_dev, m->tgt_pin, sizeof(int32_t) * m->TB, cudaMemcpyHostToDevice, m->st));
    CUDA_TRY(cudaEventRecord(m->ev_tgt, m->st));
    NNCU_TRY(gradient_common(m));
    NNCU_TRY(queue_loss(m));
    if (loss_out)
        return nncu_read_loss(m, loss_out);
    return NNCU_OK;
}

int nncu_eval_gradient_dev(nncu_model *m, const int32_t *expected_dev)
{
    if (!m || !expected_dev)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(m->device));
    CUDA_TRY(cudaMemcpyAsync(m->tgt_dev, expected_dev, sizeof(int32_t) * m->TB, cudaMemcpyDeviceToDevice, m->st));
    NNCU_TRY(gradient_common(m));
    return queue_loss(m);
}

int nncu_eval_gradient_update(nncu_model *m, const int32_t *expected_host, float *loss_out)
{
    if (!m || !expected_host)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(m->device));
    CUDA_TRY(cudaEventSynchronize(m->ev_tgt));
    memcpy(m->tgt_pin, expected_host, sizeof(int32_t) * m->TB);
    CUDA_TRY(cudaMemcpyAsync(m->tgt_dev, m->tgt_pin, sizeof(int32_t) * m->TB, cudaMemcpyHostToDevice, m->st));
    CUDA_TRY(cudaEventRecord(m->ev_tgt, m->st));
    NNCU_TRY(gradient_common(m, true));
    NNCU_TRY(queue_loss(m));
    if (loss_out)
        return nncu_read_loss(m, loss_out);
    return NNCU_OK;
}

int nncu_eval_gradient_update_dev(nncu_model *m, const int32_t *expected_dev)
{
    if (!m || !expected_dev)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(m->device));
    CUDA_TRY(cudaMemcpyAsync(m->tgt_dev, expected_dev, sizeof(int32_t) * m->TB, cudaMemcpyDeviceToDevice, m->st));
    NNCU_TRY(gradient_common(m, true));
    return queue_loss(m);
}

int nncu_optimizer_step(nncu_model *m)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    CUDA_TRY(cudaSetDevice(m->device));
    if (m->master_stale)
        return nncu_fail(NNCU_ERR_STATE, "the optimizer state is sharded over the ranks: nncu_comm_gather_master first");
    m->step++;
    float corr = 1.0f;
    if (m->p.bias_correction)
        corr = 1.0f / (1.0f - powf(m->p.beta2, (float)m->step));
    size_t n4 = m->n_floats / 4;
    launch_k(rmsprop_kernel, dim3(ceil_div(n4, 256)), dim3(256), 0, m->st, m->W, m->G, m->Vm, m->Wb, n4, m->lr, m->p.beta2,
                                                         m->p.eps, m->p.gradient_clip, corr, (const float *)nullptr);
    KERNEL_CHECK();
    return refresh_transposed(m);
}

int nncu_memory_shift(nncu_model *m)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    CUDA_TRY(cudaSetDevice(m->device));
    if (m->M > 0) {
        // memory <- last M time steps of [memory ; segment], every layer in one 2-D copy
        size_t pitch = (size_t)m->LB * m->D * m->esz;
        CUDA_TRY(cudaMemcpy2DAsync(m->hcat[m->cur ^ 1], pitch,
                                   m->hcat[m->cur] + (size_t)m->T * m->B * m->D * m->esz, pitch,
                                   (size_t)m->M * m->B * m->D * m->esz, m->nl, cudaMemcpyDeviceToDevice, m->st));
        m->cur ^= 1;
    }
    m->steps_done = 0;
    m->have_forward = false;
    return NNCU_OK;
}

int nncu_update(nncu_model *m)
{
    NNCU_TRY(nncu_optimizer_step(m));
    return nncu_memory_shift(m);
}

// NCCL picks algorithm, protocol and channel count from the message size and the machine it finds
// itself on, and each choice sums the ranks' contributions in a different order.  Pinned here
// (unless the caller's environment already says otherwise, or NNCU_NCCL_PIN=0), the order of every
// bucket's sum depends on the number of ranks alone, which is what a file's header records.  The
// variables are read when a communicator is created, so they also have to be in place before any
// other NCCL communicator of the process is.
static void pin_nccl_choices()
{
    const char *e = getenv("NNCU_NCCL_PIN");
    if (e && e[0] == '0')
        return;
    // measured on the 32-stream step, symbols/s at 2 and 4 GPUs: Ring/LL128 on 32 channels 844 k and
    // 949 k (NCCL's own choice for the 12.9 MB layer buckets; 945 k at 4 unpinned); 24 channels 830 k
    // and 860 k; Ring/Simple on 16 channels 854 k and 788 k, on 8 channels 641 k at 4; Tree 794 k at 4
    setenv("NCCL_ALGO", "Ring", 0);
    setenv("NCCL_PROTO", "LL128", 0);
    setenv("NCCL_MIN_NCHANNELS", "32", 0);
    setenv("NCCL_MAX_NCHANNELS", "32", 0);
}

int nncu_comm_unique_id(void *id_out)
{
    pin_nccl_choices();
    NcclApi *nc = nccl_api();
    if (!nc)
        return nncu_fail(NNCU_ERR_CUDA, "libnccl.so.2 could not be loaded");
    if (!id_out)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    int r = nc->GetUniqueId(id_out);
    if (r != 0)
        return nncu_fail(NNCU_ERR_CUDA, "ncclGetUniqueId: %s", nc->GetErrorString(r));
    return NNCU_OK;
}

int nncu_comm_init(nncu_model *m, int n_ranks, int rank, const void *id)
{
    if (!m || !id || n_ranks < 1 || rank < 0 || rank >= n_ranks)
        return nncu_fail(NNCU_ERR_INVALID, "bad communicator arguments");
    if (m->comm)
        return nncu_fail(NNCU_ERR_STATE, "the model already has a communicator");
    pin_nccl_choices();
    NcclApi *nc = nccl_api();
    if (!nc)
        return nncu_fail(NNCU_ERR_CUDA, "libnccl.so.2 could not be loaded");
    CUDA_TRY(cudaSetDevice(m->device));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    if (!m->st3) {
        CUDA_TRY(cudaStreamCreateWithFlags(&m->st3, cudaStreamNonBlocking));
        CUDA_TRY(cudaEventCreateWithFlags(&m->ev_bucket, cudaEventDisableTiming));
        CUDA_TRY(cudaEventCreateWithFlags(&m->ev_comm, cudaEventDisableTiming));
    }
    nccl_id_t uid;
    memcpy(&uid, id, sizeof(uid));
    void *comm = nullptr;
    int r = nc->CommInitRank(&comm, n_ranks, uid, rank);
    if (r != 0)
        return nncu_fail(NNCU_ERR_CUDA, "ncclCommInitRank: %s", nc->GetErrorString(r));
    m->comm = comm;
    m->comm_ranks = n_ranks;
    m->comm_rank = rank;
    if (n_ranks > 1) { // landing areas of the embedding-gradient gather
        CUDA_TRY(cudaMalloc(&m->ids_all, sizeof(int32_t) * (size_t)m->TB * n_ranks));
        CUDA_TRY(cudaMalloc(&m->dx_all, m->esz * (size_t)m->TB * m->D * n_ranks));
    }
    return NNCU_OK;
}

// After fused steps under a communicator each rank holds current second moments (and fp32 master
// weights, in a bf16 model) only for its own shard of every matrix.  This collective -- every rank
// calls it -- completes them everywhere, which nncu_param_get, nncu_param_set, nncu_weights_hash,
// nncu_eval_gradient and nncu_optimizer_step require; the fused step itself never needs it.
int nncu_comm_gather_master(nncu_model *m)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    if (!m->master_stale)
        return NNCU_OK;
    CUDA_TRY(cudaSetDevice(m->device));
    NcclApi *nc = nccl_api();
    const size_t N = (size_t)m->comm_ranks;
    auto gather = [&](size_t begin, size_t mid) -> int {
        const size_t nbig = mid - begin;
        if (!nbig || nbig % (4 * N))
            return NNCU_OK; // this range was all-reduced and updated whole
        const size_t chunk = nbig / N, mine = begin + chunk * (size_t)m->comm_rank;
        NNCU_TRY(nccl_ok(nc->AllGather(m->Vm + mine, m->Vm + begin, chunk, NCCL_F32, m->comm, m->st), "ncclAllGather"));
        if (m->Wb)
            NNCU_TRY(nccl_ok(nc->AllGather(m->W + mine, m->W + begin, chunk, NCCL_F32, m->comm, m->st), "ncclAllGather"));
        return NNCU_OK;
    };
    for (int l = 0; l < m->nl; l++)
        NNCU_TRY(gather(m->lo[l].w_q, m->lo[l].small));
    NNCU_TRY(gather(m->embed_out, m->out_bias != NONE ? m->out_bias : m->n_floats));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    m->master_stale = false;
    return NNCU_OK;
}

int nncu_synchronize(nncu_model *m)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    CUDA_TRY(cudaSetDevice(m->device));
    return check_err_flag(m);
}

int nncu_param_count(const nncu_model *m) { return m ? (int)m->pinfo.size() : 0; }

int nncu_param_info(const nncu_model *m, int index, char *name_out, size_t name_cap, size_t *numel_out,
                    size_t *offset_out)
{
    if (!m || index < 0 || index >= (int)m->pinfo.size())
        return nncu_fail(NNCU_ERR_INVALID, "bad parameter index");
    const ParamInfo &pi = m->pinfo[index];
    if (name_out && name_cap)
        snprintf(name_out, name_cap, "%s", pi.name);
    if (numel_out) *numel_out = pi.numel;
    if (offset_out) *offset_out = pi.off;
    return NNCU_OK;
}

static int param_io(nncu_model *m, int index, float *host, size_t numel, float *base, bool to_host)
{
    if (!m || !host || index < 0 || index >= (int)m->pinfo.size())
        return nncu_fail(NNCU_ERR_INVALID, "bad parameter index or buffer");
    const ParamInfo &pi = m->pinfo[index];
    if (numel != pi.numel)
        return nncu_fail(NNCU_ERR_INVALID, "%s has %zu elements, caller passed %zu", pi.name, pi.numel, numel);
    CUDA_TRY(cudaSetDevice(m->device));
    if (m->master_stale && base != m->G)
        return nncu_fail(NNCU_ERR_STATE, "the master weights are sharded over the ranks: nncu_comm_gather_master first");
    CUDA_TRY(cudaStreamSynchronize(m->st));
    if (to_host)
        CUDA_TRY(cudaMemcpy(host, base + pi.off, numel * 4, cudaMemcpyDeviceToHost));
    else
        CUDA_TRY(cudaMemcpy(base + pi.off, host, numel * 4, cudaMemcpyHostToDevice));
    return NNCU_OK;
}

int nncu_param_get(nncu_model *m, int index, float *host_out, size_t numel)
{
    return param_io(m, index, host_out, numel, m ? m->W : nullptr, true);
}

int nncu_param_set(nncu_model *m, int index, const float *host_in, size_t numel)
{
    NNCU_TRY(param_io(m, index, const_cast<float *>(host_in), numel, m ? m->W : nullptr, false));
    NNCU_TRY(refresh_shadows(m));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    return NNCU_OK;
}

int nncu_grad_get(nncu_model *m, int index, float *host_out, size_t numel)
{
    return param_io(m, index, host_out, numel, m ? m->G : nullptr, true);
}

int nncu_flat_buffers(nncu_model *m, float **master_dev, float **grad_dev, float **moment_dev, size_t *n_floats)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    if (master_dev) *master_dev = m->W;
    if (grad_dev) *grad_dev = m->G;
    if (moment_dev) *moment_dev = m->Vm;
    if (n_floats) *n_floats = m->n_floats;
    return NNCU_OK;
}

int nncu_weights_hash(nncu_model *m, uint64_t *hash_out)
{
    if (!m || !hash_out)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(m->device));
    if (m->master_stale)
        return nncu_fail(NNCU_ERR_STATE, "the master weights are sharded over the ranks: nncu_comm_gather_master first");
    CUDA_TRY(cudaMemsetAsync(m->hash_dev, 0, 8, m->st));
    hash_kernel<<<296, 256, 0, m->st>>>(m->W, m->n_floats, m->hash_dev);
    KERNEL_CHECK();
    unsigned long long h = 0;
    CUDA_TRY(cudaMemcpyAsync(&h, m->hash_dev, 8, cudaMemcpyDeviceToHost, m->st));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    *hash_out = h;
    return NNCU_OK;
}

static int coder_bits(int V)
{
    int n = 0;
    while ((1 << n) < V)
        n++;
    return ((1 << n) == V) ? n : -1;
}

// symbols up, coder kernel, 15-bit prob0 values down into the pinned landing area; no host wait
static int coder_paths_enqueue(nncu_model *m, int t0, int nt, const int32_t *sym_host)
{
    if (!m || !sym_host || t0 < 0 || nt < 1 || t0 + nt > m->T)
        return nncu_fail(NNCU_ERR_INVALID, "bad coder range");
    const bool pow2 = coder_bits(m->V) >= 1;
    const int nb = coder_depth(m->V), P = 1 << nb;
    if (m->V < 2)
        return nncu_fail(NNCU_ERR_INVALID, "coder-ready output needs at least two symbols");
    if ((size_t)2 * P * 4 > 200 * 1024)
        return nncu_fail(NNCU_ERR_RANGE, "n_symbols %d is beyond the limit of the coder kernels (16384; 25600 for a power of two)", m->V);
    CUDA_TRY(cudaSetDevice(m->device));
    int rows = nt * m->B;
    CUDA_TRY(cudaEventSynchronize(m->ev_sym));   // the symbol staging area is free again
    CUDA_TRY(cudaEventSynchronize(m->ev_coder)); // and so is the landing area
    memcpy(m->sym_pin, sym_host, sizeof(int32_t) * rows);
    // The coder values only read the probabilities: they are produced on the side stream, beside the
    // backward pass the caller queues next.  The next forward pass, which overwrites the
    // probabilities, is ordered behind them either by nncu_coder_paths_end (the host has waited for
    // them) or, if it is queued earlier, by a wait on their event in nncu_eval.
    cudaStream_t st = side_fork(m);
    CUDA_TRY(cudaMemcpyAsync(m->sym_dev, m->sym_pin, sizeof(int32_t) * rows, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaEventRecord(m->ev_sym, st));
    if (!pow2)
        coder_paths_any_kernel<<<rows, 256, (size_t)2 * P * 4, st>>>(m->probs + (size_t)t0 * m->B * m->V, m->sym_dev,
                                                                    m->coder_dev, m->V, P, nb);
    else if (m->V >= 1024 && m->V <= 16384)
        coder_paths_fast_kernel<<<rows, 256, 0, st>>>(m->probs + (size_t)t0 * m->B * m->V, m->sym_dev, m->coder_dev, m->V, nb);
    else
        coder_paths_kernel<<<rows, 256, (size_t)2 * m->V * 4, st>>>(m->probs + (size_t)t0 * m->B * m->V, m->sym_dev,
                                                                   m->coder_dev, m->V, nb);
    KERNEL_CHECK();
    CUDA_TRY(cudaMemcpyAsync(m->coder_pin, m->coder_dev, sizeof(uint16_t) * (size_t)rows * nb, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaEventRecord(m->ev_coder, st));
    m->coder_rows = rows;
    m->coder_nb = nb;
    return NNCU_OK;
}

int nncu_coder_paths_begin(nncu_model *m, int t0, int nt, const int32_t *sym_host)
{
    if (m && m->coder_rows)
        return nncu_fail(NNCU_ERR_STATE, "nncu_coder_paths_begin: the result of the call before was not collected");
    return coder_paths_enqueue(m, t0, nt, sym_host);
}

int nncu_coder_paths_end(nncu_model *m, uint16_t *prob0_host, int *n_bits_out)
{
    if (!m || !prob0_host)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    if (!m->coder_rows)
        return nncu_fail(NNCU_ERR_STATE, "nncu_coder_paths_end without nncu_coder_paths_begin");
    CUDA_TRY(cudaSetDevice(m->device));
    CUDA_TRY(cudaEventSynchronize(m->ev_coder));
    memcpy(prob0_host, m->coder_pin, sizeof(uint16_t) * (size_t)m->coder_rows * m->coder_nb);
    if (n_bits_out) *n_bits_out = m->coder_nb;
    m->coder_rows = 0;
    return NNCU_OK;
}

int nncu_coder_paths(nncu_model *m, int t0, int nt, const int32_t *sym_host, uint16_t *prob0_host, int *n_bits_out)
{
    if (!prob0_host)
        return nncu_fail(NNCU_ERR_INVALID, "bad coder range");
    if (m && m->coder_rows)
        return nncu_fail(NNCU_ERR_STATE, "nncu_coder_paths between nncu_coder_paths_begin and _end");
    NNCU_TRY(coder_paths_enqueue(m, t0, nt, sym_host));
    return nncu_coder_paths_end(m, prob0_host, n_bits_out);
}

int nncu_coder_trees(nncu_model *m, int t0, int nt, uint16_t *tree_host)
{
    if (!m || !tree_host || t0 < 0 || nt < 1 || t0 + nt > m->T)
        return nncu_fail(NNCU_ERR_INVALID, "bad coder range");
    const bool pow2 = coder_bits(m->V) >= 1;
    const int P = 1 << coder_depth(m->V);
    if (m->V < 2)
        return nncu_fail(NNCU_ERR_INVALID, "coder-ready output needs at least two symbols");
    if ((size_t)2 * P * 4 > 200 * 1024)
        return nncu_fail(NNCU_ERR_RANGE, "n_symbols %d is beyond the limit of the coder kernels (16384; 25600 for a power of two)", m->V);
    CUDA_TRY(cudaSetDevice(m->device));
    int rows = nt * m->B;
    if (pow2)
        coder_trees_kernel<<<rows, 256, (size_t)2 * m->V * 4, m->st>>>(m->probs + (size_t)t0 * m->B * m->V, m->coder_dev, m->V);
    else
        coder_trees_any_kernel<<<rows, 256, (size_t)2 * P * 4, m->st>>>(m->probs + (size_t)t0 * m->B * m->V, m->coder_dev,
                                                                       m->V, P);
    KERNEL_CHECK();
    CUDA_TRY(cudaMemcpyAsync(tree_host, m->coder_dev, sizeof(uint16_t) * (size_t)rows * P, cudaMemcpyDeviceToHost, m->st));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    return NNCU_OK;
}

// ---- what a bounded wait does when it runs out
// A one-thread kernel waits, through the same mbar_wait the GEMM and attention kernels use, for a
// barrier that nothing ever completes, with a limit of a few hundred tries instead of millions.  The
// wait gives up, raises the model's error flag and the kernel returns normally: the next
// nncu_synchronize reports NNCU_ERR_TIMEOUT and clears the flag, and the context stays usable.
__global__ void expired_wait_kernel(int *err_flag, uint32_t tries)
{
    __shared__ uint64_t bar;
    __shared__ int abort_s;
    abort_s = 0;
    tc::mbar_init(tc::smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tc::mbar_wait(tc::smem_u32(&bar), 0, &abort_s, err_flag, 90, tries);
}

int nncu_selftest_expired_wait(nncu_model *m)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    CUDA_TRY(cudaSetDevice(m->device));
    expired_wait_kernel<<<1, 1, 0, m->st>>>(m->err_flag, 256u);
    KERNEL_CHECK();
    return NNCU_OK;
}

// ---- range decoder on the device (decoder.cuh)

int nncu_decoder_begin(nncu_model *m, const uint8_t *payload_host, size_t len)
{
    if (!m || (!payload_host && len))
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    const bool pow2 = coder_bits(m->V) >= 1;
    const int nb = coder_depth(m->V), P = 1 << nb; // a tree row has P entries (P = V for a power of two)
    const int ring = dec::ring_slots(m->B, P, nb);
    if (ring < 2 || (size_t)2 * P * 4 > 200 * 1024)
        return nncu_fail(NNCU_ERR_RANGE, "n_symbols %d with %d streams does not fit the decoder's shared memory", m->V, m->B);
    CUDA_TRY(cudaSetDevice(m->device));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    const size_t need = len + 16;
    if (need > m->dec_cap) {
        // the captured step graphs hold the old buffer's address: they are dropped and captured again
        for (auto &g : m->step_graphs) {
            if (g.exec)
                cudaGraphExecDestroy(g.exec);
            g = nncu_model::StepGraph{nullptr, 0, 0};
        }
        if (m->dec_payload)
            cudaFree(m->dec_payload);
        m->dec_payload = nullptr;
        m->dec_cap = 0;
        CUDA_TRY(cudaMalloc(&m->dec_payload, need));
        m->dec_cap = need;
    }
    if (!m->dec_state)
        CUDA_TRY(cudaMalloc(&m->dec_state, sizeof(dec::State)));
    if (len)
        CUDA_TRY(cudaMemcpyAsync(m->dec_payload, payload_host, len, cudaMemcpyHostToDevice, m->st));
    // the state after get_bit_init (arith.c:241-262): three bytes pulled into low, range at its top
    dec::State s0;
    memset(&s0, 0, sizeof(s0));
    s0.len = len;
    for (int i = 0; i < 3; i++) {
        s0.low <<= 8;
        if (s0.pos < len)
            s0.low += payload_host[s0.pos++];
    }
    s0.range = dec::R_TOP;
    CUDA_TRY(cudaMemcpyAsync(m->dec_state, &s0, sizeof(s0), cudaMemcpyHostToDevice, m->st));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    CUDA_TRY(cudaFuncSetAttribute(pow2 ? dec::decode_step_kernel<false> : dec::decode_step_kernel<true>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dec::smem_bytes(m->B, P, nb, ring)));
    m->dec_ring = ring;
    m->dec_open = true;
    if (m->step_graphs.empty())
        m->step_graphs.assign((size_t)2 * m->T, nncu_model::StepGraph{nullptr, 0, 0});
    return NNCU_OK;
}

// one decode step: the model's one-symbol forward, the prob0 trees of its B rows, and the walk that
// turns them into symbols (left in the target rows and, for t+1 < seg_len, the next step's input)
static int decode_step(nncu_model *m, int t, int limit_t, int limit_b)
{
    const int B = m->B, V = m->V, nb = coder_depth(V), P = 1 << nb;
    const bool pow2 = P == V;
    NNCU_TRY(m->bf ? forward_range<bf16>(m, t, t + 1) : forward_range<float>(m, t, t + 1));
    if (pow2)
        launch_k(coder_trees_kernel, dim3(B), dim3(256), (size_t)2 * V * 4, m->st,
                 (const float *)(m->probs + (size_t)t * B * V), m->coder_dev, V);
    else
        launch_k(coder_trees_any_kernel, dim3(B), dim3(256), (size_t)2 * P * 4, m->st,
                 (const float *)(m->probs + (size_t)t * B * V), m->coder_dev, V, P);
    KERNEL_CHECK();
    launch_k(pow2 ? dec::decode_step_kernel<false> : dec::decode_step_kernel<true>, dim3(1), dim3(32),
             dec::smem_bytes(B, P, nb, m->dec_ring), m->st, (const uint16_t *)m->coder_dev,
             (const uint8_t *)m->dec_payload, m->dec_state, m->tgt_dev + (size_t)t * B,
             t + 1 < m->T ? m->ids_dev + (size_t)(t + 1) * B : (int32_t *)nullptr, t, limit_t, limit_b, B, V, P, nb,
             m->dec_ring, m->err_flag);
    KERNEL_CHECK();
    return NNCU_OK;
}

int nncu_decode_steps(nncu_model *m, int t0, int nt, const int32_t *ids_t0_host, int limit_t, int limit_b,
                      int32_t *symbols_host)
{
    if (!m || !symbols_host || t0 < 0 || nt < 1 || t0 + nt > m->T || limit_t < 0 || limit_b < 0)
        return nncu_fail(NNCU_ERR_INVALID, "bad decode range");
    if (!m->dec_open)
        return nncu_fail(NNCU_ERR_STATE, "nncu_decode_steps without nncu_decoder_begin");
    if (t0 != m->steps_done)
        return nncu_fail(NNCU_ERR_STATE, "step %d issued after %d steps", t0, m->steps_done);
    if (t0 == 0 && !ids_t0_host)
        return nncu_fail(NNCU_ERR_INVALID, "the first step of a segment needs its input symbols");
    CUDA_TRY(cudaSetDevice(m->device));
    const int B = m->B;
    if (ids_t0_host) {
        CUDA_TRY(cudaEventSynchronize(m->ev_ids));
        memcpy(m->ids_pin + (size_t)t0 * B, ids_t0_host, sizeof(int32_t) * B);
        CUDA_TRY(cudaMemcpyAsync(m->ids_dev + (size_t)t0 * B, m->ids_pin + (size_t)t0 * B, sizeof(int32_t) * B,
                                 cudaMemcpyHostToDevice, m->st));
        CUDA_TRY(cudaEventRecord(m->ev_ids, m->st));
    }
    bind_xin(m);
    const bool full = limit_t >= m->T; // every stream active at every step: the shape the graphs hold
    for (int t = t0; t < t0 + nt; t++) {
        auto body = [&]() { return decode_step(m, t, limit_t, limit_b); };
        NNCU_TRY(full ? run_graphed(m, m->step_graphs[(size_t)2 * t + m->cur], body) : body());
        m->steps_done = t + 1;
    }
    m->have_forward = (m->steps_done == m->T);
    CUDA_TRY(cudaEventSynchronize(m->ev_sym));
    CUDA_TRY(cudaMemcpyAsync(m->sym_pin, m->tgt_dev + (size_t)t0 * B, sizeof(int32_t) * (size_t)nt * B, cudaMemcpyDeviceToHost,
                             m->st));
    NNCU_TRY(check_err_flag(m)); // drains the stream
    memcpy(symbols_host, m->sym_pin, sizeof(int32_t) * (size_t)nt * B);
    return NNCU_OK;
}

int nncu_decoder_end(nncu_model *m, size_t *bytes_consumed)
{
    if (!m)
        return nncu_fail(NNCU_ERR_INVALID, "null model");
    if (!m->dec_open)
        return nncu_fail(NNCU_ERR_STATE, "nncu_decoder_end without nncu_decoder_begin");
    CUDA_TRY(cudaSetDevice(m->device));
    dec::State s;
    CUDA_TRY(cudaMemcpyAsync(&s, m->dec_state, sizeof(s), cudaMemcpyDeviceToHost, m->st));
    CUDA_TRY(cudaStreamSynchronize(m->st));
    if (bytes_consumed)
        *bytes_consumed = (size_t)s.pos;
    m->dec_open = false;
    return NNCU_OK;
}

// ---- launch counting and per-launch timing of the dominant kernel

int nncu_profile_begin(int time_gemms)
{
    g_nncu_launches = 0;
    if (g_nncu_prof) {
        g_nncu_prof->n = 0;
    }
    if (time_gemms) {
        static GemmProfiler prof;
        if (!prof.ready) {
            for (int i = 0; i < 2 * GemmProfiler::MAX_EV; i++)
                CUDA_TRY(cudaEventCreate(&prof.ev[i]));
            prof.ready = true;
        }
        prof.n = 0;
        g_nncu_prof = &prof;
    } else {
        g_nncu_prof = nullptr;
    }
    return NNCU_OK;
}

int nncu_profile_end(nncu_profile *out)
{
    if (!out)
        return nncu_fail(NNCU_ERR_INVALID, "null argument");
    memset(out, 0, sizeof(*out));
    out->launches = g_nncu_launches;
    GemmProfiler *pr = g_nncu_prof;
    g_nncu_prof = nullptr;
    if (pr) {
        CUDA_TRY(cudaDeviceSynchronize());
        for (int i = 0; i < pr->n; i++) {
            float ms = 0.0f;
            CUDA_TRY(cudaEventElapsedTime(&ms, pr->ev[2 * i], pr->ev[2 * i + 1]));
            out->gemm_ms += ms;
            out->gemm_flops += pr->flops[i];
        }
        out->gemm_launches = (uint64_t)pr->n;
    }
    return NNCU_OK;
}

// ---- isolated attention op

int nncu_attention_forward(const nncu_attn_shape *s, const void *q, const void *kv, const float *w_r,
                           const float *b_r, void *out, float *lse, void *cuda_stream)
{
    NNCU_TRY(attn_check_shape(s));
    if (!q || !kv || !b_r || !out)
        return nncu_fail(NNCU_ERR_INVALID, "null tensor");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    return s->dtype_bf16 ? attn_forward_any<bf16>(s, q, kv, w_r, b_r, out, lse, st)
                         : attn_forward_any<float>(s, q, kv, w_r, b_r, out, lse, st);
}

int nncu_attention_backward(const nncu_attn_shape *s, const void *q, const void *kv, const float *w_r,
                            const float *b_r, const void *out, const float *lse, const void *dout, void *dq,
                            void *dkv, float *dwr_part, float *dbr_part, void *cuda_stream)
{
    NNCU_TRY(attn_check_shape(s));
    if (!q || !kv || !b_r || !out || !lse || !dout || !dq || !dkv)
        return nncu_fail(NNCU_ERR_INVALID, "null tensor");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    return s->dtype_bf16
               ? attn_backward_any<bf16>(s, q, kv, w_r, b_r, out, lse, dout, dq, dkv, dwr_part, dbr_part, st)
               : attn_backward_any<float>(s, q, kv, w_r, b_r, out, lse, dout, dq, dkv, dwr_part, dbr_part, st);
}

int nncu_attention_reduce_tables(const nncu_attn_shape *s, const float *dwr_part, const float *dbr_part,
                                 float *dw_r, float *db_r, int accumulate, void *cuda_stream)
{
    NNCU_TRY(attn_check_shape(s));
    cudaStream_t st = (cudaStream_t)cuda_stream;
    const int L = s->mem_len + s->seg_len;
    if (dbr_part && db_r) {
        size_t n = (size_t)s->n_head * L;
        launch_k(reduce_streams_kernel, dim3(ceil_div(n, 256)), dim3(256), 0, st, dbr_part, s->n_streams, n, db_r, accumulate);
        KERNEL_CHECK();
    }
    if (dwr_part && dw_r) {
        size_t n = (size_t)s->n_head * s->d_pos * s->d_key;
        launch_k(reduce_streams_kernel, dim3(ceil_div(n, 256)), dim3(256), 0, st, dwr_part, s->n_streams, n, dw_r, accumulate);
        KERNEL_CHECK();
    }
    return NNCU_OK;
}

// ---- attention backward with its scratch inside the library image
//
// For callers that cannot hand over a scratch buffer (all device memory already in their own
// pool, or no room for the synchronisation an allocation implies).  The partial table
// gradients go to a fixed file-scope device array.  In host code the array's name is only a
// handle: its device address is fetched once per device with cudaGetSymbolAddress, with that
// device current, and that pointer is what the kernels get.

static __device__ __align__(256) float g_noalloc_scratch[NNCU_NOALLOC_SCRATCH_FLOATS];

#define NNCU_MAX_DEVICES 64
static float *g_noalloc_ptr[NNCU_MAX_DEVICES];

int nncu_attention_backward_noalloc(const nncu_attn_shape *s, const void *q, const void *kv, const float *w_r,
                                    const float *b_r, const void *out, const float *lse, const void *dout,
                                    void *dq, void *dkv, float *dw_r, float *db_r, void *cuda_stream)
{
    NNCU_TRY(attn_check_shape(s));
    if (!q || !kv || !b_r || !out || !lse || !dout || !dq || !dkv || !db_r || (w_r && !dw_r))
        return nncu_fail(NNCU_ERR_INVALID, "null tensor");
    const size_t L = (size_t)s->mem_len + s->seg_len;
    const size_t bh = (size_t)s->n_streams * s->n_head;
    const size_t n_wr = w_r ? bh * s->d_pos * s->d_key : 0, n_br = bh * L;
    if (n_wr + n_br > (size_t)NNCU_NOALLOC_SCRATCH_FLOATS)
        return nncu_fail(NNCU_ERR_RANGE,
                         "attention backward without allocation: %zu scratch floats needed, the built-in "
                         "array holds %u; use nncu_attention_backward with caller-provided buffers",
                         n_wr + n_br, (unsigned)NNCU_NOALLOC_SCRATCH_FLOATS);
    int dev = -1;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NNCU_MAX_DEVICES)
        return nncu_fail(NNCU_ERR_INVALID, "device ordinal %d out of range", dev);
    if (!g_noalloc_ptr[dev]) { // first call on this device: resolve the array's device address
        float *ptr = nullptr;
        CUDA_TRY(cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch));
        g_noalloc_ptr[dev] = ptr;
    }
    float *dwr_part = w_r ? g_noalloc_ptr[dev] : nullptr;
    float *dbr_part = g_noalloc_ptr[dev] + n_wr;
    cudaStream_t st = (cudaStream_t)cuda_stream;
    NNCU_TRY(s->dtype_bf16
                 ? attn_backward_any<bf16>(s, q, kv, w_r, b_r, out, lse, dout, dq, dkv, dwr_part, dbr_part, st)
                 : attn_backward_any<float>(s, q, kv, w_r, b_r, out, lse, dout, dq, dkv, dwr_part, dbr_part, st));
    const size_t nb = (size_t)s->n_head * L;
    launch_k(reduce_streams_kernel, dim3(ceil_div(nb, 256)), dim3(256), 0, st, dbr_part, s->n_streams, nb, db_r, 0);
    KERNEL_CHECK();
    if (w_r) {
        const size_t nw = (size_t)s->n_head * s->d_pos * s->d_key;
        launch_k(reduce_streams_kernel, dim3(ceil_div(nw, 256)), dim3(256), 0, st, dwr_part, s->n_streams, nw, dw_r, 0);
        KERNEL_CHECK();
    }
    return NNCU_OK;
}

// ---- dense contraction test hooks

// the time-out flag of the stand-alone GEMM entry points: one int per device inside the library
// image (no allocation; a flag allocated on one device must not be handed to a kernel on another)
static __device__ int g_gemm_flag;
static int *g_gemm_flag_ptr[NNCU_MAX_DEVICES];

static int gemm_flag(int **out)
{
    int dev = -1;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NNCU_MAX_DEVICES)
        return nncu_fail(NNCU_ERR_INVALID, "device ordinal %d out of range", dev);
    if (!g_gemm_flag_ptr[dev]) {
        int *ptr = nullptr;
        CUDA_TRY(cudaGetSymbolAddress((void **)&ptr, g_gemm_flag));
        CUDA_TRY(cudaMemset(ptr, 0, sizeof(int)));
        g_gemm_flag_ptr[dev] = ptr;
    }
    *out = g_gemm_flag_ptr[dev];
    return NNCU_OK;
}

static int gemm_flag_check(int *flag, cudaStream_t st)
{
    int h = 0;
    CUDA_TRY(cudaMemcpyAsync(&h, flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    if (h != 0) {
        CUDA_TRY(cudaMemsetAsync(flag, 0, sizeof(int), st));
        return nncu_fail(NNCU_ERR_TIMEOUT, "tcgen05 GEMM: a bounded wait expired (code %d)", h);
    }
    return NNCU_OK;
}

#ifdef NNCU_ATTN_TRACE
extern "C" int nncu_attn_trace(long long *dev_buf)
{
    CUDA_TRY(cudaMemcpyToSymbol(amma::g_attn_trace, &dev_buf, sizeof(dev_buf)));
    CUDA_TRY(cudaMemcpyToSymbol(attc::g_trace, &dev_buf, sizeof(dev_buf)));
    return NNCU_OK;
}
#endif
#ifdef NNCU_GEMM_TRACE
extern "C" int nncu_gemm_trace(long long *dev_buf)
{
    CUDA_TRY(cudaMemcpyToSymbol(tc::g_tc_trace, &dev_buf, sizeof(dev_buf)));
    return NNCU_OK;
}
extern "C" int nncu_gemm_trace_mode(int mode)
{
    CUDA_TRY(cudaMemcpyToSymbol(tc::g_tc_mode, &mode, sizeof(mode)));
    return NNCU_OK;
}
#endif

int nncu_gemm_bf16(int backend, int mode, int M, int N, int K, const void *A, int lda, const void *B, int ldb,
                   void *C, int ldc, int c_is_f32, void *cuda_stream)
{
    if (!A || !B || !C || M < 0 || N < 0 || K < 0 || mode < 0 || mode > 2)
        return nncu_fail(NNCU_ERR_INVALID, "bad GEMM arguments");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    const bf16 *a = (const bf16 *)A, *b = (const bf16 *)B;
    if (backend == NNCU_GEMM_SIMT)
        return c_is_f32 ? gemm_simt<bf16, bf16, float>(st, mode, M, N, K, a, lda, b, ldb, (float *)C, ldc, nullptr, 0)
                        : gemm_simt<bf16, bf16, bf16>(st, mode, M, N, K, a, lda, b, ldb, (bf16 *)C, ldc, nullptr, 0);
    int *flag = nullptr;
    NNCU_TRY(gemm_flag(&flag));
    int rc;
    if (mode == GEMM_NT)
        rc = c_is_f32 ? tc::gemm<float, false, false>(st, M, N, K, a, lda, b, ldb, (float *)C, ldc, nullptr, nullptr, flag)
                      : tc::gemm<bf16, false, false>(st, M, N, K, a, lda, b, ldb, (bf16 *)C, ldc, nullptr, nullptr, flag);
    else if (mode == GEMM_NN)
        rc = c_is_f32 ? tc::gemm<float, false, true>(st, M, N, K, a, lda, b, ldb, (float *)C, ldc, nullptr, nullptr, flag)
                      : tc::gemm<bf16, false, true>(st, M, N, K, a, lda, b, ldb, (bf16 *)C, ldc, nullptr, nullptr, flag);
    else
        rc = c_is_f32 ? tc::gemm<float, true, true>(st, M, N, K, a, lda, b, ldb, (float *)C, ldc, nullptr, nullptr, flag)
                      : tc::gemm<bf16, true, true>(st, M, N, K, a, lda, b, ldb, (bf16 *)C, ldc, nullptr, nullptr, flag);
    if (rc != NNCU_OK)
        return rc;
    return gemm_flag_check(flag, st);
}


int nncu_gemm_bf16_nt(int backend, int M, int N, int K, const void *A, int lda, const void *B, int ldb, void *C,
                      int ldc, int c_is_f32, const float *bias, void *cuda_stream)
{
    if (!A || !B || !C || M < 0 || N < 0 || K < 0)
        return nncu_fail(NNCU_ERR_INVALID, "bad GEMM arguments");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    const bf16 *a = (const bf16 *)A, *b = (const bf16 *)B;
    if (backend == NNCU_GEMM_SIMT) {
        return c_is_f32 ? gemm_simt<bf16, bf16, float>(st, GEMM_NT, M, N, K, a, lda, b, ldb, (float *)C, ldc, bias, 0)
                        : gemm_simt<bf16, bf16, bf16>(st, GEMM_NT, M, N, K, a, lda, b, ldb, (bf16 *)C, ldc, bias, 0);
    }
    int *flag = nullptr;
    NNCU_TRY(gemm_flag(&flag));
    int rc = c_is_f32 ? tc::gemm_nt<float>(st, M, N, K, a, lda, b, ldb, (float *)C, ldc, bias, nullptr, flag)
                      : tc::gemm_nt<bf16>(st, M, N, K, a, lda, b, ldb, (bf16 *)C, ldc, bias, nullptr, flag);
    if (rc != NNCU_OK)
        return rc;
    return gemm_flag_check(flag, st);
}

} // extern "C"
