// attention_tc.cuh -- bf16 relative-position attention on the 5th-generation tensor cores:
// tcgen05.mma with TMEM accumulators, operands staged by TMA (cp.async.bulk.tensor.3d).
//
// Same math as attention.cuh (nncp.c:722-800 and its adjoint), for d_head 64 and at most 64
// queries per segment (every BASELINE configuration).  One CTA owns one head of TWO streams, so
// that the query rows fill the 128 rows of a UMMA tile: rows 0-63 are the queries of stream
// b0 = 2*blockIdx.x, rows 64-127 those of stream b0 + 1.  The position table R is per head, i.e.
// shared by the two streams, so E = Q R^T is one 128-row product; the key products are issued
// against the two streams' keys side by side, [K_b0 ; K_b1], and each row uses the half that
// belongs to its stream (the other half is never read).  Per block of 128 keys per stream:
//
//   S  = Q [K_b0 ; K_b1]^T          128 x 256 x 64   -> TMEM columns   0..255
//   E  = Q Rwin^T                   128 x 192 x 64   -> TMEM columns 256..447
//   a  = (S + skew(E) + b_r) / sqrt(dk), masked; online softmax over the key blocks
//   O_b = P V_b  for b = b0, b0+1   128 x 64 x 128   -> TMEM columns   0..127 (S is dead by then)
//
// Rwin is the window of 192 table rows the block can reach (row wlo + c for column c); the
// relative shift makes row i read column jj + 63 - i for key jj of the block.  A thread owns
// one row (TMEM lane), and tcgen05.ld addresses columns warp-uniformly, so the per-row skew is
// done in registers: two aligned 32-column chunks are loaded and a five-stage barrel shifter
// (shifts by 16, 8, 4, 2, 1 selected by the bits of 31 - lane) moves each lane's window into
// place; no shared memory, no dynamic register indexing.  The masked, scaled scores go back to
// TMEM (tcgen05.st) so that the second softmax pass reads them instead of recomputing the skew.
//
// Bit-exact rows whatever the query range: a row's result depends only on that row's operands
// and on the sequence of key blocks, and a key block in which the row sees nothing leaves its
// running maximum, sum and output unchanged bit for bit.
//
// Roles (320 threads): warp 0 lane 0 issues the TMA loads, warp 1 lane 0 the MMAs (warp 1 also
// owns the TMEM allocation), warps 2-9 are 256 row threads: two per row (a warp reaches the TMEM
// lanes 32 * (warp % 4) .. +31, so warps w and w + 4 share rows), each taking two of the four
// 32-key chunks of a block and half of the output columns.  Every wait is bounded; on expiry the
// kernel raises *err_flag and leaves through the common exit that frees TMEM.
#pragma once
#include "attention.cuh"
#include "gemm_tc.cuh"

namespace attc {

using tc::fence_after_sync;
using tc::fence_before_sync;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::mbar_wait;
using tc::smem_u32;
using tc::tmem_ld32;
using tc::tmem_ld_wait;
using tc::umma_bf16;
using tc::umma_commit;

#ifdef NNCU_ATTN_TRACE
// tuning aid (off in normal builds): clock64() stamps of the kernels' phases, 32 slots per CTA
__device__ long long *g_trace = nullptr;
#define ATC_STAMP(slot)                                                                    \
    do {                                                                                   \
        long long *t_ = g_trace;                                                           \
        if (t_ && blockIdx.x + blockIdx.y * gridDim.x < 64)                                \
            t_[(blockIdx.x + blockIdx.y * gridDim.x) * 32 + (slot)] = clock64();           \
    } while (0)
#else
#define ATC_STAMP(slot) \
    do {                \
    } while (0)
#endif

constexpr int DK = 64;    // head size this kernel is built for
constexpr int KB = 128;   // keys per block and stream
constexpr int WIN = 192;  // table rows one block can reach: 128 keys + 63 query offsets, rounded
constexpr int MAXL = 1024; // b_r staging

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, int z)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t *r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr)
{
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}
__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// out[k] = x[k + 31 - lane], k = 0..31, for x[0..62]: five conditional shifts, all indices
// compile-time constants (selects, no local memory)
__device__ __forceinline__ void barrel_skew(uint32_t (&x)[64], int lane)
{
    const int s = 31 - lane;
    const bool b16 = s & 16, b8 = s & 8, b4 = s & 4, b2 = s & 2, b1 = s & 1;
#pragma unroll
    for (int k = 0; k < 47; k++)
        x[k] = b16 ? x[k + 16] : x[k];
#pragma unroll
    for (int k = 0; k < 39; k++)
        x[k] = b8 ? x[k + 8] : x[k];
#pragma unroll
    for (int k = 0; k < 35; k++)
        x[k] = b4 ? x[k + 4] : x[k];
#pragma unroll
    for (int k = 0; k < 33; k++)
        x[k] = b2 ? x[k + 2] : x[k];
#pragma unroll
    for (int k = 0; k < 32; k++)
        x[k] = b1 ? x[k + 1] : x[k];
}

// UMMA instruction descriptor: fp32 accumulate, bf16 operands, M = 128
__host__ __device__ constexpr uint32_t idesc_of(int n, bool a_mn, bool b_mn)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

constexpr int NROW = 256;          // row threads
constexpr int BRS_PAD = 64;        // b_r staging starts at index -64 ...
constexpr int BRS_LEN = MAXL + 256; // ... and runs past the last slot a masked pair can name

// Masked scores (log2 domain) of the 32 keys [jc, jc + 32) for one row, in place over the S chunk.
// x: the skewed E chunk (barrel_skew done); e0: E of table row 0 (left pad); kclamp: keys k < kclamp
// of the chunk fall on the pad; [klo, khi]: visible keys of the chunk; brp[k]: the scaled b_r term.
// Warp-uniform shortcuts: no lane on the pad, every lane seeing the whole chunk.
__device__ __forceinline__ void score_chunk(uint32_t (&sv)[32], const uint32_t (&x)[64], bool has_wr, bool clampable,
                                            float e0, int kclamp, int klo, int khi, const float *brp, float sc2)
{
    const bool any_pad = clampable && __any_sync(0xffffffffu, kclamp > 0);
    const bool all_vis = __all_sync(0xffffffffu, klo <= 0 && khi >= 31);
    if (has_wr) {
        if (any_pad) {
#pragma unroll
            for (int k = 0; k < 32; k++)
                sv[k] = __float_as_uint(__uint_as_float(sv[k]) + (k < kclamp ? e0 : __uint_as_float(x[k])));
        } else {
#pragma unroll
            for (int k = 0; k < 32; k++)
                sv[k] = __float_as_uint(__uint_as_float(sv[k]) + __uint_as_float(x[k]));
        }
    }
    if (all_vis) {
#pragma unroll
        for (int k = 0; k < 32; k++)
            sv[k] = __float_as_uint(fmaf(__uint_as_float(sv[k]), sc2, brp[k]));
    } else {
#pragma unroll
        for (int k = 0; k < 32; k++) {
            const float v = fmaf(__uint_as_float(sv[k]), sc2, brp[k]);
            sv[k] = __float_as_uint((k >= klo && k <= khi) ? v : -INFINITY);
        }
    }
}

__device__ __forceinline__ uint4 pack8(const uint32_t *r)
{
    return make_uint4(tc::pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1])),
                      tc::pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3])),
                      tc::pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5])),
                      tc::pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7])));
}

// shared-memory map of the forward kernel (bytes from the 1024-aligned base)
struct FwdSmem {
    static constexpr int Q = 0;                   // [128][64] bf16: stream b0 rows, then b0 + 1
    static constexpr int K = Q + 128 * 128;       // [256][64]: keys of b0, then of b0 + 1
    static constexpr int V = K + 256 * 128;       // [256][64]
    static constexpr int R = V + 256 * 128;       // [192][64] table window
    static constexpr int P = R + WIN * 128;       // two K-major atoms [128][64] (keys 0-63, 64-127)
    static constexpr int BRS = P + 2 * 128 * 128; // BRS_LEN floats: scaled b_r[h][.], index + BRS_PAD
    static constexpr int XCH = BRS + BRS_LEN * 4; // [4][128] floats: what the two threads of a row exchange
    static constexpr int BAR = XCH + 4 * 128 * 4; // mbarriers, TMEM slot, abort flag
    static constexpr int TOTAL = BAR + 128 + 1024; // + alignment slack
};

struct KeyBlocks {
    int lo, hi; // first and last key block with a visible pair for query rows [t0, t1)
};
__host__ __device__ inline KeyBlocks key_blocks(int M, int L, int attn_len, int t0, int t1)
{
    int jlo = t0 + M - attn_len + 1;
    jlo = jlo < 0 ? 0 : jlo;
    int jhi = t1 - 1 + M;
    jhi = jhi > L - 1 ? L - 1 : jhi;
    KeyBlocks kb;
    kb.lo = jlo / KB;
    kb.hi = jhi / KB;
    return kb;
}

__global__ void __launch_bounds__(320, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                   const __grid_constant__ CUtensorMap map_wr, AttnArgs a, int has_wr, int *err_flag)
{
    extern __shared__ unsigned char smraw_[];
    unsigned char *sm = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smraw_) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + FwdSmem::BAR);
    // bars: 0 load (Q, K, table window), 1 free (V reusable), 2 se (S and E in TMEM: K and the window
    //       reusable), 3 p (P in smem, S/E consumed), 4 o (O block in TMEM), 5 tfree (O block consumed),
    //       6 load of V
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 7);
    volatile int *abort_s = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *brs = reinterpret_cast<float *>(sm + FwdSmem::BRS);
    float *xch = reinterpret_cast<float *>(sm + FwdSmem::XCH);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b0 = blockIdx.x * 2, h = blockIdx.y;
    const int T = a.T, M = a.M, L = a.L, P = a.P, HD = a.H * DK;
    const KeyBlocks kbs = key_blocks(M, L, a.attn_len, a.t0, a.t1);
    const int c0 = P - M - 1; // table row of (i, j) is max(j - i + c0, 0)
    pdl_trigger();
    if (threadIdx.x == 0)
        ATC_STAMP(0);

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_kv)) : "memory");
        if (has_wr)
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_wr)) : "memory");
        mbar_init(smem_u32(&bars[0]), 1);
        mbar_init(smem_u32(&bars[1]), 1);
        mbar_init(smem_u32(&bars[2]), 1);
        mbar_init(smem_u32(&bars[3]), NROW);
        mbar_init(smem_u32(&bars[4]), 1);
        mbar_init(smem_u32(&bars[5]), NROW);
        mbar_init(smem_u32(&bars[6]), 1);
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1)
        tc::tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    pdl_wait();
    const uint32_t tmem = *tmem_slot;
    const uint32_t sm0 = smem_u32(sm);
    if (threadIdx.x == 0)
        ATC_STAMP(1);
    const uint32_t bar_load = smem_u32(&bars[0]), bar_free = smem_u32(&bars[1]), bar_se = smem_u32(&bars[2]),
                   bar_p = smem_u32(&bars[3]), bar_o = smem_u32(&bars[4]), bar_tfree = smem_u32(&bars[5]),
                   bar_loadv = smem_u32(&bars[6]);

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            // K and the table window of the next block are fetched as soon as this block's S and E are in
            // TMEM, under its softmax and PV product; only V waits for the PV product to finish
            for (int kb = kbs.lo; kb <= kbs.hi; kb++, it++) {
                const int j0 = kb * KB;
                if (it > 0 && !mbar_wait(bar_se, (uint32_t)((it - 1) & 1), abort_s, err_flag, 11))
                    break;
                const int wlo = j0 - 63 + c0;
                const int wrow = wlo < -(WIN - 2) ? 0 : wlo; // a window wholly below the table: row 0 alone is used
                uint32_t bytes = 256 * 128 + (has_wr ? WIN * 128 : 0) + (it == 0 ? 128 * 128 : 0);
                mbar_expect_tx(bar_load, bytes);
                if (it == 0) {
                    tma_load_3d(sm0 + FwdSmem::Q, &map_q, bar_load, h * DK, b0, 0);
                    tma_load_3d(sm0 + FwdSmem::Q + 64 * 128, &map_q, bar_load, h * DK, b0 + 1, 0);
                }
                tma_load_3d(sm0 + FwdSmem::K, &map_kv, bar_load, h * DK, b0, j0);
                tma_load_3d(sm0 + FwdSmem::K + 128 * 128, &map_kv, bar_load, h * DK, b0 + 1, j0);
                if (has_wr)
                    tma_load_3d(sm0 + FwdSmem::R, &map_wr, bar_load, 0, wrow, h);
                if (it > 0 && !mbar_wait(bar_free, (uint32_t)((it - 1) & 1), abort_s, err_flag, 17))
                    break;
                mbar_expect_tx(bar_loadv, 256 * 128);
                tma_load_3d(sm0 + FwdSmem::V, &map_kv, bar_loadv, HD + h * DK, b0, j0);
                tma_load_3d(sm0 + FwdSmem::V + 128 * 128, &map_kv, bar_loadv, HD + h * DK, b0 + 1, j0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idS = idesc_of(256, false, false), idE = idesc_of(WIN, false, false),
                               idO = idesc_of(64, false, true);
            const uint64_t dQ = tc::smem_desc_sw128(sm0 + FwdSmem::Q), dK = tc::smem_desc_sw128(sm0 + FwdSmem::K),
                           dR = tc::smem_desc_sw128(sm0 + FwdSmem::R);
            int it = 0;
            for (int kb = kbs.lo; kb <= kbs.hi; kb++, it++) {
                if (!mbar_wait(bar_load, (uint32_t)(it & 1), abort_s, err_flag, 12))
                    break;
                if (it > 0 && !mbar_wait(bar_tfree, (uint32_t)((it - 1) & 1), abort_s, err_flag, 13))
                    break;
                fence_after_sync();
                if (it == 0) ATC_STAMP(2);
#pragma unroll
                for (int k = 0; k < 4; k++)
                    umma_bf16(tmem, dQ + 2 * k, dK + 2 * k, idS, k > 0);
                if (has_wr) {
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_bf16(tmem + 256, dQ + 2 * k, dR + 2 * k, idE, k > 0);
                }
                umma_commit(bar_se);
                if (it == 0) ATC_STAMP(3);
                if (!mbar_wait(bar_p, (uint32_t)(it & 1), abort_s, err_flag, 14))
                    break;
                if (!mbar_wait(bar_loadv, (uint32_t)(it & 1), abort_s, err_flag, 18))
                    break;
                fence_after_sync();
                if (it == 0) ATC_STAMP(5);
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    const uint64_t dV = tc::smem_desc_sw128_mn(sm0 + FwdSmem::V + s * 128 * 128);
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const uint64_t dP = tc::smem_desc_sw128(sm0 + FwdSmem::P + (k >> 2) * 128 * 128) + 2 * (k & 3);
                        umma_bf16(tmem + 64 * s, dP, dV + 128 * k, idO, k > 0);
                    }
                }
                umma_commit(bar_o);
                umma_commit(bar_free);
                if (it == 0) ATC_STAMP(6);
            }
        }
    } else {
        // row threads: TMEM lane = 32 * (warp % 4) + lane; `half` picks the chunks and output columns
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane, s = row >> 6, i = row & 63, i_base = i - lane;
        const int b = b0 + s;
        const int tid = threadIdx.x - 64;
        const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
        const float sc2 = a.inv_sqrt * 1.4426950408889634f; // scores in the log2 domain
        const int brs_n = min(BRS_LEN, BRS_PAD + (kbs.hi + 1) * KB + 64);
        for (int r = tid; r < brs_n; r += NROW) {
            const int rr = r - BRS_PAD;
            brs[r] = (rr >= 0 && rr < L) ? a.br_scale * a.b_r[(size_t)h * L + rr] * sc2 : 0.0f;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        float m_run = -INFINITY, l_run = 0.0f;
        float o[32];
#pragma unroll
        for (int k = 0; k < 32; k++)
            o[k] = 0.0f;
        bool ok = true;
        int it = 0;
        for (int kb = kbs.lo; kb <= kbs.hi && ok; kb++, it++) {
            const int j0 = kb * KB;
            const int wlo = j0 - 63 + c0;
            const bool all_clamp = wlo < -(WIN - 2);
            if (lane == 0)
                ok = mbar_wait(bar_se, (uint32_t)(it & 1), abort_s, err_flag, 15);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            fence_after_sync();
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(4);
            // E of table row 0 for this query row (the left pad of nc_pad duplicates it)
            float e0 = 0.0f;
            const bool clampable = has_wr && wlo < 0;
            if (clampable) {
                e0 = __uint_as_float(tmem_ld1(trow + 256 + (all_clamp ? 0 : -wlo)));
                tmem_ld_wait();
            }
            // ---- pass 1: masked, scaled scores back into the S columns; maximum of this half
            float m_blk = -INFINITY;
#pragma unroll 1
            for (int cc = 0; cc < 2; cc++) {
                const int c = half * 2 + cc;
                uint32_t sv[32], x[64];
                tmem_ld32(trow + s * 128 + c * 32, sv);
                if (has_wr && !all_clamp) {
                    const uint32_t ecol = trow + 256 + c * 32 + (i_base == 0 ? 32 : 0);
                    tmem_ld32(ecol, x);
                    tmem_ld32(ecol + 32, x + 32);
                }
                tmem_ld_wait();
                if (has_wr && !all_clamp)
                    barrel_skew(x, lane);
                const int jc = j0 + c * 32;
                score_chunk(sv, x, has_wr, clampable, e0, all_clamp ? 32 : i - c0 - jc,
                            i + M - a.attn_len + 1 - jc, i + M - jc, brs + BRS_PAD + jc + (T - 1) - i, sc2);
#pragma unroll
                for (int k = 0; k < 32; k++)
                    m_blk = fmaxf(m_blk, __uint_as_float(sv[k]));
                tmem_st32(trow + s * 128 + c * 32, sv);
            }
            xch[half * 128 + row] = m_blk;
            tmem_st_wait();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            m_blk = fmaxf(m_blk, xch[(half ^ 1) * 128 + row]);
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(7);
            // ---- pass 2: probabilities (bf16, K-major atoms in shared memory), running sum
            const float m_new = fmaxf(m_run, m_blk);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const float alpha = ex2(m_run - m_use);
            float sum = 0.0f;
#pragma unroll 1
            for (int cc = 0; cc < 2; cc++) {
                const int c = half * 2 + cc;
                uint32_t sv[32];
                tmem_ld32(trow + s * 128 + c * 32, sv);
                tmem_ld_wait();
                unsigned char *prow = sm + FwdSmem::P + (c >> 1) * 128 * 128 + row * 128;
#pragma unroll
                for (int k = 0; k < 32; k++) {
                    const float p = ex2(__uint_as_float(sv[k]) - m_use);
                    sum += p;
                    sv[k] = __float_as_uint(p);
                }
#pragma unroll
                for (int v4 = 0; v4 < 4; v4++)
                    *reinterpret_cast<uint4 *>(prow + ((((c & 1) * 4 + v4) ^ (row & 7)) << 4)) = pack8(sv + v4 * 8);
            }
            l_run = l_run * alpha + sum;
            m_run = m_new;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            fence_before_sync();
            mbar_arrive(bar_p);
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(8);
            // ---- O block of this row's stream: this thread's 32 output columns
            if (lane == 0)
                ok = mbar_wait(bar_o, (uint32_t)(it & 1), abort_s, err_flag, 16);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            fence_after_sync();
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(9);
            {
                uint32_t y[32];
                tmem_ld32(trow + s * 64 + half * 32, y);
                tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < 32; k++)
                    o[k] = o[k] * alpha + __uint_as_float(y[k]);
            }
            fence_before_sync();
            mbar_arrive(bar_tfree);
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(10);
        }
        // the row's sum is the two halves' (same sequence of maxima on both sides)
        xch[(2 + half) * 128 + row] = l_run;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const float l_tot = half == 0 ? l_run + xch[3 * 128 + row] : xch[2 * 128 + row] + l_run;
        if (ok && i >= a.t0 && i < a.t1 && i < T && b < a.B) {
            const float inv = 1.0f / l_tot;
            bf16 *dst = reinterpret_cast<bf16 *>(a.o) + ((size_t)i * a.B + b) * HD + h * DK + half * 32;
#pragma unroll
            for (int v4 = 0; v4 < 4; v4++)
                reinterpret_cast<uint4 *>(dst)[v4] =
                    make_uint4(tc::pack_bf16(o[v4 * 8] * inv, o[v4 * 8 + 1] * inv),
                               tc::pack_bf16(o[v4 * 8 + 2] * inv, o[v4 * 8 + 3] * inv),
                               tc::pack_bf16(o[v4 * 8 + 4] * inv, o[v4 * 8 + 5] * inv),
                               tc::pack_bf16(o[v4 * 8 + 6] * inv, o[v4 * 8 + 7] * inv));
            if (a.lse && half == 0)
                a.lse[((size_t)b * a.H + h) * T + i] = (m_run + __log2f(l_tot)) * 0.6931471805599453f;
        }
    }
    if (threadIdx.x == 64)
        ATC_STAMP(11);
    // common exit: nobody touches TMEM after this barrier
    fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0)
        ATC_STAMP(12);
    if (*abort_s) {
        for (int w = 0; w < 2000; w++)
            __nanosleep(500);
    }
    if (warp == 1) {
        fence_after_sync();
        tc::tmem_dealloc(tmem, 512);
    }
}

// ---------------- backward ----------------
//
// Same CTA shape (one head of two streams, two row threads per row) and the same score pass as
// the forward kernel; the saved log-sum-exp gives the probabilities directly.  Per key block:
//
//   G1  S, E                                   as in the forward pass
//   r1  P = exp(a - lse), bf16, to shared memory (PS)
//   G2  dP = dO [V_b0 ; V_b1]^T    128 x 256    -> columns   0..255
//       dV_b = P_b^T dO_b          128 x 64     -> columns 384..511   (rows = keys)
//   r2  dV out; dS = P (dP - D) / sqrt(dk) (P as the MMAs saw it): bf16 over P in PS, and scattered into the window
//       layout dE[row][jj + 63 - i] (the inverse of the forward skew; zero elsewhere); the
//       entries whose table row is negative (left pad) are also summed into column 191
//   G3  dK_b = dS_b^T Q_b  -> 0..127 (rows = keys);  dQ_b = dS K_b -> 128..255;
//       dQ  += dE Rwin -> 256..319;  dRwin = dE^T Q -> 320..447 (rows = window rows, two
//       128-row halves);  column sums of dE (an all-ones operand) -> 448..479
//   r3  dK out; dQ accumulated in registers; dRwin and the column sums go to this CTA's slices
//       of the partial table gradients (window row c is table row wlo + c; row 191 is the left
//       pad's share of table row 0; the column sums are db_r): stored when one block covers
//       the whole table, added block after block otherwise
//
// Window row 191 of Rwin is loaded with table row 0 (a one-row TMA box), so that the left pad
// costs nothing extra: the forward term of a padded entry is E[.,191], dQ gets its share
// through dE[.,191] Rwin[191], and dRwin[191] is the padded entries' gradient of table row 0.
// The partial table gradients of a stream pair go to the slice of its first stream (the second
// stream's slice is zeroed); the caller sums the slices in stream order.
struct BwdSmem {
    static constexpr int DE = 0;                    // three K-major atoms [128][64]: window columns 0..191
    static constexpr int Q = DE + 3 * 128 * 128;    // [128][64]; also what the fourth-atom reads of dRwin see
    static constexpr int DO = Q + 128 * 128;        // [128][64]
    static constexpr int K = DO + 128 * 128;        // [256][64]
    static constexpr int V = K + 256 * 128;         // [256][64]
    static constexpr int R = V + 256 * 128;         // [192][64]: 191 window rows, then table row 0
    static constexpr int PS = R + WIN * 128;        // P, later dS: two K-major atoms [128][64]
    static constexpr int ONES = PS + 2 * 128 * 128; // 2 KB of bf16 1.0
    static constexpr int BRS = ONES + 2048;
    static constexpr int XCH = BRS + BRS_LEN * 4;   // [2][128] floats
    static constexpr int BAR = XCH + 2 * 128 * 4;
    static constexpr int TOTAL = BAR + 256 + 1024;
};

__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr, uint32_t lbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// dst[0..63] (+)= y[0..63] (fp32, 16-byte accesses; all loads first, then the stores)
// dst[0..63] (+)= TMEM row (this thread's lane, columns taddr .. taddr + 63), fp32, 16-byte
// accesses.  The TMEM loads are warp-collective: every lane runs them, `active` lanes store.
__device__ __forceinline__ void tmem_row_to_global(uint32_t taddr, float *dst, bool active, bool accumulate)
{
#pragma unroll 1
    for (int h2 = 0; h2 < 2; h2++) {
        uint32_t y[32];
        tmem_ld32(taddr + 32 * h2, y);
        tmem_ld_wait();
        if (active) {
            float4 *d4 = reinterpret_cast<float4 *>(dst) + 8 * h2;
            float4 t[8];
            if (accumulate) {
#pragma unroll
                for (int v4 = 0; v4 < 8; v4++)
                    t[v4] = d4[v4];
            }
#pragma unroll
            for (int v4 = 0; v4 < 8; v4++) {
                float4 r = make_float4(__uint_as_float(y[v4 * 4]), __uint_as_float(y[v4 * 4 + 1]),
                                       __uint_as_float(y[v4 * 4 + 2]), __uint_as_float(y[v4 * 4 + 3]));
                if (accumulate) {
                    r.x += t[v4].x; r.y += t[v4].y; r.z += t[v4].z; r.w += t[v4].w;
                }
                d4[v4] = r;
            }
        }
    }
}

// dst[0..63] (bf16) = TMEM row (columns taddr .. taddr + 63); warp-collective loads, `active` lanes store
__device__ __forceinline__ void tmem_row_to_global_bf16(uint32_t taddr, bf16 *dst, bool active)
{
#pragma unroll 1
    for (int h2 = 0; h2 < 2; h2++) {
        uint32_t y[32];
        tmem_ld32(taddr + 32 * h2, y);
        tmem_ld_wait();
        if (active) {
            uint4 *d4 = reinterpret_cast<uint4 *>(dst) + 4 * h2;
#pragma unroll
            for (int v4 = 0; v4 < 4; v4++)
                d4[v4] = pack8(y + v4 * 8);
        }
    }
}

// SINGLE: the queries see one key block only, so dQ needs no accumulator across blocks
template <bool SINGLE>
__global__ void __launch_bounds__(320, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_kv, const __grid_constant__ CUtensorMap map_wr,
                   const __grid_constant__ CUtensorMap map_wr0, AttnArgs a, int has_wr, int *err_flag)
{
    extern __shared__ unsigned char smraw_[];
    unsigned char *sm = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smraw_) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + BwdSmem::BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 11);
    volatile int *abort_s = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *brs = reinterpret_cast<float *>(sm + BwdSmem::BRS);
    float *xch = reinterpret_cast<float *>(sm + BwdSmem::XCH);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b0 = blockIdx.x * 2, h = blockIdx.y;
    const int T = a.T, M = a.M, L = a.L, P = a.P, HD = a.H * DK;
    const KeyBlocks kbs = key_blocks(M, L, a.attn_len, 0, T);
    const int c0 = P - M - 1;
    // one key block whose window covers the whole table and every b_r slot: the table gradients
    // are stored, not accumulated (and need no zero fill)
    const int wlo_first = kbs.lo * KB - 63 + c0;
    const bool direct = kbs.lo == kbs.hi && wlo_first <= 0 && wlo_first + 190 >= P - 1 &&
                        kbs.lo * KB + T - 64 <= 0 && kbs.lo * KB + 190 + T - 64 >= L - 1;
    pdl_trigger();
    if (threadIdx.x == 0)
        ATC_STAMP(0);

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_do)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_kv)) : "memory");
        mbar_init(smem_u32(&bars[0]), 1);    // load
        mbar_init(smem_u32(&bars[1]), 1);    // free
        mbar_init(smem_u32(&bars[2]), 1);    // g1
        mbar_init(smem_u32(&bars[3]), NROW); // r1
        mbar_init(smem_u32(&bars[4]), 1);    // g2
        mbar_init(smem_u32(&bars[5]), NROW); // r2
        mbar_init(smem_u32(&bars[6]), 1);    // g3
        mbar_init(smem_u32(&bars[7]), NROW); // r3
        mbar_init(smem_u32(&bars[8]), 1);    // g2b: dV
        mbar_init(smem_u32(&bars[9]), 1);    // g3b: dQ (table part), dRwin, column sums
        mbar_init(smem_u32(&bars[10]), 1);   // load of dO and V (needed from G2 on)
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the all-ones operand (any layout of ones is ones)
    for (int idx = threadIdx.x; idx < 2048 / 16; idx += blockDim.x)
        reinterpret_cast<uint4 *>(sm + BwdSmem::ONES)[idx] = make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1)
        tc::tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    pdl_wait();
    const uint32_t tmem = *tmem_slot;
    const uint32_t sm0 = smem_u32(sm);
    if (threadIdx.x == 0)
        ATC_STAMP(1);
    const uint32_t bar_load = smem_u32(&bars[0]), bar_free = smem_u32(&bars[1]), bar_g1 = smem_u32(&bars[2]),
                   bar_r1 = smem_u32(&bars[3]), bar_g2 = smem_u32(&bars[4]), bar_r2 = smem_u32(&bars[5]),
                   bar_g3 = smem_u32(&bars[6]), bar_r3 = smem_u32(&bars[7]), bar_g2b = smem_u32(&bars[8]),
                   bar_g3b = smem_u32(&bars[9]), bar_load2 = smem_u32(&bars[10]);

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int kb = kbs.lo; kb <= kbs.hi; kb++, it++) {
                const int j0 = kb * KB;
                if (it > 0 && !mbar_wait(bar_free, (uint32_t)((it - 1) & 1), abort_s, err_flag, 21))
                    break;
                const int wlo = j0 - 63 + c0;
                // Q, K and the table window complete the first barrier (S and E can start), dO and V the second
                mbar_expect_tx(bar_load, 256 * 128 + (has_wr ? WIN * 128 : 0) + (it == 0 ? 128 * 128 : 0));
                mbar_expect_tx(bar_load2, 256 * 128 + (it == 0 ? 128 * 128 : 0));
                if (it == 0) {
                    tma_load_3d(sm0 + BwdSmem::Q, &map_q, bar_load, h * DK, b0, 0);
                    tma_load_3d(sm0 + BwdSmem::Q + 64 * 128, &map_q, bar_load, h * DK, b0 + 1, 0);
                }
                tma_load_3d(sm0 + BwdSmem::K, &map_kv, bar_load, h * DK, b0, j0);
                tma_load_3d(sm0 + BwdSmem::K + 128 * 128, &map_kv, bar_load, h * DK, b0 + 1, j0);
                if (has_wr) {
                    tma_load_3d(sm0 + BwdSmem::R, &map_wr, bar_load, 0, wlo, h);             // 191 rows
                    tma_load_3d(sm0 + BwdSmem::R + 191 * 128, &map_wr0, bar_load, 0, 0, h); // table row 0
                }
                if (it == 0) {
                    tma_load_3d(sm0 + BwdSmem::DO, &map_do, bar_load2, h * DK, b0, 0);
                    tma_load_3d(sm0 + BwdSmem::DO + 64 * 128, &map_do, bar_load2, h * DK, b0 + 1, 0);
                }
                tma_load_3d(sm0 + BwdSmem::V, &map_kv, bar_load2, HD + h * DK, b0, j0);
                tma_load_3d(sm0 + BwdSmem::V + 128 * 128, &map_kv, bar_load2, HD + h * DK, b0 + 1, j0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idS = idesc_of(256, false, false), idE = idesc_of(WIN, false, false),
                               idMM = idesc_of(64, true, true), idKM = idesc_of(64, false, true),
                               idKM2 = idesc_of(128, false, true),
                               idCS = idesc_of(16, true, true);
            const uint64_t dQk = desc_sw128(sm0 + BwdSmem::Q, 16), dDOk = desc_sw128(sm0 + BwdSmem::DO, 16),
                           dKk = desc_sw128(sm0 + BwdSmem::K, 16), dVk = desc_sw128(sm0 + BwdSmem::V, 16),
                           dRk = desc_sw128(sm0 + BwdSmem::R, 16);
            const uint64_t dOnes = desc_sw128(sm0 + BwdSmem::ONES, 8192);
            int it = 0;
            for (int kb = kbs.lo; kb <= kbs.hi; kb++, it++) {
                if (!mbar_wait(bar_load, (uint32_t)(it & 1), abort_s, err_flag, 22))
                    break;
                if (it > 0 && !mbar_wait(bar_r3, (uint32_t)((it - 1) & 1), abort_s, err_flag, 23))
                    break;
                fence_after_sync();
                if (it == 0) ATC_STAMP(2);
                // G1
#pragma unroll
                for (int k = 0; k < 4; k++)
                    umma_bf16(tmem, dQk + 2 * k, dKk + 2 * k, idS, k > 0);
                if (has_wr) {
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_bf16(tmem + 256, dQk + 2 * k, dRk + 2 * k, idE, k > 0);
                }
                umma_commit(bar_g1);
                if (!mbar_wait(bar_load2, (uint32_t)(it & 1), abort_s, err_flag, 31))
                    break;
                if (!mbar_wait(bar_r1, (uint32_t)(it & 1), abort_s, err_flag, 24))
                    break;
                fence_after_sync();
                // G2
#pragma unroll
                for (int k = 0; k < 4; k++)
                    umma_bf16(tmem, dDOk + 2 * k, dVk + 2 * k, idS, k > 0);
                umma_commit(bar_g2); // dP: the row threads start on dS while dV is computed
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    const uint64_t aP = desc_sw128(sm0 + BwdSmem::PS + s * 64 * 128, 128 * 128);
                    const uint64_t bDO = desc_sw128(sm0 + BwdSmem::DO + s * 64 * 128, 8192);
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_bf16(tmem + 384 + 64 * s, aP + 128 * k, bDO + 128 * k, idMM, k > 0);
                }
                umma_commit(bar_g2b);
                if (!mbar_wait(bar_r2, (uint32_t)(it & 1), abort_s, err_flag, 25))
                    break;
                fence_after_sync();
                // G3
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    const uint64_t aS = desc_sw128(sm0 + BwdSmem::PS + s * 64 * 128, 128 * 128);
                    const uint64_t bQ = desc_sw128(sm0 + BwdSmem::Q + s * 64 * 128, 8192);
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_bf16(tmem + 64 * s, aS + 128 * k, bQ + 128 * k, idMM, k > 0);
                }
                {
                    // dQ (key part) of both streams in one product: B = [K_b0 | K_b1], the second
                    // stream's keys being the next 64-column block of the MN-major operand
                    const uint64_t bK = desc_sw128(sm0 + BwdSmem::K, 128 * 128);
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const uint64_t aSk = desc_sw128(sm0 + BwdSmem::PS + (k >> 2) * 128 * 128, 16) + 2 * (k & 3);
                        umma_bf16(tmem + 128, aSk, bK + 128 * k, idKM2, k > 0);
                    }
                }
                umma_commit(bar_g3);
                if (has_wr) {
                    const uint64_t bR = desc_sw128(sm0 + BwdSmem::R, 8192);
#pragma unroll
                    for (int k = 0; k < 12; k++) {
                        const uint64_t aE = desc_sw128(sm0 + BwdSmem::DE + (k >> 2) * 128 * 128, 16) + 2 * (k & 3);
                        umma_bf16(tmem + 256, aE, bR + 128 * k, idKM, k > 0);
                    }
                }
                {
                    const uint64_t bQ = desc_sw128(sm0 + BwdSmem::Q, 8192);
#pragma unroll
                    for (int w = 0; w < 2; w++) {
                        const uint64_t aE = desc_sw128(sm0 + BwdSmem::DE + 2 * w * 128 * 128, 128 * 128);
                        if (has_wr) {
#pragma unroll
                            for (int k = 0; k < 8; k++)
                                umma_bf16(tmem + 320 + 64 * w, aE + 128 * k, bQ + 128 * k, idMM, k > 0);
                        }
#pragma unroll
                        for (int k = 0; k < 8; k++)
                            umma_bf16(tmem + 448 + 16 * w, aE + 128 * k, dOnes, idCS, k > 0);
                    }
                }
                umma_commit(bar_g3b);
                umma_commit(bar_free);
            }
        }
    } else {
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane, s = row >> 6, i = row & 63, i_base = i - lane;
        const int b = b0 + s;
        const bool rowvalid = i < T && b < a.B;
        const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
        const int tid = threadIdx.x - 64;
        const float sc2 = a.inv_sqrt * 1.4426950408889634f;
        // D_i = dO_i . O_i and the saved log-sum-exp (log2 domain); both threads of a row compute them.
        // Their loads go out first; everything else of the prologue runs under their latency.
        uint4 ox[8], dx[8];
        float lse2 = 0.0f;
        if (rowvalid) {
            const uint4 *po = reinterpret_cast<const uint4 *>(reinterpret_cast<const bf16 *>(a.out) + ((size_t)i * a.B + b) * HD + h * DK);
            const uint4 *pd = reinterpret_cast<const uint4 *>(reinterpret_cast<const bf16 *>(a.dout) + ((size_t)i * a.B + b) * HD + h * DK);
#pragma unroll
            for (int v4 = 0; v4 < 8; v4++) {
                ox[v4] = po[v4];
                dx[v4] = pd[v4];
            }
            lse2 = a.lse[((size_t)b * a.H + h) * T + i] * 1.4426950408889634f;
        }
        if (threadIdx.x == 64) ATC_STAMP(14);
        // scaled b_r, slots -64 .. what the last key block can name
        const int brs_n = min(BRS_LEN, BRS_PAD + (kbs.hi + 1) * KB + 64);
        for (int r = tid; r < brs_n; r += NROW) {
            const int rr = r - BRS_PAD;
            brs[r] = (rr >= 0 && rr < L) ? a.br_scale * a.b_r[(size_t)h * L + rr] * sc2 : 0.0f;
        }
        if (threadIdx.x == 64) ATC_STAMP(15);
        // this pair's slices of the partial table gradients; the second stream's slice stays zero
        float *dwr = (has_wr && a.dwr_part) ? a.dwr_part + ((size_t)b0 * a.H + h) * P * DK : nullptr;
        float *dbr = a.dbr_part ? a.dbr_part + ((size_t)b0 * a.H + h) * L : nullptr;
        for (int s2 = direct ? 1 : 0; s2 < 2 && b0 + s2 < a.B; s2++) {
            if (dwr)
                for (int idx = tid; idx < P * DK / 4; idx += NROW)
                    reinterpret_cast<float4 *>(dwr + (size_t)s2 * a.H * P * DK)[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (dbr)
                for (int idx = tid; idx < L; idx += NROW)
                    dbr[(size_t)s2 * a.H * L + idx] = 0.0f;
        }
        if (threadIdx.x == 64) ATC_STAMP(16);
        // keys no query attends to get zero gradients
        bf16 *dkv = reinterpret_cast<bf16 *>(a.dkv);
        for (int kb = 0; kb * KB < L; kb++) {
            if (kb >= kbs.lo && kb <= kbs.hi)
                continue;
            const int j = kb * KB + row;
            if (j < L && b0 + half < a.B) {
                uint4 *dst = reinterpret_cast<uint4 *>(dkv + ((size_t)j * a.B + b0 + half) * a.dkvp + h * DK);
                uint4 *dst2 = reinterpret_cast<uint4 *>(dkv + ((size_t)j * a.B + b0 + half) * a.dkvp + HD + h * DK);
#pragma unroll
                for (int v4 = 0; v4 < 8; v4++) {
                    dst[v4] = make_uint4(0u, 0u, 0u, 0u);
                    dst2[v4] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
        }
        if (threadIdx.x == 64) ATC_STAMP(17);
        float Di = 0.0f;
        if (rowvalid) {
#pragma unroll
            for (int v4 = 0; v4 < 8; v4++) {
                const uint32_t xw[4] = {ox[v4].x, ox[v4].y, ox[v4].z, ox[v4].w}, yw[4] = {dx[v4].x, dx[v4].y, dx[v4].z, dx[v4].w};
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const __nv_bfloat162 xa = *reinterpret_cast<const __nv_bfloat162 *>(&xw[u]);
                    const __nv_bfloat162 ya = *reinterpret_cast<const __nv_bfloat162 *>(&yw[u]);
                    Di += __low2float(xa) * __low2float(ya) + __high2float(xa) * __high2float(ya);
                }
            }
        }
        if (threadIdx.x == 64) ATC_STAMP(18);
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (threadIdx.x == 64) ATC_STAMP(3);
        float dq_acc[SINGLE ? 1 : 32];
#pragma unroll
        for (int k = 0; k < (SINGLE ? 1 : 32); k++)
            dq_acc[k] = 0.0f;
        bf16 *erow = reinterpret_cast<bf16 *>(sm + BwdSmem::DE);
        bool ok = true;
        int it = 0;
        for (int kb = kbs.lo; kb <= kbs.hi && ok; kb++, it++) {
            const int j0 = kb * KB;
            const int wlo = j0 - 63 + c0;
            // this row's dE window cells: zero (the previous block's MMAs are done with them); each
            // thread takes half of the row's 24 16-byte pieces, rotated by lane against bank conflicts
#pragma unroll
            for (int q12 = 0; q12 < 12; q12++) {
                const int piece = half * 12 + q12, at = piece >> 3, v4 = ((piece & 7) + lane) & 7;
                *reinterpret_cast<uint4 *>(sm + BwdSmem::DE + at * 128 * 128 + row * 128 + (v4 << 4)) = make_uint4(0u, 0u, 0u, 0u);
            }
            if (lane == 0)
                ok = mbar_wait(bar_g1, (uint32_t)(it & 1), abort_s, err_flag, 26);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            fence_after_sync();
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(4);
            float e0 = 0.0f;
            const bool clampable = has_wr && wlo < 0;
            if (clampable) {
                e0 = __uint_as_float(tmem_ld1(trow + 256 + 191));
                tmem_ld_wait();
            }
            // ---- r1: probabilities of this thread's two chunks, bf16, into the K-major atoms of PS
#pragma unroll 1
            for (int cc = 0; cc < 2; cc++) {
                const int c = half * 2 + cc;
                uint32_t sv[32], x[64];
                tmem_ld32(trow + s * 128 + c * 32, sv);
                if (has_wr) {
                    const uint32_t ecol = trow + 256 + c * 32 + (i_base == 0 ? 32 : 0);
                    tmem_ld32(ecol, x);
                    tmem_ld32(ecol + 32, x + 32);
                }
                tmem_ld_wait();
                if (has_wr)
                    barrel_skew(x, lane);
                const int jc = j0 + c * 32;
                score_chunk(sv, x, has_wr, clampable, e0, i - c0 - jc, i + M - a.attn_len + 1 - jc,
                            rowvalid ? i + M - jc : -1, brs + BRS_PAD + jc + (T - 1) - i, sc2);
#pragma unroll
                for (int k = 0; k < 32; k++)
                    sv[k] = __float_as_uint(ex2(__uint_as_float(sv[k]) - lse2));
                unsigned char *prow = sm + BwdSmem::PS + (c >> 1) * 128 * 128 + row * 128;
#pragma unroll
                for (int v4 = 0; v4 < 4; v4++)
                    *reinterpret_cast<uint4 *>(prow + ((((c & 1) * 4 + v4) ^ (row & 7)) << 4)) = pack8(sv + v4 * 8);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            fence_before_sync();
            mbar_arrive(bar_r1);
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(5);
            // ---- r2
            if (lane == 0)
                ok = mbar_wait(bar_g2, (uint32_t)(it & 1), abort_s, err_flag, 27);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            fence_after_sync();
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(6);
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(7);
            float sclamp = 0.0f;
#pragma unroll 1
            for (int cc = 0; cc < 2; cc++) {
                const int c = half * 2 + cc;
                uint32_t dp[32];
                tmem_ld32(trow + s * 128 + c * 32, dp);
                unsigned char *prow = sm + BwdSmem::PS + (c >> 1) * 128 * 128 + row * 128;
                // the probabilities as the MMAs saw them (bf16), read back from this thread's own cells
                uint32_t pw[16];
#pragma unroll
                for (int v4 = 0; v4 < 4; v4++) {
                    const uint4 t4 = *reinterpret_cast<const uint4 *>(prow + ((((c & 1) * 4 + v4) ^ (row & 7)) << 4));
                    pw[v4 * 4] = t4.x; pw[v4 * 4 + 1] = t4.y; pw[v4 * 4 + 2] = t4.z; pw[v4 * 4 + 3] = t4.w;
                }
                tmem_ld_wait();
                // window column of key jj is jj + 63 - i; keys below kpad are on the left pad
                const int wc0 = c * 32 + 63 - i, kpad = -wlo - wc0;
                uint32_t pk[16];
#pragma unroll
                for (int k = 0; k < 32; k += 2) {
                    const __nv_bfloat162 pp = *reinterpret_cast<const __nv_bfloat162 *>(&pw[k >> 1]);
                    const float d0 = __low2float(pp) * (__uint_as_float(dp[k]) - Di) * a.inv_sqrt;
                    const float d1 = __high2float(pp) * (__uint_as_float(dp[k + 1]) - Di) * a.inv_sqrt;
                    const __nv_bfloat162 hh = __floats2bfloat162_rn(d0, d1);
                    pk[k >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
                    if (k < kpad)
                        sclamp += __low2float(hh);
                    if (k + 1 < kpad)
                        sclamp += __high2float(hh);
                    const int w0 = wc0 + k, w1 = w0 + 1;
                    erow[(size_t)(w0 >> 6) * 128 * 64 + row * 64 + (((((w0 & 63) >> 3) ^ (row & 7)) << 3) | (w0 & 7))] = hh.x;
                    erow[(size_t)(w1 >> 6) * 128 * 64 + row * 64 + (((((w1 & 63) >> 3) ^ (row & 7)) << 3) | (w1 & 7))] = hh.y;
                }
#pragma unroll
                for (int v4 = 0; v4 < 4; v4++)
                    *reinterpret_cast<uint4 *>(prow + ((((c & 1) * 4 + v4) ^ (row & 7)) << 4)) =
                        make_uint4(pk[v4 * 4], pk[v4 * 4 + 1], pk[v4 * 4 + 2], pk[v4 * 4 + 3]);
            }
            xch[half * 128 + row] = sclamp;
            if (lane == 0)
                ok = mbar_wait(bar_g2b, (uint32_t)(it & 1), abort_s, err_flag, 29);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            fence_after_sync();
            {
                // dV of key j0 + row, stream b0 + half
                const int j = j0 + row;
                const bool act = j < L && b0 + half < a.B;
                tmem_row_to_global_bf16(trow + 384 + 64 * half,
                                        dkv + ((size_t)(act ? j : 0) * a.B + (act ? b0 + half : 0)) * a.dkvp + HD + h * DK, act);
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (half == 0) {
                const int w = 191;
                erow[(size_t)(w >> 6) * 128 * 64 + row * 64 + (((((w & 63) >> 3) ^ (row & 7)) << 3) | (w & 7))] =
                    __float2bfloat16_rn(sclamp + xch[128 + row]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            fence_before_sync();
            mbar_arrive(bar_r2);
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(8);
            // ---- r3
            if (lane == 0)
                ok = mbar_wait(bar_g3, (uint32_t)(it & 1), abort_s, err_flag, 28);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            fence_after_sync();
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(9);
            {
                // dK of key j0 + row, stream b0 + half
                const int j = j0 + row;
                const bool act = j < L && b0 + half < a.B;
                tmem_row_to_global_bf16(trow + 64 * half,
                                        dkv + ((size_t)(act ? j : 0) * a.B + (act ? b0 + half : 0)) * a.dkvp + h * DK, act);
            }
            float dq[32];
            {
                uint32_t y[32];
                tmem_ld32(trow + 128 + 64 * s + 32 * half, y);
                tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < 32; k++)
                    dq[k] = __uint_as_float(y[k]) + (SINGLE ? 0.0f : dq_acc[SINGLE ? 0 : k]);
            }
            if (lane == 0)
                ok = mbar_wait(bar_g3b, (uint32_t)(it & 1), abort_s, err_flag, 30);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            fence_after_sync();
            if (has_wr) {
                uint32_t z[32];
                tmem_ld32(trow + 256 + 32 * half, z);
                tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < 32; k++)
                    dq[k] += __uint_as_float(z[k]);
            }
            if (SINGLE || kb == kbs.hi) {
                if (rowvalid) {
                    bf16 *dst = reinterpret_cast<bf16 *>(a.dq) + ((size_t)i * a.B + b) * a.dqp + h * DK + half * 32;
#pragma unroll
                    for (int v4 = 0; v4 < 4; v4++)
                        reinterpret_cast<uint4 *>(dst)[v4] =
                            make_uint4(tc::pack_bf16(dq[v4 * 8], dq[v4 * 8 + 1]), tc::pack_bf16(dq[v4 * 8 + 2], dq[v4 * 8 + 3]),
                                       tc::pack_bf16(dq[v4 * 8 + 4], dq[v4 * 8 + 5]), tc::pack_bf16(dq[v4 * 8 + 6], dq[v4 * 8 + 7]));
                }
            } else {
#pragma unroll
                for (int k = 0; k < (SINGLE ? 1 : 32); k++)
                    dq_acc[k] = dq[k];
            }
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(10);
            // table gradients: window rows 0..127 by the first thread of each row, then window rows
            // 128..190 by the second threads of rows 0..62, then window row 191 = the left pad's
            // share of table row 0.  When they are accumulated (several key blocks) the parts may
            // meet in one table row, hence the barriers; a single block that stores them needs one
            // only in front of the pad row's addition.
            if (half == 0) {
                const int x = wlo + row;
                if (has_wr)
                    tmem_row_to_global(trow + 320, dwr + (size_t)(x >= 0 && x < P ? x : 0) * DK, dwr && x >= 0 && x < P, !direct);
                const float cs = __uint_as_float(tmem_ld1(trow + 448));
                tmem_ld_wait();
                const int r = j0 + row + T - 64;
                if (dbr && r >= 0 && r < L)
                    dbr[r] = a.br_scale * cs + (direct ? 0.0f : dbr[r]);
            }
            if (!direct)
                asm volatile("bar.sync 1, 256;" ::: "memory");
            if (half == 1 && quarter < 2) { // warp-uniform
                const int c = 128 + row, x = wlo + c;
                if (has_wr)
                    tmem_row_to_global(trow + 384, dwr + (size_t)(x >= 0 && x < P ? x : 0) * DK,
                                       dwr && c <= 190 && x >= 0 && x < P, !direct);
                const float cs = __uint_as_float(tmem_ld1(trow + 464));
                tmem_ld_wait();
                const int r = j0 + c + T - 64;
                if (dbr && c <= 190 && r >= 0 && r < L)
                    dbr[r] = a.br_scale * cs + (direct ? 0.0f : dbr[r]);
            }
            if (clampable) { // CTA-uniform
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (half == 1 && quarter == 1) // warp-uniform; lane 31 holds window row 191
                    tmem_row_to_global(trow + 384, dwr, dwr && row == 63, true);
            }
            fence_before_sync();
            mbar_arrive(bar_r3); // every TMEM read of this block is done
            if (!direct)
                asm volatile("bar.sync 1, 256;" ::: "memory");
            if (it == 0 && threadIdx.x == 64) ATC_STAMP(11);
        }
    }
    if (threadIdx.x == 64)
        ATC_STAMP(12);
    fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0)
        ATC_STAMP(13);
    if (*abort_s) {
        for (int w = 0; w < 2000; w++)
            __nanosleep(500);
    }
    if (warp == 1) {
        fence_after_sync();
        tc::tmem_dealloc(tmem, 512);
    }
}

// ---------------- host side ----------------

struct Tmap3Key {
    const void *ptr;
    long d0, d1, d2, s1, s2;
    int b0, b1, b2;
    bool operator<(const Tmap3Key &o) const
    {
        return std::tie(ptr, d0, d1, d2, s1, s2, b0, b1, b2) < std::tie(o.ptr, o.d0, o.d1, o.d2, o.s1, o.s2, o.b0, o.b1, o.b2);
    }
};

// 3-D map over bf16 data: dims (d0 contiguous, d1, d2), strides s1, s2 in elements, 128-byte swizzle
static int make_tmap3(const void *ptr, long d0, long d1, long d2, long s1, long s2, int b0, int b1, int b2,
                      CUtensorMap *out)
{
    static std::map<Tmap3Key, CUtensorMap> cache;
    static std::mutex mu;
    Tmap3Key key{ptr, d0, d1, d2, s1, s2, b0, b1, b2};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return NNCU_OK;
    }
    tc::EncodeTiledFn fn = tc::encode_fn();
    if (!fn)
        return nncu_fail(NNCU_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2};
    cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2};
    cuuint32_t box[3] = {(cuuint32_t)b0, (cuuint32_t)b1, (cuuint32_t)b2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return nncu_fail(NNCU_ERR_CUDA, "cuTensorMapEncodeTiled (3-d) failed: %d", (int)r);
    if (cache.size() > 4096)
        cache.clear();
    cache[key] = *out;
    return NNCU_OK;
}

// shapes and operand placements the tensor-core kernels take
inline bool supported(const AttnArgs &a, const void *q, const void *kv, const void *w_r16)
{
    return a.dk == DK && a.T <= 64 && a.L <= MAXL && (a.qp % 8) == 0 && (a.kvp % 8) == 0 &&
           (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(kv) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(w_r16) & 15) == 0 &&
           (w_r16 || !a.w_r || (size_t)a.H * a.P * DK <= ((size_t)1 << 20));
}

static int forward(const AttnArgs &a, const void *w_r16, int *err_flag, cudaStream_t st)
{
    CUtensorMap mq, mkv, mwr;
    NNCU_TRY(make_tmap3(a.q, a.H * DK, a.B, a.T, a.qp, (long)a.B * a.qp, DK, 1, 64, &mq));
    NNCU_TRY(make_tmap3(a.kv, 2 * a.H * DK, a.B, a.L, a.kvp, (long)a.B * a.kvp, DK, 1, KB, &mkv));
    mwr = mq;
    if (w_r16)
        NNCU_TRY(make_tmap3(w_r16, DK, a.P, a.H, DK, (long)a.P * DK, DK, WIN, 1, &mwr));
    static bool attr_done = false;
    if (!attr_done) {
        CUDA_TRY(cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem::TOTAL));
        attr_done = true;
    }
    launch_k(attn_fwd_tc_kernel, dim3((a.B + 1) / 2, a.H), dim3(320), FwdSmem::TOTAL, st, mq, mkv, mwr, a,
             w_r16 ? 1 : 0, err_flag);
    KERNEL_CHECK();
    return NNCU_OK;
}

static int backward(const AttnArgs &a, const void *w_r16, int *err_flag, cudaStream_t st)
{
    CUtensorMap mq, mdo, mkv, mwr, mwr0;
    NNCU_TRY(make_tmap3(a.q, a.H * DK, a.B, a.T, a.qp, (long)a.B * a.qp, DK, 1, 64, &mq));
    NNCU_TRY(make_tmap3(a.dout, a.H * DK, a.B, a.T, a.H * DK, (long)a.B * a.H * DK, DK, 1, 64, &mdo));
    NNCU_TRY(make_tmap3(a.kv, 2 * a.H * DK, a.B, a.L, a.kvp, (long)a.B * a.kvp, DK, 1, KB, &mkv));
    mwr = mq;
    mwr0 = mq;
    if (w_r16) {
        NNCU_TRY(make_tmap3(w_r16, DK, a.P, a.H, DK, (long)a.P * DK, DK, WIN - 1, 1, &mwr));
        NNCU_TRY(make_tmap3(w_r16, DK, a.P, a.H, DK, (long)a.P * DK, DK, 1, 1, &mwr0));
    }
    static bool attr_done = false;
    if (!attr_done) {
        CUDA_TRY(cudaFuncSetAttribute(attn_bwd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL));
        CUDA_TRY(cudaFuncSetAttribute(attn_bwd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL));
        attr_done = true;
    }
    const KeyBlocks kbs = key_blocks(a.M, a.L, a.attn_len, 0, a.T);
    if (kbs.lo == kbs.hi)
        launch_k(attn_bwd_tc_kernel<true>, dim3((a.B + 1) / 2, a.H), dim3(320), BwdSmem::TOTAL, st, mq, mdo, mkv, mwr, mwr0,
                 a, w_r16 ? 1 : 0, err_flag);
    else
        launch_k(attn_bwd_tc_kernel<false>, dim3((a.B + 1) / 2, a.H), dim3(320), BwdSmem::TOTAL, st, mq, mdo, mkv, mwr, mwr0,
                 a, w_r16 ? 1 : 0, err_flag);
    KERNEL_CHECK();
    return NNCU_OK;
}

inline bool supported_bwd(const AttnArgs &a, const void *w_r16)
{
    return supported(a, a.q, a.kv, w_r16) && a.t0 == 0 && a.t1 == a.T && (a.dqp % 8) == 0 && (a.dkvp % 8) == 0 &&
           (reinterpret_cast<uintptr_t>(a.dq) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.dkv) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(a.dout) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0 && a.lse;
}

// ---- per-device scratch inside the library image: a time-out flag for callers without a model
// and a bf16 copy of the position table for callers that pass it in fp32 only (the isolated op)
constexpr size_t TABLE16_ELEMS = (size_t)1 << 20; // n_head * d_pos * 64 up to 1 Mi entries (2 MiB)
static __device__ int g_flag;
static __device__ __align__(256) bf16 g_table16[TABLE16_ELEMS];
constexpr int MAX_DEVICES = 64;
static int *g_flag_ptr[MAX_DEVICES];
static bf16 *g_table_ptr[MAX_DEVICES];

static int device_scratch(int **flag, bf16 **table)
{
    int dev = -1;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES)
        return nncu_fail(NNCU_ERR_INVALID, "device ordinal %d out of range", dev);
    if (!g_flag_ptr[dev]) {
        int *f = nullptr;
        bf16 *t = nullptr;
        CUDA_TRY(cudaGetSymbolAddress((void **)&f, g_flag));
        CUDA_TRY(cudaGetSymbolAddress((void **)&t, g_table16));
        CUDA_TRY(cudaMemset(f, 0, sizeof(int)));
        g_flag_ptr[dev] = f;
        g_table_ptr[dev] = t;
    }
    *flag = g_flag_ptr[dev];
    *table = g_table_ptr[dev];
    return NNCU_OK;
}

__global__ void table_to_bf16_kernel(const float *__restrict__ src, bf16 *__restrict__ dst, size_t n)
{
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n)
        dst[i] = __float2bfloat16_rn(src[i]);
}

inline bool enabled()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("NNCU_ATTN_TC");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

inline bool bwd_enabled()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("NNCU_ATTN_TC_BWD");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// Forward pass through the tcgen05 kernel.  w_r16 may be NULL while a.w_r is not: the table is
// then converted into the library's own bf16 scratch first (calls that overlap on the GPU and
// both need that conversion race on the scratch; a model always passes its bf16 shadow).
static int forward_any(const AttnArgs &a, const void *w_r16, int *err_flag, cudaStream_t st)
{
    int *flag = nullptr;
    bf16 *table = nullptr;
    if (!err_flag || (a.w_r && !w_r16))
        NNCU_TRY(device_scratch(&flag, &table));
    if (a.w_r && !w_r16) {
        const size_t n = (size_t)a.H * a.P * DK;
        launch_k(table_to_bf16_kernel, dim3((unsigned)ceil_div((long long)n, 256)), dim3(256), 0, st, a.w_r, table, n);
        KERNEL_CHECK();
        w_r16 = table;
    }
    return forward(a, a.w_r ? w_r16 : nullptr, err_flag ? err_flag : flag, st);
}

static int backward_any(const AttnArgs &a, const void *w_r16, int *err_flag, cudaStream_t st)
{
    int *flag = nullptr;
    bf16 *table = nullptr;
    if (!err_flag || (a.w_r && !w_r16))
        NNCU_TRY(device_scratch(&flag, &table));
    if (a.w_r && !w_r16) {
        const size_t n = (size_t)a.H * a.P * DK;
        launch_k(table_to_bf16_kernel, dim3((unsigned)ceil_div((long long)n, 256)), dim3(256), 0, st, a.w_r, table, n);
        KERNEL_CHECK();
        w_r16 = table;
    }
    return backward(a, a.w_r ? w_r16 : nullptr, err_flag ? err_flag : flag, st);
}

} // namespace attc
