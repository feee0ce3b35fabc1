// gemm_tc.cuh -- bf16 x bf16 -> fp32 GEMM on the 5th-generation tensor cores.
//
//   C[M][N] = sum_k A(m,k) B(n,k) (+ bias[N]) (+ addsrc)
//
// Each operand is either K-major (stored [rows = m or n][k], the forward y = x W^T form) or
// MN-major (stored [k][m or n]): dx = dy W reads W MN-major, dW = dy^T x reads both operands
// MN-major, so no transposed copy of a weight or an activation is ever made.
//
// Replaces nc_matmul (libnc.h:270-276) for every projection of the bf16 model.
// sm_100a only: operands are staged by TMA (cp.async.bulk.tensor, 128-byte
// swizzle, each CTA loading its own tiles) into a 3- or 4-stage shared-memory ring, one
// elected thread issues tcgen05.mma (UMMA 128 x BN x 16, cta_group::1) into a
// TMEM accumulator, and four epilogue warps read it back with tcgen05.ld.
//
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocation, MMA issue of the even k-blocks (one lane), TMEM release
//   warps 2-5   epilogue: warp w owns TMEM lanes 32*(w%4) .. +31 = tile rows
//   warp 6      MMA issue of the odd k-blocks (one lane), into a second accumulator
//   warp 7      TMA producer of the odd k-blocks (one lane); warp 0 loads the even ones
//
// Out-of-range rows/columns/k are zero-filled by TMA on load and clipped by TMA
// on store (the tile is staged in the idle operand ring, 128-byte swizzled), so M, N are arbitrary and K only needs 16-byte row strides.
// Every wait is bounded: on expiry the kernel raises *err_flag and leaves
// through the common exit that releases TMEM.
//
// Output element (m, n) is the accumulation, in k order, of UMMA K=16 steps of
// one fixed instruction shape; it does not depend on what else is in the tile,
// so a row of a one-symbol step equals the same row of a full-segment launch.
#pragma once
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace tc {

constexpr int BM = 128;
constexpr int BK = 64; // 64 bf16 = 128 bytes = one swizzle row

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// bounded wait; returns false (and raises the flags) when the limit is hit.  The thread
// suspends inside try_wait (up to about a microsecond per try) instead of polling; the loop is
// PTX so that the path of a barrier that is already complete is a try and a branch.
#ifdef NNCU_TC_SPIN
constexpr uint32_t WAIT_TRIES = 1u << 24;
#else
constexpr uint32_t WAIT_TRIES = 1u << 21;
#endif
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_s,
                                          int *err_flag, int code, uint32_t tries = WAIT_TRIES)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p, q;\n\t.reg .u32 c;\n\t"
                 "mov.u32 c, 0;\n"
                 "NNCU_WAIT:\n\t"
                 #ifdef NNCU_TC_SPIN
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#else
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %4;\n\t"
#endif

                 "@p bra NNCU_DONE;\n\t"
                 "add.u32 c, c, 1;\n\t"
                 "setp.lt.u32 q, c, %3;\n\t"
                 "@q bra NNCU_WAIT;\n"
                 "NNCU_DONE:\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity), "r"(tries), "r"(1000u)
                 : "memory");
    if (!ok) {
        *abort_s = 1;
        atomicExch(err_flag, code);
    }
    return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// The four UMMAs of one 64-wide k-block.  alo / blo: low words of the operand descriptors of the
// block's first 16-wide slice; a later slice adds ASTEP / BSTEP to the address field.  The
// high descriptor word is constant (DESC_HI).  `accumulate` = 0 makes the first UMMA overwrite.
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
template <uint32_t ASTEP, uint32_t BSTEP>
__device__ __forceinline__ void umma_bf16_x4(uint32_t tmem_d, uint32_t alo, uint32_t blo, uint32_t idesc,
                                             uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p, t;\n\t.reg .b64 da, db;\n\t.reg .b32 la, lb;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "setp.eq.b32 t, %4, %4;\n\t"
                 "mov.b64 da, {%1, %5};\n\t"
                 "mov.b64 db, {%2, %5};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
                 "add.u32 la, %1, %6;\n\t"
                 "add.u32 lb, %2, %7;\n\t"
                 "mov.b64 da, {la, %5};\n\t"
                 "mov.b64 db, {lb, %5};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, t;\n\t"
                 "add.u32 la, %1, %8;\n\t"
                 "add.u32 lb, %2, %9;\n\t"
                 "mov.b64 da, {la, %5};\n\t"
                 "mov.b64 db, {lb, %5};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, t;\n\t"
                 "add.u32 la, %1, %10;\n\t"
                 "add.u32 lb, %2, %11;\n\t"
                 "mov.b64 da, {la, %5};\n\t"
                 "mov.b64 db, {lb, %5};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, t;\n\t}" ::"r"(tmem_d),
                 "r"(alo), "r"(blo), "r"(idesc), "r"(accumulate), "r"(DESC_HI), "n"(ASTEP), "n"(BSTEP),
                 "n"(2 * ASTEP), "n"(2 * BSTEP), "n"(3 * ASTEP), "n"(3 * BSTEP)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t gets row (lane base + t).  Asynchronous:
// the registers are valid after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// r = 32 columns at taddr (+ the same columns of the second accumulator `other` columns further
// on, when `dual`), complete on return
__device__ __forceinline__ void tmem_ld32_pair(uint32_t taddr, uint32_t other, bool dual, uint32_t *r)
{
    tmem_ld32(taddr, r);
    if (dual) {
        uint32_t q[32];
        tmem_ld32(taddr + other, q);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j++)
            r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(q[j]));
    } else {
        tmem_ld_wait();
    }
}

// shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)1 << 16;                   // leading-dimension byte offset (unused here)
    d |= (uint64_t)(1024u >> 4) << 32;        // stride-dimension byte offset
    d |= (uint64_t)1 << 46;                   // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
    return d;
}

// MN-major tile: [k rows][64 elements along m/n] per 8 KB box, 128-byte swizzle; boxes for
// the next 64 m/n elements follow at +8192 bytes (leading offset), the next 8 k rows at
// +1024 bytes (stride offset)
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(8192u >> 4) << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

#ifdef NNCU_GEMM_TRACE
// tuning aid (off in normal builds): per-CTA clock64() stamps of the kernel's phases
__device__ long long *g_tc_trace = nullptr;
__device__ int g_tc_mode = 0; // 1: no loads (barriers only), 2: no MMAs (commits only)
#define TC_MODE(bit) (tc_mode_ & (bit))
#define TC_MODE_LOAD const int tc_mode_ = g_tc_mode; long long *const tc_trace_ = g_tc_trace;
#define TC_STAMP(slot)                                                   \
    do {                                                                 \
        long long *t_ = tc_trace_;                                       \
        if (t_ && blockIdx.x + blockIdx.y * gridDim.x < 128)             \
            t_[(blockIdx.x + blockIdx.y * gridDim.x) * 16 + (slot)] = clock64(); \
    } while (0)
#else
#define TC_MODE(bit) 0
#define TC_MODE_LOAD
#define TC_STAMP(slot) \
    do {               \
    } while (0)
#endif

template <int BN>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
#ifndef NNCU_TC_STAGES64
#define NNCU_TC_STAGES64 8
#endif
    // The ring is bound by its round trip (commit -> empty -> TMA issue -> data -> full), about 2000
    // cycles, divided by its depth: a 64-wide tile, whose launches have at most one CTA per SM anyway,
    // takes the whole shared memory (8 x 24 KB); 128-wide tiles keep 3 x 32 KB so that two CTAs share an SM
    static constexpr int STAGES = (BN == 128) ? 3 : (BN == 64 ? NNCU_TC_STAGES64 : 4);
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int BIAS_OFFSET = BAR_OFFSET + 256;      // BN floats of bias for the epilogue
    static constexpr int TOTAL = BIAS_OFFSET + BN * 4 + 1024; // + alignment slack
    static constexpr int CTAS_PER_SM = (2 * TOTAL <= 227 * 1024) ? 2 : 1;
};

template <int BN, typename TC, bool AMN, bool BMN>
__global__ void __launch_bounds__(256, SmemLayout<BN>::CTAS_PER_SM)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, int staged, TC *C, long ldc, const float *__restrict__ bias, const TC *addsrc, int M, int N,
               int K, int *err_flag, int bias_n)
{
    using SL = SmemLayout<BN>;
    extern __shared__ unsigned char smraw_[];
    // 1024-byte alignment for the 128-byte swizzle atoms
    unsigned char *sm = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smraw_) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + SL::BAR_OFFSET);
    uint64_t *full = bars, *empty = bars + SL::STAGES, *tmem_full = bars + 2 * SL::STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * SL::STAGES + 1);
    volatile int *abort_s = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *bias_s = reinterpret_cast<float *>(sm + SL::BIAS_OFFSET);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // split-K: gridDim.z CTAs share an output tile, each taking a contiguous run of k-blocks and
    // writing its partial product to rows [z*M, (z+1)*M) of C (a workspace of gridDim.z * M rows;
    // the host adds the partials in z order).  gridDim.z = 1 is the plain GEMM.
    const int nkb_all = (K + BK - 1) / BK;
    const int kper = (nkb_all + (int)gridDim.z - 1) / (int)gridDim.z;
    const int kb_first = (int)blockIdx.z * kper;
    const int nkb = max(0, min(nkb_all, kb_first + kper) - kb_first);
    const int mz = (int)blockIdx.z * M;
    TC_MODE_LOAD
    pdl_trigger();

    if (threadIdx.x == 0) {
        TC_STAMP(0);
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
        for (int s = 0; s < SL::STAGES; s++) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(tmem_full), (SL::STAGES % 2) == 0 ? 2 : 1); // one commit from each issuing thread
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1)
        tmem_alloc(smem_u32(tmem_slot), 2 * BN);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    // everything above (barriers, tensor-map prefetch, TMEM allocation) may overlap the tail of the
    // kernel before this one on the stream; from here on its results are read
    pdl_wait();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0)
        TC_STAMP(1);

    // The producer and the MMA issuer are single threads, and what bounds their loops is their
    // own instruction count (one dependent instruction every 4-6 cycles): a k-block used to cost
    // the issuer 350-600 cycles whatever the tile width, four times the tensor time of a
    // 128 x 64 tile.  So both loops carry their state incrementally (barrier addresses and the
    // low descriptor words step by constants, the phase bit flips at the ring's wrap), the four
    // UMMAs of a k-block are one asm block, and a wait is a try_wait with a branch.
    // Two loading and two issuing threads when the ring has an even number of stages: each pair then
    // owns its own stages (even / odd k-blocks).  With an odd ring the pairs would share stages, and
    // a thread two rounds ahead of its partner would mistake the parity of a barrier that has not
    // completed once for a completion: there one thread loads and one issues, as before.
    constexpr bool DUAL = (SL::STAGES % 2) == 0;
    constexpr int KSTEP = DUAL ? 2 : 1;
    if (warp == 0 || (DUAL && warp == 7)) {
        if (lane == 0) {
            // warp 0 fills the stages of the even k-blocks, warp 7 those of the odd ones (a k-block
            // costs its loading thread some 360 cycles of barrier handshake and TMA issue)
            const int which = warp == 0 ? 0 : 1;
            const uint32_t sm0 = smem_u32(sm), full0 = smem_u32(full), empty0 = smem_u32(empty);
            int s = which % SL::STAGES;
            int kx = (kb_first + which) * BK;
            for (int kb = which; kb < nkb; kb += KSTEP, kx += KSTEP * BK) {
                const uint32_t fb = full0 + 8 * s, eb = empty0 + 8 * s, dst = sm0 + s * SL::STAGE_BYTES;
                if (kb >= SL::STAGES && !mbar_wait(eb, (uint32_t)(((kb / SL::STAGES) - 1) & 1), abort_s, err_flag, 1))
                    break;
                if (kb == 0)
                    TC_STAMP(2);
                if (TC_MODE(1)) {
                    mbar_expect_tx(fb, 0);
                } else {
                    mbar_expect_tx(fb, SL::STAGE_BYTES);
                    if (AMN) {
#pragma unroll
                        for (int mb = 0; mb < BM / 64; mb++)
                            tma_load_2d(dst + mb * 8192, &map_a, fb, m0 + mb * 64, kx);
                    } else {
                        tma_load_2d(dst, &map_a, fb, kx, m0);
                    }
                    if (BMN) {
#pragma unroll
                        for (int nb = 0; nb < BN / 64; nb++)
                            tma_load_2d(dst + SL::A_BYTES + nb * 8192, &map_b, fb, n0 + nb * 64, kx);
                    } else {
                        tma_load_2d(dst + SL::A_BYTES, &map_b, fb, kx, n0);
                    }
                }
                s += KSTEP;
                if (s >= SL::STAGES)
                    s -= SL::STAGES;
            }
        }
    } else if (warp == 1 || (DUAL && warp == 6)) {
        if (lane == 0) {
            // Two issuing threads (even ring): warp 1 takes the even k-blocks into the accumulator at
            // TMEM column 0, warp 6 the odd ones into the accumulator at column BN (with an odd ring
            // warp 1 issues both, alternating); the epilogue adds the two.  A
            // k-block costs its issuing thread some 470 cycles (barrier handshake plus four UMMAs of
            // 57 cycles of issue each) whatever the tile width, more than the tensor pipe needs below
            // 256 columns, and the two threads' streams run side by side.  The association, (sum of
            // the even k-blocks) + (sum of the odd ones), each in k order, is the same for every tile
            // width and launch, so a row's bits still do not depend on what is computed with it.
            const int which = warp == 1 ? 0 : 1;
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((AMN ? 1u : 0u) << 15) |
                                       ((BMN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(BM >> 4) << 24);
            const uint32_t sm0 = smem_u32(sm), full0 = smem_u32(full), empty0 = smem_u32(empty);
            // low descriptor words of stage 0 (address and leading offset); the high word is the
            // same constant for both layouts (stride offset 1024, sm_100 version, 128-byte swizzle)
            const uint32_t alo0 = (uint32_t)(AMN ? smem_desc_sw128_mn(sm0) : smem_desc_sw128(sm0));
            const uint32_t blo0 = (uint32_t)(BMN ? smem_desc_sw128_mn(sm0 + SL::A_BYTES)
                                                 : smem_desc_sw128(sm0 + SL::A_BYTES));
            // one UMMA covers 16 along k: 32 bytes inside a K-major row (+2 in 16-byte units),
            // 16 rows of 128 bytes in an MN-major tile (+128)
            constexpr uint32_t astep = AMN ? 128u : 2u, bstep = BMN ? 128u : 2u;
            int s = which % SL::STAGES;
            uint32_t ph = (uint32_t)((which / SL::STAGES) & 1);
            bool ok = true;
            for (int kb = which; kb < nkb; kb += KSTEP) {
                // even k-blocks into the accumulator at column 0, odd ones into the one at column BN;
                // the first k-block of each overwrites
                const uint32_t tacc = tmem_base + (uint32_t)((kb & 1) * BN), acc = kb >= 2 ? 1u : 0u;
                ok = mbar_wait(full0 + 8 * s, ph, abort_s, err_flag, 2);
                if (!ok)
                    break;
                if (kb == 0)
                    TC_STAMP(3);
                fence_after_sync();
                if (!TC_MODE(2))
                    umma_bf16_x4<astep, bstep>(tacc, alo0 + s * (SL::STAGE_BYTES >> 4), blo0 + s * (SL::STAGE_BYTES >> 4), idesc,
                                               acc);
                umma_commit(empty0 + 8 * s); // frees the stage when these MMAs retire
                s += KSTEP;
                if (s >= SL::STAGES) {
                    s -= SL::STAGES;
                    ph ^= 1;
                }
            }
            if (which == 0)
                TC_STAMP(4);
            if (ok)
                umma_commit(smem_u32(tmem_full));
        }
    }
    if (warp >= 2 && warp < 6) {
        // epilogue warps 2..5
        const int quarter = warp & 3;
        bool ok = true;
        if (bias) {
            // the tile's bias values go to shared memory while the mainloop runs (a load from
            // global memory inside the chunk loop would expose its latency once per chunk)
            const int lim = min(N, bias_n) - n0;
            for (int i = threadIdx.x - 64; i < BN; i += 128)
                bias_s[i] = i < lim ? __ldg(bias + n0 + i) : 0.0f;
            asm volatile("bar.sync 1, 128;" ::: "memory"); // the four epilogue warps only
        }
        if (nkb > 0)
        {
            // one lane per warp watches the barrier: every probe of a waiting thread queues in
            // front of the producer's and the MMA thread's own barrier operations
            if (lane == 0 || TC_MODE(4))
                ok = mbar_wait(smem_u32(tmem_full), 0, abort_s, err_flag, 3);
            __syncwarp();
        }
        ok = __all_sync(0xffffffffu, ok); // tcgen05.ld below is warp-collective
        if (threadIdx.x == 64) {
            TC_STAMP(5);
            pdl_trigger_late(); // the mainloop is over: the next kernel may set itself up
        }
        fence_after_sync();
        const int row = m0 + quarter * 32 + lane;
        if (ok) {
            // Each thread holds one output row, so storing straight from registers would touch 32
            // different lines per instruction.  The warp parks 32 rows x 128 bytes in shared
            // memory (the operand ring is idle by now; 128-byte swizzle) and a TMA store, which
            // also clips the ragged edges, takes them out; two buffers per warp.  (Reading the
            // block back for row-wise global stores measured slower than the TMA store.)
            constexpr int CPB = (sizeof(TC) == 2) ? 2 : 1; // 32-column chunks per 128-byte block
            constexpr int NCH = BN / 32;
            unsigned char *stage0 = sm + quarter * 8192;
            const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16);
            // chunks still inside the matrix (uniform over the CTA)
            const int nch = min(NCH, (N - n0 + 31) / 32);
            // Each chunk is the sum of the two issuing threads' accumulators (the second one only
            // exists from two k-blocks on).  The loop is kept rolled: unrolled over the tile it would
            // run once through code larger than the instruction cache.
            const bool dual = nkb > 1;
            uint32_t ra[32];
            auto chunk = [&](int ch, const uint32_t(&r)[32]) {
                const int c0 = ch * 32, cc = ch % CPB, blk = ch / CPB;
                unsigned char *stg = stage0 + (blk & 1) * 4096;
                if (staged && cc == 0) {
                    if (lane == 0) // the store issued two blocks ago has finished reading this buffer
                        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    __syncwarp();
                }
                const int nvalid = N - (n0 + c0); // > 0 here, may exceed 32
                const bool full = nvalid >= 32;
                float x[32];
#pragma unroll
                for (int j = 0; j < 32; j++)
                    x[j] = __uint_as_float(r[j]);
                // Straight-line vector paths for whole chunks; element-wise code (one branch per
                // element) only at ragged edges.
                if (bias) {
                    const float4 *bp = reinterpret_cast<const float4 *>(bias_s + c0); // zero past N or bias_n
#pragma unroll
                    for (int v = 0; v < 8; v++) {
                        const float4 t = bp[v];
                        x[v * 4] += t.x; x[v * 4 + 1] += t.y; x[v * 4 + 2] += t.z; x[v * 4 + 3] += t.w;
                    }
                }
                if (addsrc && row < M) {
                    const TC *add = addsrc + (long)row * ldc + n0 + c0;
                    if (full && (reinterpret_cast<uintptr_t>(add) & 15) == 0) {
                        if (sizeof(TC) == 2) {
#pragma unroll
                            for (int v = 0; v < 4; v++) {
                                const uint4 t = reinterpret_cast<const uint4 *>(add)[v];
                                const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                                for (int u = 0; u < 4; u++) {
                                    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162 *>(&w[u]);
                                    x[v * 8 + u * 2] += __low2float(h);
                                    x[v * 8 + u * 2 + 1] += __high2float(h);
                                }
                            }
                        } else {
#pragma unroll
                            for (int v = 0; v < 8; v++) {
                                const float4 t = reinterpret_cast<const float4 *>(add)[v];
                                x[v * 4] += t.x; x[v * 4 + 1] += t.y; x[v * 4 + 2] += t.z; x[v * 4 + 3] += t.w;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j < nvalid)
                                x[j] += to_f(add[j]);
                    }
                }
                if (staged) {
                    unsigned char *rowp = stg + lane * 128;
                    if (sizeof(TC) == 2) {
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            uint4 pk;
                            pk.x = pack_bf16(x[v * 8 + 0], x[v * 8 + 1]);
                            pk.y = pack_bf16(x[v * 8 + 2], x[v * 8 + 3]);
                            pk.z = pack_bf16(x[v * 8 + 4], x[v * 8 + 5]);
                            pk.w = pack_bf16(x[v * 8 + 6], x[v * 8 + 7]);
                            *reinterpret_cast<uint4 *>(rowp + (((cc * 4 + v) ^ (lane & 7)) << 4)) = pk;
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < 8; v++)
                            *reinterpret_cast<float4 *>(rowp + ((v ^ (lane & 7)) << 4)) =
                                make_float4(x[v * 4], x[v * 4 + 1], x[v * 4 + 2], x[v * 4 + 3]);
                    }
                    if (cc == CPB - 1 || ch == nch - 1) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            asm volatile(
                                "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                    reinterpret_cast<uint64_t>(&map_c)),
                                "r"(smem_u32(stg)), "r"(n0 + blk * 32 * CPB), "r"(mz + m0 + quarter * 32)
                                : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    }
                } else if (row < M) {
                    TC *dst = C + (long)(mz + row) * ldc + n0 + c0;
                    if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                        if (sizeof(TC) == 2) {
#pragma unroll
                            for (int v = 0; v < 4; v++)
                                reinterpret_cast<uint4 *>(dst)[v] =
                                    make_uint4(pack_bf16(x[v * 8], x[v * 8 + 1]), pack_bf16(x[v * 8 + 2], x[v * 8 + 3]),
                                               pack_bf16(x[v * 8 + 4], x[v * 8 + 5]), pack_bf16(x[v * 8 + 6], x[v * 8 + 7]));
                        } else {
#pragma unroll
                            for (int v = 0; v < 8; v++)
                                reinterpret_cast<float4 *>(dst)[v] =
                                    make_float4(x[v * 4], x[v * 4 + 1], x[v * 4 + 2], x[v * 4 + 3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j < nvalid)
                                dst[j] = from_f<TC>(x[j]);
                    }
                }
            };
#pragma unroll 1
            for (int ch = 0; ch < nch; ch++) {
                if (nkb > 0) {
                    tmem_ld32_pair(trow + (uint32_t)(ch * 32), (uint32_t)BN, dual, ra);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        ra[j] = 0u;
                }
                chunk(ch, ra);
            }
            if (threadIdx.x == 64)
                TC_STAMP(14);
            if (staged && lane == 0)
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
        }
    }
    if (threadIdx.x == 64)
        TC_STAMP(6);
    // common exit: nobody touches TMEM after this barrier
    fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0)
        TC_STAMP(7);
    if (*abort_s) {
        // a wait gave up: let copies that are still in flight land before the CTA retires
        for (int i = 0; i < 2000; i++)
            __nanosleep(500);
    }
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}

// ---------------- host side ----------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// tensor maps are pure functions of (pointer, extents, stride, box): cache them
struct TmapKey {
    const void *ptr;
    long rows, cols, ld;
    int box_rows, box_cols, elt;
    bool operator<(const TmapKey &o) const
    {
        return std::tie(ptr, rows, cols, ld, box_rows, box_cols, elt) <
               std::tie(o.ptr, o.rows, o.cols, o.ld, o.box_rows, o.box_cols, o.elt);
    }
};

// 2-D map over a row-major [rows][cols] matrix of 2-byte (bf16) or 4-byte (fp32) elements,
// boxes of box_rows x box_cols with box_cols * elt == 128 bytes, 128-byte swizzle
static int make_tmap(const void *ptr, long rows, long cols, long ld, int box_rows, CUtensorMap *out,
                     int box_cols = BK, int elt = 2)
{
    static std::map<TmapKey, CUtensorMap> cache;
    static std::mutex mu;
    TmapKey key{ptr, rows, cols, ld, box_rows, box_cols, elt};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return NNCU_OK;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn)
        return nncu_fail(NNCU_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elt};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, elt == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                    const_cast<void *>(ptr), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return nncu_fail(NNCU_ERR_CUDA, "cuTensorMapEncodeTiled failed: %d (rows %ld cols %ld ld %ld)",
                         (int)r, rows, cols, ld);
    if (cache.size() > 4096)
        cache.clear();
    cache[key] = *out;
    return NNCU_OK;
}

static bool usable(const void *A, long lda, const void *B, long ldb, int K)
{
    return K > 0 && (lda % 8) == 0 && (ldb % 8) == 0 &&
           (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0;
}

template <int BN, typename TC, bool AMN, bool BMN>
static int launch(cudaStream_t st, int M, int N, int K, const bf16 *A, long lda, const bf16 *B,
                  long ldb, TC *C, long ldc, const float *bias, const TC *addsrc, int *err_flag, int bias_n,
                  int ksplit = 1)
{
    using SL = SmemLayout<BN>;
    if (ksplit > 1 && (M % BM != 0 || bias || addsrc))
        return nncu_fail(NNCU_ERR_INVALID, "split-K needs whole row tiles and a bare product");
    CUtensorMap ma, mb;
    if (AMN)
        NNCU_TRY(make_tmap(A, K, M, lda, 64, &ma)); // [k rows][m], 64 x 64 boxes
    else
        NNCU_TRY(make_tmap(A, M, K, lda, BM, &ma));
    if (BMN)
        NNCU_TRY(make_tmap(B, K, N, ldb, 64, &mb));
    else
        NNCU_TRY(make_tmap(B, N, K, ldb, BN, &mb));
    // rows of C that are 16-byte aligned leave through shared memory and TMA stores
    CUtensorMap mc = ma;
    const int staged = ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * sizeof(TC)) % 16 == 0) ? 1 : 0;
    if (staged)
        NNCU_TRY(make_tmap(C, (long)M * ksplit, N, ldc, 32, &mc, 128 / (int)sizeof(TC), (int)sizeof(TC)));
    static bool attr_done = false;
    if (!attr_done) {
        CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<BN, TC, AMN, BMN>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, SL::TOTAL));
        attr_done = true;
    }
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM), ksplit);
    GemmProfiler *pr = g_nncu_prof;
    const bool timed = pr && pr->n < GemmProfiler::MAX_EV;
    if (timed)
        cudaEventRecord(pr->ev[2 * pr->n], st);
    launch_k(gemm_tc_kernel<BN, TC, AMN, BMN>, dim3(grid), dim3(256), SL::TOTAL, st, ma, mb, mc, staged, C, ldc, bias, addsrc,
             M, N, K, err_flag, bias_n);
    if (timed) {
        cudaEventRecord(pr->ev[2 * pr->n + 1], st);
        pr->flops[pr->n++] = 2.0 * M * N * K;
    }
    KERNEL_CHECK();
    return NNCU_OK;
}

// A: [M][K] (lda) or, AMN, [K][M]; B: [N][K] (ldb) or, BMN, [K][N].  C bf16 or fp32; addsrc
// (may be NULL, may alias C) is added to the product.  err_flag: device int raised when a
// bounded wait expires.
template <typename TC, bool AMN, bool BMN>
static int gemm(cudaStream_t st, int M, int N, int K, const bf16 *A, long lda, const bf16 *B,
                long ldb, TC *C, long ldc, const float *bias, const TC *addsrc, int *err_flag,
                int bias_n = 1 << 30)
{
    if (M <= 0 || N <= 0)
        return NNCU_OK;
    if (!usable(A, lda, B, ldb, K))
        return nncu_fail(NNCU_ERR_INVALID, "tcgen05 GEMM needs 16-byte aligned operands and strides");
    // A k-block costs the issuing thread about the same whatever the tile width, so wide tiles use
    // the tensor pipe best; but a 256-wide tile fills the shared memory of an SM, while two
    // narrower CTAs share one and the epilogue of one overlaps the mainloop of the other.  Measured
    // on the c2 train step: thresholds 96 .. 200 are within 1 %, 200 best, 64 and 400 3 % worse.
    const long mt = ceil_div(M, BM);
    static int min_tiles = 0;
    if (!min_tiles) {
        const char *e = getenv("NNCU_TC_MIN_TILES"); // tuning knob
        min_tiles = e ? atoi(e) : 200;
        if (min_tiles < 1)
            min_tiles = 200;
    }
    // fp32 output doubles the epilogue's bytes per tile: two 128-wide CTAs per SM, one's epilogue under
    // the other's mainloop, beat one 256-wide CTA (output head, 2048 x 16384 x 512, cold: 80.7 against 91.2 us)
    static int f32_wide = -1;
    if (f32_wide < 0) {
        const char *e = getenv("NNCU_TC_F32_256");
        f32_wide = (e && e[0] == '1') ? 1 : 0;
    }
    if (mt * ceil_div(N, 256) >= min_tiles && (sizeof(TC) == 2 || f32_wide))
        return launch<256, TC, AMN, BMN>(st, M, N, K, A, lda, B, ldb, C, ldc, bias, addsrc, err_flag, bias_n);
    if (mt * ceil_div(N, 128) >= min_tiles || N <= 64)
        return launch<128, TC, AMN, BMN>(st, M, N, K, A, lda, B, ldb, C, ldc, bias, addsrc, err_flag, bias_n);
    return launch<64, TC, AMN, BMN>(st, M, N, K, A, lda, B, ldb, C, ldc, bias, addsrc, err_flag, bias_n);
}

// Long contractions with few output tiles (the output head's dX: K = n_symbols): `ksplit` CTAs
// per 128 x 128 tile, fp32 partial products in `ws` ([ksplit][M][N], M a multiple of 128); the
// caller adds the partials in order (splitk_reduce_kernel).
template <bool AMN, bool BMN>
static int gemm_splitk(cudaStream_t st, int M, int N, int K, const bf16 *A, long lda, const bf16 *B, long ldb,
                       float *ws, int ksplit, int *err_flag)
{
    if (!usable(A, lda, B, ldb, K))
        return nncu_fail(NNCU_ERR_INVALID, "tcgen05 GEMM needs 16-byte aligned operands and strides");
    return launch<128, float, AMN, BMN>(st, M, N, K, A, lda, B, ldb, ws, N, nullptr, nullptr, err_flag, 1 << 30,
                                        ksplit);
}

template <typename TC>
static int gemm_nt(cudaStream_t st, int M, int N, int K, const bf16 *A, long lda, const bf16 *B,
                   long ldb, TC *C, long ldc, const float *bias, const TC *addsrc, int *err_flag,
                   int bias_n = 1 << 30)
{
    return gemm<TC, false, false>(st, M, N, K, A, lda, B, ldb, C, ldc, bias, addsrc, err_flag, bias_n);
}

} // namespace tc
