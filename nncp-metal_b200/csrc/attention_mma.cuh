// attention_mma.cuh -- bf16 relative-position attention on the warp-level tensor path
// (mma.sync m16n8k16, fp32 accumulate), forward and backward, one CTA per (stream, head).
//
// Same math as attention.cuh (nncp.c:722-800 and its adjoint).  Per (stream, head) the
// contractions are 64 x 128 x 64: too small for a 128-row tcgen05 tile to pay, and the
// relative shift needs a per-row skew of the position scores that a register-fragment
// kernel can do through a few KB of shared memory.  Each warp owns 16 query rows:
//
//   S  = Q K^T                 (16 x 64 per key block)
//   E  = Q R^T                 (16 x 80 window of the position table for that block)
//   s  = (S + skew(E) + b_r) / sqrt(dk), masked, online softmax over key blocks of 64
//   O += P V
//
// Tile origins are multiples of 16 queries / 64 keys counted from 0 whatever range of
// queries is requested, so query row i goes through the same sequence of instructions
// and gives the same bits in a one-symbol step as in a whole-segment launch.
//
// Keys are walked in super-blocks of 128 (two key blocks): K, V and the window of the position
// table that the super-block can touch are staged per super-block, so shared memory does not
// grow with the memory length.
//
// Backward, per super-block: P and dS (bf16) of the 64 x 128 tile and the inverse-skewed dE
// window go to shared memory, then dV = P^T dO and dK = dS^T Q (complete for these keys, all
// queries being in the CTA) are written out, dQ += dS K + dE R stays in registers, and the
// table gradients dR += dE^T Q, db_r are accumulated into this (stream, head)'s slice of the
// caller's partial buffers by plain read-add-write (one CTA owns the slice; super-blocks run
// in order).  All sums have a fixed order; the caller reduces the partials over streams.
#pragma once
#include "attention.cuh"
#include "attention_tc.cuh"

namespace amma {

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const bf16 *p)
{
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const bf16 *p)
{
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

#ifdef NNCU_ATTN_TRACE
// tuning aid (off in normal builds): clock64() stamps of the backward kernel's phases
__device__ long long *g_attn_trace = nullptr;
#define AT_STAMP(slot)                                                        \
    do {                                                                      \
        if (at_trace_ && threadIdx.x == 0 && blockIdx.x < 64)                 \
            at_trace_[blockIdx.x * 16 + (slot)] = clock64();                  \
    } while (0)
#define AT_TRACE_LOAD long long *const at_trace_ = g_attn_trace;
#else
#define AT_STAMP(slot) \
    do {               \
    } while (0)
#define AT_TRACE_LOAD
#endif

constexpr int EW = 88; // fp32 row stride of the per-warp skew scratch (80 columns used)

// shared-memory geometry; identical on host and device
struct Dims {
    int SBK;  // keys per super-block: 64 or 128
    int WR;   // rows of the staged position-table window
    int LDS;  // bf16 row stride of Q, K, V, R, dO tiles
    int LPS;  // bf16 row stride of the P / dS tiles
    int PPS;  // bf16 row stride of the dE window
};
__host__ __device__ inline Dims dims_of(int L, int P, int dk)
{
    Dims d;
    d.SBK = (L <= 64 || dk > 64) ? 64 : 128; // wide heads: smaller key tiles keep the backward in shared memory
    const int whole = (P + 1 + 15) / 16 * 16;   // the table and at least one zero row
    const int window = d.SBK + 64 + 16;         // reach of 64 query rows over SBK keys, plus slack
    d.WR = whole < window ? whole : window;
    d.LDS = dk + 8;
    d.LPS = d.SBK + 8;
    d.PPS = d.WR + 8;
    return d;
}
// first table row a super-block starting at key j0 can touch, for query rows up to q_last
__device__ __forceinline__ int window_base(const AttnArgs &a, int j0, int q_last)
{
    const int w = j0 + (a.T - 1) - q_last - (a.L - a.P);
    return w > 0 ? w : 0;
}

// rows [0, nrows) of a [.. x dk] bf16 matrix with row pitch `pitch` elements -> shared tile;
// rows that fail `valid` are zero.  16-byte chunks.
template <typename F>
__device__ __forceinline__ void load_tile(bf16 *dst, int lds, const bf16 *src, size_t pitch, int nrows,
                                          int dk, F valid)
{
    // asynchronous 16-byte copies (no register staging, so a thread's copies are all in flight
    // together); complete at the next tiles_ready()
    const int cpr = dk / 8;
    for (int idx = threadIdx.x; idx < nrows * cpr; idx += blockDim.x) {
        int r = idx / cpr, c = (idx % cpr) * 8;
        bf16 *d = dst + (size_t)r * lds + c;
        if (valid(r)) {
            const uint32_t da = (uint32_t)__cvta_generic_to_shared(d);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(da), "l"(src + (size_t)r * pitch + c) : "memory");
        } else {
            *reinterpret_cast<uint4 *>(d) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
}
// every load_tile copy of this thread has landed (call before the barrier that publishes the tiles)
__device__ __forceinline__ void tiles_ready()
{
    asm volatile("cp.async.wait_all;" ::: "memory");
}

// rows [wbase, wbase + WR) of one head's position table -> shared; rows >= P are zero.  From the
// bf16 copy (16-byte chunks) when there is one, else converted from fp32.
__device__ __forceinline__ void load_table(bf16 *dst, int lds, const float *w_r_h, const bf16 *w16_h, int P,
                                           int wbase, int WR, int dk)
{
    if (w16_h) {
        load_tile(dst, lds, w16_h + (size_t)wbase * dk, (size_t)dk, WR, dk, [&](int r) { return wbase + r < P; });
        return;
    }
    for (int idx = threadIdx.x; idx < WR * dk; idx += blockDim.x) {
        int p = idx / dk, e = idx % dk;
        dst[(size_t)p * lds + e] = (w_r_h && wbase + p < P) ? __float2bfloat16_rn(w_r_h[(size_t)(wbase + p) * dk + e])
                                                             : __float2bfloat16_rn(0.0f);
    }
}

// scores of one 16-query x 64-key block: s[nt][c], already scaled and masked (-inf).
// qf: Q fragments of the warp's 16 rows.  Ks: staged keys of the super-block starting at key
// j0s; Rs: staged table rows starting at row wbase.  es: the warp's skew scratch.
template <int DK>
__device__ __forceinline__ void score_block(const AttnArgs &a, const Dims &d, const uint32_t (&qf)[DK / 16][4],
                                            const bf16 *Ks, const bf16 *Rs, const float *brs, float *es,
                                            int i0, int j0, int j0s, int wbase, int iA, int iB, int jloA,
                                            int jhiA, int jloB, int jhiB, float (&s)[8][4])
{
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    constexpr int KS = DK / 16;
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++)
            s[nt][c] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
#pragma unroll
        for (int np = 0; np < 4; np++) {
            uint32_t b[4];
            ldsm4(b, Ks + (size_t)(j0 - j0s + np * 16 + (lane & 7) + (lane >> 4) * 8) * d.LDS + ks * 16 + ((lane >> 3) & 1) * 8);
            mma16816(s[2 * np], qf[ks], b[0], b[1]);
            mma16816(s[2 * np + 1], qf[ks], b[2], b[3]);
        }
    int pbase = 0;
    if (a.w_r) {
        const int pmin = j0 + (a.T - 1) - (i0 + 15) - (a.L - a.P);
        pbase = pmin > 0 ? pmin : 0;
        float e[10][4];
#pragma unroll
        for (int nt = 0; nt < 10; nt++)
#pragma unroll
            for (int c = 0; c < 4; c++)
                e[nt][c] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++)
#pragma unroll
            for (int np = 0; np < 5; np++) {
                int row = pbase - wbase + np * 16 + (lane & 7) + (lane >> 4) * 8;
                row = row < d.WR - 1 ? row : d.WR - 1; // past the rows this block can use
                uint32_t b[4];
                ldsm4(b, Rs + (size_t)row * d.LDS + ks * 16 + ((lane >> 3) & 1) * 8);
                mma16816(e[2 * np], qf[ks], b[0], b[1]);
                mma16816(e[2 * np + 1], qf[ks], b[2], b[3]);
            }
        __syncwarp();
#pragma unroll
        for (int nt = 0; nt < 10; nt++) {
            es[g * EW + nt * 8 + 2 * t] = e[nt][0];
            es[g * EW + nt * 8 + 2 * t + 1] = e[nt][1];
            es[(g + 8) * EW + nt * 8 + 2 * t] = e[nt][2];
            es[(g + 8) * EW + nt * 8 + 2 * t + 1] = e[nt][3];
        }
        __syncwarp();
    }
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int j = j0 + nt * 8 + 2 * t + (c & 1);
            const bool hi = c >= 2;
            const int i = hi ? iB : iA;
            const bool vis = hi ? (j >= jloB && j <= jhiB) : (j >= jloA && j <= jhiA);
            float v = -INFINITY;
            if (vis) {
                const int r = j + (a.T - 1) - i;
                float z = brs[r];
                if (a.w_r) {
                    int pi = r - (a.L - a.P);
                    pi = pi < 0 ? 0 : pi;
                    z += es[(g + (hi ? 8 : 0)) * EW + pi - pbase];
                }
                v = (s[nt][c] + z) * a.inv_sqrt;
            }
            s[nt][c] = v;
        }
}

template <int DK>
size_t fwd_smem(int L, int P)
{
    Dims d = dims_of(L, P, DK);
    return ((size_t)64 * d.LDS + (size_t)2 * d.SBK * d.LDS + (size_t)d.WR * d.LDS) * sizeof(bf16) +
           ((size_t)L + 4 + 4 * 16 * EW) * sizeof(float) + 64;
}

template <int DK>
__global__ void __launch_bounds__(128) attn_fwd_mma_kernel(AttnArgs a)
{
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smraw[];
    const Dims d = dims_of(a.L, a.P, DK);
    bf16 *Qs = reinterpret_cast<bf16 *>(smraw);
    bf16 *Ks = Qs + (size_t)64 * d.LDS;
    bf16 *Vs = Ks + (size_t)d.SBK * d.LDS;
    bf16 *Rs = Vs + (size_t)d.SBK * d.LDS;
    float *brs = reinterpret_cast<float *>(Rs + (size_t)d.WR * d.LDS);
    float *Es = brs + ((a.L + 3) & ~3);
    constexpr int KS = DK / 16, NT = DK / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int HD = a.H * DK;
    const int qt0 = (a.t0 / 16) * 16 + blockIdx.y * 64; // first query row of this CTA's tiles

    const bf16 *q = reinterpret_cast<const bf16 *>(a.q);
    const bf16 *kv = reinterpret_cast<const bf16 *>(a.kv);
    load_tile(Qs, d.LDS, q + ((size_t)qt0 * a.B + b) * a.qp + h * DK, (size_t)a.B * a.qp, 64, DK,
              [&](int r) { return qt0 + r >= a.t0 && qt0 + r < a.t1; });
    for (int r = threadIdx.x; r < a.L; r += blockDim.x)
        brs[r] = a.br_scale * a.b_r[(size_t)h * a.L + r];
    tiles_ready();
    __syncthreads();

    // this warp's 16 query rows
    const int i0 = qt0 + warp * 16;
    const int va = max(i0, a.t0), vb = min(i0 + 16, a.t1) - 1;
    const bool active = va <= vb;
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
        ldsm4(qf[ks], Qs + (size_t)(warp * 16 + (lane & 15)) * d.LDS + ks * 16 + (lane >> 4) * 8);
    const int iA = i0 + g, iB = i0 + g + 8;
    int jloA = 0, jhiA = -1, jloB = 0, jhiB = -1;
    if (iA >= a.t0 && iA < a.t1)
        key_range(a, iA, jloA, jhiA);
    if (iB >= a.t0 && iB < a.t1)
        key_range(a, iB, jloB, jhiB);
    int jmin = 0, jmax = -1, tmp;
    if (active) {
        key_range(a, va, jmin, tmp);
        key_range(a, vb, tmp, jmax);
    }
    // key range of the whole CTA (its valid query rows are contiguous)
    const int ca = max(qt0, a.t0), cb = min(qt0 + 64, a.t1) - 1;
    int cmin, cmax;
    key_range(a, ca, cmin, tmp);
    key_range(a, cb, tmp, cmax);
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++)
            o[nt][c] = 0.0f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;
    float *es = Es + (size_t)warp * 16 * EW;

    for (int sb = cmin / d.SBK; sb <= cmax / d.SBK; sb++) {
        const int j0s = sb * d.SBK;
        const int wbase = window_base(a, j0s, qt0 + 63);
        __syncthreads(); // everyone is done with the previous super-block's tiles
        load_tile(Ks, d.LDS, kv + ((size_t)j0s * a.B + b) * a.kvp + h * DK, (size_t)a.B * a.kvp, d.SBK, DK,
                  [&](int r) { return j0s + r < a.L; });
        load_tile(Vs, d.LDS, kv + ((size_t)j0s * a.B + b) * a.kvp + HD + h * DK, (size_t)a.B * a.kvp, d.SBK, DK,
                  [&](int r) { return j0s + r < a.L; });
        load_table(Rs, d.LDS, a.w_r ? a.w_r + (size_t)h * a.P * DK : nullptr,
                   a.w_r16 ? reinterpret_cast<const bf16 *>(a.w_r16) + (size_t)h * a.P * DK : nullptr, a.P, wbase,
                   d.WR, DK);
        tiles_ready();
        __syncthreads();
        if (!active)
            continue;
        for (int kb = max(jmin / 64, j0s / 64); kb <= min(jmax / 64, (j0s + d.SBK - 1) / 64); kb++) {
            const int j0 = kb * 64;
            float s[8][4];
            score_block<DK>(a, d, qf, Ks, Rs, brs, es, i0, j0, j0s, wbase, iA, iB, jloA, jhiA, jloB, jhiB, s);
            float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                mxA = fmaxf(mxA, fmaxf(s[nt][0], s[nt][1]));
                mxB = fmaxf(mxB, fmaxf(s[nt][2], s[nt][3]));
            }
            mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
            mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
            mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
            mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
            const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
            const float uA = nA == -INFINITY ? 0.0f : nA, uB = nB == -INFINITY ? 0.0f : nB;
            const float scA = __expf(mA - uA), scB = __expf(mB - uB);
            mA = nA;
            mB = nB;
            float sumA = 0.0f, sumB = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                s[nt][0] = __expf(s[nt][0] - uA);
                s[nt][1] = __expf(s[nt][1] - uA);
                s[nt][2] = __expf(s[nt][2] - uB);
                s[nt][3] = __expf(s[nt][3] - uB);
                sumA += s[nt][0] + s[nt][1];
                sumB += s[nt][2] + s[nt][3];
            }
            lA = lA * scA + sumA;
            lB = lB * scB + sumB;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                o[nt][0] *= scA;
                o[nt][1] *= scA;
                o[nt][2] *= scB;
                o[nt][3] *= scB;
            }
#pragma unroll
            for (int k2 = 0; k2 < 4; k2++) {
                uint32_t pa[4];
                pa[0] = pack2(s[2 * k2][0], s[2 * k2][1]);
                pa[1] = pack2(s[2 * k2][2], s[2 * k2][3]);
                pa[2] = pack2(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
                pa[3] = pack2(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
#pragma unroll
                for (int np = 0; np < NT / 2; np++) {
                    uint32_t bb[4];
                    ldsm4t(bb, Vs + (size_t)(j0 - j0s + k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * d.LDS + np * 16 + (lane >> 4) * 8);
                    mma16816(o[2 * np], pa, bb[0], bb[1]);
                    mma16816(o[2 * np + 1], pa, bb[2], bb[3]);
                }
            }
            __syncwarp();
        }
    }
    if (!active)
        return;
    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    bf16 *out = reinterpret_cast<bf16 *>(a.o);
    if (iA >= a.t0 && iA < a.t1) {
        const float inv = 1.0f / lA;
        bf16 *dst = out + ((size_t)iA * a.B + b) * HD + h * DK;
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
            *reinterpret_cast<uint32_t *>(dst + nt * 8 + 2 * t) = pack2(o[nt][0] * inv, o[nt][1] * inv);
        if (t == 0 && a.lse)
            a.lse[((size_t)b * a.H + h) * a.T + iA] = mA + logf(lA);
    }
    if (iB >= a.t0 && iB < a.t1) {
        const float inv = 1.0f / lB;
        bf16 *dst = out + ((size_t)iB * a.B + b) * HD + h * DK;
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
            *reinterpret_cast<uint32_t *>(dst + nt * 8 + 2 * t) = pack2(o[nt][2] * inv, o[nt][3] * inv);
        if (t == 0 && a.lse)
            a.lse[((size_t)b * a.H + h) * a.T + iB] = mB + logf(lB);
    }
}

template <int DK>
size_t bwd_smem(int L, int P)
{
    Dims d = dims_of(L, P, DK);
    return ((size_t)2 * 64 * d.LDS + (size_t)2 * d.SBK * d.LDS + (size_t)d.WR * d.LDS + (size_t)2 * 64 * d.LPS +
            (size_t)64 * d.PPS) * sizeof(bf16) +
           ((size_t)L + 4 + 8 * 16 * EW + 128) * sizeof(float) + 64;
}

// 8 warps: warp w owns query tile (w & 3).  Phase A of a super-block: the two warps of a tile
// take one key block each.  Phase B: the row tiles of dV / dK / dR are dealt round-robin over
// the warps; dQ is split into its key part (warps 0-3) and position part (warps 4-7), kept in
// registers over the super-blocks and combined at the end.
template <int DK>
__global__ void __launch_bounds__(256) attn_bwd_mma_kernel(AttnArgs a)
{
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smraw[];
    AT_TRACE_LOAD
    AT_STAMP(0);
    const Dims d = dims_of(a.L, a.P, DK);
    bf16 *Qs = reinterpret_cast<bf16 *>(smraw);
    bf16 *dOs = Qs + (size_t)64 * d.LDS;
    bf16 *Ks = dOs + (size_t)64 * d.LDS;
    bf16 *Vs = Ks + (size_t)d.SBK * d.LDS;
    bf16 *Rs = Vs + (size_t)d.SBK * d.LDS;
    bf16 *Pm = Rs + (size_t)d.WR * d.LDS;
    bf16 *dSm = Pm + (size_t)64 * d.LPS;
    bf16 *dEm = dSm + (size_t)64 * d.LPS;
    float *brs = reinterpret_cast<float *>(dEm + (size_t)64 * d.PPS);
    float *Es = brs + ((a.L + 3) & ~3);
    float *Dr = Es + 8 * 16 * EW; // [64]
    float *lses = Dr + 64;        // [64]
    constexpr int KS = DK / 16, NT = DK / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int HD = a.H * DK, T = a.T, L = a.L, P = a.P;

    const bf16 *q = reinterpret_cast<const bf16 *>(a.q);
    const bf16 *kv = reinterpret_cast<const bf16 *>(a.kv);
    const bf16 *dout = reinterpret_cast<const bf16 *>(a.dout);
    const bf16 *outp = reinterpret_cast<const bf16 *>(a.out);
    float *dwr = (a.w_r && a.dwr_part) ? a.dwr_part + ((size_t)b * a.H + h) * P * DK : nullptr;
    float *dbr = a.dbr_part ? a.dbr_part + ((size_t)b * a.H + h) * L : nullptr;
    load_tile(Qs, d.LDS, q + (size_t)b * a.qp + h * DK, (size_t)a.B * a.qp, 64, DK, [&](int r) { return r < T; });
    load_tile(dOs, d.LDS, dout + (size_t)b * HD + h * DK, (size_t)a.B * HD, 64, DK, [&](int r) { return r < T; });
    for (int r = threadIdx.x; r < L; r += blockDim.x)
        brs[r] = a.br_scale * a.b_r[(size_t)h * L + r];
    if (threadIdx.x < 64)
        lses[threadIdx.x] = threadIdx.x < T ? a.lse[((size_t)b * a.H + h) * T + threadIdx.x] : 0.0f;
    // the forward output, parked in the skew scratch (not needed before phase A)
    bf16 *Os = reinterpret_cast<bf16 *>(Es);
    load_tile(Os, d.LDS, outp + (size_t)b * HD + h * DK, (size_t)a.B * HD, 64, DK, [&](int r) { return r < T; });
    // super-blocks with at least one visible (query, key) pair; the first one's keys, values and
    // table window are fetched here, together with the query-side tiles
    int cmin, cmax, tmp;
    key_range(a, 0, cmin, tmp);
    key_range(a, T - 1, tmp, cmax);
    const int sb_first = cmin / d.SBK, sb_last = cmax / d.SBK;
    const bool single = sb_first == sb_last; // table gradients are then stored, not accumulated
    auto load_keys = [&](int sb) {
        const int j0s = sb * d.SBK;
        const int wbase = window_base(a, j0s, 63);
        load_tile(Ks, d.LDS, kv + ((size_t)j0s * a.B + b) * a.kvp + h * DK, (size_t)a.B * a.kvp, d.SBK, DK,
                  [&](int r) { return j0s + r < L; });
        load_tile(Vs, d.LDS, kv + ((size_t)j0s * a.B + b) * a.kvp + HD + h * DK, (size_t)a.B * a.kvp, d.SBK, DK,
                  [&](int r) { return j0s + r < L; });
        load_table(Rs, d.LDS, a.w_r ? a.w_r + (size_t)h * P * DK : nullptr,
                   a.w_r16 ? reinterpret_cast<const bf16 *>(a.w_r16) + (size_t)h * P * DK : nullptr, P, wbase,
                   d.WR, DK);
    };
    load_keys(sb_first);
    // This (stream, head)'s table-gradient slices start at zero and the super-blocks add to them;
    // a single super-block whose window covers the whole table stores every entry itself.
    {
        const int j0f = sb_first * d.SBK;
        const bool all_rows = single && window_base(a, j0f, 63) == 0 && d.WR >= P;
        const bool all_slots = single && j0f == 0 && j0f + d.SBK - 1 + (T - 1) >= L - 1;
        if (dwr && !all_rows)
            for (int i = threadIdx.x; i < P * DK; i += blockDim.x)
                dwr[i] = 0.0f;
        if (dbr && !all_slots)
            for (int i = threadIdx.x; i < L; i += blockDim.x)
                dbr[i] = 0.0f;
    }
    tiles_ready();
    __syncthreads();
    // D_i = dO_i . O_i and the saved log-sum-exp, one warp per 8 rows
    for (int r = warp * 8; r < warp * 8 + 8; r++) {
        float s = 0.0f;
        for (int e = lane; e < DK; e += 32)
            s += to_f(dOs[(size_t)r * d.LDS + e]) * to_f(Os[(size_t)r * d.LDS + e]);
        s = warp_sum(s);
        if (lane == 0)
            Dr[r] = s;
    }

    AT_STAMP(1);
    // per-warp constants of phase A
    const int i0 = (warp & 3) * 16, half = warp >> 2;
    const int va = i0, vb = min(i0 + 16, T) - 1;
    const bool active = va <= vb;
    const int iA = i0 + g, iB = i0 + g + 8;
    int jloA = 0, jhiA = -1, jloB = 0, jhiB = -1;
    if (iA < T)
        key_range(a, iA, jloA, jhiA);
    if (iB < T)
        key_range(a, iB, jloB, jhiB);
    int jmin = 0, jmax = -1;
    if (active) {
        key_range(a, va, jmin, tmp);
        key_range(a, vb, tmp, jmax);
    }
    uint32_t qf[KS][4], df[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        ldsm4(qf[ks], Qs + (size_t)(i0 + (lane & 15)) * d.LDS + ks * 16 + (lane >> 4) * 8);
        ldsm4(df[ks], dOs + (size_t)(i0 + (lane & 15)) * d.LDS + ks * 16 + (lane >> 4) * 8);
    }
    float dq[NT][4]; // key part (warps 0-3) or position part (warps 4-7) of dQ for tile i0
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++)
            dq[nt][c] = 0.0f;
    bf16 *dkv = reinterpret_cast<bf16 *>(a.dkv);
    const int nsb = (L + d.SBK - 1) / d.SBK;

    for (int sb = 0; sb < nsb; sb++) {
        const int j0s = sb * d.SBK;
        const int wbase = window_base(a, j0s, 63);
        const bool touched = sb >= sb_first && sb <= sb_last; // any visible (query, key) pair here
        __syncthreads(); // previous super-block fully consumed (first trip: prologue done)
        if (touched && sb != sb_first)
            load_keys(sb);
        if (touched && a.w_r) // phase A scatters into the dE window; what it does not reach is zero
            for (int idx = threadIdx.x; idx < 64 * d.PPS / 8; idx += blockDim.x)
                reinterpret_cast<uint4 *>(dEm)[idx] = make_uint4(0u, 0u, 0u, 0u);
        tiles_ready();
        __syncthreads();
        if (sb == 0) AT_STAMP(2);
        if (!touched) {
            // keys nobody attends to: their dK, dV are zero
            for (int idx = threadIdx.x; idx < d.SBK * (DK / 8); idx += blockDim.x) {
                const int j = j0s + idx / (DK / 8), c = (idx % (DK / 8)) * 8;
                if (j < L) {
                    bf16 *dst = dkv + ((size_t)j * a.B + b) * a.dkvp + h * DK + c;
                    *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4 *>(dst + HD) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            continue;
        }
        // ---- phase A: P and dS of (tile i0, key block `half` of this super-block)
        {
            const int kb = j0s / 64 + half, j0 = kb * 64;
            if (j0 < j0s + d.SBK) {
                const bool visible = active && kb >= jmin / 64 && kb <= jmax / 64;
                if (!visible) {
                    for (int idx = lane; idx < 16 * 32; idx += 32) {
                        const size_t o2 = (size_t)(i0 + idx / 32) * d.LPS + (j0 - j0s) + (idx % 32) * 2;
                        *reinterpret_cast<uint32_t *>(Pm + o2) = 0u;
                        *reinterpret_cast<uint32_t *>(dSm + o2) = 0u;
                    }
                } else {
                    const float lseA = lses[i0 + g], lseB = lses[i0 + g + 8];
                    const float DA = Dr[i0 + g], DB = Dr[i0 + g + 8];
                    float *es = Es + (size_t)warp * 16 * EW;
                    float s[8][4], dp[8][4];
                    score_block<DK>(a, d, qf, Ks, Rs, brs, es, i0, j0, j0s, wbase, iA, iB, jloA, jhiA, jloB, jhiB, s);
#pragma unroll
                    for (int nt = 0; nt < 8; nt++)
#pragma unroll
                        for (int c = 0; c < 4; c++)
                            dp[nt][c] = 0.0f;
#pragma unroll
                    for (int ks = 0; ks < KS; ks++)
#pragma unroll
                        for (int np = 0; np < 4; np++) {
                            uint32_t bb[4];
                            ldsm4(bb, Vs + (size_t)(j0 - j0s + np * 16 + (lane & 7) + (lane >> 4) * 8) * d.LDS + ks * 16 + ((lane >> 3) & 1) * 8);
                            mma16816(dp[2 * np], df[ks], bb[0], bb[1]);
                            mma16816(dp[2 * np + 1], df[ks], bb[2], bb[3]);
                        }
#pragma unroll
                    for (int nt = 0; nt < 8; nt++) {
                        const float p0 = __expf(s[nt][0] - lseA), p1 = __expf(s[nt][1] - lseA);
                        const float p2 = __expf(s[nt][2] - lseB), p3 = __expf(s[nt][3] - lseB);
                        const int col = j0 - j0s + nt * 8 + 2 * t;
                        *reinterpret_cast<uint32_t *>(Pm + (size_t)(i0 + g) * d.LPS + col) = pack2(p0, p1);
                        *reinterpret_cast<uint32_t *>(Pm + (size_t)(i0 + g + 8) * d.LPS + col) = pack2(p2, p3);
                        const __nv_bfloat162 dsA = __floats2bfloat162_rn(p0 * (dp[nt][0] - DA) * a.inv_sqrt,
                                                                         p1 * (dp[nt][1] - DA) * a.inv_sqrt);
                        const __nv_bfloat162 dsB = __floats2bfloat162_rn(p2 * (dp[nt][2] - DB) * a.inv_sqrt,
                                                                         p3 * (dp[nt][3] - DB) * a.inv_sqrt);
                        *reinterpret_cast<__nv_bfloat162 *>(dSm + (size_t)(i0 + g) * d.LPS + col) = dsA;
                        *reinterpret_cast<__nv_bfloat162 *>(dSm + (size_t)(i0 + g + 8) * d.LPS + col) = dsB;
                        if (a.w_r) {
                            // inverse skew on the fly: dS[i][j] is dE[i][p] at table row p = j+T-1-i-(L-P)
                            // when p >= 1 (row 0 collects several slots and is summed after the barrier)
                            const int j = j0 + nt * 8 + 2 * t;
                            const int pA = j + (T - 1) - iA - (L - P), pB = pA - 8;
                            bf16 *eA = dEm + (size_t)(i0 + g) * d.PPS, *eB = dEm + (size_t)(i0 + g + 8) * d.PPS;
                            const int wA = pA - wbase, wB = pB - wbase; // columns of the window
                            if (iA < T) {
                                if (j < L && pA >= 1 && pA < P && wA >= 0 && wA < d.WR)
                                    eA[wA] = dsA.x;
                                if (j + 1 < L && pA + 1 >= 1 && pA + 1 < P && wA + 1 >= 0 && wA + 1 < d.WR)
                                    eA[wA + 1] = dsA.y;
                            }
                            if (iB < T) {
                                if (j < L && pB >= 1 && pB < P && wB >= 0 && wB < d.WR)
                                    eB[wB] = dsB.x;
                                if (j + 1 < L && pB + 1 >= 1 && pB + 1 < P && wB + 1 >= 0 && wB + 1 < d.WR)
                                    eB[wB + 1] = dsB.y;
                            }
                        }
                    }
                }
            }
        }
        __syncthreads();
        if (sb == 0) AT_STAMP(3);
        // ---- inverse skew for this super-block: dE[i][p] collects dS[i][j], p = max(j+T-1-i-(L-P), 0),
        //      over the window rows; db_r[r] += br_scale * sum_i dS[i][r-(T-1-i)]
        if (a.w_r && wbase == 0 && threadIdx.x < 64) {
            // table row 0 serves slots 0 .. L-P: the sum of those whose key is in this super-block
            const int i = threadIdx.x;
            float v = 0.0f;
            if (i < T) {
                const int off = (T - 1 - i) + j0s;
                const int rhi = min(L - P, off + min(d.SBK, L - j0s) - 1);
                for (int r = max(0, off); r <= rhi; r++)
                    v += to_f(dSm[(size_t)i * d.LPS + r - off]);
            }
            dEm[(size_t)i * d.PPS] = __float2bfloat16_rn(v);
        }
        if (dbr) {
            // slots whose (query, key) pairs can fall in this super-block
            const int rlo = j0s, rhi = min(L - 1, j0s + d.SBK - 1 + (T - 1));
            for (int r = rlo + threadIdx.x; r <= rhi; r += blockDim.x) {
                float acc0 = 0.0f, acc1 = 0.0f;
                for (int i = 0; i < T; i += 2) {
                    const int jl = r - (T - 1 - i) - j0s; // key of query i; query i+1 has the next key
                    if (jl >= 0 && jl < d.SBK && j0s + jl < L)
                        acc0 += to_f(dSm[(size_t)i * d.LPS + jl]);
                    if (i + 1 < T && jl + 1 >= 0 && jl + 1 < d.SBK && j0s + jl + 1 < L)
                        acc1 += to_f(dSm[(size_t)(i + 1) * d.LPS + jl + 1]);
                }
                const float v = (acc0 + acc1) * a.br_scale;
                dbr[r] = single ? v : dbr[r] + v;
            }
        }
        __syncthreads();
        if (sb == 0) AT_STAMP(4);

        // ---- phase B
        // dV = P^T dO and dK = dS^T Q for the keys of this super-block (K = the 64 queries)
        for (int mt = warp; mt < d.SBK / 16; mt += 8) {
            const int jm0 = mt * 16;
            float dv[NT][4], dk[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    dv[nt][c] = 0.0f;
                    dk[nt][c] = 0.0f;
                }
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                uint32_t ap[4], as[4];
                const int mi = lane >> 3;
                const size_t aoff = (size_t)(ks * 16 + (lane & 7) + (mi >> 1) * 8) * d.LPS + jm0 + (mi & 1) * 8;
                ldsm4t(ap, Pm + aoff);
                ldsm4t(as, dSm + aoff);
#pragma unroll
                for (int np = 0; np < NT / 2; np++) {
                    uint32_t bo[4], bq[4];
                    const size_t boff = (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * d.LDS + np * 16 + (lane >> 4) * 8;
                    ldsm4t(bo, dOs + boff);
                    ldsm4t(bq, Qs + boff);
                    mma16816(dv[2 * np], ap, bo[0], bo[1]);
                    mma16816(dv[2 * np + 1], ap, bo[2], bo[3]);
                    mma16816(dk[2 * np], as, bq[0], bq[1]);
                    mma16816(dk[2 * np + 1], as, bq[2], bq[3]);
                }
            }
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int j = j0s + jm0 + g + hh * 8;
                if (j < L) {
                    bf16 *dst = dkv + ((size_t)j * a.B + b) * a.dkvp + h * DK;
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        *reinterpret_cast<uint32_t *>(dst + nt * 8 + 2 * t) = pack2(dk[nt][2 * hh], dk[nt][2 * hh + 1]);
                        *reinterpret_cast<uint32_t *>(dst + HD + nt * 8 + 2 * t) = pack2(dv[nt][2 * hh], dv[nt][2 * hh + 1]);
                    }
                }
            }
        }
        if (sb == 0) AT_STAMP(5);
        // dQ += dS K (warps 0-3) / dE R (warps 4-7), tile i0
        if (i0 < T) {
            if (warp < 4) {
                for (int ks = 0; ks < d.SBK / 16; ks++) {
                    uint32_t as[4];
                    ldsm4(as, dSm + (size_t)(i0 + (lane & 15)) * d.LPS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int np = 0; np < NT / 2; np++) {
                        uint32_t bk[4];
                        ldsm4t(bk, Ks + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * d.LDS + np * 16 + (lane >> 4) * 8);
                        mma16816(dq[2 * np], as, bk[0], bk[1]);
                        mma16816(dq[2 * np + 1], as, bk[2], bk[3]);
                    }
                }
            } else if (a.w_r) {
                for (int ks = 0; ks < d.WR / 16; ks++) {
                    uint32_t ae[4];
                    ldsm4(ae, dEm + (size_t)(i0 + (lane & 15)) * d.PPS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int np = 0; np < NT / 2; np++) {
                        uint32_t br[4];
                        ldsm4t(br, Rs + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * d.LDS + np * 16 + (lane >> 4) * 8);
                        mma16816(dq[2 * np], ae, br[0], br[1]);
                        mma16816(dq[2 * np + 1], ae, br[2], br[3]);
                    }
                }
            }
        }
        if (sb == 0) AT_STAMP(6);
        // dR += dE^T Q over the window rows (this stream's share of the table gradient), fp32
        if (dwr) {
            for (int mt = warp; mt < d.WR / 16; mt += 8) {
                const int pm0 = mt * 16;
                float dr[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        dr[nt][c] = 0.0f;
#pragma unroll
                for (int ks = 0; ks < 4; ks++) {
                    uint32_t ae[4];
                    const int mi = lane >> 3;
                    ldsm4t(ae, dEm + (size_t)(ks * 16 + (lane & 7) + (mi >> 1) * 8) * d.PPS + pm0 + (mi & 1) * 8);
#pragma unroll
                    for (int np = 0; np < NT / 2; np++) {
                        uint32_t bq[4];
                        ldsm4t(bq, Qs + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * d.LDS + np * 16 + (lane >> 4) * 8);
                        mma16816(dr[2 * np], ae, bq[0], bq[1]);
                        mma16816(dr[2 * np + 1], ae, bq[2], bq[3]);
                    }
                }
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const int p = wbase + pm0 + g + hh * 8;
                    if (p < P)
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            float2 *dst = reinterpret_cast<float2 *>(dwr + (size_t)p * DK + nt * 8 + 2 * t);
                            float2 v = make_float2(dr[nt][2 * hh], dr[nt][2 * hh + 1]);
                            if (!single) {
                                const float2 old = *dst;
                                v.x += old.x;
                                v.y += old.y;
                            }
                            *dst = v;
                        }
                }
            }
        }
    }
    // ---- combine the two parts of dQ and write it
    __syncthreads();
    AT_STAMP(7);
    {
        float *dqp = Es; // [64][DK] fp32
        if (warp >= 4 && a.w_r && i0 < T) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                dqp[(size_t)(i0 + g) * DK + nt * 8 + 2 * t] = dq[nt][0];
                dqp[(size_t)(i0 + g) * DK + nt * 8 + 2 * t + 1] = dq[nt][1];
                dqp[(size_t)(i0 + g + 8) * DK + nt * 8 + 2 * t] = dq[nt][2];
                dqp[(size_t)(i0 + g + 8) * DK + nt * 8 + 2 * t + 1] = dq[nt][3];
            }
        }
        __syncthreads();
        if (i0 < T && warp < 4) {
            bf16 *dqg = reinterpret_cast<bf16 *>(a.dq);
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int i = i0 + g + hh * 8;
                if (i < T) {
                    bf16 *dst = dqg + ((size_t)i * a.B + b) * a.dqp + h * DK;
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        float x0 = dq[nt][2 * hh], x1 = dq[nt][2 * hh + 1];
                        if (a.w_r) {
                            x0 += dqp[(size_t)i * DK + nt * 8 + 2 * t];
                            x1 += dqp[(size_t)i * DK + nt * 8 + 2 * t + 1];
                        }
                        *reinterpret_cast<uint32_t *>(dst + nt * 8 + 2 * t) = pack2(x0, x1);
                    }
                }
            }
        }
    }
    AT_STAMP(8);
}

inline bool supported(const AttnArgs &a, bool backward)
{
    if (!(a.dk == 16 || a.dk == 32 || a.dk == 64 || a.dk == 128))
        return false;
    if (backward && a.T > 64)
        return false;
    size_t smem = 0;
    switch (a.dk) {
    case 16: smem = backward ? bwd_smem<16>(a.L, a.P) : fwd_smem<16>(a.L, a.P); break;
    case 32: smem = backward ? bwd_smem<32>(a.L, a.P) : fwd_smem<32>(a.L, a.P); break;
    case 64: smem = backward ? bwd_smem<64>(a.L, a.P) : fwd_smem<64>(a.L, a.P); break;
    default: smem = backward ? bwd_smem<128>(a.L, a.P) : fwd_smem<128>(a.L, a.P); break;
    }
    return smem <= 227 * 1024;
}

template <int DK>
static int launch_fwd(const AttnArgs &a, cudaStream_t st)
{
    size_t smem = fwd_smem<DK>(a.L, a.P);
    static size_t attr = 0;
    if (smem > attr) {
        CUDA_TRY(cudaFuncSetAttribute(attn_fwd_mma_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr = smem;
    }
    const int first_tile = a.t0 / 16, last_tile = (a.t1 - 1) / 16;
    const int groups = (last_tile - first_tile) / 4 + 1;
    launch_k(attn_fwd_mma_kernel<DK>, dim3(a.B * a.H, groups), dim3(128), smem, st, a);
    KERNEL_CHECK();
    return NNCU_OK;
}

template <int DK>
static int launch_bwd(const AttnArgs &a, cudaStream_t st)
{
    size_t smem = bwd_smem<DK>(a.L, a.P);
    static size_t attr = 0;
    if (smem > attr) {
        CUDA_TRY(cudaFuncSetAttribute(attn_bwd_mma_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr = smem;
    }
    launch_k(attn_bwd_mma_kernel<DK>, dim3(a.B * a.H), dim3(256), smem, st, a);
    KERNEL_CHECK();
    return NNCU_OK;
}

static int forward(const AttnArgs &a, cudaStream_t st)
{
    switch (a.dk) {
    case 16: return launch_fwd<16>(a, st);
    case 32: return launch_fwd<32>(a, st);
    case 64: return launch_fwd<64>(a, st);
    default: return launch_fwd<128>(a, st);
    }
}
static int backward(const AttnArgs &a, cudaStream_t st)
{
    switch (a.dk) {
    case 16: return launch_bwd<16>(a, st);
    case 32: return launch_bwd<32>(a, st);
    case 64: return launch_bwd<64>(a, st);
    default: return launch_bwd<128>(a, st);
    }
}

} // namespace amma

// ---- dispatch: bf16 goes to the tensor-core kernels when the shape allows, everything
// else to the CUDA-core kernels of attention.cuh.  The choice depends on the shape only,
// never on the query range, so one-symbol steps and whole segments take the same path.
static bool attn_force_simt()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("NNCU_ATTN_SIMT");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

template <typename T>
static int attn_forward_any(const nncu_attn_shape *s, const void *q, const void *kv, const float *w_r,
                            const float *b_r, void *out, float *lse, cudaStream_t st,
                            const AttnPitch *pt = nullptr, const void *w_r16 = nullptr, int *err_flag = nullptr)
{
    if (sizeof(T) == 2 && !attn_force_simt()) {
        AttnArgs a = attn_args(s, pt);
        a.q = q; a.kv = kv; a.w_r = w_r; a.b_r = b_r; a.o = out; a.lse = lse;
        a.w_r16 = w_r ? w_r16 : nullptr;
        // d_head 64: tcgen05 / TMEM / TMA kernel (the choice depends on the shape only)
        if (attc::enabled() && attc::supported(a, q, kv, a.w_r16))
            return attc::forward_any(a, a.w_r16, err_flag, st);
        if (amma::supported(a, false))
            return amma::forward(a, st);
    }
    return attn_forward_t<T>(s, q, kv, w_r, b_r, out, lse, st, pt);
}

template <typename T>
static int attn_backward_any(const nncu_attn_shape *s, const void *q, const void *kv, const float *w_r,
                             const float *b_r, const void *out, const float *lse, const void *dout,
                             void *dq, void *dkv, float *dwr_part, float *dbr_part, cudaStream_t st,
                             const AttnPitch *pt = nullptr, const void *w_r16 = nullptr, int *err_flag = nullptr)
{
    if (sizeof(T) == 2 && !attn_force_simt()) {
        AttnArgs a = attn_args(s, pt);
        a.w_r16 = w_r ? w_r16 : nullptr;
        if (a.t0 == 0 && a.t1 == a.T) {
            a.q = q; a.kv = kv; a.w_r = w_r; a.b_r = b_r; a.out = out; a.lse = const_cast<float *>(lse);
            a.dout = dout; a.dq = dq; a.dkv = dkv; a.dwr_part = dwr_part; a.dbr_part = dbr_part;
            if (attc::enabled() && attc::bwd_enabled() && attc::supported_bwd(a, a.w_r16))
                return attc::backward_any(a, a.w_r16, err_flag, st);
            if (amma::supported(a, true))
                return amma::backward(a, st);
        }
    }
    return attn_backward_t<T>(s, q, kv, w_r, b_r, out, lse, dout, dq, dkv, dwr_part, dbr_part, st, pt);
}

// Whether some kernel pair can run the forward and the backward pass of this shape (asked once,
// when a model is created, so that an unsupported shape is refused there and not in the middle
// of a file).  Mirrors the dispatch of attn_forward_any / attn_backward_any.
template <typename T>
static int attn_shape_supported(const nncu_attn_shape *s, bool has_wr)
{
    AttnArgs a = attn_args(s, nullptr);
    const bool mma = sizeof(T) == 2 && !attn_force_simt();
    if (!(mma && amma::supported(a, false))) {
        const size_t smem = attn_fwd_smem<T>(a.L, a.P, a.dk, has_wr);
        if (smem > 227 * 1024)
            return nncu_fail(NNCU_ERR_RANGE,
                             "attention forward of this shape (%d keys, d_pos %d, d_key %d) needs %zu bytes of "
                             "shared memory; the limit is %d",
                             a.L, a.P, a.dk, smem, 227 * 1024);
    }
    if (!(mma && amma::supported(a, true))) {
        const size_t smem = attn_bwd_smem<T>(a.T, a.L, a.P, a.dk, has_wr);
        if (smem > 227 * 1024)
            return nncu_fail(NNCU_ERR_RANGE,
                             "attention backward of this shape (seg_len %d, %d keys, d_pos %d, d_key %d) needs %zu "
                             "bytes of shared memory; the limit is %d",
                             a.T, a.L, a.P, a.dk, smem, 227 * 1024);
    }
    return NNCU_OK;
}
