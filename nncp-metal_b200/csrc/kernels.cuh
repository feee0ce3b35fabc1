// kernels.cuh -- the HBM-bound kernels of the train step: embedding, LayerNorm /
// RMSNorm with residual, activations, output softmax, loss gradient, column
// sums for bias gradients, the optimizer, the embedding gradient, transposes.
//
// Every reduction has a fixed association (warp butterflies, block trees and
// ordered loops; no atomics on floats), so a step is reproducible run to run
// and each forward row is independent of how many rows share the launch.
#pragma once
#include "common.cuh"

// ------------------------------------------------------------------
// embedding gather: x[r][:] = embed[id[r]][:] * mult        (nc_get_col, nncp.c:625-630)
template <typename T>
__global__ void embed_kernel(const int32_t *__restrict__ ids, const float *__restrict__ embed,
                             T *__restrict__ x, int rows, int D, float mult, int V)
{
    pdl_trigger();
    pdl_wait();
    int r = blockIdx.x;
    if (r >= rows)
        return;
    int id = ids[r];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const float *e = embed + (size_t)id * D;
    T *o = x + (size_t)r * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        o[i] = from_f<T>(e[i] * mult);
}

// ------------------------------------------------------------------
// s = a (+ res); y = norm(s) * g + b.  One warp per row.     (layer_norm, nncp.c:279-288)
// mode: 0 = copy only (y = s), 1 = LayerNorm, 2 = RMSNorm.  s_out / stats may be NULL.
// The statistics are taken from s after rounding to the storage type, so that the
// backward pass, which reads the stored s, sees exactly the normalised values.
template <typename T>
__global__ void __launch_bounds__(128)
residual_norm_kernel(const T *__restrict__ a, const T *__restrict__ res, T *__restrict__ s_out,
                     T *__restrict__ y, const float *__restrict__ g, const float *__restrict__ b,
                     float *__restrict__ stats, int rows, int D, int mode)
{
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + warp;
    if (r >= rows)
        return;
    const T *ar = a + (size_t)r * D;
    const T *rr = res ? res + (size_t)r * D : nullptr;
    float sum = 0.0f;
    for (int i = lane; i < D; i += 32) {
        float v = to_f(ar[i]);
        if (rr)
            v = round_to<T>(v + to_f(rr[i]));
        sum += v;
    }
    float mu = 0.0f, rstd = 1.0f;
    if (mode != 0) {
        if (mode == 1)
            mu = warp_sum(sum) / (float)D;
        float var = 0.0f;
        for (int i = lane; i < D; i += 32) {
            float v = to_f(ar[i]);
            if (rr)
                v = round_to<T>(v + to_f(rr[i]));
            var += (v - mu) * (v - mu);
        }
        var = warp_sum(var) / (float)D;
        rstd = 1.0f / sqrtf(var + 1e-5f);
        if (stats && lane == 0) {
            stats[2 * r] = mu;
            stats[2 * r + 1] = rstd;
        }
    }
    for (int i = lane; i < D; i += 32) {
        float v = to_f(ar[i]);
        if (rr)
            v = round_to<T>(v + to_f(rr[i]));
        if (s_out)
            s_out[(size_t)r * D + i] = from_f<T>(v);
        float o = (mode != 0) ? (v - mu) * rstd * g[i] + b[i] : v;
        y[(size_t)r * D + i] = from_f<T>(o);
    }
}

// Adjoint of y = norm(x)*g + b:  dx = (base ? base : 0) + J^T dy ; per-block partial column
// sums in part[blockIdx][3][D]: dg, db and (if want_sum) the column sums of the dx just
// written (the bias gradient of the projection that produced x).  Block = 8 warps, each warp
// walks rows blockIdx*RPB + warp, +8, ... inside the block's RPB-row chunk.
template <typename T>
__global__ void __launch_bounds__(256)
norm_bwd_kernel(const T *__restrict__ dy, const T *__restrict__ x, const float *__restrict__ g,
                const float *__restrict__ stats, const T *__restrict__ base, T *__restrict__ dx,
                float *__restrict__ part, int rows, int D, int mode, int rpb, int want_sum)
{
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[]; // [8][3][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *mydg = sm + (size_t)warp * 3 * D, *mydb = mydg + D, *mydx = mydb + D;
    for (int i = lane; i < 3 * D; i += 32)
        mydg[i] = 0.0f;
    const int r_end = min(rows, (blockIdx.x + 1) * rpb);
    for (int r = blockIdx.x * rpb + warp; r < r_end; r += 8) {
        const T *xr = x + (size_t)r * D, *dyr = dy + (size_t)r * D;
        const float mu = stats[2 * r], rstd = stats[2 * r + 1];
        float s1 = 0.0f, s2 = 0.0f;
        for (int i = lane; i < D; i += 32) {
            float xh = (to_f(xr[i]) - mu) * rstd;
            float d = to_f(dyr[i]);
            float dxh = d * g[i];
            s1 += dxh;
            s2 += dxh * xh;
            mydg[i] += d * xh;
            mydb[i] += d;
        }
        s1 = warp_sum(s1) / (float)D;
        s2 = warp_sum(s2) / (float)D;
        if (mode == 2)
            s1 = 0.0f;
        for (int i = lane; i < D; i += 32) {
            float xh = (to_f(xr[i]) - mu) * rstd;
            float dxh = to_f(dyr[i]) * g[i];
            float v = rstd * (dxh - s1 - xh * s2);
            if (base)
                v += to_f(base[(size_t)r * D + i]);
            T o = from_f<T>(v);
            dx[(size_t)r * D + i] = o;
            if (want_sum)
                mydx[i] += to_f(o);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 3 * D; i += blockDim.x) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++)
            s += sm[(size_t)w * 3 * D + i];
        part[(size_t)blockIdx.x * 3 * D + i] = s;
    }
}

// ---- bf16 rows of NC * 256 elements held in registers: 16-byte accesses, one pass over memory.
// Lane l owns elements c*256 + l*8 .. +7 of every 256-element chunk c.
template <int NC>
__device__ __forceinline__ void row_load(const bf16 *row, int lane, float (&v)[NC][8])
{
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const uint4 u = *reinterpret_cast<const uint4 *>(row + c * 256 + lane * 8);
        const bf16 *h = reinterpret_cast<const bf16 *>(&u);
#pragma unroll
        for (int e = 0; e < 8; e++)
            v[c][e] = to_f(h[e]);
    }
}
template <int NC>
__device__ __forceinline__ void row_store(bf16 *row, int lane, const float (&v)[NC][8])
{
#pragma unroll
    for (int c = 0; c < NC; c++) {
        uint4 u;
        bf16 *h = reinterpret_cast<bf16 *>(&u);
#pragma unroll
        for (int e = 0; e < 8; e++)
            h[e] = from_f<bf16>(v[c][e]);
        *reinterpret_cast<uint4 *>(row + c * 256 + lane * 8) = u;
    }
}
template <int NC>
__device__ __forceinline__ void vec_load_f32(const float *p, int lane, float (&v)[NC][8])
{
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const float4 a = *reinterpret_cast<const float4 *>(p + c * 256 + lane * 8);
        const float4 b = *reinterpret_cast<const float4 *>(p + c * 256 + lane * 8 + 4);
        v[c][0] = a.x; v[c][1] = a.y; v[c][2] = a.z; v[c][3] = a.w;
        v[c][4] = b.x; v[c][5] = b.y; v[c][6] = b.z; v[c][7] = b.w;
    }
}

// residual_norm_kernel for bf16 rows of D = NC * 256 elements; same arguments and rounding
// points (s is rounded to bf16 before the statistics), sums taken per lane, then over the warp.
template <int NC>
__global__ void __launch_bounds__(128)
residual_norm_vec_kernel(const bf16 *__restrict__ a, const bf16 *__restrict__ res, bf16 *__restrict__ s_out,
                         bf16 *__restrict__ y, const float *__restrict__ g, const float *__restrict__ b,
                         float *__restrict__ stats, int rows, int mode)
{
    pdl_trigger();
    pdl_wait();
    constexpr int D = NC * 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + warp;
    if (r >= rows)
        return;
    float v[NC][8];
    row_load<NC>(a + (size_t)r * D, lane, v);
    if (res) {
        float w[NC][8];
        row_load<NC>(res + (size_t)r * D, lane, w);
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
            for (int e = 0; e < 8; e++)
                v[c][e] = round_to<bf16>(v[c][e] + w[c][e]);
    }
    if (s_out)
        row_store<NC>(s_out + (size_t)r * D, lane, v);
    if (mode == 0) {
        row_store<NC>(y + (size_t)r * D, lane, v);
        return;
    }
    float mu = 0.0f;
    if (mode == 1) {
        float sum = 0.0f;
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
            for (int e = 0; e < 8; e++)
                sum += v[c][e];
        mu = warp_sum(sum) / (float)D;
    }
    float var = 0.0f;
#pragma unroll
    for (int c = 0; c < NC; c++)
#pragma unroll
        for (int e = 0; e < 8; e++)
            var += (v[c][e] - mu) * (v[c][e] - mu);
    var = warp_sum(var) / (float)D;
    const float rstd = 1.0f / sqrtf(var + 1e-5f);
    if (stats && lane == 0) {
        stats[2 * r] = mu;
        stats[2 * r + 1] = rstd;
    }
    float gv[NC][8], bv[NC][8];
    vec_load_f32<NC>(g, lane, gv);
    vec_load_f32<NC>(b, lane, bv);
#pragma unroll
    for (int c = 0; c < NC; c++)
#pragma unroll
        for (int e = 0; e < 8; e++)
            v[c][e] = (v[c][e] - mu) * rstd * gv[c][e] + bv[c][e];
    row_store<NC>(y + (size_t)r * D, lane, v);
}

// norm_bwd_kernel for bf16 rows of D = NC * 256 elements: one row per warp, eight rows per block,
// the block's column sums (dg, db, and the sums of the dx just written) go to part[block][3][D].
template <int NC>
__global__ void __launch_bounds__(256)
norm_bwd_vec_kernel(const bf16 *__restrict__ dy, const bf16 *__restrict__ x, const float *__restrict__ g,
                    const float *__restrict__ stats, const bf16 *__restrict__ base, bf16 *__restrict__ dx,
                    float *__restrict__ part, int rows, int mode, int want_sum)
{
    pdl_trigger();
    pdl_wait();
    constexpr int D = NC * 256;
    extern __shared__ float sm[]; // [8][3][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *mine = sm + (size_t)warp * 3 * D;
    const int r = blockIdx.x * 8 + warp;
    float xh[NC][8], d[NC][8], o[NC][8];
    if (r < rows) {
        const float mu = stats[2 * r], rstd = stats[2 * r + 1];
        float gv[NC][8];
        row_load<NC>(x + (size_t)r * D, lane, xh);
        row_load<NC>(dy + (size_t)r * D, lane, d);
        vec_load_f32<NC>(g, lane, gv);
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
            for (int e = 0; e < 8; e++) {
                xh[c][e] = (xh[c][e] - mu) * rstd;
                gv[c][e] *= d[c][e]; // dxh
                s1 += gv[c][e];
                s2 += gv[c][e] * xh[c][e];
            }
        s1 = warp_sum(s1) / (float)D;
        s2 = warp_sum(s2) / (float)D;
        if (mode == 2)
            s1 = 0.0f;
        if (base)
            row_load<NC>(base + (size_t)r * D, lane, o);
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float vv = rstd * (gv[c][e] - s1 - xh[c][e] * s2);
                o[c][e] = round_to<bf16>(base ? vv + o[c][e] : vv);
                xh[c][e] *= d[c][e]; // dg contribution
            }
        row_store<NC>(dx + (size_t)r * D, lane, o);
    } else {
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
            for (int e = 0; e < 8; e++)
                xh[c][e] = d[c][e] = o[c][e] = 0.0f;
    }
#pragma unroll
    for (int c = 0; c < NC; c++)
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int col = c * 256 + lane * 8 + e;
            mine[col] = xh[c][e];
            mine[D + col] = d[c][e];
            mine[2 * D + col] = want_sum ? o[c][e] : 0.0f;
        }
    __syncthreads();
    for (int i = threadIdx.x; i < 3 * D; i += blockDim.x) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++)
            s += sm[(size_t)w * 3 * D + i];
        part[(size_t)blockIdx.x * 3 * D + i] = s;
    }
}

// out[i] = ws[0][i] + ws[1][i] + ... (in that order) for the partial products of a split-K GEMM;
// n a multiple of 4.
template <typename TO>
__global__ void splitk_reduce_kernel(const float *__restrict__ ws, int ksplit, size_t n, TO *__restrict__ out)
{
    pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n)
        return;
    float4 acc = *reinterpret_cast<const float4 *>(ws + i);
    for (int z = 1; z < ksplit; z++) {
        const float4 v = *reinterpret_cast<const float4 *>(ws + (size_t)z * n + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    out[i] = from_f<TO>(acc.x);
    out[i + 1] = from_f<TO>(acc.y);
    out[i + 2] = from_f<TO>(acc.z);
    out[i + 3] = from_f<TO>(acc.w);
}

// Column reduction of partial sums, fixed order: out_k[c] = sum_p part[p*stride + off_k + c].
// blockIdx.y selects the output k (up to 3); a block owns 32 columns, its 8 warps each sum
// a contiguous range of parts, and the 8 range sums are added in range order.
struct ReduceOut {
    float *out[3];
    int off[3];
};
__global__ void __launch_bounds__(256)
reduce_cols_kernel(const float *__restrict__ part, int n_parts, int stride, int n, ReduceOut ro)
{
    pdl_trigger();
    pdl_wait();
    __shared__ float sm[8][33];
    const int c = blockIdx.x * 32 + (threadIdx.x & 31), grp = threadIdx.x >> 5;
    const int k = blockIdx.y;
    const int per = (n_parts + 7) / 8;
    float s = 0.0f;
    if (c < n) {
        const float *src = part + ro.off[k] + c;
        const int p1 = min(n_parts, (grp + 1) * per);
        for (int p = grp * per; p < p1; p++)
            s += src[(size_t)p * stride];
    }
    sm[grp][threadIdx.x & 31] = s;
    __syncthreads();
    if (grp == 0 && c < n) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++)
            t += sm[w][threadIdx.x];
        ro.out[k][c] = t;
    }
}

// Every column / stream reduction of one layer's backward pass in one launch.  Job kinds:
//   0  out[c] = sum over parts p of part[p*stride + off + c], the parts dealt to 8 groups of
//      consecutive parts whose sums are added in group order (reduce_cols_kernel's association)
//   1  out[i] (+)= sum over parts (streams) in order of part[p*stride + i]   (reduce_streams_kernel)
// blk0 is the job's first block; a block finds its job by a short scan (the table is a kernel
// argument, so the launch can sit in a captured graph).
struct ReduceJob {
    const float *part;
    float *out;
    int n_parts, stride, n, off, kind, accumulate, blk0;
};
constexpr int MAX_REDUCE_JOBS = 16;
struct ReduceJobs {
    int n_jobs;
    ReduceJob job[MAX_REDUCE_JOBS];
};
__global__ void __launch_bounds__(256) reduce_jobs_kernel(const __grid_constant__ ReduceJobs jobs)
{
    pdl_trigger();
    pdl_wait();
    __shared__ float sm[8][33];
    int j = 0;
    while (j + 1 < jobs.n_jobs && (int)blockIdx.x >= jobs.job[j + 1].blk0)
        j++;
    const ReduceJob &jb = jobs.job[j];
    const int blk = blockIdx.x - jb.blk0;
    if (jb.kind == 1) {
        const int i = blk * 256 + threadIdx.x;
        if (i < jb.n) {
            float s = 0.0f;
            for (int p = 0; p < jb.n_parts; p++)
                s += jb.part[(size_t)p * jb.stride + i];
            jb.out[i] = jb.accumulate ? jb.out[i] + s : s;
        }
        return;
    }
    const int c = blk * 32 + (threadIdx.x & 31), grp = threadIdx.x >> 5;
    const int per = (jb.n_parts + 7) / 8;
    float s = 0.0f;
    if (c < jb.n) {
        const float *src = jb.part + jb.off + c;
        const int p1 = min(jb.n_parts, (grp + 1) * per);
        for (int p = grp * per; p < p1; p++)
            s += src[(size_t)p * jb.stride];
    }
    sm[grp][threadIdx.x & 31] = s;
    __syncthreads();
    if (grp == 0 && c < jb.n) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++)
            t += sm[w][threadIdx.x];
        jb.out[c] = t;
    }
}

// dst = a + b (elementwise), used where a residual joins without a norm
template <typename T>
__global__ void add_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ dst,
                           size_t n)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n)
        dst[i] = from_f<T>(to_f(a[i]) + to_f(b[i]));
}

// ------------------------------------------------------------------
// LN_COEF (nncp.c:892-894, 975-977): a sub-layer's output is multiplied by the layer's learned
// scalar alpha before the residual sum.  Forward: dst = alpha * src.  Backward, one block per row:
// dt = alpha * ds for the branch, and part[r] = sum_c ds[r][c] * a[r][c] (the row's share of
// d alpha, columns added in a fixed order); the rows are summed later by one ordered job.
template <typename T>
__global__ void scale_rows_kernel(const T *__restrict__ src, const float *__restrict__ alpha, T *__restrict__ dst, size_t n)
{
    pdl_trigger();
    pdl_wait();
    const float al = alpha[0];
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = from_f<T>(al * to_f(src[i]));
}

template <typename T>
__global__ void __launch_bounds__(128)
scale_dot_kernel(const T *__restrict__ ds, const T *__restrict__ a, const float *__restrict__ alpha, T *__restrict__ dt,
                 float *__restrict__ part, int rows, int D)
{
    pdl_trigger();
    pdl_wait();
    __shared__ float red[4];
    const int r = blockIdx.x;
    if (r >= rows)
        return;
    const float al = alpha[0];
    float s = 0.0f;
    for (int c = threadIdx.x; c < D; c += 128) {
        const float d = to_f(ds[(size_t)r * D + c]);
        s += d * to_f(a[(size_t)r * D + c]);
        dt[(size_t)r * D + c] = from_f<T>(al * d);
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0)
        part[r] = (red[0] + red[1]) + (red[2] + red[3]);
}

// ------------------------------------------------------------------
// feed-forward activation (nncp.c:938-966).  hpre [rows][F1], hact [rows][F].
__device__ __forceinline__ float gelu_f(float x)
{
    return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x)
{
    float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    float t = tanhf(u);
    float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}

// The same two functions on the hardware tanh (one MUFU instruction, absolute error about 5e-4,
// below the rounding step of the bf16 values they feed): the bf16 activation kernels are bound
// by their instruction count, and tanhf is most of it.
__device__ __forceinline__ float tanh_hw(float x)
{
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float gelu_hw(float x)
{
    return 0.5f * x * (1.0f + tanh_hw(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_hw(float x)
{
    float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    float t = tanh_hw(u);
    float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}

// x * sigmoid(x), the gate function of FF_ACT_GATED_SILU (nc_gated_swish with beta 1, nncp.c:957-962),
// and its derivative; the _hw forms take the sigmoid from the hardware tanh.
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_grad_f(float x)
{
    const float s = 1.0f / (1.0f + expf(-x));
    return s * (1.0f + x * (1.0f - s));
}
__device__ __forceinline__ float silu_hw(float x) { return x * (0.5f + 0.5f * tanh_hw(0.5f * x)); }
__device__ __forceinline__ float silu_grad_hw(float x)
{
    const float s = 0.5f + 0.5f * tanh_hw(0.5f * x);
    return s * (1.0f + x * (1.0f - s));
}
// the gated activations: value and derivative of the function applied to the first half
__device__ __forceinline__ float gate_f(float x, int act) { return act == NNCU_FF_GATED_SILU ? silu_f(x) : gelu_f(x); }
__device__ __forceinline__ float gate_grad_f(float x, int act) { return act == NNCU_FF_GATED_SILU ? silu_grad_f(x) : gelu_grad_f(x); }
__device__ __forceinline__ float gate_hw(float x, int act) { return act == NNCU_FF_GATED_SILU ? silu_hw(x) : gelu_hw(x); }
__device__ __forceinline__ float gate_grad_hw(float x, int act) { return act == NNCU_FF_GATED_SILU ? silu_grad_hw(x) : gelu_grad_hw(x); }

template <typename T>
__global__ void act_fwd_kernel(const T *__restrict__ hpre, T *__restrict__ hact, int rows, int F,
                               int F1, int act)
{
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * F)
        return;
    int r = (int)(idx / F), i = (int)(idx % F);
    float a = to_f(hpre[(size_t)r * F1 + i]), o;
    if (act == NNCU_FF_RELU)
        o = a > 0.0f ? a : 0.0f;
    else if (act == NNCU_FF_GELU)
        o = gelu_f(a);
    else
        o = gate_f(a, act) * to_f(hpre[(size_t)r * F1 + F + i]);
    hact[idx] = from_f<T>(o);
}

// Eight columns per thread (16-byte accesses); same arithmetic per element as act_fwd_kernel.
// Needs F and F1 to be multiples of 8 and 16-byte aligned rows.
__global__ void act_fwd_vec_kernel(const bf16 *__restrict__ hpre, bf16 *__restrict__ hact, int rows, int F,
                                   int F1, int act)
{
    pdl_trigger();
    pdl_wait();
    const int cpr = F / 8;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * cpr)
        return;
    const int r = (int)(idx / cpr), i = (int)(idx % cpr) * 8;
    const uint4 va = *reinterpret_cast<const uint4 *>(hpre + (size_t)r * F1 + i);
    const bf16 *a = reinterpret_cast<const bf16 *>(&va);
    uint4 vo;
    bf16 *o = reinterpret_cast<bf16 *>(&vo);
    if (act == NNCU_FF_RELU) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float x = to_f(a[j]);
            o[j] = from_f<bf16>(x > 0.0f ? x : 0.0f);
        }
    } else if (act == NNCU_FF_GELU) {
#pragma unroll
        for (int j = 0; j < 8; j++)
            o[j] = from_f<bf16>(gelu_hw(to_f(a[j])));
    } else {
        const uint4 vg = *reinterpret_cast<const uint4 *>(hpre + (size_t)r * F1 + F + i);
        const bf16 *g = reinterpret_cast<const bf16 *>(&vg);
#pragma unroll
        for (int j = 0; j < 8; j++)
            o[j] = from_f<bf16>(gate_hw(to_f(a[j]), act) * to_f(g[j]));
    }
    *reinterpret_cast<uint4 *>(hact + (size_t)r * F + i) = vo;
}

// Adjoint of the activation, and (part != NULL) per-chunk column sums of the result for the
// ff_bias1 gradient: part[chunk][F1].  grid (ceil(F/128), ceil(rows/32)); one column per thread.
template <typename T>
__global__ void __launch_bounds__(128)
act_bwd_kernel(const T *__restrict__ hpre, const T *__restrict__ dhact, T *__restrict__ dhpre,
               float *__restrict__ part, int rows, int F, int F1, int act)
{
    const int i = blockIdx.x * 128 + threadIdx.x;
    if (i >= F)
        return;
    const int r0 = blockIdx.y * 32, r1 = min(rows, r0 + 32);
    float s0 = 0.0f, s1 = 0.0f;
    for (int r = r0; r < r1; r++) {
        float a = to_f(hpre[(size_t)r * F1 + i]), d = to_f(dhact[(size_t)r * F + i]);
        if (act == NNCU_FF_RELU || act == NNCU_FF_GELU) {
            T o = from_f<T>(act == NNCU_FF_RELU ? (a > 0.0f ? d : 0.0f) : d * gelu_grad_f(a));
            dhpre[(size_t)r * F1 + i] = o;
            s0 += to_f(o);
        } else {
            float gate = to_f(hpre[(size_t)r * F1 + F + i]);
            T o0 = from_f<T>(d * gate * gate_grad_f(a, act)), o1 = from_f<T>(d * gate_f(a, act));
            dhpre[(size_t)r * F1 + i] = o0;
            dhpre[(size_t)r * F1 + F + i] = o1;
            s0 += to_f(o0);
            s1 += to_f(o1);
        }
    }
    if (part) {
        part[(size_t)blockIdx.y * F1 + i] = s0;
        if (F1 > F)
            part[(size_t)blockIdx.y * F1 + F + i] = s1;
    }
}

// Two columns per thread (4-byte accesses), ACT_BWD_ROWS rows per block (short serial chains:
// the kernel is bound by the latency of its per-element math, not by bytes); element
// arithmetic as in act_bwd_kernel.  F even; grid (ceil(F/256), ceil(rows/ACT_BWD_ROWS)).
constexpr int ACT_BWD_ROWS = 8;
__global__ void __launch_bounds__(128)
act_bwd_vec_kernel(const bf16 *__restrict__ hpre, const bf16 *__restrict__ dhact, bf16 *__restrict__ dhpre,
                   float *__restrict__ part, int rows, int F, int F1, int act)
{
    pdl_trigger();
    pdl_wait();
    const int i = (blockIdx.x * 128 + threadIdx.x) * 2;
    if (i >= F)
        return;
    const int r0 = blockIdx.y * ACT_BWD_ROWS, r1 = min(rows, r0 + ACT_BWD_ROWS);
    float s0[2] = {0.0f, 0.0f}, s1[2] = {0.0f, 0.0f};
#pragma unroll
    for (int rr = 0; rr < ACT_BWD_ROWS; rr++) {
        const int r = r0 + rr;
        if (r >= r1)
            break;
        const __nv_bfloat162 a2 = *reinterpret_cast<const __nv_bfloat162 *>(hpre + (size_t)r * F1 + i);
        const __nv_bfloat162 d2 = *reinterpret_cast<const __nv_bfloat162 *>(dhact + (size_t)r * F + i);
        const float a[2] = {__low2float(a2), __high2float(a2)}, d[2] = {__low2float(d2), __high2float(d2)};
        bf16 o0[2], o1[2];
        if (act == NNCU_FF_RELU || act == NNCU_FF_GELU) {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                o0[j] = from_f<bf16>(act == NNCU_FF_RELU ? (a[j] > 0.0f ? d[j] : 0.0f) : d[j] * gelu_grad_hw(a[j]));
                s0[j] += to_f(o0[j]);
            }
        } else {
            const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162 *>(hpre + (size_t)r * F1 + F + i);
            const float gate[2] = {__low2float(g2), __high2float(g2)};
#pragma unroll
            for (int j = 0; j < 2; j++) {
                o0[j] = from_f<bf16>(d[j] * gate[j] * gate_grad_hw(a[j], act));
                o1[j] = from_f<bf16>(d[j] * gate_hw(a[j], act));
                s0[j] += to_f(o0[j]);
                s1[j] += to_f(o1[j]);
            }
            *reinterpret_cast<__nv_bfloat162 *>(dhpre + (size_t)r * F1 + F + i) = __halves2bfloat162(o1[0], o1[1]);
        }
        *reinterpret_cast<__nv_bfloat162 *>(dhpre + (size_t)r * F1 + i) = __halves2bfloat162(o0[0], o0[1]);
    }
    if (part) {
        float *row = part + (size_t)blockIdx.y * F1;
        row[i] = s0[0];
        row[i + 1] = s0[1];
        if (F1 > F) {
            row[F + i] = s1[0];
            row[F + i + 1] = s1[1];
        }
    }
}

// ------------------------------------------------------------------
// block-wide fixed-order reductions for 256-thread blocks
__device__ __forceinline__ float block_sum_256(float v, float *red)
{
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++)
        s += red[w];
    return s;
}
__device__ __forceinline__ float block_max_256(float v, float *red)
{
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = red[0];
#pragma unroll
    for (int w = 1; w < 8; w++)
        s = fmaxf(s, red[w]);
    return s;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// in-place softmax over the V symbols of each row of fp32 logits (nc_soft_max, nncp.c:1008).
// The output kernel of the forward pass: besides the probabilities it leaves dz = p * scale, the
// gradient of the loss with respect to the logits of every symbol but the target (which
// loss_fix_kernel corrects once the targets are known), so that the backward pass does not read
// the probability tables again.  *dz_fixed = 0 says that dz holds no target correction.
template <typename T>
__global__ void __launch_bounds__(256) softmax_rows_kernel(float *__restrict__ z, int rows, int V, T *__restrict__ dz, float scale,
                                                           int *__restrict__ dz_fixed)
{
    pdl_trigger();
    pdl_wait();
    __shared__ float red[8];
    int r = blockIdx.x;
    if (r >= rows)
        return;
    if (r == 0 && threadIdx.x == 0)
        *dz_fixed = 0;
    float *zr = z + (size_t)r * V;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += 256)
        mx = fmaxf(mx, zr[i]);
    mx = block_max_256(mx, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < V; i += 256) {
        float e = expf(zr[i] - mx);
        zr[i] = e;
        s += e;
    }
    s = block_sum_256(s, red);
    float rs = 1.0f / s;
    T *d = dz + (size_t)r * V;
    for (int i = threadIdx.x; i < V; i += 256) {
        const float pv = zr[i] * rs;
        zr[i] = pv;
        d[i] = from_f<T>(pv * scale);
    }
}

// The same for rows of up to 16384 logits, V a multiple of 1024: the row stays in registers
// (one read and one write of memory, 16-byte accesses).  Thread t owns logits (k*256 + t)*4 .. +3.
template <typename T>
__global__ void __launch_bounds__(256) softmax_rows_reg_kernel(float *__restrict__ z, int rows, int V, T *__restrict__ dz,
                                                               float scale, int *__restrict__ dz_fixed)
{
    pdl_trigger();
    pdl_wait();
    __shared__ float red[8];
    const int r = blockIdx.x;
    if (r >= rows)
        return;
    if (r == 0 && threadIdx.x == 0)
        *dz_fixed = 0;
    float4 *zr = reinterpret_cast<float4 *>(z + (size_t)r * V);
    const int nv = V / 1024;
    float4 v[16];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < 16; k++)
        if (k < nv) {
            v[k] = zr[k * 256 + threadIdx.x];
            mx = fmaxf(mx, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
        }
    mx = block_max_256(mx, red);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < 16; k++)
        if (k < nv) {
            v[k].x = expf(v[k].x - mx);
            v[k].y = expf(v[k].y - mx);
            v[k].z = expf(v[k].z - mx);
            v[k].w = expf(v[k].w - mx);
            s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
    s = block_sum_256(s, red);
    const float rs = 1.0f / s;
#pragma unroll
    for (int k = 0; k < 16; k++)
        if (k < nv) {
            v[k].x *= rs;
            v[k].y *= rs;
            v[k].z *= rs;
            v[k].w *= rs;
            zr[k * 256 + threadIdx.x] = v[k];
            T *d = dz + (size_t)r * V + (size_t)(k * 256 + threadIdx.x) * 4;
            if (sizeof(T) == 2) {
                uint2 pk;
                pk.x = pack_bf16x2(v[k].x * scale, v[k].y * scale);
                pk.y = pack_bf16x2(v[k].z * scale, v[k].w * scale);
                *reinterpret_cast<uint2 *>(d) = pk;
            } else {
                *reinterpret_cast<float4 *>(d) = make_float4(v[k].x * scale, v[k].y * scale, v[k].z * scale, v[k].w * scale);
            }
        }
}

// The target correction of dz: for every row r, dz[r][t_r] = (p[r][t_r] - 1) * scale and
// logp[r] = ln p[r][t_r] (nc_indexed_log and the adjoint of the softmax, nncp.c:1170-1175).  A
// second call for the same forward pass (*dz_fixed != 0) first puts the old targets' entries back
// to p * scale.  loss_sum_kernel, queued behind it, adds the logp in a fixed order (thread i adds
// rows i, i + 256, ...; then the block sum) and raises the flag.
template <typename T>
__global__ void __launch_bounds__(256)
loss_fix_kernel(const float *__restrict__ probs, const int32_t *__restrict__ targets, int32_t *__restrict__ fixed_targets,
                const int *__restrict__ dz_fixed, T *__restrict__ dz, float *__restrict__ logp, int rows, int V, float scale)
{
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * 256 + threadIdx.x;
    if (r >= rows)
        return;
    const float *pr = probs + (size_t)r * V;
    T *d = dz + (size_t)r * V;
    if (*dz_fixed != 0) {
        const int old = fixed_targets[r];
        d[old] = from_f<T>(pr[old] * scale);
    }
    int t = targets[r];
    t = t < 0 ? 0 : (t >= V ? V - 1 : t);
    const float pt = pr[t];
    d[t] = from_f<T>((pt - 1.0f) * scale);
    fixed_targets[r] = t;
    logp[r] = logf(pt);
}

__global__ void __launch_bounds__(256) loss_sum_kernel(const float *__restrict__ v, int n, float *__restrict__ out,
                                                       int *__restrict__ dz_fixed)
{
    pdl_trigger();
    pdl_wait();
    __shared__ float red[8];
    float s = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256)
        s += v[i];
    s = block_sum_256(s, red);
    if (threadIdx.x == 0) {
        *out = s;
        *dz_fixed = 1;
    }
}

// column sums of A [R][N] over row chunks: part[chunk][n]   (bias gradients)
template <typename T>
__global__ void colsum_part_kernel(const T *__restrict__ A, long lda, int R, int N, int rows_per,
                                   float *__restrict__ part)
{
    pdl_trigger();
    pdl_wait();
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N)
        return;
    int r0 = blockIdx.y * rows_per, r1 = min(R, r0 + rows_per);
    float s = 0.0f;
    for (int r = r0; r < r1; r++)
        s += to_f(A[(long)r * lda + n]);
    part[(size_t)blockIdx.y * N + n] = s;
}

// ------------------------------------------------------------------
// optimizer (nc_sgd_opt_update, nncp.c:1229; constants libnc.h:547-561):
//   g' = clamp(g) ; v = b2*v + (1-b2)*g'^2 ; w -= lr*g'/(sqrt(v*corr)+eps)
// and the bf16 shadow of w refreshed in the same pass.
__global__ void __launch_bounds__(256)
rmsprop_kernel(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ v,
               bf16 *__restrict__ shadow, size_t n4, float lr, float beta2, float eps,
               float clip, float corr, const float *__restrict__ hyper)
{
    pdl_trigger();
    pdl_wait();
    if (hyper) { // {lr, corr} from device memory: a captured launch must not freeze them
        lr = hyper[0];
        corr = hyper[1];
    }
    // grid-stride: correct for any grid; the library launches one thread per group of four
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 ww = reinterpret_cast<float4 *>(w)[i];
    float4 gg = reinterpret_cast<const float4 *>(g)[i];
    float4 vv = reinterpret_cast<float4 *>(v)[i];
    float *pw = &ww.x, *pg = &gg.x, *pv = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        float x = pg[k];
        if (clip != 0.0f)
            x = fminf(fmaxf(x, -clip), clip);
        pv[k] = beta2 * pv[k] + (1.0f - beta2) * x * x;
        if (x != 0.0f)
            pw[k] -= lr * x / (sqrtf(pv[k] * corr) + eps);
    }
    reinterpret_cast<float4 *>(w)[i] = ww;
    reinterpret_cast<float4 *>(v)[i] = vv;
    if (shadow) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(ww.x, ww.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn(ww.z, ww.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t *>(&lo);
        pk.y = *reinterpret_cast<uint32_t *>(&hi);
        reinterpret_cast<uint2 *>(shadow)[i] = pk;
    }
    }
}

__global__ void f32_to_bf16_kernel(const float *__restrict__ src, bf16 *__restrict__ dst, size_t n)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n)
        dst[i] = __float2bfloat16_rn(src[i]);
}

// ------------------------------------------------------------------
// dense embedding gradient (adjoint of nc_get_col): g[v][:] = mult * sum over rows r with
// id[r]==v, in ascending r, of dx[r][:].  g must be zero on entry.
// first_rows_kernel leaves in first[v] the smallest row that carries symbol v (first[] holds a
// value >= rows on entry; integer atomicMin, so the result does not depend on the order of
// arrival).  embed_grad_kernel runs one block per row: the block of a symbol's first row lists the
// rows behind it that carry the symbol (ordered compaction by warp ballots), and every thread adds
// them, in ascending order, into the four columns it owns; the other blocks leave after two loads.
__global__ void first_rows_kernel(const int32_t *__restrict__ ids, int rows, int V, int *__restrict__ first)
{
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows)
        return;
    int id = ids[r];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    atomicMin(first + id, r);
}

template <typename T>
__global__ void __launch_bounds__(128)
embed_grad_kernel(const int32_t *__restrict__ ids, const T *__restrict__ dx, float *__restrict__ g,
                  const int *__restrict__ first, int rows, int D, float mult, int V)
{
    pdl_trigger();
    pdl_wait();
    constexpr int SPAN = 2048; // rows listed per pass
    __shared__ int list[SPAN];
    __shared__ int wcnt[2][4]; // per-warp hit counts of a chunk, double-buffered by chunk parity
    const int r0 = blockIdx.x;
    int v = ids[r0];
    v = v < 0 ? 0 : (v >= V ? V - 1 : v);
    if (first[v] != r0)
        return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c0 = 0; c0 < D; c0 += 512) { // four columns per thread and pass
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int span0 = r0; span0 < rows; span0 += SPAN) {
            // ordered list of the rows of this span that carry the symbol (compaction by warp ballots).
            // Every thread keeps the running total in a register: the counts of a chunk are read by all
            // threads after one barrier, and the buffer they sit in is not written again before the
            // barrier of the next chunk has been passed by everyone.
            __syncthreads(); // the list of the span before has been read
            const int span1 = min(rows, span0 + SPAN);
            int idr[SPAN / 128]; // all of the span's ids are requested before the first is looked at
#pragma unroll
            for (int j = 0; j < SPAN / 128; j++) {
                const int r = span0 + 128 * j + threadIdx.x;
                idr[j] = r < span1 ? ids[r] : -1;
            }
            int n = 0;
#pragma unroll
            for (int j = 0; j < SPAN / 128; j++) {
                const int base = span0 + 128 * j;
                if (base >= span1)
                    break;
                const int r = base + threadIdx.x;
                int id = idr[j];
                if (r < span1)
                    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
                const bool hit = id == v;
                const unsigned bal = __ballot_sync(0xffffffffu, hit);
                if (lane == 0)
                    wcnt[j & 1][warp] = __popc(bal);
                __syncthreads();
                const int w0 = wcnt[j & 1][0], w1 = wcnt[j & 1][1], w2 = wcnt[j & 1][2], w3 = wcnt[j & 1][3];
                const int pos = n + (warp > 0 ? w0 : 0) + (warp > 1 ? w1 : 0) + (warp > 2 ? w2 : 0);
                if (hit)
                    list[pos + __popc(bal & ((1u << lane) - 1u))] = r;
                n += w0 + w1 + w2 + w3;
            }
            __syncthreads(); // the list is complete
            // sixteen rows' loads go out before the first is added: the sum of a frequent symbol is a
            // chain of additions in row order, but its loads need not wait for one another
            for (int k0 = 0; k0 < n; k0 += 16) {
                float x[16][4];
#pragma unroll
                for (int u = 0; u < 16; u++) {
                    const T *src = dx + (size_t)list[min(k0 + u, n - 1)] * D + c0;
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int c = threadIdx.x + 128 * k;
                        x[u][k] = (c0 + c < D) ? to_f(src[c]) : 0.0f;
                    }
                }
#pragma unroll
                for (int u = 0; u < 16; u++)
                    if (k0 + u < n) {
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            acc[k] += x[u][k];
                    }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int c = c0 + threadIdx.x + 128 * k;
            if (c < D)
                g[(size_t)v * D + c] = acc[k] * mult;
        }
    }
}

// ------------------------------------------------------------------
// dst[c][r] = src[r][c]  (bf16 32x32 tiles through shared memory)
__global__ void __launch_bounds__(256)
transpose_bf16_kernel(const bf16 *__restrict__ src, long lds, bf16 *__restrict__ dst, long ldd,
                      int R, int Ccols)
{
    __shared__ bf16 tile[32][33];
    int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 32; j += 8) {
        int r = r0 + j, c = c0 + tx;
        if (r < R && c < Ccols)
            tile[j][tx] = src[(long)r * lds + c];
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        int c = c0 + j, r = r0 + tx;
        if (r < R && c < Ccols)
            dst[(long)c * ldd + r] = tile[tx][j];
    }
}

// ------------------------------------------------------------------
// order-independent 64-bit digest of a float buffer: sum of mix(index, bits) mod 2^64
__device__ __forceinline__ unsigned long long mix64(unsigned long long x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__global__ void hash_kernel(const float *__restrict__ w, size_t n, unsigned long long *out)
{
    unsigned long long s = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        s += mix64((i << 32) ^ (unsigned long long)__float_as_uint(w[i]));
    atomicAdd(out, s); // integer addition: the order of arrival does not change the sum
}
