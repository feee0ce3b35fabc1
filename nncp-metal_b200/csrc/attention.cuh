// attention.cuh -- relative-position causal attention over [memory | segment],
// forward and backward, one CTA per (stream, head).
//
// Follows the sub-graph of trf_eval at nncp.c:722-800:
//   score(i,j) = ( q_i.k_j + q_i.w_r[max(r-(L-P),0)] + br_scale*b_r[r] ) / sqrt(dk)
//   r = j + (T-1) - i          nc_rel_shift(-(T-1))            nncp.c:784
//   left pad by duplication    nc_pad(L-P, NC_PAD_DUP)         nncp.c:777
//   key j visible to query i   iff 0 <= (i+M)-j < attn_len     nncp.c:357-361
// and its adjoint (LibNC's autograd is not part of the reference tree).
//
// CUDA-core kernels: at the sizes NNCP uses (T <= 64, L <= 576, dk <= 128 per
// (stream, head)) the op is bound by HBM traffic and launch latency, not by the
// tensor pipe.  K, V and the w_r table of the CTA's (stream, head) are staged
// once in shared memory; all reductions run in a fixed order (lanes own keys,
// butterflies combine them), so query row i gives the same bits whether it is
// computed alone (one-symbol step) or with the whole segment.
#pragma once
#include "common.cuh"

struct AttnArgs {
    const void *q, *kv, *out, *dout;
    const float *w_r, *b_r;
    const void *w_r16; // optional bf16 copy of w_r (same layout), used by the tensor-core kernels
    void *o, *dq, *dkv;
    float *lse, *dwr_part, *dbr_part;
    int B, H, dk, T, M, L, P, attn_len, t0, t1, qchunk;
    int qp, kvp, dqp, dkvp; // row pitches (elements) of q, kv, dq, dkv; K then V inside a kv row
    float br_scale, inv_sqrt;
};

template <typename T> struct SmemRow; // padded row strides that avoid bank conflicts
template <> struct SmemRow<float> { static __host__ __device__ int stride(int dk) { return dk + 1; } };
template <> struct SmemRow<bf16> { static __host__ __device__ int stride(int dk) { return dk + 2; } };

template <typename T>
__device__ __forceinline__ float dot_q(const float *__restrict__ qf, const T *__restrict__ row, int dk)
{
    float s = 0.0f;
    for (int e = 0; e < dk; e++)
        s = fmaf(qf[e], to_f(row[e]), s);
    return s;
}

// score of (query i, key j) for an unmasked pair
template <typename T>
__device__ __forceinline__ float score_ij(const AttnArgs &a, int h, int i, int j, const float *qf,
                                          const T *Ks, const T *Rs, int ks)
{
    float s = dot_q<T>(qf, Ks + (size_t)j * ks, a.dk);
    int r = j + (a.T - 1) - i;
    float z = a.br_scale * a.b_r[(size_t)h * a.L + r];
    if (a.w_r) {
        int pi = r - (a.L - a.P);
        pi = pi < 0 ? 0 : pi;
        z += dot_q<T>(qf, Rs + (size_t)pi * ks, a.dk);
    }
    return (s + z) * a.inv_sqrt;
}

__device__ __forceinline__ void key_range(const AttnArgs &a, int i, int &jlo, int &jhi)
{
    jhi = min(a.L - 1, i + a.M);                 // (i+M)-j >= 0
    jlo = max(0, i + a.M - a.attn_len + 1);      // (i+M)-j < attn_len
}

template <typename T>
size_t attn_fwd_smem(int L, int P, int dk, bool has_wr)
{
    int ks = SmemRow<T>::stride(dk);
    size_t b = (size_t)L * ks * sizeof(T) + (size_t)L * dk * sizeof(T);
    if (has_wr)
        b += (size_t)P * ks * sizeof(T);
    b = (b + 15) & ~(size_t)15;
    b += 8 * ((size_t)dk + L) * sizeof(float);
    return b;
}

template <typename T>
__global__ void __launch_bounds__(256) attn_fwd_kernel(AttnArgs a)
{
    extern __shared__ __align__(16) unsigned char smraw[];
    const int ks = SmemRow<T>::stride(a.dk);
    T *Ks = reinterpret_cast<T *>(smraw);
    T *Vs = Ks + (size_t)a.L * ks;
    T *Rs = Vs + (size_t)a.L * a.dk;
    size_t off = ((size_t)a.L * ks + (size_t)a.L * a.dk + (a.w_r ? (size_t)a.P * ks : 0)) * sizeof(T);
    off = (off + 15) & ~(size_t)15;
    float *fs = reinterpret_cast<float *>(smraw + off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *qf = fs + (size_t)warp * (a.dk + a.L);
    float *ps = qf + a.dk;

    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int HD = a.H * a.dk;
    const int i_first = a.t0 + blockIdx.y * a.qchunk;
    const int i_last = min(a.t1, i_first + a.qchunk) - 1;
    if (i_first > i_last)
        return;
    int jlo_all, jhi_all, tmp;
    key_range(a, i_first, jlo_all, tmp);
    key_range(a, i_last, tmp, jhi_all);

    const T *kv = reinterpret_cast<const T *>(a.kv);
    const int nj = jhi_all - jlo_all + 1;
    for (int idx = threadIdx.x; idx < nj * a.dk; idx += blockDim.x) {
        int j = jlo_all + idx / a.dk, e = idx % a.dk;
        const T *src = kv + ((size_t)j * a.B + b) * a.kvp + h * a.dk + e;
        Ks[(size_t)j * ks + e] = src[0];
        Vs[(size_t)j * a.dk + e] = src[HD];
    }
    if (a.w_r) {
        for (int idx = threadIdx.x; idx < a.P * a.dk; idx += blockDim.x) {
            int p = idx / a.dk, e = idx % a.dk;
            Rs[(size_t)p * ks + e] = from_f<T>(a.w_r[((size_t)h * a.P + p) * a.dk + e]);
        }
    }
    __syncthreads();

    const T *q = reinterpret_cast<const T *>(a.q);
    T *o = reinterpret_cast<T *>(a.o);
    for (int i = i_first + warp; i <= i_last; i += 8) {
        const T *qi = q + ((size_t)i * a.B + b) * a.qp + h * a.dk;
        for (int e = lane; e < a.dk; e += 32)
            qf[e] = to_f(qi[e]);
        __syncwarp();
        int jlo, jhi;
        key_range(a, i, jlo, jhi);
        float mx = -INFINITY;
        for (int j = jlo + lane; j <= jhi; j += 32) {
            float s = score_ij<T>(a, h, i, j, qf, Ks, Rs, ks);
            ps[j] = s;
            mx = fmaxf(mx, s);
        }
        mx = warp_max(mx);
        float sum = 0.0f;
        for (int j = jlo + lane; j <= jhi; j += 32) {
            float p = expf(ps[j] - mx);
            ps[j] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float rs = 1.0f / sum;
        __syncwarp();
        for (int e = lane; e < a.dk; e += 32) {
            float acc = 0.0f;
            for (int j = jlo; j <= jhi; j++)
                acc = fmaf(ps[j] * rs, to_f(Vs[(size_t)j * a.dk + e]), acc);
            o[((size_t)i * a.B + b) * HD + h * a.dk + e] = from_f<T>(acc);
        }
        if (lane == 0 && a.lse)
            a.lse[((size_t)b * a.H + h) * a.T + i] = mx + logf(sum);
        __syncwarp();
    }
}

template <typename T>
size_t attn_bwd_smem(int T_, int L, int P, int dk, bool has_wr)
{
    int ks = SmemRow<T>::stride(dk);
    size_t b = (size_t)L * ks * sizeof(T) + (size_t)L * dk * sizeof(T);
    if (has_wr)
        b += (size_t)P * ks * sizeof(T);
    b = (b + 15) & ~(size_t)15;
    b += ((size_t)2 * T_ * dk + (size_t)2 * T_ * (L + 1) + T_) * sizeof(float);
    return b;
}

template <typename T>
__global__ void __launch_bounds__(256) attn_bwd_kernel(AttnArgs a)
{
    extern __shared__ __align__(16) unsigned char smraw[];
    const int ks = SmemRow<T>::stride(a.dk);
    const int Tn = a.T, L = a.L, dk = a.dk, P = a.P, M = a.M;
    T *Ks = reinterpret_cast<T *>(smraw);
    T *Vs = Ks + (size_t)L * ks;
    T *Rs = Vs + (size_t)L * dk;
    size_t off = ((size_t)L * ks + (size_t)L * dk + (a.w_r ? (size_t)P * ks : 0)) * sizeof(T);
    off = (off + 15) & ~(size_t)15;
    float *qs = reinterpret_cast<float *>(smraw + off); // [T][dk]
    float *dos = qs + (size_t)Tn * dk;                  // [T][dk]
    float *Pm = dos + (size_t)Tn * dk;                  // [T][L+1]
    float *dS = Pm + (size_t)Tn * (L + 1);              // [T][L+1]
    float *Dr = dS + (size_t)Tn * (L + 1);              // [T]
    const int ls = L + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int HD = a.H * dk;

    const T *kv = reinterpret_cast<const T *>(a.kv);
    const T *q = reinterpret_cast<const T *>(a.q);
    const T *outp = reinterpret_cast<const T *>(a.out);
    const T *dout = reinterpret_cast<const T *>(a.dout);
    for (int idx = threadIdx.x; idx < L * dk; idx += blockDim.x) {
        int j = idx / dk, e = idx % dk;
        const T *src = kv + ((size_t)j * a.B + b) * a.kvp + h * dk + e;
        Ks[(size_t)j * ks + e] = src[0];
        Vs[(size_t)j * dk + e] = src[HD];
    }
    if (a.w_r)
        for (int idx = threadIdx.x; idx < P * dk; idx += blockDim.x) {
            int p = idx / dk, e = idx % dk;
            Rs[(size_t)p * ks + e] = from_f<T>(a.w_r[((size_t)h * P + p) * dk + e]);
        }
    for (int idx = threadIdx.x; idx < Tn * dk; idx += blockDim.x) {
        int i = idx / dk, e = idx % dk;
        qs[idx] = to_f(q[((size_t)i * a.B + b) * a.qp + h * dk + e]);
        dos[idx] = to_f(dout[((size_t)i * a.B + b) * HD + h * dk + e]);
    }
    for (int idx = threadIdx.x; idx < Tn * ls; idx += blockDim.x) {
        Pm[idx] = 0.0f;
        dS[idx] = 0.0f;
    }
    __syncthreads();
    // D_i = dO_i . O_i  (= sum_j P_ij dP_ij)
    for (int i = warp; i < Tn; i += 8) {
        float s = 0.0f;
        for (int e = lane; e < dk; e += 32)
            s += dos[(size_t)i * dk + e] * to_f(outp[((size_t)i * a.B + b) * HD + h * dk + e]);
        s = warp_sum(s);
        if (lane == 0)
            Dr[i] = s;
    }
    __syncthreads();
    // P and dS
    for (int i = warp; i < Tn; i += 8) {
        int jlo, jhi;
        key_range(a, i, jlo, jhi);
        const float lse = a.lse[((size_t)b * a.H + h) * Tn + i];
        const float *qf = qs + (size_t)i * dk, *dof = dos + (size_t)i * dk;
        for (int j = jlo + lane; j <= jhi; j += 32) {
            float s = score_ij<T>(a, h, i, j, qf, Ks, Rs, ks);
            float p = expf(s - lse);
            float dp = 0.0f;
            for (int e = 0; e < dk; e++)
                dp = fmaf(dof[e], to_f(Vs[(size_t)j * dk + e]), dp);
            Pm[(size_t)i * ls + j] = p;
            dS[(size_t)i * ls + j] = p * (dp - Dr[i]) * a.inv_sqrt;
        }
    }
    __syncthreads();
    // dV[j] = sum_i P_ij dO_i ; dK[j] = sum_i dS_ij q_i     (i ascending)
    T *dkv = reinterpret_cast<T *>(a.dkv);
    for (int idx = threadIdx.x; idx < L * dk; idx += blockDim.x) {
        int j = idx / dk, e = idx % dk;
        float av = 0.0f, ak = 0.0f;
        for (int i = max(0, j - M); i < Tn; i++) {
            av = fmaf(Pm[(size_t)i * ls + j], dos[(size_t)i * dk + e], av);
            ak = fmaf(dS[(size_t)i * ls + j], qs[(size_t)i * dk + e], ak);
        }
        T *dst = dkv + ((size_t)j * a.B + b) * a.dkvp + h * dk + e;
        dst[0] = from_f<T>(ak);
        dst[HD] = from_f<T>(av);
    }
    // dQ[i] = sum_j dS_ij (k_j + w_r[pi(i,j)])               (j ascending)
    T *dq = reinterpret_cast<T *>(a.dq);
    for (int idx = threadIdx.x; idx < Tn * dk; idx += blockDim.x) {
        int i = idx / dk, e = idx % dk;
        int jlo, jhi;
        key_range(a, i, jlo, jhi);
        float acc = 0.0f;
        for (int j = jlo; j <= jhi; j++) {
            float w = to_f(Ks[(size_t)j * ks + e]);
            if (a.w_r) {
                int pi = j + (Tn - 1) - i - (L - P);
                pi = pi < 0 ? 0 : pi;
                w += to_f(Rs[(size_t)pi * ks + e]);
            }
            acc = fmaf(dS[(size_t)i * ls + j], w, acc);
        }
        dq[((size_t)i * a.B + b) * a.dqp + h * dk + e] = from_f<T>(acc);
    }
    // table gradients of this (stream, head): slot r collects pairs (i, j = r-(T-1-i))
    if (a.w_r && a.dwr_part) {
        float *dst = a.dwr_part + ((size_t)b * a.H + h) * P * dk;
        for (int idx = threadIdx.x; idx < P * dk; idx += blockDim.x) {
            int p = idx / dk, e = idx % dk;
            int rlo = (p == 0) ? 0 : p + (L - P), rhi = p + (L - P);
            float acc = 0.0f;
            for (int r = rlo; r <= rhi; r++)
                for (int i = 0; i < Tn; i++) {
                    int j = r - (Tn - 1 - i);
                    if (j >= 0 && j < L)
                        acc = fmaf(dS[(size_t)i * ls + j], qs[(size_t)i * dk + e], acc);
                }
            dst[idx] = acc;
        }
    }
    if (a.dbr_part) {
        float *dst = a.dbr_part + ((size_t)b * a.H + h) * L;
        for (int r = threadIdx.x; r < L; r += blockDim.x) {
            float acc = 0.0f;
            for (int i = 0; i < Tn; i++) {
                int j = r - (Tn - 1 - i);
                if (j >= 0 && j < L)
                    acc += dS[(size_t)i * ls + j];
            }
            dst[r] = acc * a.br_scale;
        }
    }
}

// table[h][x] (+)= sum over streams b (ascending) of part[b][h][x]
__global__ void reduce_streams_kernel(const float *__restrict__ part, int B, size_t per_stream,
                                      float *__restrict__ out, int accumulate)
{
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per_stream)
        return;
    float s = 0.0f;
    for (int b = 0; b < B; b++)
        s += part[(size_t)b * per_stream + i];
    out[i] = accumulate ? out[i] + s : s;
}

static int attn_check_shape(const nncu_attn_shape *s)
{
    if (!s || s->n_streams < 1 || s->n_head < 1 || s->d_key < 1 || s->seg_len < 1 ||
        s->mem_len < 0 || s->d_pos < 1 || s->d_pos > s->mem_len + s->seg_len || s->t0 < 0 ||
        s->t1 > s->seg_len || s->t0 >= s->t1 || s->attn_len < 0 ||
        s->attn_len > s->mem_len + s->seg_len)
        return nncu_fail(NNCU_ERR_INVALID, "attention: bad shape");
    if (s->dtype_bf16 && (s->d_key & 1))
        return nncu_fail(NNCU_ERR_INVALID, "attention: bf16 needs an even d_key");
    return NNCU_OK;
}

// row pitches when q / kv / dq / dkv are column ranges of wider buffers (0 = packed)
struct AttnPitch {
    int qp, kvp, dqp, dkvp;
};

static AttnArgs attn_args(const nncu_attn_shape *s, const AttnPitch *pt = nullptr)
{
    AttnArgs a;
    memset(&a, 0, sizeof(a));
    a.B = s->n_streams; a.H = s->n_head; a.dk = s->d_key; a.T = s->seg_len; a.M = s->mem_len;
    a.L = s->mem_len + s->seg_len; a.P = s->d_pos;
    a.attn_len = s->attn_len ? s->attn_len : a.L;
    a.t0 = s->t0; a.t1 = s->t1;
    a.br_scale = s->br_scale;
    a.inv_sqrt = 1.0f / sqrtf((float)s->d_key);
    a.qp = a.dqp = a.H * a.dk;
    a.kvp = a.dkvp = 2 * a.H * a.dk;
    if (pt) {
        if (pt->qp) a.qp = pt->qp;
        if (pt->kvp) a.kvp = pt->kvp;
        if (pt->dqp) a.dqp = pt->dqp;
        if (pt->dkvp) a.dkvp = pt->dkvp;
    }
    return a;
}

template <typename T>
static int attn_forward_t(const nncu_attn_shape *s, const void *q, const void *kv, const float *w_r,
                          const float *b_r, void *out, float *lse, cudaStream_t st,
                          const AttnPitch *pt = nullptr)
{
    AttnArgs a = attn_args(s, pt);
    a.q = q; a.kv = kv; a.w_r = w_r; a.b_r = b_r; a.o = out; a.lse = lse;
    const int nq = a.t1 - a.t0;
    // enough CTAs to fill the GPU, but at least 8 queries (one per warp) per CTA
    int chunks = max(1, min(ceil_div(nq, 8), ceil_div(2 * 148, a.B * a.H)));
    a.qchunk = ceil_div(nq, chunks);
    chunks = ceil_div(nq, a.qchunk);
    size_t smem = attn_fwd_smem<T>(a.L, a.P, a.dk, w_r != nullptr);
    if (smem > 227 * 1024)
        return nncu_fail(NNCU_ERR_RANGE, "attention forward: %zu bytes of shared memory needed", smem);
    CUDA_TRY(cudaFuncSetAttribute(attn_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_fwd_kernel<T><<<dim3(a.B * a.H, chunks), 256, smem, st>>>(a);
    KERNEL_CHECK();
    return NNCU_OK;
}

template <typename T>
static int attn_backward_t(const nncu_attn_shape *s, const void *q, const void *kv,
                           const float *w_r, const float *b_r, const void *out, const float *lse,
                           const void *dout, void *dq, void *dkv, float *dwr_part,
                           float *dbr_part, cudaStream_t st, const AttnPitch *pt = nullptr)
{
    AttnArgs a = attn_args(s, pt);
    if (a.t0 != 0 || a.t1 != a.T)
        return nncu_fail(NNCU_ERR_INVALID, "attention backward runs over the whole segment");
    a.q = q; a.kv = kv; a.w_r = w_r; a.b_r = b_r; a.out = out; a.lse = const_cast<float *>(lse);
    a.dout = dout; a.dq = dq; a.dkv = dkv; a.dwr_part = dwr_part; a.dbr_part = dbr_part;
    size_t smem = attn_bwd_smem<T>(a.T, a.L, a.P, a.dk, w_r != nullptr);
    if (smem > 227 * 1024)
        return nncu_fail(NNCU_ERR_RANGE, "attention backward: %zu bytes of shared memory needed", smem);
    CUDA_TRY(cudaFuncSetAttribute(attn_bwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_bwd_kernel<T><<<a.B * a.H, 256, smem, st>>>(a);
    KERNEL_CHECK();
    return NNCU_OK;
}
