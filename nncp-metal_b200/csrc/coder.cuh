// coder.cuh -- coder-ready output: turns a row of fp32 probabilities into the
// 15-bit prob0 values that write_sym / read_sym (cp_utils.c:299-349) hand to the
// range coder, with the float arithmetic of those functions reproduced bit for
// bit:
//   p0    = vec_sum_f32(left half)      one node of a bottom-up pairwise fp32 tree
//   prob0 = clamp(lrintf(p0 * 32768 / p), 1, 32767)
//   p     <- p0 (bit 0)  or  p - p0 (bit 1),  starting from p = 1.0f at the root
// V must be a power of two: then the halving recursion of vec_sum_f32 is exactly
// the heap-ordered tree  S[k] = S[2k] + S[2k+1], leaves S[V+i] = prob[i].
#pragma once
#include "common.cuh"

// `int prob0 = lrintf(x)` as x86-64 computes it: lrintf returns a 64-bit long
// (cvtss2si: round half to even; LONG_MIN for NaN or anything outside int64), and
// the assignment keeps its low 32 bits.  Only reachable when the running mass p
// has collapsed to ~0 by cancellation, but encoder and decoder must agree there too.
__device__ __forceinline__ int prob0_of(float p0, float p)
{
    float x = __fdiv_rn(__fmul_rn(p0, 32768.0f), p);
    long long v64;
    if (!(fabsf(x) < 9.2233720368547758e18f))
        v64 = LLONG_MIN;
    else
        v64 = __float2ll_rn(x);
    int v = (int)(unsigned int)(unsigned long long)v64;
    return v < 1 ? 1 : (v > 32767 ? 32767 : v);
}

// builds S[1..2V) in shared memory from one row of probabilities
__device__ __forceinline__ void build_sum_tree(float *S, const float *__restrict__ prob, int V)
{
    for (int i = threadIdx.x; i < V; i += blockDim.x)
        S[V + i] = prob[i];
    __syncthreads();
    for (int n = V >> 1; n >= 1; n >>= 1) {
        for (int k = n + threadIdx.x; k < 2 * n; k += blockDim.x)
            S[k] = __fadd_rn(S[2 * k], S[2 * k + 1]);
        __syncthreads();
    }
}

// one block per row: the prob0 values on the root-to-leaf path of sym[row]
__global__ void __launch_bounds__(256)
coder_paths_kernel(const float *__restrict__ probs, const int32_t *__restrict__ sym,
                   uint16_t *__restrict__ out, int V, int n_bits)
{
    extern __shared__ float S[];
    const int row = blockIdx.x;
    build_sum_tree(S, probs + (size_t)row * V, V);
    if (threadIdx.x == 0) {
        int s = sym[row];
        s = s < 0 ? 0 : (s >= V ? V - 1 : s);
        float p = 1.0f;
        int k = 1;
        for (int lvl = 0; lvl < n_bits; lvl++) {
            float p0 = S[2 * k];
            out[(size_t)row * n_bits + lvl] = (uint16_t)prob0_of(p0, p);
            int bit = (s >> (n_bits - 1 - lvl)) & 1;
            p = bit ? __fsub_rn(p, p0) : p0;
            k = 2 * k + bit;
        }
    }
}

// one block per row: prob0 of every internal node, heap order, entry 0 unused
__global__ void __launch_bounds__(256)
coder_trees_kernel(const float *__restrict__ probs, uint16_t *__restrict__ out, int V)
{
    extern __shared__ float S[];
    const int row = blockIdx.x;
    build_sum_tree(S, probs + (size_t)row * V, V);
    uint16_t *o = out + (size_t)row * V;
    if (threadIdx.x == 0) {
        S[1] = 1.0f; // running mass p at the root
        o[0] = 0;
    }
    __syncthreads();
    // top-down: slot k holds p(k) once its parent has been processed
    for (int n = 1; n < V; n <<= 1) {
        for (int k = n + threadIdx.x; k < 2 * n; k += blockDim.x) {
            float p = S[k], p0 = S[2 * k];
            o[k] = (uint16_t)prob0_of(p0, p);
            S[2 * k + 1] = __fsub_rn(p, p0); // p(right); p(left) = p0 is already in S[2k]
        }
        __syncthreads();
    }
}
