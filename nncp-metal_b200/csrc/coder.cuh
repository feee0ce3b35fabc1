// coder.cuh -- coder-ready output: turns a row of fp32 probabilities into the
// 15-bit prob0 values that write_sym / read_sym (cp_utils.c:299-349) hand to the
// range coder, with the float arithmetic of those functions reproduced bit for
// bit:
//   p0    = vec_sum_f32(left half)      one node of a bottom-up pairwise fp32 tree
//   prob0 = clamp(lrintf(p0 * 32768 / p), 1, 32767)
//   p     <- p0 (bit 0)  or  p - p0 (bit 1),  starting from p = 1.0f at the root
// When V is a power of two the halving recursion of vec_sum_f32 is exactly the
// heap-ordered tree  S[k] = S[2k] + S[2k+1], leaves S[V+i] = prob[i].  For any
// other V (a word dictionary's alphabet) the recursion still is a binary tree in
// heap order, complete down to depth L-1 (L = ceil(log2 V)), whose nodes there
// cover one symbol (a leaf) or two (the last split): the *_any kernels below.
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

// The same values for V = 1024 .. 16384 without building the tree in shared memory: the row is
// read once (coalesced float4), the pairwise sums run through registers, warp shuffles and a
// 128-entry heap, and a thread that holds the left child of a node on the symbol's path drops it
// into p0s[depth].  Nodes carry their heap index K (root 1, children 2K and 2K+1, leaf i = V+i),
// so "left child of the path node at depth d" is K == 2 * ((V + sym) >> (L - d)).  Every sum is
// S[2K] + S[2K+1] of the same heap as build_sum_tree (fp32 addition commutes, so which of the two
// lanes adds first does not matter): the results are bit-identical to coder_paths_kernel.
__global__ void __launch_bounds__(256)
coder_paths_fast_kernel(const float *__restrict__ probs, const int32_t *__restrict__ sym,
                        uint16_t *__restrict__ out, int V, int n_bits)
{
    __shared__ float heap[256]; // top of the tree: entries [1, 2*NW), NW = V/128 <= 128
    __shared__ float p0s[16];
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int L = n_bits, nv4 = V >> 10, NW = V >> 7;
    int s = sym[row];
    s = s < 0 ? 0 : (s >= V ? V - 1 : s);
    const unsigned leafK = (unsigned)(V + s);
    auto keep = [&](unsigned K, float v) { // K: heap index of a node at depth d+1
        const int d = 30 - __clz((int)K);  // floor(log2 K) - 1 = depth of its parent
        if (!(K & 1u) && (K >> 1) == (leafK >> (L - d)))
            p0s[d] = v;
    };
    const float4 *pr = reinterpret_cast<const float4 *>(probs + (size_t)row * V);
#pragma unroll
    for (int j = 0; j < 16; j++) {
        if (j < nv4) {
            const unsigned g = (unsigned)(j * 256 + tid);
            const float4 q = pr[g];
            keep((unsigned)V + 4u * g, q.x); // a leaf that is a left child
            keep((unsigned)V + 4u * g + 2u, q.z);
            const float a = __fadd_rn(q.x, q.y), b = __fadd_rn(q.z, q.w);
            keep((unsigned)(V >> 1) + 2u * g, a);
            float v = __fadd_rn(a, b);
            keep((unsigned)(V >> 2) + g, v);
#pragma unroll
            for (int q2 = 1; q2 <= 5; q2++) {
                v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1 << (q2 - 1)));
                if ((lane & ((1 << q2) - 1)) == 0)
                    keep((unsigned)(V >> (2 + q2)) + (g >> q2), v);
            }
            if (lane == 0)
                heap[NW + j * 8 + w] = v; // depth log2(NW): node NW + (g >> 5)
        }
    }
    __syncthreads();
    if (w == 0) {
        for (int n = NW >> 1; n >= 1; n >>= 1) {
            for (int k = n + lane; k < 2 * n; k += 32) {
                const float v = __fadd_rn(heap[2 * k], heap[2 * k + 1]);
                heap[k] = v;
                if (k > 1)
                    keep((unsigned)k, v);
            }
            __syncwarp();
        }
        if (lane == 0) {
            float p = 1.0f;
            for (int lvl = 0; lvl < n_bits; lvl++) {
                const float p0 = p0s[lvl];
                out[(size_t)row * n_bits + lvl] = (uint16_t)prob0_of(p0, p);
                const int bit = (s >> (n_bits - 1 - lvl)) & 1;
                p = bit ? __fsub_rn(p, p0) : p0;
            }
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

// ---------------------------------------------------------------- any alphabet size
// write_sym splits a range of n symbols into n >> 1 on the left and the rest on the right, and
// vec_sum_f32 sums by the same halving, so node k of the heap (root 1, children 2k, 2k+1) covers
// the range found by following the bits of k below its leading one.  With P = 2^L >= V > P/2,
// every node above depth L-1 covers at least two symbols and every node at depth L-1 one or two.

// the range [lo, lo + n) of heap node k
__device__ __forceinline__ void node_range(unsigned k, int V, int &lo, int &n)
{
    lo = 0;
    n = V;
    for (int b = 30 - __clz((int)k); b >= 0; b--) {
        const int h = n >> 1;
        if ((k >> b) & 1u) {
            lo += h;
            n -= h;
        } else {
            n = h;
        }
    }
}

// S[1..2P): sums of the nodes; a one-symbol node at depth L-1 has no children (their slots are 0)
__device__ __forceinline__ void build_sum_tree_any(float *S, const float *__restrict__ prob, int V, int P)
{
    for (int k = (P >> 1) + threadIdx.x; k < P; k += blockDim.x) {
        int lo, n;
        node_range((unsigned)k, V, lo, n);
        if (n == 2) {
            const float a = prob[lo], b = prob[lo + 1];
            S[2 * k] = a;
            S[2 * k + 1] = b;
            S[k] = __fadd_rn(a, b);
        } else {
            S[2 * k] = 0.0f;
            S[2 * k + 1] = 0.0f;
            S[k] = prob[lo];
        }
    }
    __syncthreads();
    for (int n = P >> 2; n >= 1; n >>= 1) {
        for (int k = n + threadIdx.x; k < 2 * n; k += blockDim.x)
            S[k] = __fadd_rn(S[2 * k], S[2 * k + 1]);
        __syncthreads();
    }
}

// one block per row: the prob0 values on the path of sym[row], root first, L entries per row; a
// symbol whose leaf sits at depth L-1 uses L-1 of them and the last is 0
__global__ void __launch_bounds__(256)
coder_paths_any_kernel(const float *__restrict__ probs, const int32_t *__restrict__ sym,
                       uint16_t *__restrict__ out, int V, int P, int L)
{
    extern __shared__ float S[];
    const int row = blockIdx.x;
    build_sum_tree_any(S, probs + (size_t)row * V, V, P);
    if (threadIdx.x == 0) {
        int s = sym[row];
        s = s < 0 ? 0 : (s >= V ? V - 1 : s);
        float p = 1.0f;
        int k = 1, lo = 0, n = V, lvl = 0;
        while (n > 1 && lvl < L) {
            const int h = n >> 1;
            const float p0 = S[2 * k];
            out[(size_t)row * L + lvl++] = (uint16_t)prob0_of(p0, p);
            if (s >= lo + h) {
                lo += h;
                n -= h;
                p = __fsub_rn(p, p0);
                k = 2 * k + 1;
            } else {
                n = h;
                p = p0;
                k = 2 * k;
            }
        }
        for (; lvl < L; lvl++)
            out[(size_t)row * L + lvl] = 0;
    }
}

// one block per row: prob0 of every internal node in heap order, P entries per row (entry 0 and the
// one-symbol nodes of depth L-1 hold 0)
__global__ void __launch_bounds__(256)
coder_trees_any_kernel(const float *__restrict__ probs, uint16_t *__restrict__ out, int V, int P)
{
    extern __shared__ float S[];
    const int row = blockIdx.x;
    build_sum_tree_any(S, probs + (size_t)row * V, V, P);
    uint16_t *o = out + (size_t)row * P;
    if (threadIdx.x == 0) {
        S[1] = 1.0f; // running mass p at the root
        o[0] = 0;
    }
    __syncthreads();
    for (int n = 1; n < P; n <<= 1) {
        for (int k = n + threadIdx.x; k < 2 * n; k += blockDim.x) {
            bool split = true;
            if (2 * n == P) { // depth L-1: one symbol or two
                int lo, cnt;
                node_range((unsigned)k, V, lo, cnt);
                split = cnt == 2;
            }
            const float p = S[k], p0 = S[2 * k];
            o[k] = split ? (uint16_t)prob0_of(p0, p) : (uint16_t)0;
            S[2 * k + 1] = __fsub_rn(p, p0); // p(right); p(left) = p0 is already in S[2k]
        }
        __syncthreads();
    }
}
