// decoder.cuh -- the range decoder on the device: one step's symbols are decoded from the trees
// that coder_trees_kernel left in device memory, so a decode step needs no host round trip.
//
// The arithmetic is get_bit / read_sym of the reference coder (arith.c:241-310,
// cp_utils.c:326-349) bit for bit: split = (range * prob0) >> 15, bit = low >= split,
// renormalisation one byte at a time while range < 0xFF01, zero bytes past the end of the input.
// The streams of one step share ONE bit stream, so their symbols decode strictly one after the
// other: a single thread walks the trees.  What can run ahead is the data movement: a ring of
// shared-memory slots is filled with the next streams' trees by bulk copies (2 V bytes each,
// completion on an mbarrier) while the current one is walked, and the payload bytes the step can
// consume at most (two per bit) are staged in shared memory by the whole warp up front.
//
// An alphabet that is not a power of two has the uneven tree of write_sym (a node of n symbols
// sends n >> 1 left): the walk then carries the node's range beside its heap index and ends when
// one symbol is left (template argument ANY); a tree row has P = 2^ceil(log2 V) entries.
#pragma once
#include "common.cuh"
#include "gemm_tc.cuh"

namespace dec {

struct State {
    unsigned long long pos, len; // next payload byte, payload size
    uint32_t low, range;
    int err, pad;
};

constexpr uint32_t R_LOW = (0xffu << 8) + 1u, R_TOP = 0xffu << 16;
constexpr int MAX_RING = 8, MAX_SMEM = 200 * 1024;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

// window bytes a step of `B` streams with `nb` bits per symbol can consume, as a multiple of 16
__host__ __device__ inline int window_bytes(int B, int nb) { return (2 * B * nb + 15) & ~15; }

// slots of the ring for trees of P entries (0: the trees do not fit)
inline int ring_slots(int B, int P, int nb)
{
    const long avail = (long)MAX_SMEM - window_bytes(B, nb) - 128;
    long n = avail / ((long)P * 2);
    if (P < 8 || n < 2)
        return 0;
    return (int)std::min<long>(n, MAX_RING);
}
inline size_t smem_bytes(int B, int P, int nb, int ring) { return (size_t)ring * P * 2 + window_bytes(B, nb) + 128; }

// trees: [B][P] prob0 in heap order (entry 0 unused), P = 2^nb >= V.  sym_out[b] and ids_next[b]
// (when not null) receive the decoded symbol, 0 for the streams past the end of the block: those at
// step `t` are b >= limit_b when t == limit_t, and all of them when t > limit_t.
template <bool ANY>
__global__ void __launch_bounds__(32)
decode_step_kernel(const uint16_t *__restrict__ trees, const uint8_t *__restrict__ payload, State *state,
                   int32_t *__restrict__ sym_out, int32_t *__restrict__ ids_next, int t, int limit_t, int limit_b,
                   int B, int V, int P, int nb, int ring, int *err_flag)
{
    extern __shared__ __align__(128) uint8_t dsm[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(dsm);           // [MAX_RING] of 8 bytes, 128 reserved
    uint16_t *slots = reinterpret_cast<uint16_t *>(dsm + 128);    // [ring][P]
    uint8_t *win = dsm + 128 + (size_t)ring * P * 2;              // payload window
    __shared__ int abort_s;
    const int lane = threadIdx.x;
    const int n_act = t < limit_t ? B : (t == limit_t ? min(limit_b, B) : 0);
    const uint32_t slot_bytes = (uint32_t)P * 2u;
    unsigned long long pos = state->pos;
    const unsigned long long len = state->len, pos0 = pos;
    uint32_t low = state->low, range = state->range;

    if (lane == 0) {
        abort_s = 0;
        for (int i = 0; i < ring; i++)
            tc::mbar_init(tc::smem_u32(bars + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (lane == 0) {
        for (int b = 0; b < ring && b < n_act; b++) {
            tc::mbar_expect_tx(tc::smem_u32(bars + b), slot_bytes);
            bulk_load(tc::smem_u32(slots + (size_t)b * P), trees + (size_t)b * P, slot_bytes, tc::smem_u32(bars + b));
        }
    }
    const int wbytes = window_bytes(B, nb);
    for (int i = lane; i < wbytes; i += 32)
        win[i] = (pos0 + i < len) ? payload[pos0 + i] : (uint8_t)0;
    __syncwarp();

    if (lane == 0) {
        bool ok = true;
        int issued = min(ring, n_act); // streams whose copy has been issued
        for (int b = 0; b < B; b++) {
            int c = 0;
            if (b < n_act && ok) {
                const int s = b % ring;
                ok = tc::mbar_wait(tc::smem_u32(bars + s), (uint32_t)((b / ring) & 1), &abort_s, err_flag, 41);
                if (ok) {
                    const uint16_t *tree = slots + (size_t)s * P;
                    int k = 1;
                    auto next_bit = [&]() { // get_bit at node k: the branch taken, low / range / pos advanced
                        const uint32_t prob0 = tree[k];
                        const uint32_t split = (uint32_t)(((unsigned long long)range * prob0) >> 15);
                        const bool bit = low >= split;
                        if (bit) {
                            low -= split;
                            range -= split;
                        } else {
                            range = split;
                        }
                        while (range < R_LOW) {
                            range <<= 8;
                            low <<= 8;
                            if (pos < len) {
                                low += win[pos - pos0];
                                pos++;
                            }
                        }
                        k = 2 * k + (bit ? 1 : 0);
                        return bit;
                    };
                    if constexpr (ANY) {
                        int lo = 0, n = V;
                        for (int lvl = 0; lvl < nb && n > 1; lvl++) {
                            const int h = n >> 1;
                            if (next_bit()) {
                                lo += h;
                                n -= h;
                            } else {
                                n = h;
                            }
                        }
                        c = lo;
                    } else {
                        for (int lvl = 0; lvl < nb; lvl++)
                            next_bit();
                        c = k - V;
                    }
                    if (issued < n_act) { // the slot just walked takes the tree of stream b + ring
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        tc::mbar_expect_tx(tc::smem_u32(bars + s), slot_bytes);
                        bulk_load(tc::smem_u32(slots + (size_t)s * P), trees + (size_t)issued * P, slot_bytes,
                                  tc::smem_u32(bars + s));
                        issued++;
                    }
                }
            }
            sym_out[b] = c;
            if (ids_next)
                ids_next[b] = c;
        }
        if (!ok) {
            // copies still in flight land in this CTA's shared memory: give each a bounded chance to finish
            for (int b2 = max(issued - ring, 0); b2 < issued; b2++)
                tc::mbar_wait(tc::smem_u32(bars + b2 % ring), (uint32_t)((b2 / ring) & 1), &abort_s, err_flag, 42);
            state->err = 1;
        }
        state->pos = pos;
        state->low = low;
        state->range = range;
    }
    __syncwarp();
}

} // namespace dec
