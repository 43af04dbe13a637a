// Exact top-Z of one row of scores by a whole CTA of kSelThreads threads.
//
// Four 8-bit radix passes over the order-preserving keys find the Z-th largest key theta and how many
// entries equal to theta belong to the result; an ordered compaction then writes the selected indices in
// ascending order (entries > theta, and the first `want` entries == theta): lower index wins ties.
#pragma once

#include "common.cuh"

namespace fm {

constexpr int kSelThreads = 1024;

__device__ __forceinline__ void topz_row(const float *__restrict__ y, int64_t N, int Z, int32_t index_base,
                                         int32_t *__restrict__ out)
{
    __shared__ int hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_want;
    __shared__ int warp_gt[32], warp_eq[32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;

    if (t == 0) { s_prefix = 0; s_want = Z; }
    uint32_t mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (t < 256) hist[t] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int64_t j = t; j < N; j += kSelThreads) {
            uint32_t key = float_key(y[j]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
        }
        __syncthreads();
        if (t == 0) {
            int want = s_want, b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= want) break;
                want -= hist[b];
            }
            s_prefix = prefix | (uint32_t(b) << shift);
            s_want = want;
        }
        mask |= 255u << shift;
        __syncthreads();
    }
    const uint32_t theta = s_prefix;
    const int want = s_want;
    int gt_base = 0, eq_base = 0;
    for (int64_t j0 = 0; j0 < N; j0 += kSelThreads) {
        const int64_t j = j0 + t;
        uint32_t key = j < N ? float_key(y[j]) : 0u;
        const bool gt = j < N && key > theta;
        const bool eq = j < N && key == theta;
        const unsigned bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
        const unsigned lt_mask = (1u << lane) - 1u;
        int gt_ex = __popc(bg & lt_mask), eq_ex = __popc(be & lt_mask);
        if (lane == 0) { warp_gt[warp] = __popc(bg); warp_eq[warp] = __popc(be); }
        __syncthreads();
        if (warp == 0) {
            int g = warp_gt[lane], e = warp_eq[lane];
            int gi = g, ei = e;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                int tg = __shfl_up_sync(0xffffffffu, gi, off), te = __shfl_up_sync(0xffffffffu, ei, off);
                if (lane >= off) { gi += tg; ei += te; }
            }
            warp_gt[lane] = gi - g;
            warp_eq[lane] = ei - e;
            if (lane == 31) { hist[0] = gi; hist[1] = ei; }          // chunk totals
        }
        __syncthreads();
        gt_ex += gt_base + warp_gt[warp];
        eq_ex += eq_base + warp_eq[warp];
        if (gt || (eq && eq_ex < want)) {
            int pos = gt_ex + min(eq_ex, want);
            if (pos < Z) out[pos] = int32_t(j) + index_base;
        }
        gt_base += hist[0];
        eq_base += hist[1];
        __syncthreads();
    }
}

}  // namespace fm
