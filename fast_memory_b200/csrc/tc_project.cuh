// Interface of the tensor-core projection kernel (tc_project.cu) for the fused index build.
#pragma once

#include "tc_utils.cuh"

namespace fm {

constexpr int kTcBM = 128;                  // bucket rows per tile
constexpr int kTcBN = 256;                  // keys per tile

struct TcSeg {
    int a_row0;        // first row of A of this segment (tensor-map row)
    int n_buckets;
    int k_row0;        // first key row of this segment in the key tensor map's row coordinate
    int n_keys;        // columns of this segment's projection (keys, or sampled keys)
    int mtile0;        // index of the segment's first bucket tile in the global list
    int out_row0;      // row of the segment's first bucket in Y / tau / cand / cand_count
    int rank;          // threshold pass: which order statistic of the sample scores the threshold is (1 = largest)
};

struct TcParams {
    const TcSeg *segs;
    int n_seg;
    int n_ranges;          // key ranges per bucket tile
    // dense epilogue: scores in the blocked layout of dense_offset()
    float *Y;
    int64_t ldy;           // columns per row, a multiple of 32
    // candidate epilogue
    const float *tau;      // [total buckets] threshold of every bucket
    uint4 *cand;           // [total buckets][cap] groups of four scores (bits) of four consecutive keys, kept when any of
                           // the four reaches tau; one buffer of cap / n_ranges slots per range, filled upward by
                           // epilogue group 0 (first half of the range's tiles) and downward by group 1 (second half):
                           // both in ascending key order
    uint2 *cand_mask;      // [key tile of the segment][mask_ld] one bit per group of the tile (bit i = keys 4i .. 4i+3 of
                           // the tile): the groups that were appended, i.e. which keys the entries hold
    int64_t mask_ld;       // rows of cand_mask (>= total buckets)
    int cap;
    int *cand_count;       // [total buckets][n_ranges][2]; cap / n_ranges + 1 marks an overflow
    int *status;           // set non-zero when a wait gave up
    // how long a pipeline wait may take before the CTA gives up (0: the library's two seconds), and - a hook for the
    // test of that path only - the tile of every CTA whose load the producer leaves out (-1: none)
    uint64_t wait_limit_ns;
    int skip_tile;
};

// The test hooks above as set by fm_test_set_tc_hooks (process-wide, host side).
void tc_apply_test_hooks(TcParams &p);

// Dense scores are stored in blocks of 32 rows x 32 columns (4 KB); inside a block the element (r, c) sits at
// (c / 4) * 128 + r * 4 + c % 4, so that the 32 threads of an epilogue warp (one row each) write 512 contiguous
// bytes per instruction.  Blocks are ordered row-block major.  ldy = columns per row (multiple of 32); the
// array must cover rows rounded up to a multiple of 32.
__host__ __device__ inline size_t dense_block_offset(int64_t row, int64_t col, int64_t ldy)
{
    return (size_t(row >> 5) * size_t(ldy >> 5) + size_t(col >> 5)) * 1024;
}
__host__ __device__ inline size_t dense_offset(int64_t row, int64_t col, int64_t ldy)
{
    return dense_block_offset(row, col, ldy) + size_t((col & 31) >> 2) * 128 + size_t(row & 31) * 4 + size_t(col & 3);
}

// Thresholds straight from the projection of the key sample (tc_tau.cu): tau[row] = a lower bound, tight to 2^-15 of the
// row's score range, of the rank-th largest sample score of the bucket.  One CTA per bucket tile.
struct TauParams {
    const TcSeg *segs;     // k_row0 / n_keys in sampled rows
    int n_seg;
    float *tau;
    int *status;
    uint64_t wait_limit_ns;
};
int tc_tau_launch(const CUtensorMap &tmA, const CUtensorMap &tmKs, const TauParams &p, int mtiles, int d, bool bf16, cudaStream_t st);

// units = (total bucket tiles) * n_ranges CTAs
int tc_project_launch(const CUtensorMap &tmA, const CUtensorMap &tmK, const TcParams &p, int units, int d, bool dense, bool bf16,
                      cudaStream_t st);

}  // namespace fm
