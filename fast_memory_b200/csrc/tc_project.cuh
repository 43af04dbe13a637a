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
};

struct TcParams {
    const TcSeg *segs;
    int n_seg;
    int n_ranges;          // key ranges per bucket tile
    // dense epilogue
    float *Y;              // row = global bucket, column = key of the segment
    int64_t ldy;
    // candidate epilogue
    const float *tau;      // [total buckets] threshold of every bucket
    uint2 *cand;           // [total buckets][cap] (score bits, key index local to the segment); one buffer of
                           // cap / n_ranges slots per range, filled upward by epilogue group 0 (even tiles of the
                           // range) and downward by group 1 (odd tiles)
    int cap;
    int *cand_count;       // [total buckets][n_ranges][2]; cap / n_ranges + 1 marks an overflow
    int *status;           // set non-zero when a wait gave up
};

// units = (total bucket tiles) * n_ranges CTAs
int tc_project_launch(const CUtensorMap &tmA, const CUtensorMap &tmK, const TcParams &p, int units, int d, bool dense, bool bf16,
                      cudaStream_t st);

}  // namespace fm
