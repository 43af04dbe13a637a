// Interface between the index-build driver (index_build.cu) and the fused tensor-core path (index_fused.cu).
#pragma once

#include "common.cuh"

namespace fm {

constexpr int kFusedMaxCap = 25000;        // candidate slots per bucket the selection can deal out to its threads
constexpr size_t kFusedMaxSelSmem = 208u << 10;   // dynamic shared memory the selection may ask for (beside ~17 KB static)

struct FusedPlan {
    int step;                  // every step-th key is sampled for the threshold estimate
    int cap;                   // candidate slots per bucket
    int64_t max_keys;          // longest segment
    int64_t group_buckets;     // buckets processed per group of segments
    size_t sel_smem;           // dynamic shared memory of the selection kernel
    size_t off_status, off_segs, off_tcseg, off_tau, off_count, off_fail, off_cand, off_mask, off_yf, total;
};

// Can a segment of n_keys keys with buckets of zc keys take the fused path?
bool fused_eligible(int dtype, int d, int64_t n_keys, int64_t zc);
// Workspace layout for the listed (eligible) segments.
FusedPlan fused_plan(int n, const int64_t *n_keys, const int64_t *n_buckets, const int64_t *zc);
// Table rows of the listed segments; status word at ws + 0 (0 = ok).
int fused_index_build(const void *K, const void *A, int dtype, int d, int64_t total_key_rows, int64_t total_buckets, int n,
                      const int64_t *kb, const int64_t *nk, const int64_t *cb, const int64_t *nbk, const int64_t *zc,
                      const int64_t *table_off, int32_t *table, void *ws, bool single_range, cudaStream_t st);

}  // namespace fm
