// Work decomposition shared by the hashed-attention kernels.
//
// A work item is (bucket, block of <= kQB queries hashed to it, chunk of its key list).  Items are
// listed by a planning kernel and pulled by persistent CTAs through an atomic counter, so long and
// short buckets balance over the SMs.  When a bucket is cut into several key chunks every item writes
// an un-normalised partial (acc, m, l) per query and a combine kernel folds them.
#pragma once

#include "common.cuh"

namespace fm {

constexpr int kQB = 16;                    // queries per work item

struct AttnParams {
    const void *q, *k, *v;
    void *o;
    float *lse;
    const void *table;
    int idx_bytes;
    const int64_t *bucket_off;
    const int32_t *bucket_kbase;
    const int32_t *group_off;
    const int32_t *perm;
    int total_buckets;
    int n_q_rows;
    int64_t n_k_rows;
    int key_chunk;
    int nkc_max;
    float scale2;                          // sm_scale * log2(e)
    // workspace
    int *counters;                         // [0] = number of items, [1] = next item to hand out, [2] = a bucket longer than the
                                           // workspace was sized for, [3] = a bounded wait gave up; [8], [9] = the same pair as
                                           // [0], [1] for the list of items to serve again (`redo`)
    int4 *items;                           // {bucket, first query position, key chunk, chunks of the bucket}
    int max_items;
    int q_block;                            // queries per work item: 16 (CUDA-core kernel) or 32 (tensor-core kernel)
    int32_t *qparts;                       // per query position: number of partials to combine
    float *partials;                       // [query position][chunk][d + 2]
};

__device__ __forceinline__ int64_t load_index(const void *table, int idx_bytes, int64_t pos)
{
    return idx_bytes == 8 ? reinterpret_cast<const int64_t *>(table)[pos]
                          : int64_t(reinterpret_cast<const int32_t *>(table)[pos]);
}

struct AttnLayout {
    int key_chunk, nkc_max;
    int64_t max_items;
    size_t off_items, off_redo, off_qparts, off_partials, total;
};

inline AttnLayout attn_layout(int64_t n_q_rows, int64_t total_buckets, int64_t max_bucket_len, int d, int64_t key_chunk,
                              int sms)
{
    AttnLayout L;
    if (max_bucket_len < 1) max_bucket_len = 1;
    if (key_chunk <= 0) {
        // enough (bucket, query block) groups to fill the machine -> whole buckets; otherwise cut buckets
        // so that about 4 items per SM exist
        int64_t groups = std::max<int64_t>(1, std::min(total_buckets, n_q_rows));
        int64_t want = int64_t(4) * sms;
        if (groups >= want) key_chunk = max_bucket_len;
        else {
            int64_t parts = std::min<int64_t>(64, ceil_div(want, groups));
            key_chunk = std::max<int64_t>(256, ceil_div(ceil_div(max_bucket_len, parts), 64) * 64);
        }
    }
    key_chunk = std::min<int64_t>(std::max<int64_t>(key_chunk, 64), std::max<int64_t>(max_bucket_len, 64));
    L.key_chunk = (int)key_chunk;
    L.nkc_max = (int)ceil_div(max_bucket_len, key_chunk);
    L.max_items = (ceil_div(n_q_rows, kQB) + std::min(total_buckets, n_q_rows)) * L.nkc_max;
    size_t off = 256;                                      // counters
    L.off_items = off;
    off += align_up(size_t(L.max_items) * sizeof(int4), 256);
    L.off_redo = off;                                      // items the tcgen05 kernel hands back (same capacity)
    off += align_up(size_t(L.max_items) * sizeof(int4), 256);
    L.off_qparts = off;
    off += align_up(size_t(n_q_rows) * 4, 256);
    L.off_partials = off;
    if (L.nkc_max > 1) off += align_up(size_t(n_q_rows) * L.nkc_max * (d + 2) * sizeof(float), 256);
    L.total = off;
    return L;
}

}  // namespace fm
