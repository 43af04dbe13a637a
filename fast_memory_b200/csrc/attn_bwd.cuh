// Parameters shared by the two backward kernels of the hashed attention (hashed_attn_bwd.cu: CUDA cores, any
// element type and head dim; hashed_attn_bwd_mma.cu: mma.sync, 16-bit inputs with head dim 64 or 128).
#pragma once

#include "attn_common.cuh"

namespace fm {

struct BwdParams {
    const void *q, *k, *v, *o, *d_o;
    const float *lse;
    const void *table;
    int idx_bytes;
    const int64_t *bucket_off;
    const int32_t *bucket_kbase;
    const int32_t *group_off, *perm;
    int64_t n_k_rows;
    float sm_scale;
    float *dq, *dk, *dv;
};

// dtype FM_BF16 / FM_F16, d 64 / 128, every row 16-byte aligned
int launch_bwd_mma(const BwdParams &p, int dtype, int d, int64_t total_buckets, cudaStream_t st);

}  // namespace fm
