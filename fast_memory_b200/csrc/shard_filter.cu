// Shard filter + compaction of a globally indexed bucket table.
// Stands in for the range mask / per-row count / boolean compaction / rebase of the reference
// (memory.py:128-142): keep the entries of every (head, bucket) row whose global key index lies in
// [lo, hi), rebased to the shard (index - lo), in their original slot order, packed (head, bucket, slot).
#include "common.cuh"

namespace fm {

__global__ void exclusive_scan_kernel(const int32_t *in, int n, int32_t *out, int32_t *cursor);   // group_rows.cu

// One warp per (head, bucket) row of the [C, H, Z] table.
__global__ void shard_count_kernel(const int64_t *__restrict__ k_hashes, int C, int H, int Z, int64_t lo, int64_t hi,
                                   int32_t *__restrict__ counts, int64_t *__restrict__ counts_out)
{
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);       // row = h * C + c
    if (row >= H * C) return;
    const int lane = threadIdx.x & 31, h = row / C, c = row - h * C;
    const int64_t *src = k_hashes + (size_t(c) * H + h) * Z;
    int n = 0;
    for (int z = lane; z < Z; z += 32) {
        const int64_t idx = src[z];
        n += (idx >= lo && idx < hi) ? 1 : 0;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) n += __shfl_xor_sync(0xffffffffu, n, off);
    if (lane == 0) { counts[row] = n; counts_out[row] = n; }
}

__global__ void shard_compact_kernel(const int64_t *__restrict__ k_hashes, int C, int H, int Z, int64_t lo, int64_t hi,
                                     const int32_t *__restrict__ offsets, int64_t *__restrict__ flat_out)
{
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= H * C) return;
    const int lane = threadIdx.x & 31, h = row / C, c = row - h * C;
    const int64_t *src = k_hashes + (size_t(c) * H + h) * Z;
    int64_t *dst = flat_out + offsets[row];
    int base = 0;
    for (int z0 = 0; z0 < Z; z0 += 32) {
        const int z = z0 + lane;
        const int64_t idx = z < Z ? src[z] : -1;
        const bool keep = z < Z && idx >= lo && idx < hi;
        const unsigned bal = __ballot_sync(0xffffffffu, keep);
        if (keep) dst[base + __popc(bal & ((1u << lane) - 1u))] = idx - lo;
        base += __popc(bal);
    }
}

}  // namespace fm

extern "C" size_t fm_shard_filter_workspace_bytes(int64_t C, int64_t H)
{
    return fm::align_up(size_t(C * H) * 4, 256) + fm::align_up(size_t(C * H + 1) * 4, 256);
}

extern "C" int fm_shard_filter(const int64_t *k_hashes, int64_t C, int64_t H, int64_t Z, int64_t lo, int64_t hi,
                               int64_t *flat_out, int64_t *counts_out, void *workspace, size_t workspace_bytes, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(k_hashes && flat_out && counts_out && workspace, "fm_shard_filter: null pointer");
    FM_REQUIRE(C > 0 && H > 0 && Z > 0 && lo <= hi, "fm_shard_filter: bad sizes");
    FM_REQUIRE(C * H * Z < (int64_t(1) << 31), "fm_shard_filter: table exceeds int32 offsets");
    if (workspace_bytes < fm_shard_filter_workspace_bytes(C, H)) {
        set_error("fm_shard_filter: workspace %zu too small", workspace_bytes);
        return FM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    int32_t *counts = (int32_t *)workspace;
    int32_t *offsets = (int32_t *)((char *)workspace + align_up(size_t(C * H) * 4, 256));
    const unsigned blocks = (unsigned)ceil_div(C * H, 8);
    shard_count_kernel<<<blocks, 256, 0, st>>>(k_hashes, (int)C, (int)H, (int)Z, lo, hi, counts, counts_out);
    FM_LAUNCHED("shard_count_kernel");
    exclusive_scan_kernel<<<1, 1024, 0, st>>>(counts, (int)(C * H), offsets, nullptr);
    FM_LAUNCHED("exclusive_scan_kernel");
    shard_compact_kernel<<<blocks, 256, 0, st>>>(k_hashes, (int)C, (int)H, (int)Z, lo, hi, offsets, flat_out);
    FM_LAUNCHED("shard_compact_kernel");
    return FM_OK;
}
