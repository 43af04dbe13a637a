// Grouping of rows by bucket: a counting sort (histogram, exclusive scan, scatter).
// Stands in for the stable sort / unique_consecutive / cumsum block of the reference wrapper
// (triton_kernel.py:75-88); empty buckets simply get an empty range.
#include "common.cuh"

#include <mutex>

namespace fm {

__device__ __forceinline__ int global_bucket(const int32_t *__restrict__ hash, int r, int n_seg,
                                             const int32_t *__restrict__ seg_xb, const int32_t *__restrict__ seg_cb)
{
    int h = hash[r];
    if (seg_xb == nullptr) return h;
    int s = find_segment(seg_xb, n_seg, r);
    return seg_cb[s] + h;
}

__global__ void bucket_histogram_kernel(const int32_t *__restrict__ hash, int n_rows, int total_buckets, int n_seg,
                                        const int32_t *__restrict__ seg_xb, const int32_t *__restrict__ seg_cb,
                                        int32_t *__restrict__ counts)
{
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
        int gb = global_bucket(hash, r, n_seg, seg_xb, seg_cb);
        if (gb >= 0 && gb < total_buckets) atomicAdd(&counts[gb], 1);
    }
}

// One CTA: out[i] = sum of in[0..i), out[n] = total; `cursor` (optional) receives a copy of out[0..n).
__global__ void __launch_bounds__(1024)
exclusive_scan_kernel(const int32_t *__restrict__ in, int n, int32_t *__restrict__ out, int32_t *__restrict__ cursor)
{
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        int i = base + threadIdx.x;
        int v = i < n ? in[i] : 0;
        int inc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += t;
        }
        if (lane == 31) warp_sums[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
            int winc = w;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                int t = __shfl_up_sync(0xffffffffu, winc, off);
                if (lane >= off) winc += t;
            }
            warp_sums[lane] = winc - w;                    // exclusive prefix of the warp totals
        }
        __syncthreads();
        int carry = carry_s;
        int excl = carry + warp_sums[warp] + inc - v;
        if (i < n) {
            out[i] = excl;
            if (cursor) cursor[i] = excl;
        }
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) out[n] = carry_s;
}

__global__ void bucket_scatter_kernel(const int32_t *__restrict__ hash, int n_rows, int total_buckets, int n_seg,
                                      const int32_t *__restrict__ seg_xb, const int32_t *__restrict__ seg_cb,
                                      int32_t *__restrict__ cursor, int32_t *__restrict__ perm)
{
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
        int gb = global_bucket(hash, r, n_seg, seg_xb, seg_cb);
        if (gb >= 0 && gb < total_buckets) perm[atomicAdd(&cursor[gb], 1)] = r;
    }
}

// ---- scratch that lives in the library image, for callers that must not allocate ---------------------
// Counts and cursors of fm_group_rows_static.  Every GPU that loads the library carries these 512 KiB
// until the process exits.
constexpr int kStaticMaxBuckets = 65536;
static __device__ __align__(256) int32_t g_static_group_scratch[2 * kStaticMaxBuckets];

// Device address of g_static_group_scratch on the current device.  In host code the symbol's name is
// only a handle for the runtime, never a pointer a kernel may be given, so the address is asked for
// once per device (with that device current) and remembered.
static int static_group_scratch(int32_t **out)
{
    static std::mutex mu;
    static int32_t *cached[64];
    int dev = -1;
    FM_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("fm_group_rows_static: device ordinal %d out of range", dev);
        return FM_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void *p = nullptr;
        FM_CUDA_OK(cudaGetSymbolAddress(&p, g_static_group_scratch));
        cached[dev] = static_cast<int32_t *>(p);
    }
    *out = cached[dev];
    return FM_OK;
}

}  // namespace fm

extern "C" size_t fm_group_rows_workspace_bytes(int64_t n_rows, int64_t total_buckets)
{
    (void)n_rows;
    return fm::align_up(size_t(total_buckets) * 4, 256) * 2;      // counts, cursor
}

extern "C" int fm_group_rows(const int32_t *hash, int64_t n_rows, int64_t total_buckets, int n_seg,
                             const int32_t *seg_xb, const int32_t *seg_cb, int32_t *group_off, int32_t *perm,
                             void *workspace, size_t workspace_bytes, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(group_off && workspace && (n_rows == 0 || (hash && perm)), "fm_group_rows: null pointer");
    FM_REQUIRE(n_rows >= 0 && total_buckets > 0 && n_seg >= 1, "fm_group_rows: bad sizes");
    FM_REQUIRE(n_rows < (int64_t(1) << 31) && total_buckets < (int64_t(1) << 31), "fm_group_rows: sizes exceed int32");
    FM_REQUIRE((seg_xb == nullptr) == (seg_cb == nullptr), "fm_group_rows: pass both segment arrays or neither");
    if (workspace_bytes < fm_group_rows_workspace_bytes(n_rows, total_buckets)) {
        set_error("fm_group_rows: workspace %zu < %zu", workspace_bytes, fm_group_rows_workspace_bytes(n_rows, total_buckets));
        return FM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    int32_t *counts = (int32_t *)workspace;
    int32_t *cursor = (int32_t *)((char *)workspace + align_up(size_t(total_buckets) * 4, 256));
    FM_CUDA_OK(cudaMemsetAsync(counts, 0, size_t(total_buckets) * 4, st));
    int blocks = (int)std::min<int64_t>(std::max<int64_t>(ceil_div(n_rows, 256), 1), 4 * sm_count());
    if (n_rows > 0) {
        bucket_histogram_kernel<<<blocks, 256, 0, st>>>(hash, (int)n_rows, (int)total_buckets, n_seg, seg_xb, seg_cb, counts);
        FM_LAUNCHED("bucket_histogram_kernel");
    }
    exclusive_scan_kernel<<<1, 1024, 0, st>>>(counts, (int)total_buckets, group_off, cursor);
    FM_LAUNCHED("exclusive_scan_kernel");
    if (n_rows > 0) {
        bucket_scatter_kernel<<<blocks, 256, 0, st>>>(hash, (int)n_rows, (int)total_buckets, n_seg, seg_xb, seg_cb, cursor, perm);
        FM_LAUNCHED("bucket_scatter_kernel");
    }
    return FM_OK;
}

extern "C" int64_t fm_group_rows_static_max_buckets(void) { return fm::kStaticMaxBuckets; }

extern "C" int fm_group_rows_static(const int32_t *hash, int64_t n_rows, int64_t total_buckets, int n_seg,
                                    const int32_t *seg_xb, const int32_t *seg_cb, int32_t *group_off, int32_t *perm,
                                    fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(group_off && (n_rows == 0 || (hash && perm)), "fm_group_rows_static: null pointer");
    FM_REQUIRE(n_rows >= 0 && total_buckets > 0 && n_seg >= 1, "fm_group_rows_static: bad sizes");
    FM_REQUIRE(n_rows < (int64_t(1) << 31), "fm_group_rows_static: sizes exceed int32");
    FM_REQUIRE((seg_xb == nullptr) == (seg_cb == nullptr), "fm_group_rows_static: pass both segment arrays or neither");
    if (total_buckets > kStaticMaxBuckets) {
        set_error("fm_group_rows_static: %lld buckets exceed the built-in scratch (%d buckets); use fm_group_rows "
                  "with a caller-provided workspace", (long long)total_buckets, kStaticMaxBuckets);
        return FM_ERR_UNSUPPORTED;
    }
    int32_t *scratch = nullptr;
    int rc = static_group_scratch(&scratch);
    if (rc != FM_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int32_t *counts = scratch;
    int32_t *cursor = scratch + kStaticMaxBuckets;
    // the array keeps whatever the previous call left: the counts must start at zero (the cursors are
    // overwritten by the scan)
    FM_CUDA_OK(cudaMemsetAsync(counts, 0, size_t(total_buckets) * 4, st));
    int blocks = (int)std::min<int64_t>(std::max<int64_t>(ceil_div(n_rows, 256), 1), 4 * sm_count());
    if (n_rows > 0) {
        bucket_histogram_kernel<<<blocks, 256, 0, st>>>(hash, (int)n_rows, (int)total_buckets, n_seg, seg_xb, seg_cb, counts);
        FM_LAUNCHED("bucket_histogram_kernel");
    }
    exclusive_scan_kernel<<<1, 1024, 0, st>>>(counts, (int)total_buckets, group_off, cursor);
    FM_LAUNCHED("exclusive_scan_kernel");
    if (n_rows > 0) {
        bucket_scatter_kernel<<<blocks, 256, 0, st>>>(hash, (int)n_rows, (int)total_buckets, n_seg, seg_xb, seg_cb, cursor, perm);
        FM_LAUNCHED("bucket_scatter_kernel");
    }
    return FM_OK;
}
