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

// ---- one launch: a CTA per segment -------------------------------------------------------------------------------------
// When every hash is known to lie inside its segment's buckets (the hashes of fm_hash_rows do), the rows of segment s
// fill perm[seg_xb[s] .. seg_xb[s + 1]) exactly, so a segment's part of the result depends on nothing outside the
// segment: one CTA counts the segment's rows per bucket in shared memory, scans the counts, writes group_off and
// scatters the rows - the memset and the three launches of the general path become one launch.  A hash outside the
// segment's buckets is clamped into them (memory-safe; callers with untrusted hashes use fm_group_rows).
constexpr int kSegGroupThreads = 1024;
constexpr int kSegGroupMaxBuckets = 12288;  // counts + cursors of one segment in shared memory (96 KB)
constexpr int kSegGroupMaxRows = 32768;     // beyond this a single CTA per segment is slower than the general path

__global__ void __launch_bounds__(kSegGroupThreads)
group_rows_segment_kernel(const int32_t *__restrict__ hash, int n_rows, int total_buckets, int n_seg,
                          const int32_t *__restrict__ seg_xb, const int32_t *__restrict__ seg_cb,
                          int32_t *__restrict__ group_off, int32_t *__restrict__ perm)
{
    extern __shared__ int32_t seg_sm[];
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    const int s = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int r0 = seg_xb ? seg_xb[s] : 0, r1 = seg_xb ? seg_xb[s + 1] : n_rows;
    const int c0 = seg_cb ? seg_cb[s] : 0, C = (seg_cb ? seg_cb[s + 1] : total_buckets) - c0;
    int32_t *counts = seg_sm, *cursor = seg_sm + C;
    for (int c = t; c < C; c += kSegGroupThreads) counts[c] = 0;
    if (t == 0) carry_s = 0;
    __syncthreads();
    for (int r = r0 + t; r < r1; r += kSegGroupThreads) atomicAdd(&counts[min(max(hash[r], 0), C - 1)], 1);
    __syncthreads();
    for (int base = 0; base < C; base += kSegGroupThreads) {
        const int c = base + t;
        const int v = c < C ? counts[c] : 0;
        int inc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += o;
        }
        if (lane == 31) warp_sums[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            const int w = warp_sums[lane];
            int winc = w;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, winc, off);
                if (lane >= off) winc += o;
            }
            warp_sums[lane] = winc - w;
        }
        __syncthreads();
        const int excl = carry_s + warp_sums[warp] + inc - v;
        if (c < C) { cursor[c] = excl; group_off[c0 + c] = r0 + excl; }
        __syncthreads();
        if (t == kSegGroupThreads - 1) carry_s = excl + v;
        __syncthreads();
    }
    for (int r = r0 + t; r < r1; r += kSegGroupThreads) perm[r0 + atomicAdd(&cursor[min(max(hash[r], 0), C - 1)], 1)] = r;
    // buckets outside the listed segments (a caller serving a slice of the heads) hold no rows
    if (s == 0)
        for (int c = t; c < c0; c += kSegGroupThreads) group_off[c] = 0;
    if (s == n_seg - 1)
        for (int c = c0 + C + t; c <= total_buckets; c += kSegGroupThreads) group_off[c] = n_rows;
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

extern "C" int fm_group_rows_segmented(const int32_t *hash, int64_t n_rows, int64_t total_buckets, int n_seg,
                                       const int32_t *seg_xb, const int32_t *seg_cb, int64_t max_seg_rows, int64_t max_seg_buckets,
                                       int32_t *group_off, int32_t *perm, void *workspace, size_t workspace_bytes,
                                       fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(group_off && (n_rows == 0 || (hash && perm)), "fm_group_rows_segmented: null pointer");
    FM_REQUIRE(n_rows >= 0 && total_buckets > 0 && n_seg >= 1, "fm_group_rows_segmented: bad sizes");
    FM_REQUIRE(n_rows < (int64_t(1) << 31) && total_buckets < (int64_t(1) << 31), "fm_group_rows_segmented: sizes exceed int32");
    FM_REQUIRE((seg_xb == nullptr) == (seg_cb == nullptr), "fm_group_rows_segmented: pass both segment arrays or neither");
    FM_REQUIRE(seg_xb || n_seg == 1, "fm_group_rows_segmented: n_seg > 1 needs segment arrays");
    if (n_rows == 0 || max_seg_rows > kSegGroupMaxRows || max_seg_buckets > kSegGroupMaxBuckets || max_seg_buckets <= 0)
        return fm_group_rows(hash, n_rows, total_buckets, n_seg, seg_xb, seg_cb, group_off, perm, workspace, workspace_bytes, stream);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t dyn = size_t(max_seg_buckets) * 8;
    FM_CUDA_OK(func_attr_cached((const void *)group_rows_segment_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    group_rows_segment_kernel<<<n_seg, kSegGroupThreads, dyn, st>>>(hash, (int)n_rows, (int)total_buckets, n_seg, seg_xb, seg_cb,
                                                                  group_off, perm);
    FM_LAUNCHED("group_rows_segment_kernel");
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
