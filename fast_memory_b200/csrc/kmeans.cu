// Projection matrix by spherical k-means (distance 1 - c.x; README.md:37-45 of the reference, whose
// code has no k-means).  Every step is order-independent or has a fixed order, so the result is
// bit-reproducible: assignment = fm_hash_rows (canonical projection, first maximum wins); cluster sums =
// integer sums of the unit rows in units of 2^-40; normalisation = sequential fp64 sum of squares.
#include "common.cuh"

#include <algorithm>
#include <vector>

namespace fm {

constexpr float kFixScale = 1099511627776.0f;              // 2^40
constexpr double kFixInv = 1.0 / 1099511627776.0;

// nrm[r] = max(sqrt(sum_i x_i^2), 1e-6) with the sum a sequential FMA chain; optional U = x / nrm.
template <typename T>
__global__ void row_norm_kernel(const T *__restrict__ X, int64_t n_rows, int d, float *__restrict__ nrm,
                                float *__restrict__ U)
{
    int64_t r = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const T *x = X + r * d;
    float n2 = 0.f;
    for (int i = 0; i < d; ++i) {
        float v = Elem<T>::to_f32(x[i]);
        n2 = fmaf(v, v, n2);
    }
    float n = fmaxf(__fsqrt_rn(n2), 1e-6f);
    if (nrm) nrm[r] = n;
    if (U)
        for (int i = 0; i < d; ++i) U[r * d + i] = __fdiv_rn(Elem<T>::to_f32(x[i]), n);
}

// The same norms for 16-bit rows whose length is a multiple of 32 (up to 256): four lanes per row, each loading a
// quarter of the row in 16-byte pieces (all loads in flight at once, whole rows coalesced), the FMA chain running through
// the quarters in order, handed from lane to lane - the same summation order, so the same bits, at memory speed instead
// of one 2-byte load per element and thread.
template <typename T>
__global__ void __launch_bounds__(256)
row_norm4_kernel(const T *__restrict__ X, int64_t n_rows, int d, float *__restrict__ nrm)
{
    const int lane = threadIdx.x & 31, sub = lane & 3;
    const int64_t r = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 2;
    const bool ok = r < n_rows;
    const int quarter = d / 4;                               // elements per lane: a multiple of 8, at most 64
    const T *x = X + (ok ? r : 0) * d + sub * quarter;
    uint4 raw[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
        if (u * 8 < quarter) raw[u] = *reinterpret_cast<const uint4 *>(x + u * 8);
    float n2 = 0.f;
    for (int step = 0; step < 4; ++step) {
        if (sub == step) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (u * 8 < quarter) {
                    float f[8];
                    widen8(raw[u], f, T());
#pragma unroll
                    for (int k = 0; k < 8; ++k) n2 = fmaf(f[k], f[k], n2);
                }
        }
        n2 = __shfl_sync(0xffffffffu, n2, (lane & ~3) | step);            // the chain so far, to every lane of the four
    }
    if (ok && sub == 0) nrm[r] = fmaxf(__fsqrt_rn(n2), 1e-6f);
}

// One CTA per cluster: integer sum of its members' unit rows, then the new centroid.
// blockDim = (d, lanes): thread (c, m) sums column c over members m, m + lanes, ...
template <typename T>
__global__ void centroid_update_kernel(const T *__restrict__ X, const float *__restrict__ nrm, int d,
                                       const int32_t *__restrict__ group_off, const int32_t *__restrict__ perm,
                                       int row_base, float *__restrict__ cent_f32, T *__restrict__ A_out)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    long long *sums = reinterpret_cast<long long *>(smem_raw);             // [lanes][d]
    __shared__ double s_norm;
    const int c = threadIdx.x, m = threadIdx.y, lanes = blockDim.y;
    const int b = blockIdx.x;
    const int m0 = group_off[b], m1 = group_off[b + 1];
    long long acc = 0;
    for (int i = m0 + m; i < m1; i += lanes) {
        const int64_t r = int64_t(row_base) + perm[i];
        const float u = __fdiv_rn(Elem<T>::to_f32(X[r * d + c]), nrm[r]);
        acc += __float2ll_rn(u * kFixScale);
    }
    sums[m * d + c] = acc;
    __syncthreads();
    if (m == 0) {
        for (int k = 1; k < lanes; ++k) acc += sums[k * d + c];
        sums[c] = acc;
    }
    __syncthreads();
    if (m == 0 && c == 0) {
        double n2 = 0.0;
        for (int i = 0; i < d; ++i) {
            double s = __dmul_rn(double(sums[i]), kFixInv);
            n2 = __dadd_rn(n2, __dmul_rn(s, s));
        }
        s_norm = __dsqrt_rn(n2);
    }
    __syncthreads();
    if (m == 0) {
        float val = cent_f32[size_t(b) * d + c];                            // empty cluster keeps its centroid
        if (m1 > m0 && s_norm > 0.0) {
            double s = __dmul_rn(double(sums[c]), kFixInv);
            val = __double2float_rn(__ddiv_rn(s, s_norm));
            cent_f32[size_t(b) * d + c] = val;
        }
        A_out[size_t(b) * d + c] = Elem<T>::from_f32(val);
    }
}

template <typename T>
__global__ void cast_rows_kernel(const float *__restrict__ src, T *__restrict__ dst, int64_t n)
{
    int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = Elem<T>::from_f32(src[i]);
}

struct KmLayout { size_t off_nrm, off_hash, off_goff, off_perm, off_group, off_hws, off_seg, total; };
static KmLayout km_layout(int n_seg, const int64_t *seg_xb, const int64_t *seg_cb)
{
    // every iteration handles all segments at once: one assignment (hash), one grouping, one centroid update
    const int64_t rows = std::max<int64_t>(seg_xb[n_seg], 1), total_c = std::max<int64_t>(seg_cb[n_seg], 1);
    KmLayout L;
    size_t off = 0;
    L.off_nrm = off;  off += align_up(size_t(rows) * 4, 256);
    L.off_hash = off; off += align_up(size_t(rows) * 4, 256);
    L.off_goff = off; off += align_up(size_t(total_c + 1) * 4, 256);
    L.off_perm = off; off += align_up(size_t(rows) * 4, 256);
    L.off_group = off; off += fm_group_rows_workspace_bytes(rows, total_c);
    L.off_hws = off; off += fm_hash_rows_workspace_bytes(rows, n_seg);
    L.off_seg = off; off += 2 * align_up(size_t(n_seg + 1) * 4, 256);       // int32 copies of the segment prefixes
    L.total = off;
    return L;
}

template <typename T>
static int kmeans_impl(const void *Xv, int d, int n_seg, const int64_t *seg_xb, const int64_t *seg_cb, int iters,
                       float *cent_f32, void *A_out, char *ws, cudaStream_t st)
{
    const T *X = (const T *)Xv;
    T *A = (T *)A_out;
    KmLayout L = km_layout(n_seg, seg_xb, seg_cb);
    float *nrm = (float *)(ws + L.off_nrm);
    int32_t *hash = (int32_t *)(ws + L.off_hash);
    int32_t *goff = (int32_t *)(ws + L.off_goff);
    int32_t *perm = (int32_t *)(ws + L.off_perm);
    void *gws = ws + L.off_group;
    int32_t *d_xb = (int32_t *)(ws + L.off_seg), *d_cb = (int32_t *)(ws + L.off_seg + align_up(size_t(n_seg + 1) * 4, 256));
    const int64_t rows = seg_xb[n_seg], total_c = seg_cb[n_seg];
    if (rows <= 0 || total_c <= 0) return FM_OK;
    int64_t max_rows = 0;
    {
        std::vector<int32_t> h(2 * size_t(n_seg + 1));
        for (int s = 0; s <= n_seg; ++s) { h[s] = (int32_t)seg_xb[s]; h[n_seg + 1 + s] = (int32_t)seg_cb[s]; }
        for (int s = 0; s < n_seg; ++s) max_rows = std::max(max_rows, seg_xb[s + 1] - seg_xb[s]);
        FM_CUDA_OK(cudaMemcpyAsync(d_xb, h.data(), size_t(n_seg + 1) * 4, cudaMemcpyHostToDevice, st));
        FM_CUDA_OK(cudaMemcpyAsync(d_cb, h.data() + n_seg + 1, size_t(n_seg + 1) * 4, cudaMemcpyHostToDevice, st));
        FM_CUDA_OK(cudaStreamSynchronize(st));               // (the host vector goes away; a set-up step, once per call)
    }
    if (sizeof(T) == 2 && d % 32 == 0 && d <= 256) {
        if constexpr (sizeof(T) == 2) row_norm4_kernel<T><<<(unsigned)ceil_div(rows * 4, 256), 256, 0, st>>>(X, rows, d, nrm);
    } else {
        row_norm_kernel<T><<<(unsigned)ceil_div(rows, 128), 128, 0, st>>>(X, rows, d, nrm, nullptr);
    }
    FM_LAUNCHED("row_norm_kernel");
    cast_rows_kernel<T><<<(unsigned)ceil_div(total_c * d, 256), 256, 0, st>>>(cent_f32, A, total_c * d);
    FM_LAUNCHED("cast_rows_kernel");
    const int lanes = std::max(1, 512 / d);
    const bool one = n_seg == 1;
    for (int it = 0; it < iters; ++it) {
        int rc = fm_hash_rows(X, A, Elem<T>::id, rows, total_c, d, n_seg, one ? nullptr : d_xb, one ? nullptr : d_cb, max_rows, hash,
                              ws + L.off_hws, fm_hash_rows_workspace_bytes(rows, n_seg), st);
        if (rc != FM_OK) return rc;
        rc = fm_group_rows(hash, rows, total_c, n_seg, one ? nullptr : d_xb, one ? nullptr : d_cb, goff, perm, gws,
                           fm_group_rows_workspace_bytes(rows, total_c), st);
        if (rc != FM_OK) return rc;
        // (perm holds global row numbers and goff runs over the clusters of all segments: one launch)
        centroid_update_kernel<T><<<(unsigned)total_c, dim3(d, lanes), size_t(lanes) * d * 8, st>>>(X, nrm, d, goff, perm, 0, cent_f32, A);
        FM_LAUNCHED("centroid_update_kernel");
    }
    return FM_OK;
}

}  // namespace fm

extern "C" size_t fm_kmeans_workspace_bytes(int n_seg, const int64_t *seg_xb, const int64_t *seg_cb, int d)
{
    (void)d;
    return fm::km_layout(n_seg, seg_xb, seg_cb).total;
}

extern "C" int fm_kmeans(const void *X, int dtype, int d, int n_seg, const int64_t *seg_xb, const int64_t *seg_cb,
                         int iters, float *cent_f32, void *A_out, void *workspace, size_t workspace_bytes,
                         fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(X && seg_xb && seg_cb && cent_f32 && A_out && workspace, "fm_kmeans: null pointer");
    FM_REQUIRE(n_seg >= 1 && iters >= 0, "fm_kmeans: bad sizes");
    FM_REQUIRE(seg_xb[n_seg] < (int64_t(1) << 31), "fm_kmeans: rows exceed int32");
    if (d < 16 || d > 256 || d % 16) {
        set_error("fm_kmeans: head dim %d not supported (multiple of 16 in [16, 256])", d);
        return FM_ERR_UNSUPPORTED;
    }
    if (workspace_bytes < fm_kmeans_workspace_bytes(n_seg, seg_xb, seg_cb, d)) {
        set_error("fm_kmeans: workspace %zu too small", workspace_bytes);
        return FM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
    case FM_F32: return kmeans_impl<float>(X, d, n_seg, seg_xb, seg_cb, iters, cent_f32, A_out, (char *)workspace, st);
    case FM_BF16: return kmeans_impl<__nv_bfloat16>(X, d, n_seg, seg_xb, seg_cb, iters, cent_f32, A_out, (char *)workspace, st);
    case FM_F16: return kmeans_impl<__half>(X, d, n_seg, seg_xb, seg_cb, iters, cent_f32, A_out, (char *)workspace, st);
    default: set_error("fm_kmeans: unknown dtype %d", dtype); return FM_ERR_UNSUPPORTED;
    }
}

namespace fm {
// out[i, :] = mean_j U[rows[i * per_out + j], :], one CTA per output row (the rows are scattered: every thread owns a
// few columns and walks the row list).
__global__ void __launch_bounds__(128)
gather_mean_kernel(const float *__restrict__ U, int d, const int32_t *__restrict__ rows, int per_out, float *__restrict__ out)
{
    const int32_t *list = rows + size_t(blockIdx.x) * per_out;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < per_out; ++j) acc += U[size_t(list[j]) * d + c];
        out[size_t(blockIdx.x) * d + c] = acc / float(per_out);
    }
}
}  // namespace fm

extern "C" int fm_gather_mean(const float *U, int64_t n_rows, int d, const int32_t *rows, int64_t n_out, int64_t per_out, float *out,
                              fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(U && rows && out && n_rows > 0 && d > 0 && n_out >= 0 && per_out > 0, "fm_gather_mean: bad argument");
    FM_REQUIRE(per_out < (int64_t(1) << 31) && n_out < (int64_t(1) << 31), "fm_gather_mean: sizes exceed int32");
    if (n_out == 0) return FM_OK;
    gather_mean_kernel<<<(unsigned)n_out, 128, 0, (cudaStream_t)stream>>>(U, d, rows, (int)per_out, out);
    FM_LAUNCHED("gather_mean_kernel");
    return FM_OK;
}

extern "C" int fm_unit_rows(const void *X, int dtype, int64_t n_rows, int d, float *U, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(X && U && n_rows >= 0 && d > 0, "fm_unit_rows: bad argument");
    if (n_rows == 0) return FM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned blocks = (unsigned)ceil_div(n_rows, 128);
    switch (dtype) {
    case FM_F32: row_norm_kernel<float><<<blocks, 128, 0, st>>>((const float *)X, n_rows, d, nullptr, U); break;
    case FM_BF16: row_norm_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>((const __nv_bfloat16 *)X, n_rows, d, nullptr, U); break;
    case FM_F16: row_norm_kernel<__half><<<blocks, 128, 0, st>>>((const __half *)X, n_rows, d, nullptr, U); break;
    default: set_error("fm_unit_rows: unknown dtype %d", dtype); return FM_ERR_UNSUPPORTED;
    }
    FM_LAUNCHED("row_norm_kernel");
    return FM_OK;
}
