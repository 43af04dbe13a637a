// Index build: projection Y = A K^T in the canonical fp32 order, exact top-Z selection per bucket, and
// the per-segment driver.  Stands in for einsum + topk of the reference (memory.py:261, 273;
// triton_kernel.py:277-278; README.md:25-27).
#include "index_fused.cuh"
#include "simt_tile.cuh"
#include "topz_row.cuh"

#include <vector>

namespace fm {

// ---- projection (CUDA cores, canonical order) ---------------------------------------------------------
// One CTA per 64-key tile; the bucket rows of A stream through in tiles of 64.
template <typename T>
__global__ void __launch_bounds__(kTileThreads)
project_kernel(const T *__restrict__ A, const T *__restrict__ K, int C, int64_t N, int d, float *__restrict__ Y,
               int64_t ldy)
{
    extern __shared__ __align__(16) float smem[];
    float *As = smem;                                  // bucket rows ("X" operand of tile_dot)
    float *Ks = smem + kTile * tile_ld(d);             // key rows
    const int64_t j0 = int64_t(blockIdx.x) * kTile;
    const int nk = (int)min(int64_t(kTile), N - j0);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    load_tile_f32(Ks, K + size_t(j0) * d, nk, d);
    for (int c0 = 0; c0 < C; c0 += kTile) {
        __syncthreads();
        load_tile_f32(As, A + size_t(c0) * d, min(kTile, C - c0), d);
        __syncthreads();
        float acc[4][4];
        tile_dot(As, Ks, d, acc);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int c = c0 + ty + 16 * i;
            if (c >= C) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int jj = tx + 16 * j;
                if (jj < nk) Y[size_t(c) * ldy + j0 + jj] = acc[i][j];
            }
        }
    }
}

// ---- exact top-Z of a row: see topz_row.cuh ---------------------------------------------------------------
__global__ void __launch_bounds__(kSelThreads)
topz_select_kernel(const float *__restrict__ Y, int64_t N, int64_t ldy, int Z, int32_t index_base,
                   int32_t *__restrict__ table, int64_t ld_table)
{
    topz_row(Y + size_t(blockIdx.x) * ldy, N, Z, index_base, table + size_t(blockIdx.x) * ld_table);
}

template <typename T>
static int launch_project(const void *A, const void *K, int64_t C, int64_t N, int d, float *Y, int64_t ldy,
                          cudaStream_t st)
{
    size_t smem = tile_smem_bytes(d);
    FM_CUDA_OK(func_attr_cached((const void *)project_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    project_kernel<T><<<(unsigned)ceil_div(N, kTile), kTileThreads, smem, st>>>((const T *)A, (const T *)K, (int)C, N, d, Y, ldy);
    FM_LAUNCHED("project_kernel");
    return FM_OK;
}

static int check_dim(const char *who, int d)
{
    if (d < 16 || d > 256 || d % 16) {
        set_error("%s: head dim %d not supported (multiple of 16 in [16, 256])", who, d);
        return FM_ERR_UNSUPPORTED;
    }
    return FM_OK;
}

constexpr size_t kBuildBudget = size_t(1) << 30;           // bytes of projection scores held at once

static int64_t rows_per_pass(int64_t C, int64_t N)
{
    int64_t rows = std::max<int64_t>(64, int64_t(kBuildBudget / (size_t(N) * 4)) / 64 * 64);
    return std::min(C, rows);
}

}  // namespace fm

extern "C" int fm_project(const void *A, const void *K, int dtype, int64_t C, int64_t N, int d, float *Y, int64_t ldy,
                          fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(A && K && Y, "fm_project: null pointer");
    FM_REQUIRE(C > 0 && N > 0 && ldy >= N && C < (int64_t(1) << 31), "fm_project: bad sizes");
    int rc = check_dim("fm_project", d);
    if (rc != FM_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
    case FM_F32: return launch_project<float>(A, K, C, N, d, Y, ldy, st);
    case FM_BF16: return launch_project<__nv_bfloat16>(A, K, C, N, d, Y, ldy, st);
    case FM_F16: return launch_project<__half>(A, K, C, N, d, Y, ldy, st);
    default: set_error("fm_project: unknown dtype %d", dtype); return FM_ERR_UNSUPPORTED;
    }
}

namespace fm {
// scores[e] = canonical A[b] . K[table[e]] for the entries e of bucket b: what a table's keys scored, in the fixed fp32
// order, so that tables of different key shards can be merged exactly.
template <typename T>
__global__ void __launch_bounds__(128)
table_scores_kernel(const T *__restrict__ K, const T *__restrict__ A, int d, const int32_t *__restrict__ table,
                    const int64_t *__restrict__ bucket_off, float *__restrict__ scores)
{
    const int b = blockIdx.x;
    const T *a_row = A + size_t(b) * d;
    for (int64_t e = bucket_off[b] + threadIdx.x; e < bucket_off[b + 1]; e += blockDim.x)
        scores[e] = canonical_dot(a_row, K + size_t(table[e]) * d, d);
}
}  // namespace fm

extern "C" int fm_table_scores(const void *K, const void *A, int dtype, int d, int64_t total_buckets, const int32_t *table,
                               const int64_t *bucket_off, float *scores, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(K && A && table && bucket_off && scores, "fm_table_scores: null pointer");
    FM_REQUIRE(total_buckets > 0 && total_buckets < (int64_t(1) << 31), "fm_table_scores: bad bucket count");
    int rc = check_dim("fm_table_scores", d);
    if (rc != FM_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
    case FM_F32: table_scores_kernel<float><<<(unsigned)total_buckets, 128, 0, st>>>((const float *)K, (const float *)A, d, table, bucket_off, scores); break;
    case FM_BF16: table_scores_kernel<__nv_bfloat16><<<(unsigned)total_buckets, 128, 0, st>>>((const __nv_bfloat16 *)K, (const __nv_bfloat16 *)A, d, table, bucket_off, scores); break;
    case FM_F16: table_scores_kernel<__half><<<(unsigned)total_buckets, 128, 0, st>>>((const __half *)K, (const __half *)A, d, table, bucket_off, scores); break;
    default: set_error("fm_table_scores: unknown dtype %d", dtype); return FM_ERR_UNSUPPORTED;
    }
    FM_LAUNCHED("table_scores_kernel");
    return FM_OK;
}

extern "C" int fm_topz_select(const float *Y, int64_t n_rows, int64_t N, int64_t ldy, int64_t Z, int32_t index_base,
                              int32_t *table, int64_t ld_table, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(Y && table, "fm_topz_select: null pointer");
    FM_REQUIRE(n_rows > 0 && N > 0 && ldy >= N && Z > 0 && Z <= N && ld_table >= Z, "fm_topz_select: bad sizes");
    FM_REQUIRE(N + int64_t(index_base) < (int64_t(1) << 31), "fm_topz_select: indices exceed int32");
    topz_select_kernel<<<(unsigned)n_rows, kSelThreads, 0, (cudaStream_t)stream>>>(Y, N, ldy, (int)Z, index_base, table, ld_table);
    FM_LAUNCHED("topz_select_kernel");
    return FM_OK;
}

namespace fm {
// segments that take the tensor-core path, as parallel arrays
struct FusedList {
    std::vector<int64_t> kb, nk, cb, nbk, zc, toff;
    std::vector<int> seg;
};
static FusedList fused_segments(int n_seg, const int64_t *seg_kb, const int64_t *seg_cb, const int64_t *seg_z,
                                const int64_t *table_off, int d, int dtype, int flags)
{
    FusedList F;
    if (flags & FM_BUILD_EXACT_ONLY) return F;
    for (int s = 0; s < n_seg; ++s) {
        const int64_t N = seg_kb[s + 1] - seg_kb[s], C = seg_cb[s + 1] - seg_cb[s];
        if (N <= 0 || C <= 0 || seg_z[s] <= 0) continue;
        const int64_t zc = std::min(seg_z[s], N);
        if (!fused_eligible(dtype, d, N, zc)) continue;
        F.kb.push_back(seg_kb[s]); F.nk.push_back(N); F.cb.push_back(seg_cb[s]); F.nbk.push_back(C); F.zc.push_back(zc);
        F.toff.push_back(table_off ? table_off[s] : 0);
        F.seg.push_back(s);
    }
    // the selection holds a bucket's candidates in shared memory; the projection addresses a group's candidate array
    // with 32-bit byte offsets
    if (!F.seg.empty()) {
        const FusedPlan P = fused_plan((int)F.seg.size(), F.nk.data(), F.nbk.data(), F.zc.data());
        if (P.cap > kFusedMaxCap || P.sel_smem > kFusedMaxSelSmem || uint64_t(P.group_buckets) * uint64_t(P.cap) * 16 >= (uint64_t(1) << 32)) return FusedList();
    }
    return F;
}
}  // namespace fm

extern "C" size_t fm_index_build_workspace_bytes(int n_seg, const int64_t *seg_kb, const int64_t *seg_cb,
                                                 const int64_t *seg_z, int d, int dtype, int flags)
{
    using namespace fm;
    size_t need = 256;
    FusedList F = fused_segments(n_seg, seg_kb, seg_cb, seg_z, nullptr, d, dtype, flags);
    size_t fi = 0;
    for (int s = 0; s < n_seg; ++s) {
        if (fi < F.seg.size() && F.seg[fi] == s) { ++fi; continue; }
        int64_t N = seg_kb[s + 1] - seg_kb[s], C = seg_cb[s + 1] - seg_cb[s];
        if (N <= 0 || C <= 0) continue;
        need = std::max(need, 256 + size_t(rows_per_pass(C, N)) * size_t(N) * 4);
    }
    if (!F.seg.empty()) need = std::max(need, fused_plan((int)F.seg.size(), F.nk.data(), F.nbk.data(), F.zc.data()).total);
    return align_up(need, 256);
}

extern "C" int fm_index_build(const void *K, const void *A, int dtype, int d, int n_seg, const int64_t *seg_kb,
                              const int64_t *seg_cb, const int64_t *seg_z, const int64_t *table_off, int32_t *table,
                              int flags, void *workspace, size_t workspace_bytes, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(K && A && seg_kb && seg_cb && seg_z && table_off && table && workspace, "fm_index_build: null pointer");
    FM_REQUIRE(n_seg >= 1, "fm_index_build: bad segment count");
    int rc = check_dim("fm_index_build", d);
    if (rc != FM_OK) return rc;
    if (workspace_bytes < fm_index_build_workspace_bytes(n_seg, seg_kb, seg_cb, seg_z, d, dtype, flags)) {
        set_error("fm_index_build: workspace %zu too small", workspace_bytes);
        return FM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const size_t eb = elem_bytes(dtype);
    FM_CUDA_OK(cudaMemsetAsync(workspace, 0, 256, st));              // status word
    FusedList F = fused_segments(n_seg, seg_kb, seg_cb, seg_z, table_off, d, dtype, flags);
    if (!F.seg.empty()) {
        FM_REQUIRE(((uintptr_t)K | (uintptr_t)A) % 16 == 0, "fm_index_build: K and A must be 16-byte aligned");
        rc = fused_index_build(K, A, dtype, d, seg_kb[n_seg], seg_cb[n_seg], (int)F.seg.size(), F.kb.data(), F.nk.data(),
                               F.cb.data(), F.nbk.data(), F.zc.data(), F.toff.data(), table, workspace, (flags & FM_BUILD_SINGLE_RANGE) != 0, st);
        if (rc != FM_OK) return rc;
    }
    float *Y = (float *)((char *)workspace + 256);
    size_t fi = 0;
    for (int s = 0; s < n_seg; ++s) {
        if (fi < F.seg.size() && F.seg[fi] == s) { ++fi; continue; }
        const int64_t N = seg_kb[s + 1] - seg_kb[s], C = seg_cb[s + 1] - seg_cb[s];
        if (N <= 0 || C <= 0) continue;
        FM_REQUIRE(seg_z[s] > 0, "fm_index_build: bucket size of segment %d must be positive", s);
        FM_REQUIRE(seg_kb[s + 1] < (int64_t(1) << 31), "fm_index_build: key rows exceed int32");
        const int64_t Zc = std::min(seg_z[s], N);
        const int64_t step = rows_per_pass(C, N);
        const char *Ks = (const char *)K + size_t(seg_kb[s]) * d * eb;
        for (int64_t c0 = 0; c0 < C; c0 += step) {
            const int64_t rows = std::min(step, C - c0);
            const char *As = (const char *)A + size_t(seg_cb[s] + c0) * d * eb;
            rc = fm_project(As, Ks, dtype, rows, N, d, Y, N, stream);
            if (rc != FM_OK) return rc;
            rc = fm_topz_select(Y, rows, N, N, Zc, (int32_t)seg_kb[s], table + table_off[s] + c0 * Zc, Zc, stream);
            if (rc != FM_OK) return rc;
        }
    }
    return FM_OK;
}
