// Index build: projection Y = A K^T in the canonical fp32 order, exact top-Z selection per bucket, and
// the per-segment driver.  Stands in for einsum + topk of the reference (memory.py:261, 273;
// triton_kernel.py:277-278; README.md:25-27).
#include "simt_tile.cuh"

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

// ---- exact top-Z of a row ------------------------------------------------------------------------------
// One CTA per row.  Four 8-bit radix passes over the order-preserving keys find the Z-th largest key
// theta and how many entries equal to theta belong to the result; an ordered compaction then writes
// the selected indices in ascending order (entries > theta, and the first `want` entries == theta).
constexpr int kSelThreads = 1024;

__global__ void __launch_bounds__(kSelThreads)
topz_select_kernel(const float *__restrict__ Y, int64_t N, int64_t ldy, int Z, int32_t index_base,
                   int32_t *__restrict__ table, int64_t ld_table)
{
    __shared__ int hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_want;
    __shared__ int warp_gt[32], warp_eq[32];
    const float *y = Y + size_t(blockIdx.x) * ldy;
    int32_t *out = table + size_t(blockIdx.x) * ld_table;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;

    if (t == 0) { s_prefix = 0; s_want = Z; }
    uint32_t mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (t < 256) hist[t] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int64_t j = t; j < N; j += kSelThreads) {
            uint32_t key = float_key(y[j]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
        }
        __syncthreads();
        if (t == 0) {
            int want = s_want, b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= want) break;
                want -= hist[b];
            }
            s_prefix = prefix | (uint32_t(b) << shift);
            s_want = want;
        }
        mask |= 255u << shift;
        __syncthreads();
    }
    const uint32_t theta = s_prefix;
    const int want = s_want;
    int gt_base = 0, eq_base = 0;
    for (int64_t j0 = 0; j0 < N; j0 += kSelThreads) {
        const int64_t j = j0 + t;
        uint32_t key = j < N ? float_key(y[j]) : 0u;
        const bool gt = j < N && key > theta;
        const bool eq = j < N && key == theta;
        const unsigned bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
        const unsigned lt_mask = (1u << lane) - 1u;
        int gt_ex = __popc(bg & lt_mask), eq_ex = __popc(be & lt_mask);
        if (lane == 0) { warp_gt[warp] = __popc(bg); warp_eq[warp] = __popc(be); }
        __syncthreads();
        if (warp == 0) {
            int g = warp_gt[lane], e = warp_eq[lane];
            int gi = g, ei = e;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                int tg = __shfl_up_sync(0xffffffffu, gi, off), te = __shfl_up_sync(0xffffffffu, ei, off);
                if (lane >= off) { gi += tg; ei += te; }
            }
            warp_gt[lane] = gi - g;
            warp_eq[lane] = ei - e;
            if (lane == 31) { hist[0] = gi; hist[1] = ei; }          // chunk totals
        }
        __syncthreads();
        gt_ex += gt_base + warp_gt[warp];
        eq_ex += eq_base + warp_eq[warp];
        if (gt || (eq && eq_ex < want)) {
            int pos = gt_ex + min(eq_ex, want);
            if (pos < Z) out[pos] = int32_t(j) + index_base;
        }
        gt_base += hist[0];
        eq_base += hist[1];
        __syncthreads();
    }
}

template <typename T>
static int launch_project(const void *A, const void *K, int64_t C, int64_t N, int d, float *Y, int64_t ldy,
                          cudaStream_t st)
{
    size_t smem = tile_smem_bytes(d);
    FM_CUDA_OK(cudaFuncSetAttribute(project_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
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

extern "C" size_t fm_index_build_workspace_bytes(int n_seg, const int64_t *seg_kb, const int64_t *seg_cb,
                                                 const int64_t *seg_z, int d, int dtype)
{
    (void)seg_z; (void)d; (void)dtype;
    size_t need = 256;
    for (int s = 0; s < n_seg; ++s) {
        int64_t N = seg_kb[s + 1] - seg_kb[s], C = seg_cb[s + 1] - seg_cb[s];
        if (N <= 0 || C <= 0) continue;
        need = std::max(need, size_t(fm::rows_per_pass(C, N)) * size_t(N) * 4);
    }
    return fm::align_up(need, 256);
}

extern "C" int fm_index_build(const void *K, const void *A, int dtype, int d, int n_seg, const int64_t *seg_kb,
                              const int64_t *seg_cb, const int64_t *seg_z, const int64_t *table_off, int32_t *table,
                              void *workspace, size_t workspace_bytes, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(K && A && seg_kb && seg_cb && seg_z && table_off && table && workspace, "fm_index_build: null pointer");
    FM_REQUIRE(n_seg >= 1, "fm_index_build: bad segment count");
    int rc = check_dim("fm_index_build", d);
    if (rc != FM_OK) return rc;
    if (workspace_bytes < fm_index_build_workspace_bytes(n_seg, seg_kb, seg_cb, seg_z, d, dtype)) {
        set_error("fm_index_build: workspace %zu too small", workspace_bytes);
        return FM_ERR_WORKSPACE;
    }
    const size_t eb = elem_bytes(dtype);
    float *Y = (float *)workspace;
    for (int s = 0; s < n_seg; ++s) {
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
