// Query / key hashing: hash[r] = argmax_c A[c, :] . x[r, :] over the buckets of r's segment.
// Stands in for the einsum + argmax of the reference (memory.py:281-283, triton_kernel.py:280-281).
#include "simt_tile.cuh"

namespace fm {

// grid = (row tiles of the longest segment, segments).  A CTA keeps its 64 rows in shared memory and
// streams the segment's buckets through in tiles of 64, tracking the running (best, argbest) of each
// row with "first maximum wins".
template <typename T>
__global__ void __launch_bounds__(kTileThreads)
hash_rows_kernel(const T *__restrict__ x, const T *__restrict__ A, int d, int n_rows, int total_buckets,
                 const int32_t *__restrict__ seg_xb, const int32_t *__restrict__ seg_cb,
                 int32_t *__restrict__ hash_out)
{
    extern __shared__ __align__(16) float smem[];
    float *Xs = smem;
    float *As = smem + kTile * tile_ld(d);

    const int s = blockIdx.y;
    const int row0 = seg_xb ? seg_xb[s] : 0;
    const int row1 = seg_xb ? seg_xb[s + 1] : n_rows;
    const int cb0 = seg_cb ? seg_cb[s] : 0;
    const int C = (seg_cb ? seg_cb[s + 1] : total_buckets) - cb0;
    const int r0 = row0 + blockIdx.x * kTile;
    if (r0 >= row1) return;
    const int n_valid = min(kTile, row1 - r0);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

    load_tile_f32(Xs, x + size_t(r0) * d, n_valid, d);

    float best[4];
    int arg[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { best[i] = -INFINITY; arg[i] = 0x7fffffff; }

    for (int c0 = 0; c0 < C; c0 += kTile) {
        __syncthreads();                                   // previous tile fully consumed (and Xs visible)
        load_tile_f32(As, A + size_t(cb0 + c0) * d, min(kTile, C - c0), d);
        __syncthreads();
        float acc[4][4];
        tile_dot(Xs, As, d, acc);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int c = c0 + tx + 16 * j;                      // ascending in j: strict > keeps the first maximum
            if (c < C) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (acc[i][j] > best[i] || arg[i] == 0x7fffffff) { best[i] = acc[i][j]; arg[i] = c; }
            }
        }
    }
    // reduce over the 16 tx lanes that share a row (lanes of one half-warp): larger value, then lower index
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best[i], off);
            int oa = __shfl_xor_sync(0xffffffffu, arg[i], off);
            if (oa != 0x7fffffff && (arg[i] == 0x7fffffff || ob > best[i] || (ob == best[i] && oa < arg[i]))) {
                best[i] = ob;
                arg[i] = oa;
            }
        }
        int r = ty + 16 * i;
        if (tx == 0 && r < n_valid) hash_out[r0 + r] = arg[i] == 0x7fffffff ? 0 : arg[i];
    }
}

template <typename T>
static int launch_hash(const void *x, const void *A, int64_t n_rows, int64_t total_buckets, int d, int n_seg,
                       const int32_t *seg_xb, const int32_t *seg_cb, int64_t max_seg_rows, int32_t *hash_out,
                       cudaStream_t st)
{
    size_t smem = tile_smem_bytes(d);
    FM_CUDA_OK(cudaFuncSetAttribute(hash_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)ceil_div(max_seg_rows, kTile), (unsigned)n_seg);
    hash_rows_kernel<T><<<grid, kTileThreads, smem, st>>>((const T *)x, (const T *)A, d, (int)n_rows,
                                                         (int)total_buckets, seg_xb, seg_cb, hash_out);
    FM_LAUNCHED("hash_rows_kernel");
    return FM_OK;
}

}  // namespace fm

extern "C" int fm_hash_rows(const void *x, const void *A, int dtype, int64_t n_rows, int64_t total_buckets, int d,
                            int n_seg, const int32_t *seg_xb, const int32_t *seg_cb, int64_t max_seg_rows,
                            int32_t *hash_out, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(x && A && hash_out, "fm_hash_rows: null pointer");
    FM_REQUIRE(n_rows >= 0 && total_buckets > 0 && n_seg >= 1, "fm_hash_rows: bad sizes");
    FM_REQUIRE(n_rows < (int64_t(1) << 31) && total_buckets < (int64_t(1) << 31), "fm_hash_rows: sizes exceed int32");
    FM_REQUIRE((seg_xb == nullptr) == (seg_cb == nullptr), "fm_hash_rows: pass both segment arrays or neither");
    FM_REQUIRE(seg_xb || n_seg == 1, "fm_hash_rows: n_seg > 1 needs segment arrays");
    if (d < 16 || d > 256 || d % 16) {
        set_error("fm_hash_rows: head dim %d not supported (multiple of 16 in [16, 256])", d);
        return FM_ERR_UNSUPPORTED;
    }
    if (n_rows == 0) return FM_OK;
    if (max_seg_rows <= 0) max_seg_rows = n_rows;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
    case FM_F32: return launch_hash<float>(x, A, n_rows, total_buckets, d, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, st);
    case FM_BF16: return launch_hash<__nv_bfloat16>(x, A, n_rows, total_buckets, d, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, st);
    case FM_F16: return launch_hash<__half>(x, A, n_rows, total_buckets, d, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, st);
    default: set_error("fm_hash_rows: unknown dtype %d", dtype); return FM_ERR_UNSUPPORTED;
    }
}
