// 64 x 64 fp32 tile contraction on CUDA cores with a FIXED summation order.
//
// out[r][c] = sum_i X[r][i] * A[c][i] is accumulated as  y = fmaf(x_i, a_i, y)  for i = 0 .. d-1,
// one chain per output.  This is the canonical projection of the library: every table entry and every
// hash that has to be bit-identical to the CPU oracle is decided by values computed in this order.
//
// 256 threads as 16 (ty) x 16 (tx); thread (ty, tx) owns rows ty + 16 i and columns tx + 16 j
// (i, j = 0..3).  Both operand tiles sit in shared memory as fp32 rows of d + 4 floats, which makes
// the 16-byte reads of one quarter-warp (same ty, tx = 0..7) a broadcast for X and conflict-free for A.
#pragma once

#include "common.cuh"

namespace fm {

constexpr int kTile = 64;
constexpr int kTileThreads = 256;

__host__ __device__ inline int tile_ld(int d) { return d + 4; }
inline size_t tile_smem_bytes(int d) { return size_t(2) * kTile * tile_ld(d) * sizeof(float); }

// Load `rows` x d elements starting at src (row stride d) into dst (row stride d + 4) as fp32;
// rows beyond n_valid are zero-filled.
template <typename T>
__device__ __forceinline__ void load_tile_f32(float *__restrict__ dst, const T *__restrict__ src, int n_valid, int d)
{
    const int ld = tile_ld(d);
    if constexpr (sizeof(T) == 4) {
        const int per_row = d >> 2;
        for (int e = threadIdx.x; e < kTile * per_row; e += kTileThreads) {
            int r = e / per_row, c4 = e - r * per_row;
            float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < n_valid) val = *reinterpret_cast<const float4 *>(src + size_t(r) * d + c4 * 4);
            *reinterpret_cast<float4 *>(dst + r * ld + c4 * 4) = val;
        }
    } else {
        const int per_row = d >> 3;
        for (int e = threadIdx.x; e < kTile * per_row; e += kTileThreads) {
            int r = e / per_row, c8 = e - r * per_row;
            float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (r < n_valid) {
                uint4 raw = *reinterpret_cast<const uint4 *>(src + size_t(r) * d + c8 * 8);
                widen8(raw, f, T());
            }
            float *p = dst + r * ld + c8 * 8;
            *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4 *>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
        }
    }
}

// acc[i][j] = canonical dot(Xs[ty + 16 i], As[tx + 16 j]).
__device__ __forceinline__ void tile_dot(const float *__restrict__ Xs, const float *__restrict__ As, int d,
                                         float (&acc)[4][4])
{
    const int ld = tile_ld(d);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k = 0; k < d; k += 4) {
        float4 x[4], a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = *reinterpret_cast<const float4 *>(Xs + (ty + 16 * i) * ld + k);
#pragma unroll
        for (int j = 0; j < 4; ++j) a[j] = *reinterpret_cast<const float4 *>(As + (tx + 16 * j) * ld + k);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float y = acc[i][j];
                y = fmaf(x[i].x, a[j].x, y);
                y = fmaf(x[i].y, a[j].y, y);
                y = fmaf(x[i].z, a[j].z, y);
                y = fmaf(x[i].w, a[j].w, y);
                acc[i][j] = y;
            }
    }
}

// One canonical dot product by a single thread (slow path for isolated re-checks).
template <typename T>
__device__ __forceinline__ float canonical_dot(const T *__restrict__ a, const T *__restrict__ x, int d)
{
    float y = 0.f;
    for (int i = 0; i < d; ++i) y = fmaf(Elem<T>::to_f32(a[i]), Elem<T>::to_f32(x[i]), y);
    return y;
}

}  // namespace fm
