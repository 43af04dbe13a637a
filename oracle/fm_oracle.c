/*
 * TEST INFRASTRUCTURE ONLY - CPU oracle for the LSH attention-memory path.
 *
 * Plain-C restatement of the arithmetic whose bit pattern matters (projection,
 * argmax hash, top-Z selection).  It is the checker the parity tests compare the
 * CUDA kernels against and the port that the CPU baseline times; nothing in the
 * product package links or calls it.
 *
 * Canonical projection.  The reference computes Y = A.K^T with a library GEMM
 * (memory.py:261, triton_kernel.py:277) whose summation order is unspecified.
 * "Bit-exact bucket tables given identical fp32 projections" needs ONE defined
 * order, so both this file and the CUDA kernels use
 *     y = 0;  for i = 0 .. d-1:  y = fmaf(a[i], k[i], y)
 * in fp32 (inputs widened exactly from bf16/fp16 when they are 16-bit).
 *
 * Tie-breaking.  torch.topk / torch.argmax leave ties implementation-defined
 * (memory.py:273, 283; triton_kernel.py:278, 281); the canonical rule here is
 * "lower index wins" for both the top-Z set and the argmax.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define FMO_TILE 256

/* Y[c, j] = canonical dot(A[c, :], K[j, :]).  README.md:25 (Y = A K^T), memory.py:261. */
void fmo_project(const float *A, const float *K, int64_t C, int64_t N, int64_t d, float *Y)
{
#pragma omp parallel for schedule(static)
    for (int64_t j0 = 0; j0 < N; j0 += FMO_TILE) {
        int64_t jn = (N - j0 < FMO_TILE) ? (N - j0) : FMO_TILE;
        float kt[FMO_TILE];            /* one feature of the key tile, contiguous for the vector loop */
        float acc[FMO_TILE];
        for (int64_t c = 0; c < C; ++c) {
            const float *a = A + c * d;
            for (int64_t j = 0; j < jn; ++j) acc[j] = 0.0f;
            for (int64_t i = 0; i < d; ++i) {
                float ai = a[i];
                for (int64_t j = 0; j < jn; ++j) kt[j] = K[(j0 + j) * d + i];
                for (int64_t j = 0; j < jn; ++j) acc[j] = fmaf(ai, kt[j], acc[j]);
            }
            memcpy(Y + c * N + j0, acc, (size_t)jn * sizeof(float));
        }
    }
}

/* Same projection with the key tile transposed once per tile (faster for large C). */
void fmo_project_fast(const float *A, const float *K, int64_t C, int64_t N, int64_t d, float *Y)
{
#pragma omp parallel
    {
        float *kt = (float *)malloc((size_t)d * FMO_TILE * sizeof(float));
        float acc[FMO_TILE];
#pragma omp for schedule(static)
        for (int64_t j0 = 0; j0 < N; j0 += FMO_TILE) {
            int64_t jn = (N - j0 < FMO_TILE) ? (N - j0) : FMO_TILE;
            for (int64_t j = 0; j < jn; ++j)
                for (int64_t i = 0; i < d; ++i) kt[i * FMO_TILE + j] = K[(j0 + j) * d + i];
            for (int64_t c = 0; c < C; ++c) {
                const float *a = A + c * d;
                for (int64_t j = 0; j < jn; ++j) acc[j] = 0.0f;
                for (int64_t i = 0; i < d; ++i) {
                    float ai = a[i];
                    const float *kr = kt + i * FMO_TILE;
                    for (int64_t j = 0; j < jn; ++j) acc[j] = fmaf(ai, kr[j], acc[j]);
                }
                memcpy(Y + c * N + j0, acc, (size_t)jn * sizeof(float));
            }
        }
        free(kt);
    }
}

/* h[r] = argmax_c canonical dot(A[c, :], X[r, :]), first maximum wins.
 * README.md:29, memory.py:281-283, triton_kernel.py:280-281. */
void fmo_argmax_hash(const float *A, const float *X, int64_t C, int64_t R, int64_t d, int32_t *h)
{
    /* rows are processed in tiles, transposed once, so that the FMA chain of every (row, bucket) pair
     * keeps its sequential order over i while the compiler vectorises across the rows of the tile */
#pragma omp parallel
    {
        float *xt = (float *)malloc((size_t)d * FMO_TILE * sizeof(float));
        float acc[FMO_TILE], best[FMO_TILE];
        int32_t arg[FMO_TILE];
#pragma omp for schedule(static)
        for (int64_t r0 = 0; r0 < R; r0 += FMO_TILE) {
            int64_t rn = (R - r0 < FMO_TILE) ? (R - r0) : FMO_TILE;
            for (int64_t j = 0; j < rn; ++j)
                for (int64_t i = 0; i < d; ++i) xt[i * FMO_TILE + j] = X[(r0 + j) * d + i];
            for (int64_t c = 0; c < C; ++c) {
                const float *a = A + c * d;
                for (int64_t j = 0; j < rn; ++j) acc[j] = 0.0f;
                for (int64_t i = 0; i < d; ++i) {
                    float ai = a[i];
                    const float *xr = xt + i * FMO_TILE;
                    for (int64_t j = 0; j < rn; ++j) acc[j] = fmaf(ai, xr[j], acc[j]);
                }
                for (int64_t j = 0; j < rn; ++j)
                    if (c == 0 || acc[j] > best[j]) { best[j] = acc[j]; arg[j] = (int32_t)c; }
            }
            for (int64_t j = 0; j < rn; ++j) h[r0 + j] = arg[j];
        }
        free(xt);
    }
}

/* Order-preserving map float -> uint32 (larger float <=> larger key). */
static inline uint32_t fmo_key(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

/* Per row of Y[R, N]: the Z indices with the largest values, ties broken toward the lower
 * index, written in ascending index order (README.md:27 argtop_Z; memory.py:273).
 * Z must be <= N.  -0.0 and +0.0 compare equal, as they do for torch.topk. */
void fmo_topz(const float *Y, int64_t R, int64_t N, int64_t Z, int32_t *table)
{
#pragma omp parallel
    {
        uint32_t *keys = (uint32_t *)malloc((size_t)N * sizeof(uint32_t));
#pragma omp for schedule(dynamic, 1)
        for (int64_t r = 0; r < R; ++r) {
            const float *y = Y + r * N;
            for (int64_t j = 0; j < N; ++j) {
                float f = y[j];
                if (f == 0.0f) f = 0.0f;          /* fold -0.0 onto +0.0 */
                keys[j] = fmo_key(f);
            }
            /* radix descent for the Z-th largest key */
            uint32_t prefix = 0, mask = 0;
            int64_t want = Z;
            for (int shift = 24; shift >= 0; shift -= 8) {
                int64_t hist[256];
                memset(hist, 0, sizeof(hist));
                for (int64_t j = 0; j < N; ++j)
                    if ((keys[j] & mask) == prefix) hist[(keys[j] >> shift) & 255u]++;
                int b = 255;
                for (; b > 0; --b) {
                    if (hist[b] >= want) break;
                    want -= hist[b];
                }
                prefix |= (uint32_t)b << shift;
                mask |= 255u << shift;
            }
            /* prefix = key of the Z-th largest; `want` = how many equal to it are taken */
            int32_t *out = table + r * Z;
            int64_t n = 0, eq = 0;
            for (int64_t j = 0; j < N; ++j) {
                if (keys[j] > prefix) out[n++] = (int32_t)j;
                else if (keys[j] == prefix && eq < want) { out[n++] = (int32_t)j; ++eq; }
            }
        }
        free(keys);
    }
}

/* U[r, :] = X[r, :] / max(||X[r, :]||, 1e-6) in fp32; ||x||^2 is a sequential FMA chain
 * (unit-sphere projection of README.md:39; clamp as in memory.py:215-217). */
void fmo_unit_rows(const float *X, int64_t R, int64_t d, float *U)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < R; ++r) {
        const float *x = X + r * d;
        float n2 = 0.0f;
        for (int64_t i = 0; i < d; ++i) n2 = fmaf(x[i], x[i], n2);
        float nrm = sqrtf(n2);
        if (nrm < 1e-6f) nrm = 1e-6f;
        for (int64_t i = 0; i < d; ++i) U[r * d + i] = x[i] / nrm;
    }
}

int fmo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
