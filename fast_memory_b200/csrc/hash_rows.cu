// Query / key hashing: hash[r] = argmax_c A[c, :] . x[r, :] over the buckets of r's segment.
// Stands in for the einsum + argmax of the reference (memory.py:281-283, triton_kernel.py:280-281).
#include "mma_utils.cuh"
#include "simt_tile.cuh"
#include "tc_utils.cuh"

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

// ---- tensor-core path for 16-bit inputs ------------------------------------------------------------------
// The scores are computed with mma.sync (fp32 accumulate, unspecified summation order), which is only a
// FILTER: per row the kernel keeps the best and second-best score; when they are closer than a bound on
// the accumulation error the row goes on a re-check list and a second kernel decides it with the canonical
// fp32 chain.  A row whose gap exceeds the bound has the same argmax under both orders, so the result is
// bit-identical to the all-fp32 kernel above.
//
// Error bound: each value is within 2^-16 M of the exact dot product and the canonical chain within
// 2^-17 M (d <= 256), M = ||x|| max_c ||a_c|| >= sum_i |a_ci x_i|; two scores can therefore swap order
// only if their tensor-core gap is below 3 * 2^-16 M.  The test uses 2^-12 M.
constexpr float kHashEps = 1.0f / 4096.0f;
constexpr int kHashThreads = 128;

// running top three scores of a row (indices kept for the best two)
struct Top3 {
    float best, second, third;
    int arg, arg2;
};
// Branch-free (the lanes of a warp hold different rows, so a branchy insert runs every arm): the earlier score keeps its
// place on a tie, like "first maximum wins".
__device__ __forceinline__ void top3_push(Top3 &t, float v, int c)
{
    const bool gb = v > t.best, gs = v > t.second;
    t.third = fmaxf(t.third, fminf(t.second, v));
    t.second = fmaxf(t.second, fminf(t.best, v));
    t.arg2 = gb ? t.arg : (gs ? c : t.arg2);
    t.arg = gb ? c : t.arg;
    t.best = fmaxf(t.best, v);
}

// amax[s] = max row norm of the A rows of segment s (as the bits of a non-negative float, via atomicMax)
template <typename T>
__global__ void a_norm_max_kernel(const T *__restrict__ A, int total_buckets, int d, int n_seg,
                                  const int32_t *__restrict__ seg_cb, unsigned *__restrict__ amax)
{
    const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (c >= total_buckets) return;
    const int lane = threadIdx.x & 31;
    float n2 = 0.f;
    for (int i = lane; i < d; i += 32) {
        float v = Elem<T>::to_f32(A[size_t(c) * d + i]);
        n2 = fmaf(v, v, n2);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, off);
    if (lane == 0) {
        const int s = seg_cb ? find_segment(seg_cb, n_seg, c) : 0;
        atomicMax(&amax[s], __float_as_uint(sqrtf(n2) * 1.0001f));
    }
}

template <typename T, int D>
__global__ void __launch_bounds__(kHashThreads)
hash_rows_mma_kernel(const T *__restrict__ x, const T *__restrict__ A, int n_rows, int total_buckets,
                     const int32_t *__restrict__ seg_xb, const int32_t *__restrict__ seg_cb,
                     const unsigned *__restrict__ amax, int32_t *__restrict__ hash_out,
                     int32_t *__restrict__ recheck, int *__restrict__ n_recheck)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int CPR = D / 8;                                   // 16-byte chunks per row
    constexpr int TILE_BYTES = kTile * D * 2;
    const int s = blockIdx.y;
    const int row0 = seg_xb ? seg_xb[s] : 0;
    const int row1 = seg_xb ? seg_xb[s + 1] : n_rows;
    const int cb0 = seg_cb ? seg_cb[s] : 0;
    const int C = (seg_cb ? seg_cb[s + 1] : total_buckets) - cb0;
    const int r0 = row0 + blockIdx.x * kTile;
    if (r0 >= row1) return;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, g = lane >> 2, tq = lane & 3;
    const uint32_t smem_base = smem_u32(smem_raw);
    const char *Ab = reinterpret_cast<const char *>(A + size_t(cb0) * D);

    auto issue = [&](int ta) {
        const int c0 = ta * kTile;
        if (c0 < C) {
            const uint32_t dst = smem_base + (ta & 1) * TILE_BYTES;
            for (int e = t; e < kTile * CPR; e += kHashThreads) {
                const int j = e / CPR, c = e - j * CPR;
                const bool ok = c0 + j < C;
                cp_async16(dst + swz<D>(j, c), Ab + (ok ? size_t(c0 + j) * (D * 2) + c * 16 : 0), ok);
            }
        }
        cp_async_commit();
    };
    issue(0);

    // this warp's 16 rows as A-operand fragments, and their norms
    uint32_t qf[D / 16][4];
    float xn2[2] = {0.f, 0.f};
    {
        const int ra = r0 + warp * 16 + g, rb = ra + 8;
        const T *q0 = ra < row1 ? x + size_t(ra) * D : nullptr;
        const T *q1 = rb < row1 ? x + size_t(rb) * D : nullptr;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int c = ks * 16 + tq * 2;
            qf[ks][0] = q0 ? *reinterpret_cast<const uint32_t *>(q0 + c) : 0u;
            qf[ks][1] = q1 ? *reinterpret_cast<const uint32_t *>(q1 + c) : 0u;
            qf[ks][2] = q0 ? *reinterpret_cast<const uint32_t *>(q0 + c + 8) : 0u;
            qf[ks][3] = q1 ? *reinterpret_cast<const uint32_t *>(q1 + c + 8) : 0u;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const T *h = reinterpret_cast<const T *>(&qf[ks][e]);
                const float a = Elem<T>::to_f32(h[0]), b = Elem<T>::to_f32(h[1]);
                xn2[e & 1] += a * a + b * b;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            xn2[r] += __shfl_xor_sync(0xffffffffu, xn2[r], 1);
            xn2[r] += __shfl_xor_sync(0xffffffffu, xn2[r], 2);
        }
    }

    Top3 top[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) top[r] = Top3{-INFINITY, -INFINITY, -INFINITY, 0, 0};
    const int n_at = (C + kTile - 1) / kTile;
    for (int ta = 0; ta < n_at; ++ta) {
        issue(ta + 1);
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t a_base = smem_base + (ta & 1) * TILE_BYTES;
        const int c0 = ta * kTile;
#pragma unroll
        for (int nt2 = 0; nt2 < kTile / 16; ++nt2) {
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int j = nt2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int c = ks * 2 + ((lane >> 3) & 1);
                uint32_t b[4];
                ldmatrix_x4(b, a_base + swz<D>(j, c));
                mma16816<T>(s0, qf[ks], b[0], b[1]);
                mma16816<T>(s1, qf[ks], b[2], b[3]);
            }
            const int ca = c0 + nt2 * 16 + tq * 2;             // bucket of s0[0] / s0[2]; s1 is 8 further
            if (c0 + nt2 * 16 + 16 > C) {                       // the segment's last, partial group of 16 buckets
                if (ca >= C) { s0[0] = -INFINITY; s0[2] = -INFINITY; }
                if (ca + 1 >= C) { s0[1] = -INFINITY; s0[3] = -INFINITY; }
                if (ca + 8 >= C) { s1[0] = -INFINITY; s1[2] = -INFINITY; }
                if (ca + 9 >= C) { s1[1] = -INFINITY; s1[3] = -INFINITY; }
            }
            // a score enters the top three only if it beats the third: one test for the four scores of a row
            if (fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1])) > top[0].third) {
                top3_push(top[0], s0[0], ca); top3_push(top[0], s0[1], ca + 1);
                top3_push(top[0], s1[0], ca + 8); top3_push(top[0], s1[1], ca + 9);
            }
            if (fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3])) > top[1].third) {
                top3_push(top[1], s0[2], ca); top3_push(top[1], s0[3], ca + 1);
                top3_push(top[1], s1[2], ca + 8); top3_push(top[1], s1[3], ca + 9);
            }
        }
        __syncthreads();                                         // tile consumed before its buffer is refilled
    }
    cp_async_wait<0>();

    const float a_max = __uint_as_float(amax[s]);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
#pragma unroll
        for (int off = 1; off <= 2; off <<= 1) {                 // fold the 4 lanes of the quad that share a row
            const float ob = __shfl_xor_sync(0xffffffffu, top[r].best, off), os = __shfl_xor_sync(0xffffffffu, top[r].second, off);
            const float ot = __shfl_xor_sync(0xffffffffu, top[r].third, off);
            const int oa = __shfl_xor_sync(0xffffffffu, top[r].arg, off), oa2 = __shfl_xor_sync(0xffffffffu, top[r].arg2, off);
            top3_push(top[r], ob, oa);
            top3_push(top[r], os, oa2);
            top3_push(top[r], ot, 0);                           // can only land in `third`, whose index is not kept
        }
        const int row = r0 + warp * 16 + g + 8 * r;
        if (tq == 0 && row < row1) {
            // Scores closer than eps to the best may beat it under the canonical order.  None: done.  Exactly one
            // (the usual near-tie): the two are compared with the fp32 chain right here.  More: full re-check.
            const float eps = kHashEps * sqrtf(xn2[r]) * a_max;
            int choice = top[r].arg;
            if (!(top[r].best - top[r].second > eps)) {
                if (top[r].best - top[r].third > eps) {
                    const T *xr = x + size_t(row) * D;
                    const float y1 = canonical_dot(A + size_t(cb0 + top[r].arg) * D, xr, D);
                    const float y2 = canonical_dot(A + size_t(cb0 + top[r].arg2) * D, xr, D);
                    if (y2 > y1 || (y2 == y1 && top[r].arg2 < top[r].arg)) choice = top[r].arg2;
                } else {
                    recheck[atomicAdd(n_recheck, 1)] = row;
                }
            }
            hash_out[row] = choice;
        }
    }
}

// One CTA per listed row: canonical argmax (fp32 FMA chain per bucket, first maximum wins).  The list is short and
// a chain is a long string of dependent steps, so the row's buckets are spread over the whole CTA and a thread fetches
// a bucket's row in one go (up to 16 loads in flight) before it runs the chain.
constexpr int kRecheckThreads = 256;
template <typename T>
__global__ void __launch_bounds__(kRecheckThreads)
hash_recheck_kernel(const T *__restrict__ x, const T *__restrict__ A, int d, int n_rows, int total_buckets, int n_seg,
                    const int32_t *__restrict__ seg_xb, const int32_t *__restrict__ seg_cb,
                    const int32_t *__restrict__ recheck, const int *__restrict__ n_recheck,
                    int32_t *__restrict__ hash_out)
{
    __shared__ float xs[256];
    __shared__ float wbest[kRecheckThreads / 32];
    __shared__ int warg[kRecheckThreads / 32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int n = min(*n_recheck, n_rows);
    for (int i = blockIdx.x; i < n; i += gridDim.x) {
        const int row = recheck[i];
        const int s = seg_xb ? find_segment(seg_xb, n_seg, row) : 0;
        const int cb0 = seg_cb ? seg_cb[s] : 0;
        const int C = (seg_cb ? seg_cb[s + 1] : total_buckets) - cb0;
        __syncthreads();
        for (int e = t; e < d; e += kRecheckThreads) xs[e] = Elem<T>::to_f32(x[size_t(row) * d + e]);
        __syncthreads();
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int c = t; c < C; c += kRecheckThreads) {
            const T *a = A + size_t(cb0 + c) * d;
            float y = 0.f;
            for (int e0 = 0; e0 < d; e0 += 128) {
                uint4 raw[16];
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (e0 + 8 * u < d) raw[u] = *reinterpret_cast<const uint4 *>(a + e0 + 8 * u);
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (e0 + 8 * u < d) {
                        float f[8];
                        widen8(raw[u], f, T());
#pragma unroll
                        for (int k = 0; k < 8; ++k) y = fmaf(f[k], xs[e0 + 8 * u + k], y);
                    }
            }
            if (y > best || arg == 0x7fffffff) { best = y; arg = c; }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
            if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
        }
        if (lane == 0) { wbest[warp] = best; warg[warp] = arg; }
        __syncthreads();
        if (t == 0) {
            for (int w = 1; w < kRecheckThreads / 32; ++w) {
                const float ob = wbest[w];
                const int oa = warg[w];
                if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
            }
            hash_out[row] = arg == 0x7fffffff ? 0 : arg;
        }
    }
}

// ---- tcgen05 path for large batches of 16-bit rows -----------------------------------------------------------
// The same filter with the scores from the 5th-generation tensor cores: a CTA takes 128 rows (the M side of the MMA,
// loaded once by TMA) and streams the segment's buckets through in tiles of 128 (the N side); the fp32 accumulators
// live in TMEM (two of 128 columns, so the MMAs of one tile run under the scan of the previous one), and each of the
// 128 epilogue threads owns one row - the 32x32b TMEM load hands a thread consecutive columns of its own lane - and
// keeps that row's running top three in registers.  warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 = epilogue.
// Every wait is bounded; if one gives up, the CTA's rows go to the re-check list, which decides them exactly.
constexpr int kThBM = 128, kThBN = 128, kThThreads = 192, kThStages = 2;
constexpr int64_t kTcHashMinRows = 2048;     // below this the set-up of the tcgen05 pipeline does not pay

template <typename T, int D>
__global__ void __launch_bounds__(kThThreads, 2)
hash_rows_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmA, const T *__restrict__ x,
                    const T *__restrict__ A, int n_rows, int total_buckets, const int32_t *__restrict__ seg_xb,
                    const int32_t *__restrict__ seg_cb, const unsigned *__restrict__ amax, int32_t *__restrict__ hash_out,
                    int32_t *__restrict__ recheck, int *__restrict__ n_recheck, uint32_t idesc)
{
    constexpr int KB = D / 64;                               // 64-element (128-byte) k-blocks
    constexpr uint32_t X_BYTES = KB * kThBM * 128, STAGE_BYTES = KB * kThBN * 128;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bars[2 * kThStages + 1 + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;

    const int s = blockIdx.y;
    const int row0 = seg_xb ? seg_xb[s] : 0;
    const int row1 = seg_xb ? seg_xb[s + 1] : n_rows;
    const int cb0 = seg_cb ? seg_cb[s] : 0;
    const int C = (seg_cb ? seg_cb[s + 1] : total_buckets) - cb0;
    const int r0 = row0 + blockIdx.x * kThBM;
    if (r0 >= row1) return;                                  // before any barrier or allocation
    const int n_tiles = (C + kThBN - 1) / kThBN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (tc::smem_addr(smem_dyn) + 1023u) & ~1023u;          // 1024-byte aligned tiles
    const uint32_t x_smem = base, a_smem = base + X_BYTES;
    const uint32_t bar0 = tc::smem_addr(bars);
    auto full_bar = [&](int i) { return bar0 + 8u * i; };
    auto empty_bar = [&](int i) { return bar0 + 8u * (kThStages + i); };
    const uint32_t x_bar = bar0 + 8u * (2 * kThStages);
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kThStages + 1 + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kThStages + 3 + a); };

    if (threadIdx.x == 0) {
        for (int i = 0; i < kThStages; ++i) { tc::mbar_init(full_bar(i), 1); tc::mbar_init(empty_bar(i), 1); }
        tc::mbar_init(x_bar, 1);
        for (int a = 0; a < 2; ++a) { tc::mbar_init(tfull_bar(a), 1); tc::mbar_init(tempty_bar(a), 4); }
        tc::mbar_fence_init();
        s_abort = 0;
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_addr(&tmem_slot), 2 * kThBN);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tc::prefetch_tensormap(&tmX);
            tc::prefetch_tensormap(&tmA);
            tc::mbar_arrive_expect_tx(x_bar, X_BYTES);
            for (int kb = 0; kb < KB; ++kb) tc::tma_load_2d(x_smem + kb * (kThBM * 128), &tmX, kb * 64, r0, x_bar);
            for (int t = 0; t < n_tiles; ++t) {
                const int st = t % kThStages;
                if (!tc::mbar_wait(empty_bar(st), ((t / kThStages) & 1) ^ 1) || *(volatile int *)&s_abort) { s_abort = 1; break; }
                tc::mbar_arrive_expect_tx(full_bar(st), STAGE_BYTES);
                for (int kb = 0; kb < KB; ++kb)
                    tc::tma_load_2d(a_smem + st * STAGE_BYTES + kb * (kThBN * 128), &tmA, kb * 64, cb0 + t * kThBN, full_bar(st));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = tc::mbar_wait(x_bar, 0);
            for (int t = 0; ok && t < n_tiles; ++t) {
                const int st = t % kThStages, acc = t & 1;
                ok = tc::mbar_wait(tempty_bar(acc), ((t >> 1) & 1) ^ 1) && tc::mbar_wait(full_bar(st), (t / kThStages) & 1);
                if (!ok || *(volatile int *)&s_abort) { ok = false; break; }
                tc::fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kThBN;
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t da = tc::smem_desc_sw128(x_smem + kb * (kThBM * 128) + k * 32);
                        const uint64_t db = tc::smem_desc_sw128(a_smem + st * STAGE_BYTES + kb * (kThBN * 128) + k * 32);
                        tc::umma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
                    }
                }
                tc::umma_commit(empty_bar(st));
                tc::umma_commit(tfull_bar(acc));
            }
            if (!ok) s_abort = 1;
        }
    } else {
        const int q = warp & 3;                              // TMEM lane quarter this warp may read
        const int row = r0 + q * 32 + lane;
        const bool row_ok = row < row1;
        Top3 top = Top3{-INFINITY, -INFINITY, -INFINITY, 0, 0};
        bool ok = true;
        for (int t = 0; t < n_tiles; ++t) {
            const int acc = t & 1;
            ok = tc::mbar_wait(tfull_bar(acc), (t >> 1) & 1) && !*(volatile int *)&s_abort;
            ok = __all_sync(0xffffffffu, ok);                // the TMEM loads below need the whole warp
            if (!ok) break;
            tc::fence_after_sync();
            const int c0 = t * kThBN;
#pragma unroll 1
            for (int b = 0; b < kThBN / 32; ++b) {
                uint32_t v[32];
                tc::tmem_ld_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * kThBN + b * 32, v);
                tc::tmem_ld_wait();
                const int cb = c0 + b * 32;
                if (cb + 32 > C) {                           // the segment's last, partial batch: columns of other segments
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (cb + e >= C) v[e] = 0xff800000u;
                }
                // a score enters the top three only if it beats the third: one test per four scores
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float f0 = __uint_as_float(v[4 * j]), f1 = __uint_as_float(v[4 * j + 1]);
                    const float f2 = __uint_as_float(v[4 * j + 2]), f3 = __uint_as_float(v[4 * j + 3]);
                    if (fmaxf(fmaxf(f0, f1), fmaxf(f2, f3)) > top.third) {
                        top3_push(top, f0, cb + 4 * j);
                        top3_push(top, f1, cb + 4 * j + 1);
                        top3_push(top, f2, cb + 4 * j + 2);
                        top3_push(top, f3, cb + 4 * j + 3);
                    }
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tempty_bar(acc));
        }
        if (!ok && lane == 0) s_abort = 1;
        if (row_ok) {
            if (!ok) {
                recheck[atomicAdd(n_recheck, 1)] = row;      // decided exactly by the re-check kernel
                hash_out[row] = 0;
            } else {
                // the row itself is still in shared memory (the M-side tile, 128-byte swizzle: 16-byte chunk c of row m
                // sits at chunk c ^ (m & 7) of the row's 128 bytes inside each 64-element k-block)
                const int m = q * 32 + lane;
                tc::mbar_wait(x_bar, 0);                     // completed long ago: orders this thread after the TMA writes
                const unsigned char *xt = smem_dyn + (x_smem - tc::smem_addr(smem_dyn)) + m * 128;
                auto x_chunk = [&](int e) {                  // elements e .. e + 7 of the row
                    return *reinterpret_cast<const uint4 *>(xt + (e >> 6) * (kThBM * 128) + ((((e >> 3) & 7) ^ (m & 7)) << 4));
                };
                float xn2 = 0.f;
#pragma unroll
                for (int e = 0; e < D; e += 8) {
                    float f[8];
                    widen8(x_chunk(e), f, T());
#pragma unroll
                    for (int u = 0; u < 8; ++u) xn2 = fmaf(f[u], f[u], xn2);
                }
                // Scores closer than eps to the best may beat it under the canonical order.  None: done.  Exactly one
                // (the usual near-tie): the two are compared with the fp32 chain right here.  More: full re-check.
                const float eps = kHashEps * sqrtf(xn2) * 1.0001f * __uint_as_float(amax[s]);
                int choice = top.arg;
                if (!(top.best - top.second > eps)) {
                    if (top.best - top.third > eps) {
                        // both canonical chains at once, the two bucket rows fetched four chunks ahead
                        const T *a1 = A + size_t(cb0 + top.arg) * D, *a2 = A + size_t(cb0 + top.arg2) * D;
                        float y1 = 0.f, y2 = 0.f;
                        for (int e0 = 0; e0 < D; e0 += 32) {
                            uint4 r1[4], r2[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                r1[u] = *reinterpret_cast<const uint4 *>(a1 + e0 + 8 * u);
                                r2[u] = *reinterpret_cast<const uint4 *>(a2 + e0 + 8 * u);
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                float fx[8], f1[8], f2[8];
                                widen8(x_chunk(e0 + 8 * u), fx, T());
                                widen8(r1[u], f1, T());
                                widen8(r2[u], f2, T());
#pragma unroll
                                for (int k = 0; k < 8; ++k) { y1 = fmaf(f1[k], fx[k], y1); y2 = fmaf(f2[k], fx[k], y2); }
                            }
                        }
                        if (y2 > y1 || (y2 == y1 && top.arg2 < top.arg)) choice = top.arg2;
                    } else {
                        recheck[atomicAdd(n_recheck, 1)] = row;
                    }
                }
                hash_out[row] = choice;
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem_base, 2 * kThBN);
}

struct HashLayout { size_t off_amax, off_count, off_list, total; };
static HashLayout hash_layout(int64_t n_rows, int n_seg)
{
    HashLayout L;
    L.off_amax = 0;
    L.off_count = align_up(size_t(n_seg) * 4, 256);
    L.off_list = L.off_count + 256;
    L.total = L.off_list + align_up(size_t(std::max<int64_t>(n_rows, 1)) * 4, 256);
    return L;
}

template <typename T, int D>
static int launch_hash_mma(const void *x, const void *A, int64_t n_rows, int64_t total_buckets, int n_seg,
                           const int32_t *seg_xb, const int32_t *seg_cb, int64_t max_seg_rows, int32_t *hash_out,
                           char *ws, cudaStream_t st)
{
    HashLayout L = hash_layout(n_rows, n_seg);
    unsigned *amax = (unsigned *)(ws + L.off_amax);
    int *count = (int *)(ws + L.off_count);
    int32_t *list = (int32_t *)(ws + L.off_list);
    FM_CUDA_OK(cudaMemsetAsync(ws, 0, L.off_list, st));
    a_norm_max_kernel<T><<<(unsigned)ceil_div(total_buckets, 4), 128, 0, st>>>((const T *)A, (int)total_buckets, D, n_seg, seg_cb, amax);
    FM_LAUNCHED("a_norm_max_kernel");
    if (n_rows >= kTcHashMinRows && (D == 64 || D == 128)) {
        CUtensorMap tmX, tmA;
        int rc = make_tensor_map_2d(&tmX, x, Elem<T>::id, (uint64_t)n_rows, D, (uint64_t)D * 2, kThBM);
        if (rc != FM_OK) return rc;
        rc = make_tensor_map_2d(&tmA, A, Elem<T>::id, (uint64_t)total_buckets, D, (uint64_t)D * 2, kThBN);
        if (rc != FM_OK) return rc;
        const size_t smem = size_t(D / 64) * (kThBM * 128 + kThStages * kThBN * 128) + 1024;
        FM_CUDA_OK(func_attr_cached((const void *)hash_rows_tc_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid((unsigned)ceil_div(max_seg_rows, kThBM), (unsigned)n_seg);
        hash_rows_tc_kernel<T, D><<<grid, kThThreads, smem, st>>>(tmX, tmA, (const T *)x, (const T *)A, (int)n_rows, (int)total_buckets,
                                                                seg_xb, seg_cb, amax, hash_out, list, count,
                                                                tc::instr_desc_f16(Elem<T>::id == FM_BF16, kThBM, kThBN));
        FM_LAUNCHED("hash_rows_tc_kernel");
    } else {
        const size_t smem = 2 * size_t(kTile) * D * 2;
        FM_CUDA_OK(func_attr_cached((const void *)hash_rows_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid((unsigned)ceil_div(max_seg_rows, kTile), (unsigned)n_seg);
        hash_rows_mma_kernel<T, D><<<grid, kHashThreads, smem, st>>>((const T *)x, (const T *)A, (int)n_rows, (int)total_buckets,
                                                                   seg_xb, seg_cb, amax, hash_out, list, count);
        FM_LAUNCHED("hash_rows_mma_kernel");
    }
    const int blocks = (int)std::min<int64_t>(n_rows, int64_t(sm_count()) * 4);
    hash_recheck_kernel<T><<<blocks, kRecheckThreads, 0, st>>>((const T *)x, (const T *)A, D, (int)n_rows, (int)total_buckets, n_seg,
                                                  seg_xb, seg_cb, list, count, hash_out);
    FM_LAUNCHED("hash_recheck_kernel");
    return FM_OK;
}

template <typename T>
static int launch_hash(const void *x, const void *A, int64_t n_rows, int64_t total_buckets, int d, int n_seg,
                       const int32_t *seg_xb, const int32_t *seg_cb, int64_t max_seg_rows, int32_t *hash_out,
                       cudaStream_t st)
{
    size_t smem = tile_smem_bytes(d);
    FM_CUDA_OK(func_attr_cached((const void *)hash_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)ceil_div(max_seg_rows, kTile), (unsigned)n_seg);
    hash_rows_kernel<T><<<grid, kTileThreads, smem, st>>>((const T *)x, (const T *)A, d, (int)n_rows,
                                                         (int)total_buckets, seg_xb, seg_cb, hash_out);
    FM_LAUNCHED("hash_rows_kernel");
    return FM_OK;
}

}  // namespace fm

extern "C" size_t fm_hash_rows_workspace_bytes(int64_t n_rows, int n_seg)
{
    return fm::hash_layout(n_rows, std::max(n_seg, 1)).total;
}

extern "C" int fm_hash_rows(const void *x, const void *A, int dtype, int64_t n_rows, int64_t total_buckets, int d,
                            int n_seg, const int32_t *seg_xb, const int32_t *seg_cb, int64_t max_seg_rows,
                            int32_t *hash_out, void *workspace, size_t workspace_bytes, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(x && A && hash_out && workspace, "fm_hash_rows: null pointer");
    FM_REQUIRE(n_rows >= 0 && total_buckets > 0 && n_seg >= 1, "fm_hash_rows: bad sizes");
    FM_REQUIRE(n_rows < (int64_t(1) << 31) && total_buckets < (int64_t(1) << 31), "fm_hash_rows: sizes exceed int32");
    FM_REQUIRE((seg_xb == nullptr) == (seg_cb == nullptr), "fm_hash_rows: pass both segment arrays or neither");
    FM_REQUIRE(seg_xb || n_seg == 1, "fm_hash_rows: n_seg > 1 needs segment arrays");
    if (d < 16 || d > 256 || d % 16) {
        set_error("fm_hash_rows: head dim %d not supported (multiple of 16 in [16, 256])", d);
        return FM_ERR_UNSUPPORTED;
    }
    if (workspace_bytes < fm_hash_rows_workspace_bytes(n_rows, n_seg)) {
        set_error("fm_hash_rows: workspace %zu < %zu", workspace_bytes, fm_hash_rows_workspace_bytes(n_rows, n_seg));
        return FM_ERR_WORKSPACE;
    }
    if (n_rows == 0) return FM_OK;
    if (max_seg_rows <= 0) max_seg_rows = n_rows;
    cudaStream_t st = (cudaStream_t)stream;
    char *ws = (char *)workspace;
    const bool aligned = ((uintptr_t)x | (uintptr_t)A) % 16 == 0;
    if (dtype == FM_BF16 && aligned && d == 128) return launch_hash_mma<__nv_bfloat16, 128>(x, A, n_rows, total_buckets, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, ws, st);
    if (dtype == FM_BF16 && aligned && d == 64) return launch_hash_mma<__nv_bfloat16, 64>(x, A, n_rows, total_buckets, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, ws, st);
    if (dtype == FM_F16 && aligned && d == 128) return launch_hash_mma<__half, 128>(x, A, n_rows, total_buckets, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, ws, st);
    if (dtype == FM_F16 && aligned && d == 64) return launch_hash_mma<__half, 64>(x, A, n_rows, total_buckets, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, ws, st);
    switch (dtype) {
    case FM_F32: return launch_hash<float>(x, A, n_rows, total_buckets, d, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, st);
    case FM_BF16: return launch_hash<__nv_bfloat16>(x, A, n_rows, total_buckets, d, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, st);
    case FM_F16: return launch_hash<__half>(x, A, n_rows, total_buckets, d, n_seg, seg_xb, seg_cb, max_seg_rows, hash_out, st);
    default: set_error("fm_hash_rows: unknown dtype %d", dtype); return FM_ERR_UNSUPPORTED;
    }
}
