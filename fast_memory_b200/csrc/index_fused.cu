// Fused index build for 16-bit keys (d = 64 / 128): projection on the tcgen05 tensor cores, selection without
// ever writing Y.  Stands in for einsum + topk of the reference (memory.py:261, 273; triton_kernel.py:277-278).
//
//   1. key_norm_max:   kmax_s = max_j ||k_j|| per segment (bounds the accumulation error of a score).
//   2. sample scores:  tensor-core projection of every `step`-th key (dense epilogue, small).
//   3. thresholds:     tau_b = the r-th largest sample score of bucket b, r chosen so that about
//                      (r / z) Z keys pass and fewer than Z pass with probability ~1e-6 per bucket (z = Z / step;
//                      such a bucket goes to the fallback).
//   4. candidates:     tensor-core projection of ALL keys; the epilogue appends every group of four consecutive
//                      keys with a score >= tau_b (the four scores) to the bucket's candidate list, in key order,
//                      and records the group in a bit mask per (bucket, key tile).
//   5. selection:      per bucket, theta = Z-th largest candidate score.  Scores come from the tensor cores
//                      (hardware summation order), so only candidates whose score is outside
//                      [theta - eps, theta + eps] are decided by them; the band in between is re-scored
//                      with the canonical fp32 chain and ranked exactly (lower index wins ties).  The table row
//                      (ascending key rows) is therefore bit-identical to the all-fp32 build.
//   6. fallback:       a bucket whose list overflowed, or whose threshold was too high to prove completeness,
//                      is rebuilt from canonical scores of all its segment's keys.
#include "index_fused.cuh"
#include "simt_tile.cuh"
#include "tc_project.cuh"
#include "topz_row.cuh"

#include <cmath>
#include <cstring>
#include <mutex>
#include <vector>

namespace fm {

// eps = kBandEps * ||a_b|| * kmax.  A tensor-core score is within 2^-16 M of the exact dot product and the
// canonical chain within 2^-17 M (M = ||a|| ||k|| >= sum |a_i k_i|, d <= 128), so two keys can compare
// differently under the two orders only if their tensor-core scores differ by less than 3 * 2^-16 M; the band's
// half-width is 4 * 2^-16 M.  (Measured on 2.7e8 scores of the benchmark data: the two differ by at most 2^-21.9 M.)
// The band is what the selection re-scores with the canonical chain, about 20 keys per bucket on the benchmark.
constexpr float kBandEps = 1.0f / 16384.0f;
constexpr int kMaxBand = 512;               // largest band re-scored exactly; beyond it the bucket goes to the fallback
constexpr int kMaxFail = 64;                // buckets the fallback can take per group of segments
constexpr int kMaxSample = 49152;           // sample scores of one bucket (the key step is raised to stay below it)
constexpr int kMaxRanges = 8;               // key ranges a bucket tile's keys may be split into (one CTA each)

struct FusedSeg {
    int kb, n_keys;            // first key row (absolute), key count
    int cb, n_buckets;         // first bucket (global), bucket count
    int zc;                    // min(Z, N)
    int rank;                  // which sample order statistic is the threshold (1 = largest)
    int ns0, ns;               // first sampled row in units of `step`, number of sampled rows
    int out_row0;              // first bucket of the segment inside the group's arrays
    unsigned kmax_bits;        // max key norm, as float bits (atomicMax)
    long long table_off;       // where the segment's table starts
};

// ---- 1. max key norm per segment ---------------------------------------------------------------------------
// Sum of squares of the eight elements of a 16-byte piece, never more than 2 % below the exact value.  bf16: packed
// multiply-adds (four instructions for the eight elements; every step rounds to 8 bits: at most 2^-9 relative each).
__device__ __forceinline__ float piece_norm2(const uint4 &raw, __nv_bfloat16)
{
    const __nv_bfloat162 *x = reinterpret_cast<const __nv_bfloat162 *>(&raw);
    __nv_bfloat162 acc = __hmul2(x[0], x[0]);
    acc = __hfma2(x[1], x[1], acc);
    acc = __hfma2(x[2], x[2], acc);
    acc = __hfma2(x[3], x[3], acc);
    return __low2float(acc) + __high2float(acc);
}
__device__ __forceinline__ float piece_norm2(const uint4 &raw, __half)      // (fp16 sums would overflow: fp32)
{
    float f[8];
    widen8(raw, f, __half());
    float n2 = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) n2 = fmaf(f[e], f[e], n2);
    return n2;
}

// One CTA per SM, no shared memory: the kernel runs on a second stream beside the candidate projection, whose CTAs take
// nearly all of an SM's shared memory (one CTA of this kernel still fits) but leave most of the memory bandwidth idle.
// What it costs the projection is issue slots (the projection's epilogue warps are its bottleneck), so the kernel is
// written for few instructions per byte: packed squares, and ONE reduction over the lanes for four rows (a butterfly
// that halves the number of live values at each of its first two steps).  The result only scales the band of the
// selection and is inflated by 3 %.
template <typename T>
__global__ void __launch_bounds__(512) key_norm_max_kernel(const T *__restrict__ K, int d, FusedSeg *__restrict__ segs, int n_seg)
{
    const int lanes_per_row = d / 8;                         // 16-byte pieces per row: 8 or 16
    const int rows_per_warp = 32 / lanes_per_row;
    const int lane = threadIdx.x & 31, sub = lane % lanes_per_row, rsel = lane / lanes_per_row;
    const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * (blockDim.x >> 5);
    const int stride = n_warps * rows_per_warp;
    for (int s = 0; s < n_seg; ++s) {
        const int kb = segs[s].kb, n_keys = segs[s].n_keys;
        float best = 0.f;
        // four rows per iteration: the loads are issued together, which is what keeps enough bytes in flight
        for (int r0 = warp_global * rows_per_warp + rsel; r0 < n_keys; r0 += 4 * stride) {
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int r = r0 + u * stride;
                // (streaming loads: the rows are marked to leave L2 first, where the projection keeps the key tiles its CTAs share)
                raw[u] = r < n_keys ? __ldcs(reinterpret_cast<const uint4 *>(K + size_t(kb + r) * d + sub * 8)) : make_uint4(0, 0, 0, 0);
            }
            float n0 = piece_norm2(raw[0], T()), n1 = piece_norm2(raw[1], T()), n2 = piece_norm2(raw[2], T()), n3 = piece_norm2(raw[3], T());
            // lanes with bit 0 clear go on with rows 0 and 1, the others with rows 2 and 3; then bit 1 splits again
            const bool odd = sub & 1;
            const float k0 = odd ? n2 : n0, k1 = odd ? n3 : n1, s0 = odd ? n0 : n2, s1 = odd ? n1 : n3;
            const float a0 = k0 + __shfl_xor_sync(0xffffffffu, s0, 1), a1 = k1 + __shfl_xor_sync(0xffffffffu, s1, 1);
            const bool hi = sub & 2;
            float b = (hi ? a1 : a0) + __shfl_xor_sync(0xffffffffu, hi ? a0 : a1, 2);
            for (int off = 4; off < lanes_per_row; off <<= 1) b += __shfl_xor_sync(0xffffffffu, b, off);
            best = fmaxf(best, b);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, off));
        if (lane == 0 && best > 0.f) atomicMax(&segs[s].kmax_bits, __float_as_uint(sqrtf(best) * 1.03f));
    }
}

__device__ __forceinline__ int seg_of_out_row(const FusedSeg *__restrict__ segs, int n_seg, int row)
{
    int lo = 0, hi = n_seg;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (segs[mid].out_row0 <= row) lo = mid; else hi = mid;
    }
    return lo;
}

// ---- 3. (the thresholds come from tc_tau.cu) helpers of the selection --------------------------------------------------
// Values held in shared memory.
struct SmemValues {
    const float *v;
    int n;
    template <class F> __device__ __forceinline__ void for_each(F f) const
    {
        for (int i = threadIdx.x; i < n; i += blockDim.x) f(i, v[i]);
    }
};

// ---- block-wide helpers of the selection kernels -------------------------------------------------------------------
// Exclusive prefix sum of one int per thread over the CTA (any multiple of 32 threads up to 1024); `total` receives the sum.
// `ws` holds 33 ints.  Three barriers.
__device__ __forceinline__ int block_exclusive_scan(int v, int *ws, int &total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += o;
    }
    __syncthreads();                                         // ws may still be read by an earlier call
    if (lane == 31) ws[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int w = lane < nw ? ws[lane] : 0;
        int winc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, winc, off);
            if (lane >= off) winc += o;
        }
        ws[lane] = winc - w;
        if (lane == 31) ws[32] = winc;
    }
    __syncthreads();
    total = ws[32];
    return ws[warp] + incl - v;
}

// The same with ONE barrier: every warp adds up the warp totals for itself.  `ws` holds 32 ints; two calls in a row
// without a barrier between them must use different arrays (a slow warp may still be reading the first).
__device__ __forceinline__ int block_exclusive_scan1(int v, int *ws, int &total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += o;
    }
    if (lane == 31) ws[warp] = incl;
    __syncthreads();
    const int w = lane < nw ? ws[lane] : 0;
    int winc = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, winc, off);
        if (lane >= off) winc += o;
    }
    total = __shfl_sync(0xffffffffu, winc, 31);
    return __shfl_sync(0xffffffffu, winc - w, warp) + incl - v;
}

// The r-th largest of the n floats in shared memory `vals` (n >= r >= 1, all inside [lo, hi]) by ONE warp, without a
// CTA-wide barrier: a 256-bin histogram finds the bin, its members (few when n is a few hundred) are ranked directly.
// `hist` holds 256 ints, `small` kWarpSmall floats, `ctl` 2 ints.  When more than kWarpSmall values crowd the bin
// the smallest of them is returned (at most the r-th largest) and `exact` is cleared.  Every lane returns the result.
constexpr int kWarpSmall = 128;

__device__ __forceinline__ float warp_select_small(const float *vals, int n, int r, float lo, float hi, int *hist, float *small,
                                                   int *ctl, bool &exact)
{
    const int lane = threadIdx.x & 31;
    exact = true;
    if (!(hi > lo)) return lo;
    for (int i = lane; i < 256; i += 32) hist[i] = 0;
    if (lane == 0) { ctl[0] = 0; ctl[1] = 0; }
    __syncwarp();
    const float scale = 256.f / (hi - lo);
    for (int i = lane; i < n; i += 32) atomicAdd(&hist[min(255, int((vals[i] - lo) * scale))], 1);
    __syncwarp();
    int mine = 0;                                            // lane 0 owns the 8 highest bins
#pragma unroll
    for (int k = 0; k < 8; ++k) mine += hist[255 - (lane * 8 + k)];
    int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += o;
    }
    int bin = -1, want = 0;
    {
        int acc = incl - mine;
        if (acc < r && r <= incl) {
            for (int k = 0; k < 8; ++k) {
                const int b = 255 - (lane * 8 + k);
                if (r <= acc + hist[b]) { bin = b; want = r - acc; break; }
                acc += hist[b];
            }
        }
    }
    const unsigned owner = __ballot_sync(0xffffffffu, bin >= 0);
    const int src_lane = __ffs(owner) - 1;
    bin = __shfl_sync(0xffffffffu, bin, src_lane);
    want = __shfl_sync(0xffffffffu, want, src_lane);
    float mmin = INFINITY;
    for (int i = lane; i < n; i += 32) {
        const float v = vals[i];
        if (min(255, int((v - lo) * scale)) == bin) {
            const int slot = atomicAdd(&ctl[0], 1);
            if (slot < kWarpSmall) small[slot] = v;
            mmin = fminf(mmin, v);
        }
    }
    __syncwarp();
    const int cnt = ctl[0];
    if (cnt > kWarpSmall) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) mmin = fminf(mmin, __shfl_xor_sync(0xffffffffu, mmin, off));
        exact = false;
        return mmin;
    }
    float theta = -INFINITY;
    for (int i = lane; i < cnt; i += 32) {
        const float v = small[i];
        int gt = 0, eq = 0;
        for (int o = 0; o < cnt; ++o) { gt += small[o] > v; eq += small[o] == v; }
        if (gt < want && want <= gt + eq) theta = v;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) theta = fmaxf(theta, __shfl_xor_sync(0xffffffffu, theta, off));
    return theta;
}

// The r-th largest of the floats a value source yields (at least r of them), all of them inside [lo, hi]; a source exposes
//  template <class F> void for_each(F f)  which calls f(ordinal, value) for the values this thread owns.  One histogram of
// kFineBins linear bins finds the bin that holds it; the members of that bin are ranked directly when they are few, else
// the bin is cut into kFineBins finer ones (a few rounds at most: scores near a threshold crowd a narrow interval).
// If the crowd does not thin out the lower edge of the bin is returned, which is at most the r-th largest - callers
// that need the exact order statistic pass exact = true and get `ok = false` then.  Every thread returns the same value.
constexpr int kFineBins = 2048;
constexpr int kFineSmall = 512;

struct FineScratch {
    int hist[kFineBins];
    float small[kFineSmall];
    float wsmall[kWarpSmall];
    int scan[33];
    int bin, want, count, n_small, exact;
    int ctl[2];
    float theta, mlo, mhi;
};

template <class Source>
__device__ __forceinline__ float select_rth_fine(const Source &src, int r, float lo, float hi, FineScratch &S, bool &ok)
{
    const int t = threadIdx.x, nthreads = blockDim.x;
    int want = r;
    ok = true;
    for (int round = 0; round < 6; ++round) {
        if (!(hi > lo)) return lo;                           // everything left is one value
        __syncthreads();
        for (int i = t; i < kFineBins; i += nthreads) S.hist[i] = 0;
        __syncthreads();
        const float scale = float(kFineBins) / (hi - lo);
        src.for_each([&](int, float v) {
            if (v >= lo && v <= hi) atomicAdd(&S.hist[min(kFineBins - 1, int((v - lo) * scale))], 1);
        });
        __syncthreads();
        // suffix sums from the top: thread t owns `per` consecutive bins, highest bins in thread 0
        const int per = (kFineBins + nthreads - 1) / nthreads;
        int mine = 0;
        for (int k = 0; k < per; ++k) {
            const int b = kFineBins - 1 - (t * per + k);
            mine += b >= 0 ? S.hist[b] : 0;
        }
        int total;
        const int above = block_exclusive_scan(mine, S.scan, total);
        if (mine > 0 && above < want && want <= above + mine) {
            int acc = above;
            for (int k = 0; k < per; ++k) {
                const int b = kFineBins - 1 - (t * per + k);
                const int h = b >= 0 ? S.hist[b] : 0;
                if (want <= acc + h) { S.bin = b; S.want = want - acc; S.count = h; break; }
                acc += h;
            }
        }
        if (t == 0) S.n_small = 0;
        __syncthreads();
        const int bin = S.bin, cnt = S.count;
        want = S.want;
        if (cnt <= kFineSmall) {
            // the bin's members go to a list that warp 0 ranks by itself
            float mlo = INFINITY, mhi = -INFINITY;
            src.for_each([&](int, float v) {
                if (v >= lo && v <= hi && min(kFineBins - 1, int((v - lo) * scale)) == bin) {
                    S.small[atomicAdd(&S.n_small, 1)] = v;
                    mlo = fminf(mlo, v);
                    mhi = fmaxf(mhi, v);
                }
            });
            if (cnt > 32) {                                  // (a handful is ranked without knowing its range)
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    mlo = fminf(mlo, __shfl_xor_sync(0xffffffffu, mlo, off));
                    mhi = fmaxf(mhi, __shfl_xor_sync(0xffffffffu, mhi, off));
                }
                float *red = reinterpret_cast<float *>(S.hist);   // the histogram has been consumed
                __syncthreads();
                if ((t & 31) == 0) { red[t >> 5] = mlo; red[32 + (t >> 5)] = mhi; }
            }
            __syncthreads();
            if (t < 32) {
                float th;
                bool ex = true;
                if (cnt > 32) {
                    const float *red = reinterpret_cast<const float *>(S.hist);
                    mlo = INFINITY; mhi = -INFINITY;
                    for (int w = 0; w < (nthreads >> 5); ++w) { mlo = fminf(mlo, red[w]); mhi = fmaxf(mhi, red[32 + w]); }
                    __syncwarp();
                    th = warp_select_small(S.small, cnt, want, mlo, mhi, S.hist + 128, S.wsmall, S.ctl, ex);
                } else {
                    th = -INFINITY;
                    for (int i = t; i < cnt; i += 32) {
                        const float v = S.small[i];
                        int gt = 0, eq = 0;
                        for (int o = 0; o < cnt; ++o) { gt += S.small[o] > v; eq += S.small[o] == v; }
                        if (gt < want && want <= gt + eq) th = v;
                    }
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) th = fmaxf(th, __shfl_xor_sync(0xffffffffu, th, off));
                }
                if (t == 0) { S.theta = th; S.exact = ex ? 1 : 0; }
            }
            __syncthreads();
            ok = S.exact != 0;
            return S.theta;
        }
        // narrow to the exact value range of the bin's members
        float nlo = INFINITY, nhi = -INFINITY;
        src.for_each([&](int, float v) {
            if (v >= lo && v <= hi && min(kFineBins - 1, int((v - lo) * scale)) == bin) { nlo = fminf(nlo, v); nhi = fmaxf(nhi, v); }
        });
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            nlo = fminf(nlo, __shfl_xor_sync(0xffffffffu, nlo, off));
            nhi = fmaxf(nhi, __shfl_xor_sync(0xffffffffu, nhi, off));
        }
        float *red = reinterpret_cast<float *>(S.hist);       // the histogram has been consumed
        __syncthreads();
        if ((t & 31) == 0) { red[t >> 5] = nlo; red[32 + (t >> 5)] = nhi; }
        __syncthreads();
        nlo = INFINITY; nhi = -INFINITY;
        for (int w = 0; w < (nthreads >> 5); ++w) { nlo = fminf(nlo, red[w]); nhi = fmaxf(nhi, red[32 + w]); }
        lo = nlo; hi = nhi;
    }
    ok = false;                                              // masses of nearly equal values
    return lo;
}

// ---- 5. exact selection among the candidates ---------------------------------------------------------------------
struct SelParams {
    const FusedSeg *segs;
    int n_seg;
    int n_ranges, cap;
    const uint4 *cand;         // groups of four scores
    const uint2 *cand_mask;    // [key tile][mask_ld] the groups of every tile that were appended (one bit each)
    int64_t mask_ld;           // rows
    const int *cand_count;     // [rows][n_ranges][2]
    const float *tau;
    const void *A, *K;
    int d;
    int32_t *table;
    int *fail_count;           // buckets handed to the fallback
    int *fail_list;            // their rows inside the group
    int max_tiles;             // key tiles of the longest segment (sizes the mask arrays in shared memory)
};

// One CTA per bucket.  The bucket's candidate groups - sub-lists (range 0, group 0), (range 0, group 1), (range 1,
// group 0), ...; group 0 of a range was written upward from the start of the range's buffer, group 1 downward from
// its end, so concatenated in this order they are in key order - are dealt out in key order, E consecutive entries per
// thread.  That makes every ordered step a matter of one count per thread and one prefix sum over the CTA:
//   1. the tile masks go to shared memory with their prefix population counts (entry ordinal -> key tile and bit);
//   2. every thread loads its entries (KEEP: they stay in registers; otherwise they are read a second time in step 3)
//      and counts the scores that reach tau; a prefix sum gives each thread its place among the hits;
//   3. the hits are written, in key order, to shared memory with their key indices (found by walking the masks from
//      the thread's first entry);
//   4. theta = the Z-th largest hit (histogram of 2048 bins over the hits' range, refined inside one bin);
//   5. hits above theta + eps are in, the band around theta is re-scored with the canonical chain and ranked exactly;
//   6. every thread counts the selected hits of its stretch of positions, a prefix sum places them, and the table row
//      comes out in ascending key order.
template <typename T, int THREADS, int EMAX, bool KEEP>
__global__ void __launch_bounds__(THREADS, (KEEP ? 1024 : 1536) / THREADS)
candidate_select_kernel(SelParams p)
{
    extern __shared__ __align__(16) unsigned char sel_dyn[];
    float *cy = reinterpret_cast<float *>(sel_dyn);                     // [cap] candidate scores, in key order
    int *cid = reinterpret_cast<int *>(cy + p.cap);                     // [cap] their key indices; bit 31 = band entry that made it
    unsigned long long *m64 = reinterpret_cast<unsigned long long *>(cid + p.cap + (p.cap & 1));   // [n_tiles] tile masks
    int *tile_pre = reinterpret_cast<int *>(m64 + p.max_tiles);         // [n_tiles + 1] entries before each tile
    __shared__ FineScratch S;
    __shared__ int band[kMaxBand];                                      // positions of the band entries in cy / cid
    __shared__ float band_y[kMaxBand];                                  // their canonical scores
    __shared__ int band_rank[kMaxBand];
    __shared__ float a_f32[256];
    __shared__ float red_s[64];
    __shared__ int scan_ws[2][32];
    __shared__ int s_fail, s_nband, s_nent, s_in;
    __shared__ int s_start[2 * kMaxRanges + 1];                         // entries before each sub-list
    __shared__ float s_anorm;

    const int row = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    constexpr int nthreads = THREADS, nwarps = THREADS / 32;
    const FusedSeg sg = p.segs[seg_of_out_row(p.segs, p.n_seg, row)];
    if (row - sg.out_row0 >= sg.n_buckets) return;           // padding between segments
    const int bucket = sg.cb + (row - sg.out_row0);
    const int Z = sg.zc;
    const T *a_row = reinterpret_cast<const T *>(p.A) + size_t(bucket) * p.d;
    const int sub_cap = p.cap / p.n_ranges;
    const int n_sl = 2 * p.n_ranges;
    const uint4 *lists = p.cand + size_t(row) * p.cap;
    const float tau = p.tau[row];
    const int n_tiles = (sg.n_keys + kTcBN - 1) / kTcBN;

    // ---- 1. sub-list sizes (the two groups of a range share a buffer and must not have met in the middle); masks ----
    if (t == 0) {
        int n = 0, fail = 0;
        for (int r = 0; r < p.n_ranges; ++r) {
            const int c0 = p.cand_count[(size_t(row) * p.n_ranges + r) * 2], c1 = p.cand_count[(size_t(row) * p.n_ranges + r) * 2 + 1];
            if (c0 > sub_cap || c1 > sub_cap || c0 + c1 > sub_cap) fail = 1;
            s_start[2 * r] = n;      n += c0;
            s_start[2 * r + 1] = n;  n += c1;
        }
        s_start[n_sl] = n;
        if (n > EMAX * THREADS) fail = 1;
        s_nent = fail ? 0 : n;
        s_fail = fail;
        s_nband = 0;
        s_in = 0;
    }
    for (int i = t; i < p.d; i += nthreads) a_f32[i] = Elem<T>::to_f32(a_row[i]);
    {
        const uint2 *mcol = p.cand_mask + row;
        for (int tile = t; tile < n_tiles; tile += nthreads) {
            const uint2 w = mcol[size_t(tile) * p.mask_ld];
            m64[tile] = (unsigned long long)w.x | ((unsigned long long)w.y << 32);
        }
    }
    __syncthreads();
    if (warp == 0) {                                         // ||a_b||
        float n2 = 0.f;
        for (int i = lane; i < p.d; i += 32) n2 = fmaf(a_f32[i], a_f32[i], n2);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, off);
        if (lane == 0) s_anorm = sqrtf(n2) * 1.0001f;
    }
    const int n_ent = s_nent;
    // ---- 2. this thread's entries [e0, e1), in key order; entries before each key tile --------------------------------
    const int E = (n_ent + nthreads - 1) / nthreads;
    const int e0 = min(n_ent, t * E), e1 = min(n_ent, e0 + E);
    auto entry_ptr = [&](int e, int &sl) {                   // sl: sub-list of e, carried from the previous entry
        while (e >= s_start[sl + 1]) ++sl;
        const int j = e - s_start[sl], cnt = s_start[sl + 1] - s_start[sl];
        (void)cnt;
        return lists + size_t(sl >> 1) * sub_cap + ((sl & 1) ? sub_cap - 1 - j : j);
    };
    uint4 ent[KEEP ? EMAX : 1];
    int my_hits = 0;
    float hmax = -INFINITY;
    if constexpr (KEEP) {                                    // ask for the entries now: they arrive while the masks are summed up
#pragma unroll
        for (int u = 0; u < EMAX; ++u) ent[u] = make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u);
        if (e0 < e1) {
            int sl = 0;
            const uint4 *first = entry_ptr(e0, sl);
            if (e1 <= s_start[sl + 1]) {                     // the usual case: one sub-list holds the whole stretch
                const int step = (sl & 1) ? -1 : 1;
#pragma unroll
                for (int u = 0; u < EMAX; ++u)
                    if (e0 + u < e1) ent[u] = first[u * step];
            } else {
#pragma unroll
                for (int u = 0; u < EMAX; ++u)
                    if (e0 + u < e1) ent[u] = *entry_ptr(e0 + u, sl);
            }
        }
    }
    {
        // entries before every tile: a stretch of consecutive tiles per thread, then a prefix sum over the threads
        const int per_t = (n_tiles + nthreads - 1) / nthreads;
        const int t0 = min(n_tiles, t * per_t), t1 = min(n_tiles, t0 + per_t);
        int c = 0;
        for (int tile = t0; tile < t1; ++tile) c += __popcll(m64[tile]);
        int total;
        int before = block_exclusive_scan1(c, scan_ws[0], total);
        for (int tile = t0; tile < t1; ++tile) { tile_pre[tile] = before; before += __popcll(m64[tile]); }
        if (t == 0) {
            tile_pre[n_tiles] = total;
            if (total != n_ent) s_fail = 1;                  // masks and list lengths disagree (an overflowed list)
        }
    }
    // hits = scores that reach tau.  Their range for the selection is [tau, largest score]: no score below tau is
    // larger than a hit, so the maximum needs no predicate.
    if constexpr (KEEP) {
#pragma unroll
        for (int u = 0; u < EMAX; ++u) {
            const float f[4] = {__uint_as_float(ent[u].x), __uint_as_float(ent[u].y), __uint_as_float(ent[u].z), __uint_as_float(ent[u].w)};
#pragma unroll
            for (int k = 0; k < 4; ++k) my_hits += f[k] >= tau ? 1 : 0;
            hmax = fmaxf(fmaxf(hmax, fmaxf(f[0], f[1])), fmaxf(f[2], f[3]));
        }
    } else {
        int sl = 0;
        for (int e = e0; e < e1; ++e) {
            const uint4 x = *entry_ptr(e, sl);
            const float f[4] = {__uint_as_float(x.x), __uint_as_float(x.y), __uint_as_float(x.z), __uint_as_float(x.w)};
#pragma unroll
            for (int k = 0; k < 4; ++k) my_hits += f[k] >= tau ? 1 : 0;
            hmax = fmaxf(fmaxf(hmax, fmaxf(f[0], f[1])), fmaxf(f[2], f[3]));
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, off));
    if (lane == 0) red_s[warp] = hmax;
    int n;
    int pos = block_exclusive_scan1(my_hits, scan_ws[1], n);    // (its barrier also publishes red_s and s_fail)
    hmax = lane < nwarps ? red_s[lane] : -INFINITY;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, off));
    const float hmin = tau;
    if (t == 0 && (n < Z || n > p.cap)) s_fail = 1;
    __syncthreads();

    if (!s_fail) {
        // ---- 3. the hits with their key indices, in key order --------------------------------------------------------
        if (e0 < e1) {
            int lo = 0, hi = n_tiles;                        // largest tile with tile_pre[tile] <= e0
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (tile_pre[mid] <= e0) lo = mid; else hi = mid;
            }
            int tile = lo;
            unsigned long long m = m64[tile];
            for (int skip = e0 - tile_pre[tile]; skip > 0; --skip) m &= m - 1;
            int sl = 0;
            auto emit = [&](const uint4 &x) {
                while (m == 0) m = m64[++tile];              // ends inside the masks: their population is n_ent
                const int key0 = tile * kTcBN + 4 * (__ffsll((long long)m) - 1);
                m &= m - 1;
                const uint32_t s4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float y = __uint_as_float(s4[k]);
                    if (y >= tau) { cy[pos] = y; cid[pos] = key0 + k; ++pos; }
                }
            };
            if constexpr (KEEP) {
#pragma unroll
                for (int u = 0; u < EMAX; ++u)
                    if (e0 + u < e1) emit(ent[u]);
            } else {
                for (int e = e0; e < e1; ++e) emit(*entry_ptr(e, sl));
            }
        }
        __syncthreads();

        // ---- 4. theta ---------------------------------------------------------------------------------------------
        bool exact = true;
        const float theta = select_rth_fine(SmemValues{cy, n}, Z, hmin, hmax, S, exact);
        const float eps = kBandEps * s_anorm * __uint_as_float(sg.kmax_bits);
        const float lo = theta - eps, hi = theta + eps;
        // everything at or above lo has to be among the candidates, i.e. the threshold was low enough
        if (t == 0 && (!exact || (!(tau <= lo) && n < sg.n_keys))) s_fail = 1;

        // ---- 5. certain entries (score > hi) and the band [lo, hi], per stretch of positions --------------------------
        const int per = ((n + nthreads - 1) / nthreads) | 1;               // odd: stretches start in different banks
        const int i0 = min(n, t * per), i1 = min(n, i0 + per);
        int my_in = 0;
        for (int i = i0; i < i1; ++i) {
            const float y = cy[i];
            if (y > hi) ++my_in;
            else if (y >= lo) {
                const int slot = atomicAdd(&s_nband, 1);
                if (slot < kMaxBand) band[slot] = i;
            }
        }
        my_in = __reduce_add_sync(0xffffffffu, my_in);
        if (lane == 0 && my_in) atomicAdd(&s_in, my_in);
        __syncthreads();
        const int total_in = s_in;
        const int n_band = s_nband, need = Z - total_in;
        if (t == 0 && (n_band > kMaxBand || need < 0 || need > n_band)) s_fail = 1;
        __syncthreads();
        if (!s_fail) {
            // canonical scores of the band, then an exact rank: better = larger score, then lower key index
            const T *Kseg = reinterpret_cast<const T *>(p.K) + size_t(sg.kb) * p.d;
            // four lanes per key row: each loads a quarter of the row (all loads in flight together), then the
            // chain runs through the quarters in order, handed from lane to lane
            const int quarter = p.d / 4, sub = lane & 3;
            for (int b0 = 0; b0 < n_band; b0 += nthreads / 4) {
                if (b0 + warp * 8 >= n_band) break;          // this warp's eight entries lie beyond the band
                const int b = b0 + (t >> 2);
                const T *krow = Kseg + size_t(cid[band[min(b, n_band - 1)]]) * p.d + sub * quarter;
                uint4 raw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (u * 8 < quarter) raw[u] = *reinterpret_cast<const uint4 *>(krow + u * 8);
                float y = 0.f;
                for (int step = 0; step < 4; ++step) {
                    if (sub == step) {
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (u * 8 < quarter) {
                                float f[8];
                                if constexpr (sizeof(T) == 2) widen8(raw[u], f, T());
#pragma unroll
                                for (int k = 0; k < 8; ++k) y = fmaf(a_f32[sub * quarter + u * 8 + k], f[k], y);
                            }
                    }
                    y = __shfl_sync(0xffffffffu, y, (lane & ~3) | step);      // the chain so far, to every lane of the four
                }
                if (b < n_band && sub == 0) { band_y[b] = y; band_rank[b] = 0; }
            }
            __syncthreads();
            {
                const int parts = max(1, nthreads / max(n_band, 1));
                for (int w = t; w < n_band * parts; w += nthreads) {
                    const int b = w / parts, part = w - b * parts;
                    const float y = band_y[b];
                    const int id = cid[band[b]];
                    int rank = 0;
                    for (int o = part; o < n_band; o += parts) {
                        const float yo = band_y[o];
                        rank += (yo > y) || (yo == y && cid[band[o]] < id);
                    }
                    if (rank) atomicAdd(&band_rank[b], rank);
                }
            }
            __syncthreads();
            for (int b = t; b < n_band; b += nthreads)
                if (band_rank[b] < need) cid[band[b]] |= int(0x80000000u);
            __syncthreads();
            // ---- 6. ordered write: the candidates are in key order, so is the table row ------------------------------
            int my_sel = 0;
            for (int i = i0; i < i1; ++i) {
                const float y = cy[i];
                my_sel += (y > hi || (y >= lo && cid[i] < 0)) ? 1 : 0;
            }
            int total_sel;
            int out_pos = block_exclusive_scan1(my_sel, scan_ws[0], total_sel);
            int32_t *out = p.table + sg.table_off + size_t(row - sg.out_row0) * Z;
            for (int i = i0; i < i1; ++i) {
                const float y = cy[i];
                const int id = cid[i];
                if (y > hi || (y >= lo && id < 0)) {
                    if (out_pos < Z) out[out_pos] = sg.kb + (id & 0x7fffffff);
                    ++out_pos;
                }
            }
            if (t == 0 && total_sel != Z) s_fail = 1;
        }
    }
    __syncthreads();
    if (t == 0 && s_fail) {
        const int slot = atomicAdd(p.fail_count, 1);
        if (slot < kMaxFail) p.fail_list[slot] = row;
    }
}

template <typename T, int THREADS, int EMAX, bool KEEP>
static int launch_select(const SelParams &sp, unsigned rows, size_t dyn, cudaStream_t st)
{
    FM_CUDA_OK(func_attr_cached((const void *)candidate_select_kernel<T, THREADS, EMAX, KEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    candidate_select_kernel<T, THREADS, EMAX, KEEP><<<rows, THREADS, dyn, st>>>(sp);
    FM_LAUNCHED("candidate_select_kernel");
    return FM_OK;
}

// ---- 6. fallback: canonical scores of a whole segment for the listed buckets, then the exact row select ---------
template <typename T>
__global__ void fallback_scores_kernel(const FusedSeg *__restrict__ segs, int n_seg, const int *__restrict__ fail_count,
                                       const int *__restrict__ fail_list, const T *__restrict__ A, const T *__restrict__ K, int d,
                                       float *__restrict__ Yf, int64_t ldf)
{
    const int n_fail = min(*fail_count, kMaxFail);
    for (int f = blockIdx.y; f < n_fail; f += gridDim.y) {   // (no failures as a rule: the grid is kept small)
        const int row = fail_list[f];
        const FusedSeg sg = segs[seg_of_out_row(segs, n_seg, row)];
        const T *a_row = A + size_t(sg.cb + (row - sg.out_row0)) * d;
        for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < sg.n_keys; j += gridDim.x * blockDim.x)
            Yf[size_t(f) * ldf + j] = canonical_dot(a_row, K + size_t(sg.kb + j) * d, d);
    }
}

__global__ void __launch_bounds__(kSelThreads)
fallback_select_kernel(const FusedSeg *__restrict__ segs, int n_seg, const int *__restrict__ fail_count,
                       const int *__restrict__ fail_list, const float *__restrict__ Yf, int64_t ldf, int32_t *__restrict__ table,
                       int *__restrict__ status)
{
    if (blockIdx.x == 0 && threadIdx.x == 0 && *fail_count > kMaxFail) atomicExch(status, 4);
    if ((int)blockIdx.x >= min(*fail_count, kMaxFail)) return;
    const int row = fail_list[blockIdx.x];
    const FusedSeg sg = segs[seg_of_out_row(segs, n_seg, row)];
    topz_row(Yf + size_t(blockIdx.x) * ldf, sg.n_keys, sg.zc, sg.kb, table + sg.table_off + size_t(row - sg.out_row0) * sg.zc);
}

// ---- host ----------------------------------------------------------------------------------------------------------
bool fused_eligible(int dtype, int d, int64_t n_keys, int64_t zc)
{
    // buckets much smaller than the segment (otherwise a threshold filters nothing), yet not so small that the
    // key sample needed to estimate the threshold outgrows shared memory
    return (dtype == FM_BF16 || dtype == FM_F16) && (d == 64 || d == 128) && n_keys >= 8192 && zc * 4 <= n_keys && zc >= 64 &&
           n_keys <= zc * 4096 && zc <= 12288;      // and a bucket's candidates have to fit the selection bitmap
}

// Key ranges per bucket tile for the candidate pass: units = mtiles * ranges CTAs of one tile row each.  The fewest
// ranges that fill the last wave of CTAs to 95 % (else the best found), never cutting a segment below 16 key tiles
// per range: every range costs a pipeline fill and a slice of the list capacity.
static int choose_ranges(int64_t mtiles, int64_t min_tiles, int sms)
{
    int best = 1;
    double best_eff = 0.0;
    for (int r = 1; r <= kMaxRanges && (r == 1 || min_tiles / r >= 16); ++r) {
        const int64_t units = mtiles * r;
        const double eff = double(units) / double(ceil_div(units, sms) * sms);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = r; }
        if (eff >= 0.95) break;
    }
    return best;
}

// Which order statistic of the sample scores serves as the threshold: z sampled keys of a bucket are expected among its
// top Z; the threshold is too high - and the bucket goes to the fallback - when more than the chosen rank are.  Four
// standard deviations: about one bucket in 10^5 (a fifth of a bucket per benchmark build); every half deviation more
// costs the selection 3 % more candidates.
static int sample_rank(double z) { return (int)std::ceil(z + 4.0 * std::sqrt(z) + 2.0); }

// Layout of the workspace for the eligible segments.  Groups are sized so that the candidate lists of one group stay
// within ~3 GB.
FusedPlan fused_plan(int n, const int64_t *n_keys, const int64_t *n_buckets, const int64_t *zc)
{
    FusedPlan P = {};
    int64_t zmin = INT64_MAX, total_b = 0;
    for (int i = 0; i < n; ++i) { zmin = std::min(zmin, zc[i]); P.max_keys = std::max(P.max_keys, n_keys[i]); total_b += n_buckets[i]; }
    // about 128 of a bucket's keys in the sample; a coarser step for very long segments (at most kMaxSample sampled keys),
    // never so coarse that fewer than 8 of a bucket's keys are expected in the sample
    P.step = (int)std::max<int64_t>(std::min<int64_t>(64, zmin / 128), ceil_div(P.max_keys, kMaxSample));
    P.step = (int)std::max<int64_t>(1, std::min<int64_t>(P.step, zmin / 8));
    int cap = 0;
    for (int i = 0; i < n; ++i) {
        const double z = double(zc[i]) / P.step;
        const double r = sample_rank(z);
        cap = std::max(cap, (int)std::ceil(P.step * (r + 6.0 * std::sqrt(r))) + 64);
    }
    P.cap = (cap + 7) / 8 * 8;
    // shared memory of the selection kernel: candidate scores + key indices, tile masks, entries before each tile
    P.sel_smem = size_t(P.cap) * 8 + size_t(ceil_div(P.max_keys, kTcBN)) * 12 + 32;
    const size_t per_bucket = size_t(P.cap) * 16 + size_t(ceil_div(P.max_keys, kTcBN)) * 8;
    // rows of a group: every segment starts on a multiple of 32 rows
    int64_t max_b = 0, total_pad = 0;
    for (int i = 0; i < n; ++i) { max_b = std::max(max_b, ceil_div(n_buckets[i], 32) * 32); total_pad += ceil_div(n_buckets[i], 32) * 32; }
    // (also keeps the candidate array of a group below 4 GB: the epilogue addresses it with 32-bit byte offsets)
    P.group_buckets = std::max<int64_t>(max_b, std::min<int64_t>(total_pad, int64_t((size_t(3) << 30) / per_bucket)));
    size_t off = 0;
    P.off_status = off; off += 256;
    P.off_fail = off;   off += align_up(size_t(kMaxFail + 1) * 4, 256);
    P.off_segs = off;   off += align_up(size_t(n) * sizeof(FusedSeg), 256);
    P.off_tcseg = off;  off += align_up(size_t(n) * sizeof(TcSeg) * 2, 256);
    P.off_tau = off;    off += align_up(size_t(P.group_buckets) * 4, 256);
    P.off_count = off;  off += align_up(size_t(P.group_buckets) * kMaxRanges * 2 * 4, 256);
    P.off_cand = off;   off += align_up(size_t(P.group_buckets) * P.cap * 16, 256);
    P.off_mask = off;   off += align_up(size_t(ceil_div(P.max_keys, kTcBN)) * P.group_buckets * 8, 256);
    P.off_yf = off;     off += align_up(size_t(kMaxFail) * P.max_keys * 4, 256);
    P.total = off;
    return P;
}

// Per-device helpers of a build, made once: an extra stream for work that may run beside the main sequence with the two
// events that fork and join it (stream == nullptr if they cannot be made: the work then stays on the caller's stream),
// and a small ring of pinned staging buffers for the segment descriptors, so that their copies to the device never
// make the host wait for the stream (a copy from pageable memory may).  A slot is reused only after the copies that
// read it have run (its event).
constexpr int kStageSlots = 4;
constexpr size_t kStageBytes = 64 << 10;
struct BuildSide {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    char *stage[kStageSlots] = {};
    cudaEvent_t stage_done[kStageSlots] = {};
    int next = 0;
    bool tried = false;
};
static std::mutex g_side_mu;
static std::mutex g_enqueue_mu;                // held while one build enqueues its group: the fork / join events are per device
static BuildSide g_side[64];

static BuildSide *build_side()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_side_mu);
    BuildSide &b = g_side[dev];
    if (!b.tried) {
        b.tried = true;
        // the side stream has the highest priority: its one small CTA per SM is placed as soon as it may run, not
        // after the last CTA of a long grid on the caller's stream has been placed
        int prio_least = 0, prio_greatest = 0;
        if (cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest) != cudaSuccess) { prio_greatest = 0; cudaGetLastError(); }
        bool ok = cudaStreamCreateWithPriority(&b.stream, cudaStreamNonBlocking, prio_greatest) == cudaSuccess &&
                  cudaEventCreateWithFlags(&b.fork, cudaEventDisableTiming) == cudaSuccess &&
                  cudaEventCreateWithFlags(&b.join, cudaEventDisableTiming) == cudaSuccess;
        if (!ok) { b.stream = nullptr; cudaGetLastError(); }
        for (int i = 0; i < kStageSlots; ++i) {
            if (cudaMallocHost((void **)&b.stage[i], kStageBytes) != cudaSuccess ||
                cudaEventCreateWithFlags(&b.stage_done[i], cudaEventDisableTiming) != cudaSuccess) {
                b.stage[i] = nullptr;
                cudaGetLastError();
            }
        }
    }
    return &b;
}

// Copies `bytes` of host data to the device on `st` through a pinned staging slot when one is to be had.
static int stage_to_device(BuildSide *side, void *dst, const void *src, size_t bytes, cudaStream_t st)
{
    int slot = -1;
    if (side && bytes <= kStageBytes) {
        std::lock_guard<std::mutex> lock(g_side_mu);
        if (side->stage[side->next]) { slot = side->next; side->next = (side->next + 1) % kStageSlots; }
    }
    if (slot < 0) {
        FM_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, st));
        return FM_OK;
    }
    FM_CUDA_OK(cudaEventSynchronize(side->stage_done[slot]));             // the slot's previous copy has run (long ago, as a rule)
    memcpy(side->stage[slot], src, bytes);
    FM_CUDA_OK(cudaMemcpyAsync(dst, side->stage[slot], bytes, cudaMemcpyHostToDevice, st));
    FM_CUDA_OK(cudaEventRecord(side->stage_done[slot], st));
    return FM_OK;
}

// Builds the table rows of the listed segments.  status word (ws + 0): 0 = ok, 1-3 = a tensor-core pipeline
// wait gave up, 4 = more buckets needed the fallback than it can take.
template <typename T>
static int fused_build_impl(const void *K, const void *A, int d, int64_t total_key_rows, int64_t total_buckets, int n,
                            const int64_t *kb, const int64_t *nk, const int64_t *cb, const int64_t *nbk, const int64_t *zc,
                            const int64_t *table_off, int32_t *table, char *ws, bool single_range, cudaStream_t st)
{
    const int dtype = Elem<T>::id;
    FusedPlan P = fused_plan(n, nk, nbk, zc);
    CUtensorMap tmA, tmK, tmKs;
    int rc = make_tensor_map_2d(&tmA, A, dtype, (uint64_t)total_buckets, (uint64_t)d, (uint64_t)d * 2, kTcBM);
    if (rc != FM_OK) return rc;
    rc = make_tensor_map_2d(&tmK, K, dtype, (uint64_t)total_key_rows, (uint64_t)d, (uint64_t)d * 2, kTcBN);
    if (rc != FM_OK) return rc;
    rc = make_tensor_map_2d(&tmKs, K, dtype, (uint64_t)ceil_div(total_key_rows, P.step), (uint64_t)d, (uint64_t)d * 2 * P.step, kTcBN);
    if (rc != FM_OK) return rc;
    // (the status word at ws + 0 has been cleared by the caller)
    // host mirror of the descriptor area [FusedSeg x n | pad | TcSeg x 2n]: one copy when a group covers every segment
    const size_t desc_bytes = (P.off_tcseg - P.off_segs) + size_t(2 * n) * sizeof(TcSeg);
    std::vector<char> hdesc(desc_bytes, 0);
    FusedSeg *hs = reinterpret_cast<FusedSeg *>(hdesc.data());
    TcSeg *ht = reinterpret_cast<TcSeg *>(hdesc.data() + (P.off_tcseg - P.off_segs));
    int g0 = 0;
    while (g0 < n) {
        // one group: consecutive segments whose buckets fit the group arrays
        int g1 = g0;
        int64_t rows = 0, mtiles = 0;
        while (g1 < n && rows + ceil_div(nbk[g1], 32) * 32 <= P.group_buckets) {
            FusedSeg &s = hs[g1];
            s.kb = (int)kb[g1]; s.n_keys = (int)nk[g1]; s.cb = (int)cb[g1]; s.n_buckets = (int)nbk[g1]; s.zc = (int)zc[g1];
            s.rank = sample_rank(double(zc[g1]) / P.step);
            s.ns0 = (int)ceil_div(kb[g1], P.step);
            s.ns = (int)(ceil_div(kb[g1] + nk[g1], P.step) - s.ns0);
            s.out_row0 = (int)rows; s.kmax_bits = 0; s.table_off = table_off[g1];
            ht[g1] = TcSeg{s.cb, s.n_buckets, s.ns0, s.ns, (int)mtiles, s.out_row0, s.rank};    // threshold pass (sampled rows)
            ht[n + g1] = TcSeg{s.cb, s.n_buckets, s.kb, s.n_keys, (int)mtiles, s.out_row0, 0};      // candidate pass
            rows += ceil_div(nbk[g1], 32) * 32;
            mtiles += ceil_div(nbk[g1], kTcBM);
            ++g1;
        }
        const int ng = g1 - g0;
        FusedSeg *dsegs = (FusedSeg *)(ws + P.off_segs) + g0;
        TcSeg *dtc_s = (TcSeg *)(ws + P.off_tcseg) + g0, *dtc_m = (TcSeg *)(ws + P.off_tcseg) + n + g0;
        BuildSide *bs = build_side();
        // two host threads building on one device share the side stream and its two events: their record / wait pairs
        // must not interleave (the enqueue of a group takes about a hundred microseconds)
        std::lock_guard<std::mutex> enqueue_lock(g_enqueue_mu);
        if (ng == n) {
            rc = stage_to_device(bs, ws + P.off_segs, hdesc.data(), desc_bytes, st);
        } else {
            rc = stage_to_device(bs, dsegs, hs + g0, sizeof(FusedSeg) * ng, st);
            if (rc == FM_OK) rc = stage_to_device(bs, dtc_s, ht + g0, sizeof(TcSeg) * ng, st);
            if (rc == FM_OK) rc = stage_to_device(bs, dtc_m, ht + n + g0, sizeof(TcSeg) * ng, st);
        }
        if (rc != FM_OK) return rc;
        FM_CUDA_OK(cudaMemsetAsync(ws + P.off_fail, 0, 512, st));
        float *tau = (float *)(ws + P.off_tau);
        int *counts = (int *)(ws + P.off_count);
        int *fail_count = (int *)(ws + P.off_fail), *fail_list = fail_count + 1;
        uint4 *cand = (uint4 *)(ws + P.off_cand);
        uint2 *cand_mask = (uint2 *)(ws + P.off_mask);
        float *Yf = (float *)(ws + P.off_yf);

        cudaStream_t side = bs ? bs->stream : nullptr;
        cudaEvent_t ev_fork = bs ? bs->fork : nullptr, ev_join = bs ? bs->join : nullptr;

        const int sms = sm_count();
        TcParams tp = {};
        tp.segs = dtc_s; tp.n_seg = ng; tp.status = (int *)(ws + P.off_status);
        {
            // thresholds: the sample projection three times over with reducing epilogues (tc_tau.cu), no score matrix
            TauParams tq = {dtc_s, ng, tau, (int *)(ws + P.off_status), 0};
            rc = tc_tau_launch(tmA, tmKs, tq, int(mtiles), d, dtype == FM_BF16, st);
            if (rc != FM_OK) return rc;
        }

        tp.segs = dtc_m;
        tp.tau = tau; tp.cand = cand; tp.cand_mask = cand_mask; tp.mask_ld = P.group_buckets; tp.cap = P.cap; tp.cand_count = counts;
        {
            int64_t min_tiles = INT64_MAX;
            for (int i = g0; i < g1; ++i) min_tiles = std::min(min_tiles, ceil_div(nk[i], kTcBN));
            tp.n_ranges = single_range ? 1 : choose_ranges(mtiles, min_tiles, sms);
        }
        // The key norms are only needed by the selection.  They are taken on a second stream beside the candidate
        // projection - tensor-bound, it leaves most of the memory bandwidth idle - and joined before the selection:
        // the fork is recorded before the projection is launched, so both start when the thresholds are done.
        if (side) {
            FM_CUDA_OK(cudaEventRecord(ev_fork, st));
            FM_CUDA_OK(cudaStreamWaitEvent(side, ev_fork, 0));
        }
        rc = tc_project_launch(tmA, tmK, tp, int(mtiles) * tp.n_ranges, d, false, dtype == FM_BF16, st);
        if (rc != FM_OK) return rc;
        // (the projection's CTAs configure their SMs for the largest shared memory: ask for the same, or this kernel's
        // CTAs would wait for SMs to drain)
        FM_CUDA_OK(func_attr_cached((const void *)key_norm_max_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        key_norm_max_kernel<T><<<sms, 512, 0, side ? side : st>>>((const T *)K, d, dsegs, ng);
        FM_LAUNCHED("key_norm_max_kernel");
        if (side) {
            FM_CUDA_OK(cudaEventRecord(ev_join, side));
            FM_CUDA_OK(cudaStreamWaitEvent(st, ev_join, 0));
        }
        const int max_tiles = (int)ceil_div(P.max_keys, kTcBN);
        SelParams sp = {dsegs, ng, tp.n_ranges, P.cap, cand, cand_mask, P.group_buckets, counts, tau, A, K, d, table, fail_count, fail_list,
                        max_tiles};
        {
            // candidate scores + key indices, tile masks, entries before each tile
            const size_t dyn = P.sel_smem;
            // The CTA's steps are chains of memory round trips and barriers, so what counts is how many CTAs an SM holds.
            // Measured on the 32-head benchmark build: 512 threads reading their 9 entries twice (40 registers, 3 CTAs
            // per SM) 1.03 ms; the entries kept in registers (64 registers, 2 CTAs) 1.10 ms; 256 threads x 18 entries
            // 1.42 ms; 128 x 40 2.11 ms.
            if (P.cap <= 9 * 512) rc = launch_select<T, 512, 9, false>(sp, (unsigned)rows, dyn, st);
            else if (P.cap <= 8 * 1024) rc = launch_select<T, 1024, 8, true>(sp, (unsigned)rows, dyn, st);
            else rc = launch_select<T, 1024, 25, false>(sp, (unsigned)rows, dyn, st);
            if (rc != FM_OK) return rc;
        }

        fallback_scores_kernel<T><<<dim3((unsigned)std::min<int64_t>(ceil_div(P.max_keys, 256), 4 * sms), 4), 256, 0, st>>>(
            dsegs, ng, fail_count, fail_list, (const T *)A, (const T *)K, d, Yf, P.max_keys);
        FM_LAUNCHED("fallback_scores_kernel");
        fallback_select_kernel<<<kMaxFail, kSelThreads, 0, st>>>(dsegs, ng, fail_count, fail_list, Yf, P.max_keys, table,
                                                                  (int *)(ws + P.off_status));
        FM_LAUNCHED("fallback_select_kernel");
        g0 = g1;
    }
    return FM_OK;
}

int fused_index_build(const void *K, const void *A, int dtype, int d, int64_t total_key_rows, int64_t total_buckets, int n,
                      const int64_t *kb, const int64_t *nk, const int64_t *cb, const int64_t *nbk, const int64_t *zc,
                      const int64_t *table_off, int32_t *table, void *ws, bool single_range, cudaStream_t st)
{
    if (dtype == FM_BF16)
        return fused_build_impl<__nv_bfloat16>(K, A, d, total_key_rows, total_buckets, n, kb, nk, cb, nbk, zc, table_off, table, (char *)ws, single_range, st);
    return fused_build_impl<__half>(K, A, d, total_key_rows, total_buckets, n, kb, nk, cb, nbk, zc, table_off, table, (char *)ws, single_range, st);
}

}  // namespace fm
