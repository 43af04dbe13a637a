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
#include <mutex>
#include <vector>

namespace fm {

// eps = kBandEps * ||a_b|| * kmax.  A tensor-core score is within 2^-16 M of the exact dot product and the
// canonical chain within 2^-17 M (M = ||a|| ||k|| >= sum |a_i k_i|, d <= 128), so two keys can compare
// differently under the two orders only if their tensor-core scores differ by less than 3 * 2^-16 M.
constexpr float kBandEps = 1.0f / 4096.0f;
constexpr int kMaxBand = 512;               // largest band re-scored exactly; beyond it the bucket goes to the fallback
constexpr int kMaxFail = 64;                // buckets the fallback can take per group of segments
constexpr int kMaxSample = 49152;           // sample scores of one bucket held in shared memory (192 KB)
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
template <typename T>
__global__ void key_norm_max_kernel(const T *__restrict__ K, int d, FusedSeg *__restrict__ segs)
{
    FusedSeg &sg = segs[blockIdx.y];
    const int lanes_per_row = d / 8;                         // 16-byte pieces per row
    const int rows_per_warp = 32 / lanes_per_row;
    const int lane = threadIdx.x & 31, sub = lane % lanes_per_row, rsel = lane / lanes_per_row;
    const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * (blockDim.x >> 5);
    float best = 0.f;
    const int stride = n_warps * rows_per_warp;
    // four rows per iteration: the loads are issued together, which is what keeps enough bytes in flight
    for (int r0 = warp_global * rows_per_warp + rsel; r0 < sg.n_keys; r0 += 4 * stride) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int r = r0 + u * stride;
            raw[u] = r < sg.n_keys ? *reinterpret_cast<const uint4 *>(K + size_t(sg.kb + r) * d + sub * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float f[8];
            widen8(raw[u], f, T());
            float n2 = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) n2 = fmaf(f[e], f[e], n2);
            for (int off = 1; off < lanes_per_row; off <<= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, off);
            best = fmaxf(best, n2);
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, off));
    if (lane == 0 && best > 0.f) atomicMax(&sg.kmax_bits, __float_as_uint(sqrtf(best) * 1.0001f));
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

__device__ __forceinline__ float key_to_float(uint32_t key)
{
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

// ---- selection of the r-th largest of n floats ----------------------------------------------------------------------
// All threads of the CTA call; `load(i)` returns value i (from global memory / L2: the lists are re-read in a few
// passes instead of being held in shared memory, which keeps a CTA's footprint at a few KB and many CTAs per SM
// in flight).  The values are binned LINEARLY between their minimum and maximum (scores near a threshold are
// spread over a narrow interval, where the radix digits of the floats would all collide), the bin holding the
// r-th largest is found from the top, and the search recurses into that bin until it holds at most kSmallSel
// values, which are ranked directly.  Returns theta = the r-th largest value (the same in every thread).
constexpr int kSelBins = 512;
constexpr int kSmallSel = 256;

// COPIES: lanes spread their increments over that many copies of the histogram (a power of two) - scores pile up in
// a few bins and same-address shared-memory atomics serialise; small inputs do with one.
template <int COPIES> struct SelScratch {
    static constexpr int kCopies = COPIES;
    int hist[COPIES * kSelBins];
    float small[kSmallSel];
    float red[64];
    int bin, want, count, n_small;
    float lo, hi, theta;
};

// A value source exposes  template <class F> void for_each(F f)  which calls f(ordinal, score) for the values this
// thread owns.  When the caller knows an interval [lo0, hi0] that holds every value it passes it (have_range) and
// the first look at the values is saved.
template <class Source, class Scratch>
__device__ __forceinline__ float select_rth(const Source &src, int n, int r, Scratch &S, bool have_range = false, float lo0 = 0.f,
                                            float hi0 = 0.f)
{
    constexpr int kHistCopies = Scratch::kCopies;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nthreads = blockDim.x, nw = (nthreads + 31) >> 5;
    float lo = -INFINITY, hi = INFINITY;
    int want = r;                                            // rank from the top inside [lo, hi]
    for (int iter = 0; iter < 40; ++iter) {
        if (iter == 0 && have_range) {
            __syncthreads();
            for (int i = t; i < kHistCopies * kSelBins; i += nthreads) S.hist[i] = 0;
            __syncthreads();
            lo = lo0; hi = hi0;
        } else {
            // exact value range of what is left
            float mn = INFINITY, mx = -INFINITY;
            src.for_each([&](int, float v) {
                if (v >= lo && v <= hi) { mn = fminf(mn, v); mx = fmaxf(mx, v); }
            });
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            }
            __syncthreads();
            if (lane == 0) { S.red[warp] = mn; S.red[32 + warp] = mx; }
            for (int i = t; i < kHistCopies * kSelBins; i += nthreads) S.hist[i] = 0;
            __syncthreads();
            mn = INFINITY; mx = -INFINITY;
            for (int w = 0; w < nw; ++w) { mn = fminf(mn, S.red[w]); mx = fmaxf(mx, S.red[32 + w]); }
            lo = mn; hi = mx;
        }
        if (!(hi > lo)) return lo;                           // every remaining value is equal (uniform across the CTA)
        const float scale = float(kSelBins) / (hi - lo);
        src.for_each([&](int, float v) {
            if (v >= lo && v <= hi) atomicAdd(&S.hist[(lane & (kHistCopies - 1)) * kSelBins + min(kSelBins - 1, int((v - lo) * scale))], 1);
        });
        __syncthreads();
        for (int i = t; i < kSelBins; i += nthreads) {       // fold the copies into copy 0
            int sum = 0;
#pragma unroll
            for (int c = 0; c < kHistCopies; ++c) sum += S.hist[c * kSelBins + i];
            S.hist[i] = sum;
        }
        __syncthreads();
        // find the bin from the top: thread t owns bins [t * per, (t + 1) * per)
        {
            const int per = (kSelBins + nthreads - 1) / nthreads;
            int mine = 0;
            for (int k = 0; k < per; ++k) mine += t * per + k < kSelBins ? S.hist[t * per + k] : 0;
            int inc = mine;                                  // suffix sum inside the warp
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int o = __shfl_down_sync(0xffffffffu, inc, off);
                if (lane + off < 32) inc += o;
            }
            int *wsum = reinterpret_cast<int *>(S.red);
            __syncthreads();
            if (lane == 0) wsum[warp] = inc;
            __syncthreads();
            int above = inc - mine;                          // values in bins above this thread's
            for (int w = warp + 1; w < nw; ++w) above += wsum[w];
            if (mine > 0 && above < want && want <= above + mine) {
                int acc = above;
                for (int k = per - 1; k >= 0; --k) {
                    const int h = t * per + k < kSelBins ? S.hist[t * per + k] : 0;
                    if (want <= acc + h) { S.bin = t * per + k; S.want = want - acc; S.count = h; break; }
                    acc += h;
                }
            }
            __syncthreads();
        }
        const int bin = S.bin, cnt = S.count;
        want = S.want;
        if (cnt <= kSmallSel) {
            if (t == 0) S.n_small = 0;
            __syncthreads();
            src.for_each([&](int, float v) {
                if (v >= lo && v <= hi && min(kSelBins - 1, int((v - lo) * scale)) == bin) S.small[atomicAdd(&S.n_small, 1)] = v;
            });
            __syncthreads();
            for (int i = t; i < cnt; i += nthreads) {
                const float v = S.small[i];
                int gt = 0, eq = 0;
                for (int o = 0; o < cnt; ++o) { gt += S.small[o] > v; eq += S.small[o] == v; }
                if (gt < want && want <= gt + eq) S.theta = v;     // all writers hold the same value
            }
            __syncthreads();
            return S.theta;
        }
        // recurse into the bin: narrow [lo, hi] to the bin's value interval (the next round finds its exact range)
        {
            float nlo = INFINITY, nhi = -INFINITY;
            src.for_each([&](int, float v) {
                if (v >= lo && v <= hi && min(kSelBins - 1, int((v - lo) * scale)) == bin) { nlo = fminf(nlo, v); nhi = fmaxf(nhi, v); }
            });
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                nlo = fminf(nlo, __shfl_xor_sync(0xffffffffu, nlo, off));
                nhi = fmaxf(nhi, __shfl_xor_sync(0xffffffffu, nhi, off));
            }
            __syncthreads();
            if (lane == 0) { S.red[warp] = nlo; S.red[32 + warp] = nhi; }
            __syncthreads();
            nlo = INFINITY; nhi = -INFINITY;
            for (int w = 0; w < nw; ++w) { nlo = fminf(nlo, S.red[w]); nhi = fmaxf(nhi, S.red[32 + w]); }
            lo = nlo; hi = nhi;
            __syncthreads();
        }
    }
    return lo;
}

// ---- 3. thresholds from the sample scores -----------------------------------------------------------------------
constexpr int kSelCThreads = 256;           // smallest CTA of the selection kernels (they take any multiple of 32 up to 1024)

// Values held in shared memory.
struct SmemValues {
    const float *v;
    int n;
    template <class F> __device__ __forceinline__ void for_each(F f) const
    {
        for (int i = threadIdx.x; i < n; i += blockDim.x) f(i, v[i]);
    }
};

// One row of the blocked dense scores, read from global memory.
struct SampleRow {
    const float *blk;          // block row base + this row's offset inside a block
    int n;
    template <class F> __device__ __forceinline__ void for_each(F f) const
    {
        const int n4 = (n + 3) >> 2;
        for (int g = threadIdx.x; g < n4; g += blockDim.x) {
            const float4 v = *reinterpret_cast<const float4 *>(blk + size_t(g >> 3) * 1024 + size_t(g & 7) * 128);
            const int i = g * 4;
            f(i, v.x);
            if (i + 1 < n) f(i + 1, v.y);
            if (i + 2 < n) f(i + 2, v.z);
            if (i + 3 < n) f(i + 3, v.w);
        }
    }
};

// One small CTA per bucket: tau = the r-th largest score of the bucket's row of the blocked sample scores (four
// consecutive columns are 16 contiguous bytes).  r is small against the row, so most of the row is discarded cheaply:
// every thread keeps four maxima over disjoint parts of what it loads; the r-th largest of all these maxima is a
// lower bound of tau (r different scores reach it), and only the scores at or above the bound - a few hundred, found
// in a second sweep over the row, which by then sits in L2 - enter the selection.  The CTAs are small and hold a
// few KB each so that an SM keeps dozens of rows in flight: the work per row is a chain of short dependent steps.
// (Measured on the 32-head benchmark build: 64 threads 2.79 ms, 128 threads 2.72 ms, 256 threads 2.77 ms.)
constexpr int kTauThreads = 128;
constexpr int kTopCap = 1024;               // sample scores that may lie at or above the lower bound

__device__ __forceinline__ void load_sample_groups(const float *blk, int g0, int stride, int n4, int n, float4 (&v)[4])
{
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int g = min(g0 + u * stride, n4 - 1);                                // group of 4 columns
        v[u] = *reinterpret_cast<const float4 *>(blk + size_t(g >> 3) * 1024 + size_t(g & 7) * 128);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int g = g0 + u * stride;
        if (g >= n4) v[u].x = -INFINITY;                                           // groups and columns past the row's end
        if (4 * g + 1 >= n) v[u].y = -INFINITY;
        if (4 * g + 2 >= n) v[u].z = -INFINITY;
        if (4 * g + 3 >= n) v[u].w = -INFINITY;
    }
}

__global__ void __launch_bounds__(kTauThreads)
sample_tau_kernel(const float *__restrict__ Ys, int64_t ldy, const FusedSeg *__restrict__ segs, int n_seg, float *__restrict__ tau)
{
    __shared__ SelScratch<1> S;
    __shared__ float tmax_s[4 * kTauThreads];
    __shared__ float top_s[kTopCap];
    __shared__ int s_top;
    const int row = blockIdx.x, t = threadIdx.x;
    const FusedSeg sg = segs[seg_of_out_row(segs, n_seg, row)];
    if (row - sg.out_row0 >= sg.n_buckets) return;           // padding between segments
    const float *blk = Ys + dense_block_offset(row, 0, ldy) + size_t(row & 31) * 4;
    const int n = sg.ns, n4 = (n + 3) >> 2, r = min(sg.rank, n);
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    for (int g0 = t; g0 < n4; g0 += 4 * kTauThreads) {
        float4 v[4];
        load_sample_groups(blk, g0, kTauThreads, n4, n, v);
#pragma unroll
        for (int u = 0; u < 4; ++u) mx[u] = fmaxf(fmaxf(mx[u], v[u].x), fmaxf(fmaxf(v[u].y, v[u].z), v[u].w));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) tmax_s[u * kTauThreads + t] = mx[u];
    if (t == 0) s_top = 0;
    __syncthreads();
    bool pruned = false;
    if (r <= 4 * kTauThreads) {
        const float bound = select_rth(SmemValues{tmax_s, 4 * kTauThreads}, 4 * kTauThreads, r, S);
        for (int g0 = t; g0 < n4; g0 += 4 * kTauThreads) {
            float4 v[4];
            load_sample_groups(blk, g0, kTauThreads, n4, n, v);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float f[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (f[k] >= bound) {
                        const int pos = atomicAdd(&s_top, 1);
                        if (pos < kTopCap) top_s[pos] = f[k];
                    }
            }
        }
        __syncthreads();
        pruned = s_top >= r && s_top <= kTopCap;             // uniform; more than that (masses of equal scores): the plain way
    }
    float th;
    if (pruned) th = select_rth(SmemValues{top_s, s_top}, s_top, r, S);
    else th = select_rth(SampleRow{blk, n}, n, r, S);
    if (t == 0) tau[row] = th;
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
};

constexpr int kMaxItems = kFusedMaxCap / 32 + 2 * kMaxRanges + 1;   // 32-entry slabs of one bucket's sub-lists

// One CTA per bucket.  The bucket's candidate groups - sub-lists (range 0, group 0), (range 0, group 1), (range 1,
// group 0), ...; group 0 of a range was written upward from the start of the range's buffer, group 1 downward from
// its end, so concatenated in this order they are in key order - are cut into slabs of 32 entries, one warp per slab.
// The scores that reach tau are compacted, still in key order, into shared memory (count per slab, scan, write),
// where every later step runs; no step inside a loop needs a CTA-wide barrier.
template <typename T>
__global__ void __launch_bounds__(1024)
candidate_select_kernel(SelParams p)
{
    extern __shared__ __align__(16) unsigned char sel_dyn[];
    float *cy = reinterpret_cast<float *>(sel_dyn);                     // [cap] candidate scores, in key order
    int *cid = reinterpret_cast<int *>(cy + p.cap);                     // [cap] their key indices; bit 31 = band entry that made it
    __shared__ SelScratch<2> S;
    __shared__ int band[kMaxBand];                                      // positions of the band entries in cy / cid
    __shared__ float band_y[kMaxBand];                                  // their canonical scores
    __shared__ int band_rank[kMaxBand];
    __shared__ float a_f32[256];
    __shared__ int item_off[kMaxItems + 1];                             // hits before each slab
    __shared__ int s_n, s_items, s_fail, s_nband;
    __shared__ int s_start[2 * kMaxRanges + 1];                         // entries before each sub-list
    __shared__ int s_istart[2 * kMaxRanges + 1];                        // slabs before each sub-list
    __shared__ int warp_in[33];                                         // selected entries per warp range
    __shared__ int scan_tot[32];
    __shared__ float s_anorm;

    const int row = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int nthreads = blockDim.x, nwarps = blockDim.x >> 5;
    const FusedSeg sg = p.segs[seg_of_out_row(p.segs, p.n_seg, row)];
    if (row - sg.out_row0 >= sg.n_buckets) return;           // padding between segments
    const int bucket = sg.cb + (row - sg.out_row0);
    const int Z = sg.zc;
    const T *a_row = reinterpret_cast<const T *>(p.A) + size_t(bucket) * p.d;
    const int sub_cap = p.cap / p.n_ranges;
    const int n_sl = 2 * p.n_ranges;
    const uint4 *lists = p.cand + size_t(row) * p.cap;
    const float tau = p.tau[row];

    // sub-list sizes; the two groups of a range share a buffer and must not have met in the middle
    if (t == 0) {
        int n = 0, items = 0, fail = 0;
        for (int r = 0; r < p.n_ranges; ++r) {
            const int c0 = p.cand_count[(size_t(row) * p.n_ranges + r) * 2], c1 = p.cand_count[(size_t(row) * p.n_ranges + r) * 2 + 1];
            if (c0 > sub_cap || c1 > sub_cap || c0 + c1 > sub_cap) fail = 1;
            s_start[2 * r] = n;      s_istart[2 * r] = items;      n += c0; items += (c0 + 31) >> 5;
            s_start[2 * r + 1] = n;  s_istart[2 * r + 1] = items;  n += c1; items += (c1 + 31) >> 5;
        }
        s_start[n_sl] = n;
        s_istart[n_sl] = items;
        s_items = fail ? 0 : items;
        s_fail = fail;
        s_nband = 0;
    }
    for (int i = t; i < p.d; i += nthreads) a_f32[i] = Elem<T>::to_f32(a_row[i]);
    if (t < 33) warp_in[t] = 0;
    __syncthreads();
    // the lists are read twice below, a few entries per thread at a time: ask for them now (128-byte lines into L2)
    for (int sl = 0; sl < n_sl; ++sl) {
        const int cnt = s_start[sl + 1] - s_start[sl];
        const uint4 *first = lists + size_t(sl >> 1) * sub_cap + ((sl & 1) ? sub_cap - cnt : 0);
        for (int i = t * 8; i < cnt; i += nthreads * 8) asm volatile("prefetch.global.L2 [%0];" ::"l"(first + i));
    }
    if (warp == 0) {                                         // ||a_b||
        float n2 = 0.f;
        for (int i = lane; i < p.d; i += 32) n2 = fmaf(a_f32[i], a_f32[i], n2);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, off);
        if (lane == 0) s_anorm = sqrtf(n2) * 1.0001f;
    }

    // Which keys the entries hold: the tile masks, walked in key order, give the first key of the i-th entry (the
    // sub-lists concatenate in tile order).  The key indices are parked at the END of cid, entry i at
    // cid[cap - n_ent + i]: the hits are written from the front and hit position <= cap - n_ent + entry ordinal.
    const int n_items = s_items;
    const int n_ent = n_items ? s_start[n_sl] : 0;
    int *ecol = cid + (p.cap - n_ent);
    if (n_ent) {
        const int n_tiles = (sg.n_keys + kTcBN - 1) / kTcBN;
        const uint2 *mcol = p.cand_mask + row;
        int run = 0;
        const int tpt = min(4, max(1, (n_tiles + nthreads - 1) / nthreads));       // consecutive tiles per thread and step
        for (int t0 = 0; t0 < n_tiles; t0 += tpt * nthreads) {
            unsigned long long m[4];
            int c = 0;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int tile = t0 + tpt * t + u;
                uint2 w = make_uint2(0, 0);
                if (u < tpt && tile < n_tiles) w = mcol[size_t(tile) * p.mask_ld];
                m[u] = (unsigned long long)w.x | ((unsigned long long)w.y << 32);
                c += __popcll(m[u]);
            }
            int incl = c;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += o;
            }
            if (lane == 31) scan_tot[warp] = incl;
            __syncthreads();
            int before = 0, total = 0;
            for (int w = 0; w < nwarps; ++w) {
                const int cw = scan_tot[w];
                before += w < warp ? cw : 0;
                total += cw;
            }
            int e = run + before + incl - c;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int key0 = (t0 + tpt * t + u) * kTcBN;
                while (m[u]) {
                    const int bit = __ffsll((long long)m[u]) - 1;
                    m[u] &= m[u] - 1;
                    if (e < n_ent) ecol[e] = key0 + 4 * bit;
                    ++e;
                }
            }
            run += total;
            __syncthreads();
        }
        if (t == 0 && run != n_ent) s_fail = 1;              // masks and list lengths disagree (an overflowed list)
    }
    __syncthreads();

    // entry `lane` of slab `it` (all -inf past the sub-list's end); `ord` = its ordinal among the bucket's entries
    auto slab_entry = [&](int it, int &ord) {
        const int sl = __popc(__ballot_sync(0xffffffffu, lane < n_sl && it >= s_istart[lane + 1]));
        const int j = (it - s_istart[sl]) * 32 + lane, cnt = s_start[sl + 1] - s_start[sl];
        uint4 e = make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u);
        ord = -1;
        if (j < cnt) {
            e = lists[size_t(sl >> 1) * sub_cap + ((sl & 1) ? sub_cap - 1 - j : j)];
            ord = s_start[sl] + j;
        }
        return e;
    };
    // hits per slab (four slabs per step: the loads are issued together)
    const unsigned lt_mask = (1u << lane) - 1u;
    auto hit_ballots = [&](const uint4 &e, unsigned (&bal)[4]) {
        bal[0] = __ballot_sync(0xffffffffu, __uint_as_float(e.x) >= tau);
        bal[1] = __ballot_sync(0xffffffffu, __uint_as_float(e.y) >= tau);
        bal[2] = __ballot_sync(0xffffffffu, __uint_as_float(e.z) >= tau);
        bal[3] = __ballot_sync(0xffffffffu, __uint_as_float(e.w) >= tau);
    };
    for (int it0 = warp; it0 < n_items; it0 += 4 * nwarps) {
        uint4 e[4];
        int ord[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (it0 + u * nwarps < n_items) e[u] = slab_entry(it0 + u * nwarps, ord[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (it0 + u * nwarps < n_items) {
                unsigned bal[4];
                hit_ballots(e[u], bal);
                if (lane == 0) item_off[it0 + u * nwarps + 1] = __popc(bal[0]) + __popc(bal[1]) + __popc(bal[2]) + __popc(bal[3]);
            }
    }
    __syncthreads();
    if (warp == 0) {                                         // exclusive scan over the slabs
        int run = 0;
        for (int i0 = 0; i0 < n_items; i0 += 32) {
            const int c = i0 + lane < n_items ? item_off[i0 + lane + 1] : 0;
            int incl = c;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += o;
            }
            if (i0 + lane < n_items) item_off[i0 + lane + 1] = run + incl;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            item_off[0] = 0;
            s_n = run;
            if (run < Z || run > p.cap) s_fail = 1;
        }
    }
    __syncthreads();
    const int n = s_n;
    if (!s_fail) {
        // ordered write of the hits; their value range for the selection on the way
        float hmin = INFINITY, hmax = -INFINITY;
        for (int ib = 0; ib < n_items; ib += 4 * nwarps) {   // the same trip count in every warp: a barrier inside
            const int it0 = ib + warp;
            uint4 e[4];
            int col[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (it0 + u * nwarps < n_items) {
                    int ord;
                    e[u] = slab_entry(it0 + u * nwarps, ord);
                    col[u] = ord >= 0 ? ecol[ord] : 0;
                }
            __syncthreads();                                 // every key index of this step is read before hits land in cid
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (it0 + u * nwarps < n_items) {
                    const uint32_t s4[4] = {e[u].x, e[u].y, e[u].z, e[u].w};
                    unsigned bal[4];
                    hit_ballots(e[u], bal);
                    int pos = item_off[it0 + u * nwarps] + __popc(bal[0] & lt_mask) + __popc(bal[1] & lt_mask) + __popc(bal[2] & lt_mask) +
                              __popc(bal[3] & lt_mask);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float y = __uint_as_float(s4[k]);
                        if (y >= tau) {
                            cy[pos] = y;
                            cid[pos] = col[u] + k;
                            ++pos;
                            hmin = fminf(hmin, y);
                            hmax = fmaxf(hmax, y);
                        }
                    }
                }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            hmin = fminf(hmin, __shfl_xor_sync(0xffffffffu, hmin, off));
            hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, off));
        }
        if (lane == 0) { S.red[warp] = hmin; S.red[32 + warp] = hmax; }
        __syncthreads();
        for (int w = 0; w < nwarps; ++w) { hmin = fminf(hmin, S.red[w]); hmax = fmaxf(hmax, S.red[32 + w]); }

        const SmemValues src{cy, n};
        const float theta = select_rth(src, n, Z, S, true, hmin, hmax);
        const float eps = kBandEps * s_anorm * __uint_as_float(sg.kmax_bits);
        const float lo = theta - eps, hi = theta + eps;
        // everything at or above lo has to be among the candidates, i.e. the threshold was low enough
        if (t == 0 && !(tau <= lo) && n < sg.n_keys) s_fail = 1;
        // warp w owns positions [w * per, (w + 1) * per): it counts its certain entries (score > hi) and lists the
        // band [lo, hi]
        const int per = (n + nwarps - 1) / nwarps;
        const int w_begin = min(n, warp * per), w_end = min(n, w_begin + per);
        int my_in = 0;
        for (int i = w_begin + lane; i < w_end; i += 32) {
            const float y = cy[i];
            if (y > hi) ++my_in;
            else if (y >= lo) {
                const int slot = atomicAdd(&s_nband, 1);
                if (slot < kMaxBand) band[slot] = i;
            }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) my_in += __shfl_xor_sync(0xffffffffu, my_in, off);
        if (lane == 0) { warp_in[warp] = my_in; atomicAdd(&warp_in[32], my_in); }
        __syncthreads();
        const int n_band = s_nband, need = Z - warp_in[32];
        if (t == 0 && (n_band > kMaxBand || need < 0 || need > n_band)) s_fail = 1;
        __syncthreads();
        if (!s_fail) {
            // canonical scores of the band, then an exact rank: better = larger score, then lower key index
            const T *Kseg = reinterpret_cast<const T *>(p.K) + size_t(sg.kb) * p.d;
            // four lanes per key row: each loads a quarter of the row (all loads in flight together), then the
            // chain runs through the quarters in order, handed from lane to lane
            const int quarter = p.d / 4, sub = lane & 3;
            for (int b0 = 0; b0 < n_band; b0 += nthreads / 4) {
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
                if (band_rank[b] < need) {
                    cid[band[b]] |= int(0x80000000u);
                    atomicAdd(&warp_in[band[b] / per], 1);
                }
            __syncthreads();
            // ordered compaction, one warp per range: the candidates are in key order, so is the table row
            int32_t *out = p.table + sg.table_off + size_t(row - sg.out_row0) * Z;
            int base_out = 0;
            for (int w = 0; w < warp; ++w) base_out += warp_in[w];
            for (int i0 = w_begin; i0 < w_end; i0 += 32) {
                const int i = i0 + lane;
                bool sel = false;
                int id = 0;
                if (i < w_end) {
                    const float y = cy[i];
                    id = cid[i];
                    sel = y > hi || (y >= lo && id < 0);
                }
                const unsigned bal = __ballot_sync(0xffffffffu, sel);
                const int pos = base_out + __popc(bal & ((1u << lane) - 1u));
                if (sel && pos < Z) out[pos] = sg.kb + (id & 0x7fffffff);
                base_out += __popc(bal);
            }
        }
    }
    __syncthreads();
    if (t == 0 && s_fail) {
        const int slot = atomicAdd(p.fail_count, 1);
        if (slot < kMaxFail) p.fail_list[slot] = row;
    }
}

// ---- 6. fallback: canonical scores of a whole segment for the listed buckets, then the exact row select ---------
template <typename T>
__global__ void fallback_scores_kernel(const FusedSeg *__restrict__ segs, int n_seg, const int *__restrict__ fail_count,
                                       const int *__restrict__ fail_list, const T *__restrict__ A, const T *__restrict__ K, int d,
                                       float *__restrict__ Yf, int64_t ldf)
{
    if ((int)blockIdx.y >= min(*fail_count, kMaxFail)) return;
    const int row = fail_list[blockIdx.y];
    const FusedSeg sg = segs[seg_of_out_row(segs, n_seg, row)];
    const T *a_row = A + size_t(sg.cb + (row - sg.out_row0)) * d;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < sg.n_keys; j += gridDim.x * blockDim.x)
        Yf[size_t(blockIdx.y) * ldf + j] = canonical_dot(a_row, K + size_t(sg.kb + j) * d, d);
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

// CTA size of the selection kernels: what they hold in shared memory decides how many CTAs share an SM, so a
// large footprint gets more threads per CTA.
static int sel_threads(size_t dyn_smem) { return dyn_smem <= (48u << 10) ? kSelCThreads : (dyn_smem <= (100u << 10) ? 512 : 1024); }

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

static int sample_rank(double z) { return (int)std::ceil(z + 5.0 * std::sqrt(z) + 2.0); }

// Layout of the workspace for the eligible segments.  Groups are sized so that the sample scores and the candidate
// lists of one group stay within ~3 GB.
FusedPlan fused_plan(int n, const int64_t *n_keys, const int64_t *n_buckets, const int64_t *zc)
{
    FusedPlan P = {};
    int64_t zmin = INT64_MAX, total_b = 0;
    for (int i = 0; i < n; ++i) { zmin = std::min(zmin, zc[i]); P.max_keys = std::max(P.max_keys, n_keys[i]); total_b += n_buckets[i]; }
    // about 128 of a bucket's keys in the sample; a coarser step when the sampled row would not fit in shared memory
    // (kMaxSample scores), never so coarse that fewer than 8 of them are expected
    P.step = (int)std::max<int64_t>(std::min<int64_t>(64, zmin / 128), ceil_div(P.max_keys, kMaxSample));
    P.step = (int)std::max<int64_t>(1, std::min<int64_t>(P.step, zmin / 8));
    int cap = 0;
    for (int i = 0; i < n; ++i) {
        const double z = double(zc[i]) / P.step;
        const double r = sample_rank(z);
        cap = std::max(cap, (int)std::ceil(P.step * (r + 6.0 * std::sqrt(r))) + 64);
        P.ld_sample = std::max<int64_t>(P.ld_sample, n_keys[i] / P.step + 2);
    }
    P.cap = (cap + 7) / 8 * 8;
    P.ld_sample = (P.ld_sample + 31) / 32 * 32;              // the dense scores are stored in 32 x 32 blocks
    const size_t per_bucket = size_t(P.ld_sample) * 4 + size_t(P.cap) * 16 + size_t(ceil_div(P.max_keys, kTcBN)) * 8;
    // rows of a group: every segment starts on a multiple of 32 rows
    int64_t max_b = 0, total_pad = 0;
    for (int i = 0; i < n; ++i) { max_b = std::max(max_b, ceil_div(n_buckets[i], 32) * 32); total_pad += ceil_div(n_buckets[i], 32) * 32; }
    // (also keeps the candidate array of a group below 4 GB: the epilogue addresses it with 32-bit byte offsets)
    P.group_buckets = std::max<int64_t>(max_b, std::min<int64_t>(total_pad, int64_t((size_t(3) << 30) / per_bucket)));
    size_t off = 0;
    P.off_status = off; off += 256;
    P.off_segs = off;   off += align_up(size_t(n) * sizeof(FusedSeg), 256);
    P.off_tcseg = off;  off += align_up(size_t(n) * sizeof(TcSeg) * 2, 256);
    P.off_tau = off;    off += align_up(size_t(P.group_buckets) * 4, 256);
    P.off_count = off;  off += align_up(size_t(P.group_buckets) * kMaxRanges * 2 * 4, 256);
    P.off_fail = off;   off += align_up(size_t(kMaxFail + 1) * 4, 256);
    P.off_ys = off;     off += align_up(size_t(P.group_buckets) * P.ld_sample * 4, 256);
    P.off_cand = off;   off += align_up(size_t(P.group_buckets) * P.cap * 16, 256);
    P.off_mask = off;   off += align_up(size_t(ceil_div(P.max_keys, kTcBN)) * P.group_buckets * 8, 256);
    P.off_yf = off;     off += align_up(size_t(kMaxFail) * P.max_keys * 4, 256);
    P.total = off;
    return P;
}

// One extra stream per device for work that may run beside the main sequence of a build (nullptr if it cannot be made:
// the work then stays on the caller's stream).
static cudaStream_t side_stream()
{
    static std::mutex mu;
    static cudaStream_t tab[64] = {};
    static bool tried[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!tried[dev]) {
        tried[dev] = true;
        if (cudaStreamCreateWithFlags(&tab[dev], cudaStreamNonBlocking) != cudaSuccess) { tab[dev] = nullptr; cudaGetLastError(); }
    }
    return tab[dev];
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
    FM_CUDA_OK(cudaMemsetAsync(ws + P.off_status, 0, 256, st));

    std::vector<FusedSeg> hs(n);
    std::vector<TcSeg> ht(2 * n);
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
            ht[g1] = TcSeg{s.cb, s.n_buckets, s.ns0, s.ns, (int)mtiles, s.out_row0};            // sample pass
            ht[n + g1] = TcSeg{s.cb, s.n_buckets, s.kb, s.n_keys, (int)mtiles, s.out_row0};      // candidate pass
            rows += ceil_div(nbk[g1], 32) * 32;
            mtiles += ceil_div(nbk[g1], kTcBM);
            ++g1;
        }
        const int ng = g1 - g0;
        FusedSeg *dsegs = (FusedSeg *)(ws + P.off_segs) + g0;
        TcSeg *dtc_s = (TcSeg *)(ws + P.off_tcseg) + g0, *dtc_m = (TcSeg *)(ws + P.off_tcseg) + n + g0;
        FM_CUDA_OK(cudaMemcpyAsync(dsegs, hs.data() + g0, sizeof(FusedSeg) * ng, cudaMemcpyHostToDevice, st));
        FM_CUDA_OK(cudaMemcpyAsync(dtc_s, ht.data() + g0, sizeof(TcSeg) * ng, cudaMemcpyHostToDevice, st));
        FM_CUDA_OK(cudaMemcpyAsync(dtc_m, ht.data() + n + g0, sizeof(TcSeg) * ng, cudaMemcpyHostToDevice, st));
        FM_CUDA_OK(cudaMemsetAsync(ws + P.off_fail, 0, 256, st));
        float *tau = (float *)(ws + P.off_tau);
        int *counts = (int *)(ws + P.off_count);
        int *fail_count = (int *)(ws + P.off_fail), *fail_list = fail_count + 1;
        float *Ys = (float *)(ws + P.off_ys);
        uint4 *cand = (uint4 *)(ws + P.off_cand);
        uint2 *cand_mask = (uint2 *)(ws + P.off_mask);
        float *Yf = (float *)(ws + P.off_yf);

        // The key norms are only needed by the selection: they are taken on a second stream, under the sample pass and
        // the threshold selection (which leave most of the memory bandwidth idle), and joined before the selection.
        cudaStream_t side = side_stream();
        cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
        if (side) {
            FM_CUDA_OK(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
            FM_CUDA_OK(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
            FM_CUDA_OK(cudaEventRecord(ev_fork, st));
            FM_CUDA_OK(cudaStreamWaitEvent(side, ev_fork, 0));
        }
        key_norm_max_kernel<T><<<dim3(std::max(1, 8 * sm_count() / ng), ng), 256, 0, side ? side : st>>>((const T *)K, d, dsegs);
        FM_LAUNCHED("key_norm_max_kernel");
        if (side) FM_CUDA_OK(cudaEventRecord(ev_join, side));

        const int sms = sm_count();
        TcParams tp = {};
        tp.segs = dtc_s; tp.n_seg = ng; tp.status = (int *)(ws + P.off_status);
        tp.Y = Ys; tp.ldy = P.ld_sample;
        {
            const int64_t tiles = ceil_div(P.ld_sample, kTcBN);
            tp.n_ranges = (int)std::max<int64_t>(1, std::min<int64_t>(tiles, ceil_div(2 * sms, mtiles)));
            rc = tc_project_launch(tmA, tmKs, tp, int(mtiles) * tp.n_ranges, d, true, dtype == FM_BF16, st);
            if (rc != FM_OK) return rc;
        }
        {
            sample_tau_kernel<<<(unsigned)rows, kTauThreads, 0, st>>>(Ys, P.ld_sample, dsegs, ng, tau);
        }
        FM_LAUNCHED("sample_tau_kernel");

        tp.segs = dtc_m;
        tp.tau = tau; tp.cand = cand; tp.cand_mask = cand_mask; tp.mask_ld = P.group_buckets; tp.cap = P.cap; tp.cand_count = counts;
        {
            int64_t min_tiles = INT64_MAX;
            for (int i = g0; i < g1; ++i) min_tiles = std::min(min_tiles, ceil_div(nk[i], kTcBN));
            tp.n_ranges = single_range ? 1 : choose_ranges(mtiles, min_tiles, sms);
        }
        rc = tc_project_launch(tmA, tmK, tp, int(mtiles) * tp.n_ranges, d, false, dtype == FM_BF16, st);
        if (rc != FM_OK) return rc;

        if (side) {
            FM_CUDA_OK(cudaStreamWaitEvent(st, ev_join, 0));
            cudaEventDestroy(ev_fork);                       // released once the work that uses them has run
            cudaEventDestroy(ev_join);
        }
        SelParams sp = {dsegs, ng, tp.n_ranges, P.cap, cand, cand_mask, P.group_buckets, counts, tau, A, K, d, table, fail_count, fail_list};
        {
            const size_t dyn = size_t(P.cap) * 8;
            FM_CUDA_OK(cudaFuncSetAttribute(candidate_select_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
            candidate_select_kernel<T><<<(unsigned)rows, sel_threads(dyn), dyn, st>>>(sp);
        }
        FM_LAUNCHED("candidate_select_kernel");

        fallback_scores_kernel<T><<<dim3((unsigned)std::min<int64_t>(ceil_div(P.max_keys, 256), 4 * sms), kMaxFail), 256, 0, st>>>(
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
