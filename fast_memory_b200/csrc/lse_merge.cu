// LSE merge of two partial attention results, in place on fp32 accumulators.
// Stands in for update_out_and_lse of the reference (memory.py:54-71):
//     d = blk_lse - lse;  out -= sigmoid(d) * (out - blk_out);  lse -= logsigmoid(-d)
// i.e. lse <- log(e^lse + e^blk_lse) and out <- the convex combination weighted by e^lse, e^blk_lse.
#include "common.cuh"

namespace fm {

template <typename T> __device__ __forceinline__ float load_as_f32(const void *p, size_t i)
{
    return Elem<T>::to_f32(reinterpret_cast<const T *>(p)[i]);
}

__device__ __forceinline__ float load_lse(const void *p, int dtype, size_t i)
{
    if (dtype == FM_F32) return reinterpret_cast<const float *>(p)[i];
    if (dtype == FM_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    return __half2float(reinterpret_cast<const __half *>(p)[i]);
}

// One warp per row; lanes stride the head dim in 16-byte pieces.  HBM-bound: per row it moves
// d * (8 + sizeof(T)) + 12 bytes.
template <typename T>
__global__ void __launch_bounds__(256)
lse_merge_kernel(float *__restrict__ out, float *__restrict__ lse, const T *__restrict__ blk_out,
                 const void *__restrict__ blk_lse, int lse_dtype, int64_t n_rows, int d)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = int64_t(gridDim.x) * (blockDim.x >> 5);
    for (int64_t r = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n_rows; r += warps) {
        const float a = lse[r];
        const float b = load_lse(blk_lse, lse_dtype, r);
        // weight of the block: sigmoid(b - a); new lse: a + softplus(b - a).  -inf on a side = weight 0.
        float w, nl;
        if (b == -INFINITY) { w = 0.f; nl = a; }
        else if (a == -INFINITY) { w = 1.f; nl = b; }
        else {
            const float dlt = b - a;
            w = 1.f / (1.f + expf(-dlt));
            nl = a + (dlt > 0.f ? dlt + log1pf(expf(-dlt)) : log1pf(expf(dlt)));
        }
        float *orow = out + r * d;
        const T *brow = blk_out + r * d;
        for (int c = lane * 4; c < d; c += 128) {
            float4 o4 = *reinterpret_cast<const float4 *>(orow + c);
            float b0, b1, b2, b3;
            if constexpr (sizeof(T) == 4) {
                float4 b4 = *reinterpret_cast<const float4 *>(brow + c);
                b0 = b4.x; b1 = b4.y; b2 = b4.z; b3 = b4.w;
            } else {
                uint2 raw = *reinterpret_cast<const uint2 *>(brow + c);
                const T *h = reinterpret_cast<const T *>(&raw);
                b0 = Elem<T>::to_f32(h[0]); b1 = Elem<T>::to_f32(h[1]);
                b2 = Elem<T>::to_f32(h[2]); b3 = Elem<T>::to_f32(h[3]);
            }
            o4.x -= w * (o4.x - b0);
            o4.y -= w * (o4.y - b1);
            o4.z -= w * (o4.z - b2);
            o4.w -= w * (o4.w - b3);
            *reinterpret_cast<float4 *>(orow + c) = o4;
        }
        if (lane == 0) lse[r] = nl;
    }
}

// The same merge out of place: (acc_out fp32, acc_lse) and (blk_out T, blk_lse fp32) are read, the merged rows are written
// to `dst` in TO (fp32 or T) and `dst_lse`; per row it moves d * (4 + sizeof(T) + sizeof(TO)) + 12 bytes instead of the
// copy + in-place merge + cast a caller that must keep its accumulator would otherwise run.
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
lse_merge_out_kernel(const float *__restrict__ acc_out, const float *__restrict__ acc_lse, const T *__restrict__ blk_out,
                     const float *__restrict__ blk_lse, TO *__restrict__ dst, float *__restrict__ dst_lse, int64_t n_rows, int d)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = int64_t(gridDim.x) * (blockDim.x >> 5);
    for (int64_t r = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n_rows; r += warps) {
        const float a = acc_lse[r], b = blk_lse[r];
        float w, nl;
        if (b == -INFINITY) { w = 0.f; nl = a; }
        else if (a == -INFINITY) { w = 1.f; nl = b; }
        else {
            const float dlt = b - a;
            w = 1.f / (1.f + expf(-dlt));
            nl = a + (dlt > 0.f ? dlt + log1pf(expf(-dlt)) : log1pf(expf(dlt)));
        }
        const float *arow = acc_out + r * d;
        const T *brow = blk_out + r * d;
        TO *orow = dst + r * d;
        for (int c = lane * 4; c < d; c += 128) {
            float4 o4 = *reinterpret_cast<const float4 *>(arow + c);
            float b0, b1, b2, b3;
            if constexpr (sizeof(T) == 4) {
                float4 b4 = *reinterpret_cast<const float4 *>(brow + c);
                b0 = b4.x; b1 = b4.y; b2 = b4.z; b3 = b4.w;
            } else {
                uint2 raw = *reinterpret_cast<const uint2 *>(brow + c);
                const T *h = reinterpret_cast<const T *>(&raw);
                b0 = Elem<T>::to_f32(h[0]); b1 = Elem<T>::to_f32(h[1]);
                b2 = Elem<T>::to_f32(h[2]); b3 = Elem<T>::to_f32(h[3]);
            }
            o4.x -= w * (o4.x - b0);
            o4.y -= w * (o4.y - b1);
            o4.z -= w * (o4.z - b2);
            o4.w -= w * (o4.w - b3);
            if constexpr (sizeof(TO) == 4) {
                *reinterpret_cast<float4 *>(orow + c) = o4;
            } else {
                TO h[4] = {Elem<TO>::from_f32(o4.x), Elem<TO>::from_f32(o4.y), Elem<TO>::from_f32(o4.z), Elem<TO>::from_f32(o4.w)};
                *reinterpret_cast<uint2 *>(orow + c) = *reinterpret_cast<const uint2 *>(h);
            }
        }
        if (lane == 0) dst_lse[r] = nl;
    }
}

template <typename T>
static int launch_merge_out(const float *acc_out, const float *acc_lse, const void *blk_out, const float *blk_lse, void *dst,
                            int dst_dtype, float *dst_lse, int64_t n_rows, int d, cudaStream_t st)
{
    const int blocks = (int)std::min<int64_t>(ceil_div(n_rows, 8), int64_t(sm_count()) * 8);
    if (dst_dtype == FM_F32)
        lse_merge_out_kernel<T, float><<<blocks, 256, 0, st>>>(acc_out, acc_lse, (const T *)blk_out, blk_lse, (float *)dst, dst_lse, n_rows, d);
    else
        lse_merge_out_kernel<T, T><<<blocks, 256, 0, st>>>(acc_out, acc_lse, (const T *)blk_out, blk_lse, (T *)dst, dst_lse, n_rows, d);
    FM_LAUNCHED("lse_merge_out_kernel");
    return FM_OK;
}


// ---- merge of the partial results of several ranks over peer memory ------------------------------------------------
// Every rank holds, in memory its peers can address, its partial (o, lse) over ITS keys for all query rows.  Rank r owns
// the rows [row0, row1): it pulls those rows of every rank's partial, merges them -
//     M = max_p lse_p,  w_p = e^(lse_p - M),  out = sum_p w_p o_p / sum_p w_p,  lse = M + log sum_p w_p
// (the pairwise merge of memory.py:54-71 written as one sum; a rank whose LSE is -inf has weight 0) - and pushes the
// finished rows to the result buffers of all ranks, so that everyone ends up with the complete result: one kernel in the
// place of the W - 1 send / receive + merge steps of the reference's ring (memory.py:307-338).  Loads and stores to peer
// memory are plain ones.  Thread = 8 consecutive elements (16 bytes of a 16-bit o) of one row.
constexpr int kMaxPeers = 8;
struct PeerMergeParams {
    const void *o[kMaxPeers];
    const float *lse[kMaxPeers];
    float *out[kMaxPeers];
    float *lse_out[kMaxPeers];
    int world;
    int d;
    int64_t row0, row1;
};

template <typename T>
__global__ void __launch_bounds__(256)
peer_merge_kernel(PeerMergeParams p)
{
    const int tpr = p.d / 8;                                 // threads per row
    const int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t r = p.row0 + t / tpr;
    const int c = int(t % tpr) * 8;
    if (r >= p.row1) return;
    float l[kMaxPeers];
    uint4 raw[kMaxPeers][sizeof(T) == 4 ? 2 : 1];
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMaxPeers; ++w)
        if (w < p.world) {
            l[w] = p.lse[w][r];
            const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(p.o[w]) + r * p.d + c);
            raw[w][0] = src[0];
            if constexpr (sizeof(T) == 4) raw[w][1] = src[1];
        }
#pragma unroll
    for (int w = 0; w < kMaxPeers; ++w)
        if (w < p.world) M = fmaxf(M, l[w]);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, den = 0.f;
#pragma unroll
    for (int w = 0; w < kMaxPeers; ++w)
        if (w < p.world) {
            const float wt = l[w] > -INFINITY ? expf(l[w] - M) : 0.f;      // (M = -inf only if every l is)
            den += wt;
            float f[8];
            if constexpr (sizeof(T) == 4) {
                const float *g = reinterpret_cast<const float *>(&raw[w][0]);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = g[e];
            } else {
                widen8(raw[w][0], f, T());
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(wt, f[e], acc[e]);
        }
    const float inv = den > 0.f ? 1.f / den : 0.f;           // no rank has a key for this row: zeros and -inf
    const float4 lo = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    const float4 hi = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
    const float L = den > 0.f ? M + logf(den) : -INFINITY;
#pragma unroll
    for (int w = 0; w < kMaxPeers; ++w)
        if (w < p.world) {
            float4 *dst = reinterpret_cast<float4 *>(p.out[w] + r * p.d + c);
            dst[0] = lo;
            dst[1] = hi;
            if (c == 0) p.lse_out[w][r] = L;
        }
}

}  // namespace fm

extern "C" int fm_lse_merge(float *out, float *lse, const void *blk_out, int blk_dtype, const void *blk_lse,
                            int lse_dtype, int64_t n_rows, int d, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(n_rows >= 0 && d > 0, "fm_lse_merge: bad sizes");
    if (n_rows == 0) return FM_OK;
    FM_REQUIRE(out && lse && blk_out && blk_lse, "fm_lse_merge: null pointer");
    FM_REQUIRE(d % 4 == 0, "fm_lse_merge: head dim must be a multiple of 4");
    FM_REQUIRE(((uintptr_t)out) % 16 == 0 && ((uintptr_t)blk_out) % 8 == 0, "fm_lse_merge: misaligned buffer");
    if (lse_dtype != FM_F32 && lse_dtype != FM_BF16 && lse_dtype != FM_F16) {
        set_error("fm_lse_merge: unknown lse dtype %d", lse_dtype);
        return FM_ERR_UNSUPPORTED;
    }
    cudaStream_t st = (cudaStream_t)stream;
    int blocks = (int)std::min<int64_t>(ceil_div(n_rows, 8), int64_t(sm_count()) * 8);
    switch (blk_dtype) {
    case FM_F32:
        lse_merge_kernel<float><<<blocks, 256, 0, st>>>(out, lse, (const float *)blk_out, blk_lse, lse_dtype, n_rows, d);
        break;
    case FM_BF16:
        lse_merge_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(out, lse, (const __nv_bfloat16 *)blk_out, blk_lse, lse_dtype, n_rows, d);
        break;
    case FM_F16:
        lse_merge_kernel<__half><<<blocks, 256, 0, st>>>(out, lse, (const __half *)blk_out, blk_lse, lse_dtype, n_rows, d);
        break;
    default: set_error("fm_lse_merge: unknown dtype %d", blk_dtype); return FM_ERR_UNSUPPORTED;
    }
    FM_LAUNCHED("lse_merge_kernel");
    return FM_OK;
}

extern "C" int fm_lse_merge_out(const float *acc_out, const float *acc_lse, const void *blk_out, int blk_dtype, const float *blk_lse,
                                void *dst, int dst_dtype, float *dst_lse, int64_t n_rows, int d, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(n_rows >= 0 && d > 0, "fm_lse_merge_out: bad sizes");
    if (n_rows == 0) return FM_OK;
    FM_REQUIRE(acc_out && acc_lse && blk_out && blk_lse && dst && dst_lse, "fm_lse_merge_out: null pointer");
    FM_REQUIRE(d % 4 == 0, "fm_lse_merge_out: head dim must be a multiple of 4");
    FM_REQUIRE(((uintptr_t)acc_out) % 16 == 0 && ((uintptr_t)blk_out) % 8 == 0 && ((uintptr_t)dst) % 8 == 0,
               "fm_lse_merge_out: misaligned buffer");
    FM_REQUIRE(dst_dtype == FM_F32 || dst_dtype == blk_dtype, "fm_lse_merge_out: the result is fp32 or in the block's dtype");
    FM_REQUIRE(dst_dtype != FM_F32 || ((uintptr_t)dst) % 16 == 0, "fm_lse_merge_out: misaligned buffer");
    cudaStream_t st = (cudaStream_t)stream;
    switch (blk_dtype) {
    case FM_F32: return launch_merge_out<float>(acc_out, acc_lse, blk_out, blk_lse, dst, dst_dtype, dst_lse, n_rows, d, st);
    case FM_BF16: return launch_merge_out<__nv_bfloat16>(acc_out, acc_lse, blk_out, blk_lse, dst, dst_dtype, dst_lse, n_rows, d, st);
    case FM_F16: return launch_merge_out<__half>(acc_out, acc_lse, blk_out, blk_lse, dst, dst_dtype, dst_lse, n_rows, d, st);
    default: set_error("fm_lse_merge_out: unknown dtype %d", blk_dtype); return FM_ERR_UNSUPPORTED;
    }
}

extern "C" int fm_merge_peer_partials(const void *const *o_ptrs, const float *const *lse_ptrs, float *const *out_ptrs,
                                      float *const *lse_out_ptrs, int world, int o_dtype, int64_t row0, int64_t row1, int d,
                                      fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(o_ptrs && lse_ptrs && out_ptrs && lse_out_ptrs, "fm_merge_peer_partials: null pointer");
    FM_REQUIRE(world >= 1 && world <= kMaxPeers, "fm_merge_peer_partials: 1 to %d ranks, got %d", kMaxPeers, world);
    FM_REQUIRE(row0 >= 0 && row1 >= row0 && d > 0 && d % 8 == 0, "fm_merge_peer_partials: bad sizes");
    if (row1 == row0) return FM_OK;
    PeerMergeParams p = {};
    for (int w = 0; w < world; ++w) {
        FM_REQUIRE(o_ptrs[w] && lse_ptrs[w] && out_ptrs[w] && lse_out_ptrs[w], "fm_merge_peer_partials: null buffer of rank %d", w);
        FM_REQUIRE(((uintptr_t)o_ptrs[w] | (uintptr_t)out_ptrs[w]) % 16 == 0, "fm_merge_peer_partials: buffers must be 16-byte aligned");
        p.o[w] = o_ptrs[w]; p.lse[w] = lse_ptrs[w]; p.out[w] = out_ptrs[w]; p.lse_out[w] = lse_out_ptrs[w];
    }
    p.world = world; p.d = d; p.row0 = row0; p.row1 = row1;
    const int64_t threads = (row1 - row0) * (d / 8);
    const unsigned grid = (unsigned)ceil_div(threads, 256);
    cudaStream_t st = (cudaStream_t)stream;
    if (o_dtype == FM_F32) peer_merge_kernel<float><<<grid, 256, 0, st>>>(p);
    else if (o_dtype == FM_BF16) peer_merge_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
    else if (o_dtype == FM_F16) peer_merge_kernel<__half><<<grid, 256, 0, st>>>(p);
    else {
        set_error("fm_merge_peer_partials: unknown dtype %d", o_dtype);
        return FM_ERR_UNSUPPORTED;
    }
    FM_LAUNCHED("peer_merge_kernel");
    return FM_OK;
}
