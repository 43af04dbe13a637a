// Hashed attention backward: dQ, dK, dV over the gathered rows of every query's bucket.
//
// Stands in for ring_attention_masked_backward of the reference (memory.py:166-206), which rebuilds a dense
// [queries x keys] mask and runs five einsums over it; here only the (query, key) pairs that exist are touched:
//     P  = exp(q.k * sm_scale - lse)              lse = the log-sum-exp the forward pass was normalised with (it may
//     dV += P^T dO                                      cover more keys than this memory: merged results, mem:332)
//     dP = dO V^T,  D = rowsum(dO * O)
//     dS = P * (dP - D)
//     dQ = dS K * sm_scale,  dK += dS^T Q * sm_scale
// One CTA per bucket walks the bucket's query blocks (16 queries) and key tiles (64 keys) on the CUDA cores in fp32.
// A query lies in exactly one bucket, so dQ rows are written once; a key lies in several buckets, so dK and dV are
// accumulated with fp32 (16-byte vector) atomics into buffers the caller has zeroed (or is accumulating shard after shard).
// This is the training-time companion of the forward kernels, written for parity first: no tensor cores yet.
#include "attn_bwd.cuh"

#include <cstdlib>

namespace fm {

namespace {

constexpr int kBwdThreads = 128;
constexpr int kBwdQ = 16;                   // queries per block
constexpr int kBwdK = 64;                   // keys per tile
constexpr int kPLd = kBwdK + 1;


// PASSES = ceil(d / 128): in the d-wide phases a lane owns four consecutive columns of every 128-column pass and a warp
// a quarter of the tile's keys, so that dK and dV go out as 16-byte vector atomics (a quarter of the atomic traffic).
template <typename T, int PASSES>
__global__ void __launch_bounds__(kBwdThreads)
attn_bwd_kernel(BwdParams p, int d)
{
    extern __shared__ __align__(16) float bsm[];
    const int ld = d + 1;                                    // odd row stride: a warp reading one column of 32 rows hits 32 banks
    float *Qs = bsm;                                         // [kBwdQ][d]
    float *Gs = Qs + kBwdQ * d;                              // [kBwdQ][d]   dO
    float *Ks = Gs + kBwdQ * d;                              // [kBwdK][ld]
    float *Vs = Ks + kBwdK * ld;                             // [kBwdK][ld]
    float *Ps = Vs + kBwdK * ld;                             // [kBwdQ][kPLd]
    float *Ss = Ps + kBwdQ * kPLd;                           // [kBwdQ][kPLd] dS
    float *Dq = Ss + kBwdQ * kPLd;                           // [kBwdQ]
    float *Lq = Dq + kBwdQ;                                  // [kBwdQ]
    __shared__ int64_t rows_s[kBwdK];

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int gb = blockIdx.x;
    const int q0 = p.group_off[gb], nq_all = p.group_off[gb + 1] - q0;
    const int64_t kb = p.bucket_off[gb], len = p.bucket_off[gb + 1] - kb;
    if (nq_all <= 0 || len <= 0) return;
    const int64_t kbase = p.bucket_kbase ? p.bucket_kbase[gb] : 0;
    const T *qg = reinterpret_cast<const T *>(p.q), *og = reinterpret_cast<const T *>(p.o), *gg = reinterpret_cast<const T *>(p.d_o);
    const T *kg = reinterpret_cast<const T *>(p.k), *vg = reinterpret_cast<const T *>(p.v);

    for (int qb = 0; qb < nq_all; qb += kBwdQ) {
        const int nq = min(kBwdQ, nq_all - qb);
        __syncthreads();
        // queries, their output gradients, D = rowsum(dO * O) and the LSE
        for (int e = t; e < kBwdQ * d; e += kBwdThreads) {
            const int qi = e / d, c = e - qi * d;
            float qv = 0.f, gv = 0.f;
            if (qi < nq) {
                const size_t row = size_t(p.perm[q0 + qb + qi]);
                qv = Elem<T>::to_f32(qg[row * d + c]);
                gv = Elem<T>::to_f32(gg[row * d + c]);
            }
            Qs[e] = qv;
            Gs[e] = gv;
        }
        for (int qi = warp; qi < kBwdQ; qi += kBwdThreads / 32) {
            float acc = 0.f;
            if (qi < nq) {
                const size_t row = size_t(p.perm[q0 + qb + qi]);
                for (int c = lane; c < d; c += 32) acc = fmaf(Elem<T>::to_f32(gg[row * d + c]), Elem<T>::to_f32(og[row * d + c]), acc);
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (lane == 0) {
                Dq[qi] = acc;
                Lq[qi] = qi < nq ? p.lse[p.perm[q0 + qb + qi]] : INFINITY;       // +inf: P = 0 for rows that do not exist
            }
        }
        float dq_acc[PASSES][kBwdQ][4];                      // this warp's keys only; folded over the warps at the end
#pragma unroll
        for (int u = 0; u < PASSES; ++u)
#pragma unroll
            for (int a = 0; a < kBwdQ; ++a) dq_acc[u][a][0] = dq_acc[u][a][1] = dq_acc[u][a][2] = dq_acc[u][a][3] = 0.f;

        for (int64_t t0 = 0; t0 < len; t0 += kBwdK) {
            const int nk = int(min(int64_t(kBwdK), len - t0));
            __syncthreads();
            if (t < kBwdK) {
                int64_t row = -1;
                if (t < nk) {
                    row = load_index(p.table, p.idx_bytes, kb + t0 + t) + kbase;
                    row = min(max(row, int64_t(0)), p.n_k_rows - 1);
                }
                rows_s[t] = row;
            }
            __syncthreads();
            for (int e = t; e < kBwdK * d; e += kBwdThreads) {
                const int j = e / d, c = e - j * d;
                const int64_t row = rows_s[j];
                Ks[j * ld + c] = row >= 0 ? Elem<T>::to_f32(kg[size_t(row) * d + c]) : 0.f;
                Vs[j * ld + c] = row >= 0 ? Elem<T>::to_f32(vg[size_t(row) * d + c]) : 0.f;
            }
            __syncthreads();
            // P and dS: thread -> key j, 8 of the 16 queries
            {
                const int j = t & (kBwdK - 1), qh = (t >> 6) * 8;
                float s[8], dp[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) s[a] = dp[a] = 0.f;
                for (int c = 0; c < d; ++c) {
                    const float kv = Ks[j * ld + c], vv = Vs[j * ld + c];
#pragma unroll
                    for (int a = 0; a < 8; ++a) {
                        s[a] = fmaf(Qs[(qh + a) * d + c], kv, s[a]);
                        dp[a] = fmaf(Gs[(qh + a) * d + c], vv, dp[a]);
                    }
                }
#pragma unroll
                for (int a = 0; a < 8; ++a) {
                    const int qi = qh + a;
                    const float l = Lq[qi];
                    // an empty softmax (lse = -inf) or a missing row / key contributes nothing
                    const float pv = (j < nk && l > -INFINITY && l < INFINITY) ? expf(s[a] * p.sm_scale - l) : 0.f;
                    Ps[qi * kPLd + j] = pv;
                    Ss[qi * kPLd + j] = pv * (dp[a] - Dq[qi]);
                }
            }
            __syncthreads();
            // the d-wide phases: warp -> keys j = warp, warp + 4, ...; lane -> columns 4 lane .. 4 lane + 3 of each pass
#pragma unroll
            for (int u = 0; u < PASSES; ++u) {
                const int c = u * 128 + lane * 4;
                if (c < d) {
                    for (int j = warp; j < nk; j += kBwdThreads / 32) {
                        const float k0 = Ks[j * ld + c], k1 = Ks[j * ld + c + 1], k2 = Ks[j * ld + c + 2], k3 = Ks[j * ld + c + 3];
                        float4 dk4 = make_float4(0.f, 0.f, 0.f, 0.f), dv4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int a = 0; a < kBwdQ; ++a) {
                            const float ds = Ss[a * kPLd + j], pv = Ps[a * kPLd + j];
                            const float4 q4 = *reinterpret_cast<const float4 *>(Qs + a * d + c);
                            const float4 g4 = *reinterpret_cast<const float4 *>(Gs + a * d + c);
                            dq_acc[u][a][0] = fmaf(ds, k0, dq_acc[u][a][0]);      // dQ += dS K
                            dq_acc[u][a][1] = fmaf(ds, k1, dq_acc[u][a][1]);
                            dq_acc[u][a][2] = fmaf(ds, k2, dq_acc[u][a][2]);
                            dq_acc[u][a][3] = fmaf(ds, k3, dq_acc[u][a][3]);
                            dk4.x = fmaf(ds, q4.x, dk4.x); dk4.y = fmaf(ds, q4.y, dk4.y);      // dK += dS^T Q
                            dk4.z = fmaf(ds, q4.z, dk4.z); dk4.w = fmaf(ds, q4.w, dk4.w);
                            dv4.x = fmaf(pv, g4.x, dv4.x); dv4.y = fmaf(pv, g4.y, dv4.y);      // dV += P^T dO
                            dv4.z = fmaf(pv, g4.z, dv4.z); dv4.w = fmaf(pv, g4.w, dv4.w);
                        }
                        const size_t off = size_t(rows_s[j]) * d + c;
                        dk4.x *= p.sm_scale; dk4.y *= p.sm_scale; dk4.z *= p.sm_scale; dk4.w *= p.sm_scale;
                        atomicAdd(reinterpret_cast<float4 *>(p.dk + off), dk4);
                        atomicAdd(reinterpret_cast<float4 *>(p.dv + off), dv4);
                    }
                }
            }
        }
        // fold the four warps' dQ through shared memory (the key tiles are done with)
        __syncthreads();
        float *fold = Ks;                                    // [4][kBwdQ][d] <= the K and V tiles
#pragma unroll
        for (int u = 0; u < PASSES; ++u) {
            const int c = u * 128 + lane * 4;
            if (c < d) {
#pragma unroll
                for (int a = 0; a < kBwdQ; ++a)
                    *reinterpret_cast<float4 *>(fold + (warp * kBwdQ + a) * d + c) =
                        make_float4(dq_acc[u][a][0], dq_acc[u][a][1], dq_acc[u][a][2], dq_acc[u][a][3]);
            }
        }
        __syncthreads();
        for (int e = t; e < nq * d; e += kBwdThreads) {
            const int a = e / d, c = e - a * d;
            const float sum = (fold[(0 * kBwdQ + a) * d + c] + fold[(1 * kBwdQ + a) * d + c]) +
                              (fold[(2 * kBwdQ + a) * d + c] + fold[(3 * kBwdQ + a) * d + c]);
            p.dq[size_t(p.perm[q0 + qb + a]) * d + c] = sum * p.sm_scale;
        }
    }
}

template <typename T> static int launch_bwd(const BwdParams &p, int d, int64_t total_buckets, cudaStream_t st)
{
    const size_t smem = sizeof(float) * (2 * size_t(kBwdQ) * d + 2 * size_t(kBwdK) * (d + 1) + 2 * kBwdQ * kPLd + 2 * kBwdQ);
    if (d <= 128) {
        FM_CUDA_OK(func_attr_cached((const void *)attn_bwd_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attn_bwd_kernel<T, 1><<<(unsigned)total_buckets, kBwdThreads, smem, st>>>(p, d);
    } else {
        FM_CUDA_OK(func_attr_cached((const void *)attn_bwd_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attn_bwd_kernel<T, 2><<<(unsigned)total_buckets, kBwdThreads, smem, st>>>(p, d);
    }
    FM_LAUNCHED("attn_bwd_kernel");
    return FM_OK;
}

}  // namespace

}  // namespace fm

extern "C" int fm_hashed_attn_bwd(const void *q, const void *k, const void *v, int dtype, int d, int64_t n_q_rows, int64_t n_k_rows,
                                  int64_t total_buckets, const void *table, int idx_bytes, const int64_t *bucket_off,
                                  const int32_t *bucket_kbase, const int32_t *group_off, const int32_t *perm, float sm_scale,
                                  const void *o, const float *lse, const void *d_o, float *dq, float *dk, float *dv,
                                  fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(q && k && v && table && bucket_off && group_off && perm && o && lse && d_o && dq && dk && dv,
               "fm_hashed_attn_bwd: null pointer");
    FM_REQUIRE(n_q_rows >= 0 && n_k_rows > 0 && total_buckets > 0 && total_buckets < (int64_t(1) << 31), "fm_hashed_attn_bwd: bad sizes");
    FM_REQUIRE(idx_bytes == 4 || idx_bytes == 8, "fm_hashed_attn_bwd: idx_bytes must be 4 or 8");
    if (d < 16 || d > 256 || d % 16) {
        set_error("fm_hashed_attn_bwd: head dim %d not supported (multiple of 16 in [16, 256])", d);
        return FM_ERR_UNSUPPORTED;
    }
    if (n_q_rows == 0) return FM_OK;
    BwdParams p = {q, k, v, o, d_o, lse, table, idx_bytes, bucket_off, bucket_kbase, group_off, perm, n_k_rows, sm_scale, dq, dk, dv};
    cudaStream_t st = (cudaStream_t)stream;
    // rows of dq whose bucket is empty are never visited: start from zero
    FM_CUDA_OK(cudaMemsetAsync(dq, 0, size_t(n_q_rows) * d * sizeof(float), st));
    // 16-bit inputs with a head dim the tensor-core kernel is built for (rows 16-byte aligned): mma.sync
    static const bool simt_only = getenv("FASTMEM_BWD_SIMT") != nullptr;        // (the CUDA-core kernel, for comparison)
    if ((dtype == FM_BF16 || dtype == FM_F16) && (d == 64 || d == 128) &&
        (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o | (uintptr_t)d_o) % 16 == 0) && !simt_only)
        return launch_bwd_mma(p, dtype, d, total_buckets, st);
    switch (dtype) {
    case FM_F32: return launch_bwd<float>(p, d, total_buckets, st);
    case FM_BF16: return launch_bwd<__nv_bfloat16>(p, d, total_buckets, st);
    case FM_F16: return launch_bwd<__half>(p, d, total_buckets, st);
    default: set_error("fm_hashed_attn_bwd: unknown dtype %d", dtype); return FM_ERR_UNSUPPORTED;
    }
}
