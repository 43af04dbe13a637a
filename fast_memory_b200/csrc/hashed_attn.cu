// Hashed attention forward: planning, the CUDA-core (any dtype, exact fp32 arithmetic) kernel, the
// partial combine, and the C entry point.  The tensor-core kernel for 16-bit inputs lives in
// hashed_attn_mma.cu and is dispatched from here.
//
// Semantics follow the reference kernel (triton_kernel.py:177-272): per (bucket, query block) the
// bucket's key rows are gathered through the table, scores are q.k * (sm_scale * log2 e), the softmax
// runs online in base 2 with the running maximum m and denominator l (started at -inf and 1), P is
// rounded to the input dtype before P.V while l sums the unrounded p, and the epilogue writes
// acc / l and m + log2 l.  Differences by design: queries are read and outputs written through the
// grouping permutation (no sorted copy of q, no scatter of o), the LSE is returned in natural-log fp32,
// and a bucket may be cut into key chunks whose partials are combined afterwards.
#include "attn_common.cuh"

#include <cstdlib>
#include <cstring>

namespace fm {

int launch_attn_mma(const AttnParams &p, int dtype, int d, int grid, cudaStream_t st);   // hashed_attn_mma.cu
bool attn_mma_supported(int dtype, int d);
int launch_attn_tc(const AttnParams &p, int dtype, int grid, int4 *redo_items, int *redo_count, cudaStream_t st);   // hashed_attn_tc.cu
bool attn_tc_supported(int dtype, int d);

// Which tensor-core kernel serves 16-bit inputs with head dim 128: the mma.sync kernel (0, the default: it is the faster
// one, see hashed_attn_tc.cu) or the tcgen05 kernel (1).  Set by fm_set_attn_kernel, initially from FASTMEM_ATTN_KERNEL
// (= mma | tc).
static std::atomic<int> g_attn_kernel{-1};
static bool prefer_tc_kernel()
{
    int c = g_attn_kernel.load(std::memory_order_relaxed);
    if (c < 0) {
        const char *e = getenv("FASTMEM_ATTN_KERNEL");
        c = (e && !strcmp(e, "tc")) ? 1 : 0;
        g_attn_kernel.store(c, std::memory_order_relaxed);
    }
    return c == 1;
}

// ---- planning -----------------------------------------------------------------------------------
__global__ void attn_plan_kernel(AttnParams p)
{
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= p.total_buckets) return;
    int q0 = p.group_off[b], nq = p.group_off[b + 1] - q0;
    if (nq <= 0) return;
    int64_t len = p.bucket_off[b + 1] - p.bucket_off[b];
    int nkc = len > 0 ? int((len + p.key_chunk - 1) / p.key_chunk) : 1;
    if (nkc > p.nkc_max) {
        // a bucket longer than the max_bucket_len the workspace was sized for: its partials would not fit, so the keys
        // beyond nkc_max chunks are left out and the anomaly is recorded in the workspace's third counter
        nkc = p.nkc_max;
        p.counters[2] = 1;
    }
    int nqb = (nq + p.q_block - 1) / p.q_block;
    int base = atomicAdd(&p.counters[0], nqb * nkc);
    for (int qb = 0; qb < nqb; ++qb)
        for (int kc = 0; kc < nkc; ++kc) {
            int id = base + qb * nkc + kc;
            if (id < p.max_items) p.items[id] = make_int4(b, q0 + qb * p.q_block, kc, nkc);
        }
}

// ---- CUDA-core kernel -----------------------------------------------------------------------------
constexpr int kSimtThreads = 128;
constexpr int kSimtTK = 64;                 // keys per tile
constexpr int kSLd = kSimtTK + 4;           // row stride of the score tile (floats)

template <typename T, int D> struct SimtCfg {
    static constexpr int CPT = D > 128 ? D / 128 : 1;          // output columns per thread
    static constexpr int TPC = D / CPT;                         // threads across the columns
    static constexpr int QG = kSimtThreads / TPC;               // query groups
    static constexpr int QPT = kQB / QG;                        // queries per thread
    static constexpr int EPC = 16 / sizeof(T);                  // elements per 16-byte chunk
    static constexpr int LDK = D + EPC;                         // K tile row stride (elements): odd number of chunks
    static constexpr size_t smem =
        sizeof(float) * (kQB * D + kQB * kSLd + 3 * kQB) + sizeof(int64_t) * kSimtTK + sizeof(T) * (kSimtTK * LDK + kSimtTK * D);
};

template <typename T, int D>
__global__ void __launch_bounds__(kSimtThreads)
attn_simt_kernel(AttnParams p)
{
    using C = SimtCfg<T, D>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int64_t *idx_s = reinterpret_cast<int64_t *>(smem_raw);
    float *Qs = reinterpret_cast<float *>(idx_s + kSimtTK);    // [kQB][D]
    float *Ss = Qs + kQB * D;                                  // [kQB][kSLd]
    float *m_s = Ss + kQB * kSLd;                              // [kQB]
    float *l_s = m_s + kQB;
    float *a_s = l_s + kQB;
    T *Ks = reinterpret_cast<T *>(a_s + kQB);                  // [kSimtTK][LDK]
    T *Vs = Ks + kSimtTK * C::LDK;                             // [kSimtTK][D]
    __shared__ int s_item;

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const T *qg = reinterpret_cast<const T *>(p.q);
    const T *kg = reinterpret_cast<const T *>(p.k);
    const T *vg = reinterpret_cast<const T *>(p.v);
    const int n_items = min(p.counters[0], p.max_items);

    for (;;) {
        __syncthreads();
        if (t == 0) s_item = atomicAdd(&p.counters[1], 1);
        __syncthreads();
        const int item = s_item;
        if (item >= n_items) break;
        const int4 it = p.items[item];
        const int gb = it.x, q_begin = it.y, kc = it.z, nkc = it.w;
        const int nq = min(kQB, p.group_off[gb + 1] - q_begin);
        const int64_t kb = p.bucket_off[gb];
        const int64_t len = p.bucket_off[gb + 1] - kb;
        const int64_t k0 = int64_t(kc) * p.key_chunk;
        const int64_t k1 = min(len, k0 + p.key_chunk);
        const int64_t kbase = p.bucket_kbase ? p.bucket_kbase[gb] : 0;

        // queries -> fp32 in shared memory (rows beyond nq are zero)
        for (int e = t; e < kQB * D; e += kSimtThreads) {
            int qi = e / D, c = e - qi * D;
            float val = 0.f;
            if (qi < nq) val = Elem<T>::to_f32(qg[size_t(p.perm[q_begin + qi]) * D + c]);
            Qs[e] = val;
        }
        if (t < kQB) { m_s[t] = -INFINITY; l_s[t] = 1.f; }
        float acc[C::QPT][C::CPT];
#pragma unroll
        for (int a = 0; a < C::QPT; ++a)
#pragma unroll
            for (int c = 0; c < C::CPT; ++c) acc[a][c] = 0.f;
        const int col0 = (t % C::TPC) * C::CPT;
        const int qg0 = (t / C::TPC) * C::QPT;

        for (int64_t t0 = k0; t0 < k1; t0 += kSimtTK) {
            const int nk = int(min(int64_t(kSimtTK), k1 - t0));
            __syncthreads();                                    // previous tile consumed, Qs / m / l visible
            if (t < kSimtTK) {
                int64_t row = -1;
                if (t < nk) {
                    // entries outside [0, n_k_rows) are clamped: a malformed table never reads out of bounds
                    row = load_index(p.table, p.idx_bytes, kb + t0 + t) + kbase;
                    row = min(max(row, int64_t(0)), p.n_k_rows - 1);
                }
                idx_s[t] = row;
            }
            __syncthreads();
            constexpr int CPR = D / C::EPC;                     // 16-byte chunks per row
            for (int e = t; e < kSimtTK * CPR; e += kSimtThreads) {
                int j = e / CPR, ch = e - j * CPR;
                int64_t row = idx_s[j];
                uint4 kk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
                if (row >= 0) {
                    kk = *reinterpret_cast<const uint4 *>(kg + size_t(row) * D + ch * C::EPC);
                    vv = *reinterpret_cast<const uint4 *>(vg + size_t(row) * D + ch * C::EPC);
                }
                *reinterpret_cast<uint4 *>(Ks + j * C::LDK + ch * C::EPC) = kk;
                *reinterpret_cast<uint4 *>(Vs + j * D + ch * C::EPC) = vv;
            }
            __syncthreads();
            // scores: thread -> key j, 8 of the 16 queries
            {
                const int j = t & (kSimtTK - 1), qh = (t >> 6) * 8;
                float s[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) s[a] = 0.f;
                const T *krow = Ks + j * C::LDK;
                for (int c = 0; c < D; c += C::EPC) {
                    float kf[8];
                    if constexpr (sizeof(T) == 4) {
                        float4 kq = *reinterpret_cast<const float4 *>(krow + c);
                        kf[0] = kq.x; kf[1] = kq.y; kf[2] = kq.z; kf[3] = kq.w;
                    } else {
                        uint4 raw = *reinterpret_cast<const uint4 *>(krow + c);
                        widen8(raw, kf, T());
                    }
#pragma unroll
                    for (int a = 0; a < 8; ++a) {
                        const float *qrow = Qs + (qh + a) * D + c;
#pragma unroll
                        for (int e = 0; e < C::EPC; ++e) s[a] = fmaf(qrow[e], kf[e], s[a]);
                    }
                }
                const bool live = j < nk && idx_s[j] >= 0;
#pragma unroll
                for (int a = 0; a < 8; ++a) Ss[(qh + a) * kSLd + j] = live ? s[a] * p.scale2 : -INFINITY;
            }
            __syncthreads();
            // online softmax: warp w owns query rows 4w .. 4w+3
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const int qi = warp * 4 + a;
                float s0 = Ss[qi * kSLd + lane], s1 = Ss[qi * kSLd + lane + 32];
                float mx = fmaxf(s0, s1);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
                const float m_old = m_s[qi];
                const float m_new = fmaxf(m_old, mx);
                float p0 = 0.f, p1 = 0.f, alpha = 1.f;
                if (m_new > -INFINITY) {
                    p0 = exp2f(s0 - m_new);
                    p1 = exp2f(s1 - m_new);
                    alpha = exp2f(m_old - m_new);
                }
                float sum = p0 + p1;
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                Ss[qi * kSLd + lane] = Elem<T>::to_f32(Elem<T>::from_f32(p0));
                Ss[qi * kSLd + lane + 32] = Elem<T>::to_f32(Elem<T>::from_f32(p1));
                if (lane == 0) {
                    m_s[qi] = m_new;
                    l_s[qi] = l_s[qi] * alpha + sum;
                    a_s[qi] = alpha;
                }
            }
            __syncthreads();
            // acc = acc * alpha + P V
#pragma unroll
            for (int a = 0; a < C::QPT; ++a) {
                const float al = a_s[qg0 + a];
#pragma unroll
                for (int c = 0; c < C::CPT; ++c) acc[a][c] *= al;
            }
            for (int j = 0; j < kSimtTK; j += 4) {
                float vv[4][C::CPT];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj)
#pragma unroll
                    for (int c = 0; c < C::CPT; ++c) vv[jj][c] = Elem<T>::to_f32(Vs[(j + jj) * D + col0 + c]);
#pragma unroll
                for (int a = 0; a < C::QPT; ++a) {
                    float4 pp = *reinterpret_cast<const float4 *>(Ss + (qg0 + a) * kSLd + j);
#pragma unroll
                    for (int c = 0; c < C::CPT; ++c) {
                        float y = acc[a][c];
                        y = fmaf(pp.x, vv[0][c], y);
                        y = fmaf(pp.y, vv[1][c], y);
                        y = fmaf(pp.z, vv[2][c], y);
                        y = fmaf(pp.w, vv[3][c], y);
                        acc[a][c] = y;
                    }
                }
            }
        }
        __syncthreads();
        // epilogue
        if (nkc == 1) {
#pragma unroll
            for (int a = 0; a < C::QPT; ++a) {
                const int qi = qg0 + a;
                if (qi < nq) {
                    const size_t row = p.perm[q_begin + qi];
                    const float l = l_s[qi];
                    T *orow = reinterpret_cast<T *>(p.o) + row * D;
#pragma unroll
                    for (int c = 0; c < C::CPT; ++c) orow[col0 + c] = Elem<T>::from_f32(acc[a][c] / l);
                }
            }
            if (t < nq) p.lse[p.perm[q_begin + t]] = (m_s[t] + log2f(l_s[t])) * 0.6931471805599453f;
        } else {
#pragma unroll
            for (int a = 0; a < C::QPT; ++a) {
                const int qi = qg0 + a;
                if (qi < nq) {
                    float *dst = p.partials + (size_t(q_begin + qi) * p.nkc_max + kc) * (D + 2);
#pragma unroll
                    for (int c = 0; c < C::CPT; ++c) dst[col0 + c] = acc[a][c];
                }
            }
            if (t < nq) {
                float *dst = p.partials + (size_t(q_begin + t) * p.nkc_max + kc) * (D + 2);
                dst[D] = m_s[t];
                dst[D + 1] = l_s[t];
                if (kc == 0) p.qparts[q_begin + t] = nkc;
            }
        }
    }
}

// ---- combine: fold the per-chunk partials of one query ----------------------------------------------
template <typename T>
__global__ void attn_combine_kernel(AttnParams p, int d)
{
    const int qpos = blockIdx.x;
    const int n = p.qparts[qpos];
    if (n <= 1) return;                                         // unsplit buckets were written directly
    const float *base = p.partials + size_t(qpos) * p.nkc_max * (d + 2);
    float M = -INFINITY;
    for (int i = 0; i < n; ++i) M = fmaxf(M, base[size_t(i) * (d + 2) + d]);
    float L = 0.f;
    for (int i = 0; i < n; ++i) {
        float mi = base[size_t(i) * (d + 2) + d];
        L += base[size_t(i) * (d + 2) + d + 1] * (mi > -INFINITY ? exp2f(mi - M) : 0.f);
    }
    const size_t row = p.perm[qpos];
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < n; ++i) {
            float mi = base[size_t(i) * (d + 2) + d];
            acc += base[size_t(i) * (d + 2) + c] * (mi > -INFINITY ? exp2f(mi - M) : 0.f);
        }
        reinterpret_cast<T *>(p.o)[row * d + c] = Elem<T>::from_f32(acc / L);
    }
    if (threadIdx.x == 0) p.lse[row] = (M + log2f(L)) * 0.6931471805599453f;
}

template <typename T, int D>
static int launch_simt(const AttnParams &p, int grid, cudaStream_t st)
{
    size_t smem = SimtCfg<T, D>::smem;
    FM_CUDA_OK(func_attr_cached((const void *)attn_simt_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_simt_kernel<T, D><<<grid, kSimtThreads, smem, st>>>(p);
    FM_LAUNCHED("attn_simt_kernel");
    return FM_OK;
}

template <typename T>
static int dispatch_simt(const AttnParams &p, int d, int grid, cudaStream_t st)
{
    switch (d) {
    case 16: return launch_simt<T, 16>(p, grid, st);
    case 32: return launch_simt<T, 32>(p, grid, st);
    case 64: return launch_simt<T, 64>(p, grid, st);
    case 128: return launch_simt<T, 128>(p, grid, st);
    case 256: return launch_simt<T, 256>(p, grid, st);
    default:
        set_error("fm_hashed_attn_fwd: head dim %d not supported (16, 32, 64, 128, 256)", d);
        return FM_ERR_UNSUPPORTED;
    }
}

}  // namespace fm

extern "C" int fm_set_attn_kernel(int which)
{
    if (which != 0 && which != 1) {
        fm::set_error("fm_set_attn_kernel: 0 (mma.sync) or 1 (tcgen05), got %d", which);
        return FM_ERR_BAD_ARG;
    }
    fm::g_attn_kernel.store(which, std::memory_order_relaxed);
    return FM_OK;
}

extern "C" size_t fm_hashed_attn_workspace_bytes(int64_t n_q_rows, int64_t total_buckets, int64_t max_bucket_len, int d,
                                                 int64_t key_chunk)
{
    return fm::attn_layout(n_q_rows, total_buckets, max_bucket_len, d, key_chunk, fm::sm_count()).total;
}

extern "C" int fm_hashed_attn_fwd(const void *q, const void *k, const void *v, int dtype, int d, int64_t n_q_rows,
                                  int64_t n_k_rows, int64_t total_buckets, const void *table, int idx_bytes,
                                  const int64_t *bucket_off, const int32_t *bucket_kbase, int64_t max_bucket_len,
                                  const int32_t *group_off, const int32_t *perm, float sm_scale, void *o, float *lse,
                                  int64_t key_chunk, void *workspace, size_t workspace_bytes, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(n_q_rows >= 0 && n_k_rows >= 0 && total_buckets > 0, "fm_hashed_attn_fwd: bad sizes");
    if (n_q_rows == 0) return FM_OK;
    FM_REQUIRE(q && o && lse && bucket_off && group_off && perm && workspace, "fm_hashed_attn_fwd: null pointer");
    FM_REQUIRE(n_k_rows == 0 || (k && v && table), "fm_hashed_attn_fwd: null key/value/table pointer");
    FM_REQUIRE(idx_bytes == 4 || idx_bytes == 8, "fm_hashed_attn_fwd: idx_bytes must be 4 or 8");
    FM_REQUIRE(n_q_rows < (int64_t(1) << 31) && total_buckets < (int64_t(1) << 31), "fm_hashed_attn_fwd: sizes exceed int32");
    FM_REQUIRE(((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) % 16 == 0, "fm_hashed_attn_fwd: q/k/v/o must be 16-byte aligned");
    if (dtype != FM_F32 && dtype != FM_BF16 && dtype != FM_F16) {
        set_error("fm_hashed_attn_fwd: unknown dtype %d", dtype);
        return FM_ERR_UNSUPPORTED;
    }
    const int sms = sm_count();
    AttnLayout L = attn_layout(n_q_rows, total_buckets, max_bucket_len, d, key_chunk, sms);
    if (workspace_bytes < L.total) {
        set_error("fm_hashed_attn_fwd: workspace %zu < %zu", workspace_bytes, L.total);
        return FM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    char *ws = (char *)workspace;
    AttnParams p;
    p.q = q; p.k = k; p.v = v; p.o = o; p.lse = lse;
    p.table = table; p.idx_bytes = idx_bytes; p.bucket_off = bucket_off; p.bucket_kbase = bucket_kbase;
    p.group_off = group_off; p.perm = perm;
    p.total_buckets = (int)total_buckets; p.n_q_rows = (int)n_q_rows; p.n_k_rows = n_k_rows;
    p.key_chunk = L.key_chunk; p.nkc_max = L.nkc_max;
    p.scale2 = sm_scale * 1.44269504f;
    p.counters = (int *)ws;
    p.items = (int4 *)(ws + L.off_items);
    p.max_items = (int)std::min<int64_t>(L.max_items, 0x7fffffff);
    p.qparts = (int32_t *)(ws + L.off_qparts);
    p.partials = (float *)(ws + L.off_partials);

    // the tensor-core kernel tracks the row maximum before scaling, which needs a positive scale
    const bool use_mma = attn_mma_supported(dtype, d) && sm_scale > 0.f;
    // items of up to 32 queries gather a bucket once for two row tiles but take twice as long as a 16-query item: with
    // plenty of (bucket, queries) groups per CTA that is a pure gain, with few (decode) the long items leave CTAs idle
    // at the end of the launch, so the queries are cut into 16-query items there
    const int64_t groups_bound = std::min<int64_t>(total_buckets, n_q_rows);
    p.q_block = use_mma ? (groups_bound >= int64_t(24) * sms ? 32 : 16) : kQB;

    FM_CUDA_OK(cudaMemsetAsync(p.counters, 0, 64, st));
    if (L.nkc_max > 1) FM_CUDA_OK(cudaMemsetAsync(p.qparts, 0, size_t(n_q_rows) * 4, st));
    attn_plan_kernel<<<(unsigned)ceil_div(total_buckets, 256), 256, 0, st>>>(p);
    FM_LAUNCHED("attn_plan_kernel");

    int rc;
    int grid = (int)std::min<int64_t>(L.max_items, int64_t(sms) * (use_mma ? 3 : 4));
    if (use_mma && attn_tc_supported(dtype, d) && prefer_tc_kernel()) {
        // tcgen05 kernel, one CTA per SM; the items it hands back (a later score far above the first tile's best) are
        // served again by the mma.sync kernel, which reads their count from the device
        int4 *redo = (int4 *)(ws + L.off_redo);
        rc = launch_attn_tc(p, dtype, (int)std::min<int64_t>(L.max_items, sms), redo, p.counters + 8, st);
        if (rc == FM_OK) {
            AttnParams again = p;
            again.items = redo;
            again.counters = p.counters + 8;
            rc = launch_attn_mma(again, dtype, d, (int)std::min<int64_t>(L.max_items, 2 * int64_t(sms)), st);
        }
    } else if (use_mma) rc = launch_attn_mma(p, dtype, d, grid, st);
    else if (dtype == FM_F32) rc = dispatch_simt<float>(p, d, grid, st);
    else if (dtype == FM_BF16) rc = dispatch_simt<__nv_bfloat16>(p, d, grid, st);
    else rc = dispatch_simt<__half>(p, d, grid, st);
    if (rc != FM_OK) return rc;

    if (L.nkc_max > 1) {
        if (dtype == FM_F32) attn_combine_kernel<float><<<(unsigned)n_q_rows, 128, 0, st>>>(p, d);
        else if (dtype == FM_BF16) attn_combine_kernel<__nv_bfloat16><<<(unsigned)n_q_rows, 128, 0, st>>>(p, d);
        else attn_combine_kernel<__half><<<(unsigned)n_q_rows, 128, 0, st>>>(p, d);
        FM_LAUNCHED("attn_combine_kernel");
    }
    return FM_OK;
}
