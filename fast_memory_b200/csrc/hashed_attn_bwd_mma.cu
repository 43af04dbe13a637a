// Hashed attention backward on the tensor cores (mma.sync m16n8k16) for 16-bit inputs, head dim 64 or 128:
// dQ, dK, dV over the gathered rows of every query's bucket (memory.py:166-206 of the reference).
//
// One CTA (four warps) per bucket walks the bucket's query blocks (16 queries: one MMA row tile) and, inside, its key
// tiles of 64 gathered rows (K and V through a two-stage cp.async ring, XOR-swizzled); warp w takes keys 16 w .. 16 w + 15
// of every tile.  Per (query block, tile, warp), all in the orientation of the forward kernel (queries on M):
//     S  = Q K^T,  dP = dO V^T                  (A = Q / dO from shared memory, B = K / V rows, ldmatrix)
//     P  = 2^(S scale2 - lse2),  dS = P (dP - D) sm_scale,   D = rowsum(dO o O)
//     dQ += dS K                                 (A = dS from the accumulator registers, B = K through ldmatrix.trans)
//     dV += P^T dO,  dK += dS^T Q                (A = the 8x8 blocks of P / dS transposed by movmatrix, B = dO / Q through
//                                                 ldmatrix.trans), sixteen columns at a time, straight into global memory
//                                                 with 8-byte vector reductions: a key lies in several buckets
// P and dS are rounded to the input type before they become operands, as the forward kernel rounds P.  dQ stays in
// registers across the key tiles and the four warps' parts are added through shared memory at the end of a query block
// (a query lies in exactly one bucket: plain stores).  The caller has zeroed dq and zeroed or pre-loaded dk / dv.
#include "attn_bwd.cuh"
#include "mma_utils.cuh"

namespace fm {

namespace {

constexpr int kThreads = 128;
constexpr int kTK = 64;                     // keys per tile
constexpr int kQB = 16;                     // queries per block

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a)
{
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ void red_add_v2(float *addr, float a, float b)
{
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};\n" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 3)
attn_bwd_mma_kernel(BwdParams p)
{
    constexpr int CPR = D / 8;                               // 16-byte chunks per row
    constexpr int ROW_BYTES = D * 2;
    constexpr int QB_BYTES = kQB * ROW_BYTES;                // a block of queries (or of their output gradients)
    constexpr int TILE_BYTES = kTK * ROW_BYTES;              // a K (or V) tile
    constexpr int FOLD_LD = D + 4;
    static_assert(4 * kQB * FOLD_LD * 4 <= 4 * TILE_BYTES, "the dQ fold buffer must fit in the tile stages");
    extern __shared__ __align__(128) unsigned char bsm[];
    __shared__ int32_t rows_s[2][kTK];
    __shared__ float lq_s[kQB], dq_s[kQB];

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int gb = blockIdx.x;
    const int q0 = p.group_off[gb], nq_all = p.group_off[gb + 1] - q0;
    const int64_t kb = p.bucket_off[gb], len = p.bucket_off[gb + 1] - kb;
    if (nq_all <= 0 || len <= 0) return;
    const int64_t kbase = p.bucket_kbase ? p.bucket_kbase[gb] : 0;
    const T *qg = reinterpret_cast<const T *>(p.q), *og = reinterpret_cast<const T *>(p.o), *gg = reinterpret_cast<const T *>(p.d_o);
    const char *kg = reinterpret_cast<const char *>(p.k), *vg = reinterpret_cast<const char *>(p.v);
    const uint32_t sbase = smem_u32(bsm);
    const uint32_t qs = sbase, gs = sbase + QB_BYTES, kv0 = sbase + 2 * QB_BYTES;     // Q block, dO block, two (K, V) stages
    const int n_tiles = int((len + kTK - 1) / kTK);
    const int32_t row_max = int32_t(min(p.n_k_rows - 1, int64_t(0x7fffffff)));
    const float scale2 = p.sm_scale * 1.4426950408889634f;
    const int wk0 = warp * 16;

    // lane parts of the ldmatrix addresses (row, 16-byte chunk) inside a swizzled [rows][D] tile
    const int a_row = (lane & 7) + (((lane >> 3) & 1) << 3), a_chk = lane >> 4;      // A operand: Q / dO, 16 rows
    const int b_row = (lane & 7) + ((lane >> 4) << 3), b_chk = (lane >> 3) & 1;      // B operand, k = head dim: K / V rows
    const int c_row = (lane & 7) + (((lane >> 3) & 1) << 3), c_chk = lane >> 4;      // B operand, transposed loads (k = rows)

    // table entries are fetched one tile ahead of the copies that need them, so the index load never stalls the gather
    constexpr int PER_T = kTK * CPR / kThreads;              // 16-byte pieces per thread, matrix and tile
    int32_t rows[PER_T];
    auto load_rows = [&](int tile) {
#pragma unroll
        for (int i = 0; i < PER_T; ++i) {
            const int j = (t + i * kThreads) / CPR;
            const int64_t pos = int64_t(tile) * kTK + j;
            rows[i] = (tile < n_tiles && pos < len) ? min(max(int32_t(load_index(p.table, p.idx_bytes, kb + pos) + kbase), 0), row_max) : -1;
        }
    };
    auto issue = [&](int tile) {
        if (tile < n_tiles) {
            const int st = tile & 1;
            const uint32_t kdst = kv0 + st * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
#pragma unroll
            for (int i = 0; i < PER_T; ++i) {
                const int idx = t + i * kThreads, j = idx / CPR, c = idx % CPR;
                const bool ok = rows[i] >= 0;
                if (c == 0) rows_s[st][j] = rows[i];
                const size_t off = size_t(max(rows[i], 0)) * ROW_BYTES + c * 16;
                cp_async16(kdst + swz<D>(j, c), kg + off, ok);
                cp_async16(vdst + swz<D>(j, c), vg + off, ok);
            }
        }
        cp_async_commit();
    };

    for (int qb = 0; qb < nq_all; qb += kQB) {
        const int nq = min(kQB, nq_all - qb);
        __syncthreads();                                     // the previous block's fold buffer and Q / dO are done with
        // Q and dO of the block through the permutation (rows that do not exist: zeros), D and the LSE
#pragma unroll
        for (int i = 0; i < kQB * CPR / kThreads; ++i) {
            const int idx = t + i * kThreads, r = idx / CPR, c = idx % CPR;
            const bool ok = r < nq;
            const size_t row = ok ? size_t(p.perm[q0 + qb + r]) : 0;
            cp_async16(qs + swz<D>(r, c), qg + row * D + c * 8, ok);
            cp_async16(gs + swz<D>(r, c), gg + row * D + c * 8, ok);
        }
        cp_async_commit();
        for (int r = warp; r < kQB; r += kThreads / 32) {
            float acc = 0.f;
            if (r < nq) {
                const size_t row = size_t(p.perm[q0 + qb + r]);
                for (int c = lane * 2; c < D; c += 64) {
                    acc = fmaf(Elem<T>::to_f32(gg[row * D + c]), Elem<T>::to_f32(og[row * D + c]), acc);
                    acc = fmaf(Elem<T>::to_f32(gg[row * D + c + 1]), Elem<T>::to_f32(og[row * D + c + 1]), acc);
                }
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (lane == 0) {
                dq_s[r] = acc;
                float l = r < nq ? p.lse[p.perm[q0 + qb + r]] : INFINITY;
                // an empty softmax (lse = -inf), a bad value or a row that does not exist: P = 2^(-inf) = 0
                lq_s[r] = (l > -INFINITY && l < INFINITY) ? l * 1.4426950408889634f : INFINITY;
            }
        }
        load_rows(0);
        issue(0);
        load_rows(1);

        float dq[D / 8][4];
#pragma unroll
        for (int n = 0; n < D / 8; ++n) dq[n][0] = dq[n][1] = dq[n][2] = dq[n][3] = 0.f;

        for (int tile = 0; tile < n_tiles; ++tile) {
            cp_async_wait<0>();
            __syncthreads();                                 // the tile (and, first time round, Q / dO / D / LSE) landed; the other stage is free
            issue(tile + 1);
            load_rows(tile + 2);
            const int st = tile & 1;
            const uint32_t ks = kv0 + st * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
            const int live = int(min(int64_t(kTK), len - int64_t(tile) * kTK));

            // S = Q K^T and dP = dO V^T for this warp's 16 keys
            float s[2][4], dp[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[n][e] = dp[n][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t aq[4], ag[4], bk[4], bv[4];
                ldmatrix_x4(aq, qs + swz<D>(a_row, 2 * kk + a_chk));
                ldmatrix_x4(ag, gs + swz<D>(a_row, 2 * kk + a_chk));
                ldmatrix_x4(bk, ks + swz<D>(wk0 + b_row, 2 * kk + b_chk));
                ldmatrix_x4(bv, vs + swz<D>(wk0 + b_row, 2 * kk + b_chk));
                mma16816<T>(s[0], aq, bk[0], bk[1]);
                mma16816<T>(s[1], aq, bk[2], bk[3]);
                mma16816<T>(dp[0], ag, bv[0], bv[1]);
                mma16816<T>(dp[1], ag, bv[2], bv[3]);
            }
            // P and dS of rows g and g + 8, keys wk0 + 8 n + 2 tq + {0, 1}; both as A operands ([16 q x 16 keys])
            const float l2[2] = {lq_s[g], lq_s[g + 8]}, dd[2] = {dq_s[g], dq_s[g + 8]};
            uint32_t pa[4], dsa[4];
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int jk = wk0 + n * 8 + tq * 2;
                float pv[4], dv_[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    const bool ok = jk + (e & 1) < live;
                    pv[e] = ok ? fast_exp2(fmaf(s[n][e], scale2, -l2[r])) : 0.f;
                    dv_[e] = pv[e] * (dp[n][e] - dd[r]) * p.sm_scale;
                }
                pa[2 * n] = pack2<T>(pv[0], pv[1]);          // row g
                pa[2 * n + 1] = pack2<T>(pv[2], pv[3]);      // row g + 8
                dsa[2 * n] = pack2<T>(dv_[0], dv_[1]);
                dsa[2 * n + 1] = pack2<T>(dv_[2], dv_[3]);
            }
            // dQ += dS K   (k = the warp's 16 keys, n = head dim)
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, ks + swz<D>(wk0 + c_row, 2 * n2 + c_chk));
                mma16816<T>(dq[2 * n2], dsa, b[0], b[1]);
                mma16816<T>(dq[2 * n2 + 1], dsa, b[2], b[3]);
            }
            // P^T and dS^T as A operands ([16 keys x 16 q]): the 8x8 blocks transposed, the off-diagonal ones swapped
            uint32_t pta[4], dsta[4];
            pta[0] = movmatrix_trans(pa[0]);   pta[1] = movmatrix_trans(pa[2]);   pta[2] = movmatrix_trans(pa[1]);   pta[3] = movmatrix_trans(pa[3]);
            dsta[0] = movmatrix_trans(dsa[0]); dsta[1] = movmatrix_trans(dsa[2]); dsta[2] = movmatrix_trans(dsa[1]); dsta[3] = movmatrix_trans(dsa[3]);
            // dV += P^T dO and dK += dS^T Q, sixteen columns at a time, reduced straight into global memory
            const int32_t row_a = rows_s[st][wk0 + g], row_b = rows_s[st][wk0 + g + 8];
            float *dv_a = p.dv + size_t(max(row_a, 0)) * D + tq * 2, *dv_b = p.dv + size_t(max(row_b, 0)) * D + tq * 2;
            float *dk_a = p.dk + size_t(max(row_a, 0)) * D + tq * 2, *dk_b = p.dk + size_t(max(row_b, 0)) * D + tq * 2;
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                uint32_t bg[4], bq[4];
                ldmatrix_x4_trans(bg, gs + swz<D>(c_row, 2 * n2 + c_chk));
                ldmatrix_x4_trans(bq, qs + swz<D>(c_row, 2 * n2 + c_chk));
                float v0[4] = {0.f, 0.f, 0.f, 0.f}, v1[4] = {0.f, 0.f, 0.f, 0.f}, k0[4] = {0.f, 0.f, 0.f, 0.f}, k1[4] = {0.f, 0.f, 0.f, 0.f};
                mma16816<T>(v0, pta, bg[0], bg[1]);
                mma16816<T>(v1, pta, bg[2], bg[3]);
                mma16816<T>(k0, dsta, bq[0], bq[1]);
                mma16816<T>(k1, dsta, bq[2], bq[3]);
                if (row_a >= 0) {
                    red_add_v2(dv_a + n2 * 16, v0[0], v0[1]);
                    red_add_v2(dv_a + n2 * 16 + 8, v1[0], v1[1]);
                    red_add_v2(dk_a + n2 * 16, k0[0], k0[1]);
                    red_add_v2(dk_a + n2 * 16 + 8, k1[0], k1[1]);
                }
                if (row_b >= 0) {
                    red_add_v2(dv_b + n2 * 16, v0[2], v0[3]);
                    red_add_v2(dv_b + n2 * 16 + 8, v1[2], v1[3]);
                    red_add_v2(dk_b + n2 * 16, k0[2], k0[3]);
                    red_add_v2(dk_b + n2 * 16 + 8, k1[2], k1[3]);
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();                                     // all tiles consumed: the stages become the fold buffer
        float *fold = reinterpret_cast<float *>(bsm + 2 * QB_BYTES);          // [4 warps][16][FOLD_LD]
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            float *a0 = fold + (warp * kQB + g) * FOLD_LD + n * 8 + tq * 2;
            *reinterpret_cast<float2 *>(a0) = make_float2(dq[n][0], dq[n][1]);
            *reinterpret_cast<float2 *>(a0 + 8 * FOLD_LD) = make_float2(dq[n][2], dq[n][3]);
        }
        __syncthreads();
        for (int e = t * 4; e < nq * D; e += kThreads * 4) {
            const int r = e / D, c = e - r * D;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float4 x = *reinterpret_cast<const float4 *>(fold + (w * kQB + r) * FOLD_LD + c);
                sum.x += x.x; sum.y += x.y; sum.z += x.z; sum.w += x.w;
            }
            *reinterpret_cast<float4 *>(p.dq + size_t(p.perm[q0 + qb + r]) * D + c) = sum;
        }
    }
}

template <typename T, int D>
int launch(const BwdParams &p, int64_t total_buckets, cudaStream_t st)
{
    const size_t smem = 2 * size_t(kQB) * D * 2 + 4 * size_t(kTK) * D * 2;
    FM_CUDA_OK(func_attr_cached((const void *)attn_bwd_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_bwd_mma_kernel<T, D><<<(unsigned)total_buckets, kThreads, smem, st>>>(p);
    FM_LAUNCHED("attn_bwd_mma_kernel");
    return FM_OK;
}

}  // namespace

int launch_bwd_mma(const BwdParams &p, int dtype, int d, int64_t total_buckets, cudaStream_t st)
{
    if (dtype == FM_BF16 && d == 128) return launch<__nv_bfloat16, 128>(p, total_buckets, st);
    if (dtype == FM_BF16 && d == 64) return launch<__nv_bfloat16, 64>(p, total_buckets, st);
    if (dtype == FM_F16 && d == 128) return launch<__half, 128>(p, total_buckets, st);
    if (dtype == FM_F16 && d == 64) return launch<__half, 64>(p, total_buckets, st);
    set_error("tensor-core backward: needs bf16 / fp16 and head dim 64 or 128");
    return FM_ERR_UNSUPPORTED;
}

}  // namespace fm
