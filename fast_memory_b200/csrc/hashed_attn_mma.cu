// Tensor-core hashed attention for 16-bit inputs (bf16 / fp16, head dim 64 or 128).
//
// The path is HBM / L2-bound (arithmetic intensity ~ queries per bucket, far below the ridge), so the kernel is built
// around the gather and around occupancy: 128-thread CTAs that fit three to an SM (<= 168 registers, two stages of a
// 64-key K tile and V tile), each warp streaming the K and V rows it needs through its own cp.async pipeline
// (16-byte pieces, XOR-swizzled rows), and the math rides along on mma.sync m16n8k16:
//   * a work item holds <= 32 queries.  Up to 16 queries (one MMA row tile): the 4 warps split every key tile four
//     ways (16 keys each) and each warp gathers exactly the keys it consumes - no CTA-wide barrier in the tile loop,
//     the warps drift apart and hide one another's latencies.  17 to 32 queries (two row tiles): warps 2h and 2h+1
//     form a pair that shares the 32 keys of half h of every tile - each gathers 16 of them, a 64-thread named
//     barrier per tile hands them over, warp 2h+r computes row tile r over the 32 keys - so the bucket is gathered
//     once, not twice, with the register footprint of a single row tile;
//   * S = Q K^T from ldmatrix'd K rows, base-2 online softmax per warp in registers, P rounded to the
//     input dtype and fed straight back as the A operand of P V (V through ldmatrix.trans);
//   * at the end of the item the warps' (m, l, acc) states are folded through shared memory and written out
//     through the grouping permutation (or as a partial when the bucket is split over CTAs).
// Rounding points follow the reference kernel (triton_kernel.py:248-263).
#include "attn_common.cuh"
#include "mma_utils.cuh"

namespace fm {

namespace {

constexpr int kThreads = 128;
constexpr int kTK = 64;                     // keys per tile
constexpr int kStages = 2;
constexpr int kMaxQ = 32;                   // queries per work item (two row tiles)
constexpr int kCtasPerSm = 3;

template <int D> struct MmaCfg {
    static constexpr int CPR = D / 8;                           // 16-byte chunks per row
    static constexpr int ROWS_PER_PASS = 32 / CPR;              // rows covered by one sweep of a warp over its 16 keys
    static constexpr int PASSES = 16 / ROWS_PER_PASS;           // copies per thread per matrix per tile
    static constexpr int TILE_BYTES = kTK * D * 2;              // one K (or V) tile
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int ACC_LD = D + 4;                        // combine buffer row stride (floats)
    static constexpr size_t smem = size_t(kStages) * STAGE_BYTES;
    static_assert(4 * 16 * ACC_LD * 4 + 4 * 16 * 8 <= kStages * STAGE_BYTES, "combine buffer must fit in the tile stages");
};

__device__ __forceinline__ void pair_barrier(int pair)
{
    // immediate barrier numbers: a register operand makes the compiler reserve all sixteen
    if (pair == 0) asm volatile("bar.sync 1, 64;" ::: "memory");
    else asm volatile("bar.sync 2, 64;" ::: "memory");
}

// One work item.  PAIR = false: one row tile of 16 queries, every warp takes 16 keys of each tile.  PAIR = true: two
// row tiles; warp w computes row tile (w & 1) over the 32 keys of half (w >> 1) of each tile, gathered by the pair.
template <typename T, int D, bool PAIR>
__device__ __forceinline__ void run_item(const AttnParams &p, unsigned char *smem, const int4 it, const int nq)
{
    using C = MmaCfg<D>;
    constexpr int NQ = PAIR ? 32 : 16;
    constexpr int SUB = PAIR ? 2 : 1;                            // 16-key slices a warp consumes per tile
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const T *qg = reinterpret_cast<const T *>(p.q);
    const char *kg = reinterpret_cast<const char *>(p.k);
    const char *vg = reinterpret_cast<const char *>(p.v);
    const uint32_t smem_base = smem_u32(smem);
    const int rt = PAIR ? (warp & 1) : 0;                        // row tile of this warp
    const int wk0 = PAIR ? (warp >> 1) * 32 : warp * 16;         // first key of the tile this warp consumes
    // every warp gathers 16 keys of each tile: the ones it consumes itself, or half of the ones its pair consumes
    const int my_c = lane % C::CPR;                              // chunk column this thread copies
    // ldmatrix addresses inside a swizzled tile: row j, chunk c = 2 i + b sit at j 2D + ((c ^ (j & 7)) << 4).  With
    // x = j & 7 = lane & 7 this splits into ((i & 4) << 5) + (((i & 3) ^ (x >> 1)) << 5) + ((b ^ (x & 1)) << 4): a
    // compile-time term, one of four lane constants, and a lane constant - no XOR left in the tile loop.
    uint32_t sw_i[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) sw_i[i] = uint32_t((i ^ ((lane >> 1) & 3)) << 5);
    // K (S = Q K^T): matrices (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi)
    const uint32_t k_lane = uint32_t(((lane & 7) + ((lane >> 4) << 3)) * (D * 2) + ((((lane >> 3) & 1) ^ (lane & 1)) << 4));
    // V (P V, transposed loads): matrices (keys 0-7, d 16 n2 + 0-7), (keys 8-15, same d), (keys 0-7, d + 8), (keys 8-15, d + 8)
    const uint32_t v_lane = uint32_t(((lane & 7) + (((lane >> 3) & 1) << 3)) * (D * 2) + (((lane >> 4) ^ (lane & 1)) << 4));
    const int my_r = warp * 16 + lane / C::CPR;                  // first row this thread copies

    const int gb = it.x, q_begin = it.y, kc = it.z, nkc = it.w;
    const int64_t kb = p.bucket_off[gb];
    const int64_t len = p.bucket_off[gb + 1] - kb;
    const int64_t k0 = int64_t(kc) * p.key_chunk;
    const int chunk_len = int(min(len - k0, int64_t(p.key_chunk)));
    const int n_tiles = chunk_len > 0 ? (chunk_len + kTK - 1) / kTK : 0;
    const int64_t kbase = p.bucket_kbase ? p.bucket_kbase[gb] : 0;
    const int64_t tbl0 = kb + k0;

    // ---- Q (A operand) of the warp's row tile, through the permutation, in registers ----
    uint32_t qf[D / 16][4];
    {
        const int r0 = rt * 16 + g, r1 = r0 + 8;
        const T *q0 = r0 < nq ? qg + size_t(p.perm[q_begin + r0]) * D : nullptr;
        const T *q1 = r1 < nq ? qg + size_t(p.perm[q_begin + r1]) * D : nullptr;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int c = ks * 16 + tq * 2;
            qf[ks][0] = q0 ? *reinterpret_cast<const uint32_t *>(q0 + c) : 0u;
            qf[ks][1] = q1 ? *reinterpret_cast<const uint32_t *>(q1 + c) : 0u;
            qf[ks][2] = q0 ? *reinterpret_cast<const uint32_t *>(q0 + c + 8) : 0u;
            qf[ks][3] = q1 ? *reinterpret_cast<const uint32_t *>(q1 + c + 8) : 0u;
        }
    }

    // ---- gather pipeline -----------------------------------------------------------------------------
    // Table entries are fetched one tile ahead and only looked at when their copies are issued, so the
    // index load never stalls the warp.  Entries outside [0, n_k_rows) are clamped into range: a malformed
    // table gives a meaningless result but never an out-of-bounds access.
    int32_t rows[C::PASSES];
    const int32_t row_max = int32_t(min(p.n_k_rows - 1, int64_t(0x7fffffff)));
    auto load_rows = [&](int tile) {
#pragma unroll
        for (int i = 0; i < C::PASSES; ++i) {
            const int j = tile * kTK + my_r + i * C::ROWS_PER_PASS;
            rows[i] = (tile < n_tiles && j < chunk_len) ? int32_t(load_index(p.table, p.idx_bytes, tbl0 + j)) : -1;
        }
    };
    auto issue = [&](int tile) {
        if (tile < n_tiles) {
            const int st = tile % kStages;
            const uint32_t kdst = smem_base + st * C::STAGE_BYTES;
            const uint32_t vdst = kdst + C::TILE_BYTES;
            const int live = chunk_len - tile * kTK;             // rows of this tile that exist
#pragma unroll
            for (int i = 0; i < C::PASSES; ++i) {
                const int j = my_r + i * C::ROWS_PER_PASS;
                const bool ok = j < live;
                const int32_t row = min(max(rows[i] + int32_t(kbase), 0), row_max);
                const size_t off = size_t(row) * (D * 2) + my_c * 16;
                cp_async16(kdst + swz<D>(j, my_c), kg + off, ok);
                cp_async16(vdst + swz<D>(j, my_c), vg + off, ok);
            }
        }
        cp_async_commit();
    };
    load_rows(0);
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        issue(s);
        load_rows(s + 1);
    }

    // l is kept as per-thread partial sums (the four threads of a row share m, hence alpha) and added up at the end
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {tq == 0 ? 1.f : 0.f, tq == 0 ? 1.f : 0.f};
    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;

    for (int tile = 0; tile < n_tiles; ++tile) {
        cp_async_wait<kStages - 2>();
        // the rows of the tile landed and the stage refilled below is free: a matter of this warp alone, or of the pair
        if constexpr (PAIR) pair_barrier(warp >> 1);
        else __syncwarp();
        issue(tile + kStages - 1);
        load_rows(tile + kStages);
        const int st = tile % kStages;
        const uint32_t ks_base = smem_base + st * C::STAGE_BYTES;
        const uint32_t vs_base = ks_base + C::TILE_BYTES;

        // S = Q K^T for 16 queries x 16 SUB keys (two accumulation chains per 16-key slice; with 12 warps per SM
        // splitting them further into even and odd k-steps only cost instructions)
        float s[SUB][2][4];
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[sub][n][e] = 0.f;
            const uint32_t k_sub = ks_base + (wk0 + sub * 16) * (D * 2) + k_lane;
            const uint32_t k_addr[4] = {k_sub + sw_i[0], k_sub + sw_i[1], k_sub + sw_i[2], k_sub + sw_i[3]};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t b[4];
                if (ks < 4) ldmatrix_x4_off<0>(b, k_addr[ks & 3]);
                else ldmatrix_x4_off<128>(b, k_addr[ks & 3]);
                mma16816<T>(s[sub][0], qf[ks], b[0], b[1]);
                mma16816<T>(s[sub][1], qf[ks], b[2], b[3]);
            }
        }
        // mask (only the last tile can be partial), online softmax in the scaled base-2 domain over the warp's keys of
        // the tile (rows g and g + 8 of the row tile; this thread's keys: wk0 + 16 sub + 8 n + 2 tq + {0, 1})
        if (tile == n_tiles - 1) {
            const int live = chunk_len - tile * kTK;
#pragma unroll
            for (int sub = 0; sub < SUB; ++sub)
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    const int jk = wk0 + sub * 16 + n * 8 + tq * 2;
                    if (jk >= live) { s[sub][n][0] = -INFINITY; s[sub][n][2] = -INFINITY; }
                    if (jk + 1 >= live) { s[sub][n][1] = -INFINITY; s[sub][n][3] = -INFINITY; }
                }
        }
        uint32_t pa[SUB][4];
        float alpha[2];
        bool moved = false;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int sub = 0; sub < SUB; ++sub)
                mx = fmaxf(mx, fmaxf(fmaxf(s[sub][0][2 * r], s[sub][0][2 * r + 1]), fmaxf(s[sub][1][2 * r], s[sub][1][2 * r + 1])));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[r], mx * p.scale2);                 // scale2 > 0 keeps the order
            const float m_sub = m_new > -INFINITY ? m_new : 0.f;                // nothing live yet: p = 2^-inf = 0
            alpha[r] = fast_exp2(m_run[r] - m_sub);
            float sum = 0.f;
#pragma unroll
            for (int sub = 0; sub < SUB; ++sub) {
                const float p00 = fast_exp2(fmaf(s[sub][0][2 * r], p.scale2, -m_sub));
                const float p01 = fast_exp2(fmaf(s[sub][0][2 * r + 1], p.scale2, -m_sub));
                const float p10 = fast_exp2(fmaf(s[sub][1][2 * r], p.scale2, -m_sub));
                const float p11 = fast_exp2(fmaf(s[sub][1][2 * r + 1], p.scale2, -m_sub));
                sum += (p00 + p01) + (p10 + p11);
                pa[sub][r] = pack2<T>(p00, p01);                 // keys 0-7 of the slice
                pa[sub][2 + r] = pack2<T>(p10, p11);             // keys 8-15
            }
            l_run[r] = l_run[r] * alpha[r] + sum;
            m_run[r] = m_new;
            moved = moved || alpha[r] != 1.f;
        }
        // the running maxima settle after a few tiles; rescale the accumulators only when one moved
        if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                acc[n][0] *= alpha[0];
                acc[n][1] *= alpha[0];
                acc[n][2] *= alpha[1];
                acc[n][3] *= alpha[1];
            }
        }
        // acc += P V  (k = 16 keys per slice, n = head dim)
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
            const uint32_t v_sub = vs_base + (wk0 + sub * 16) * (D * 2) + v_lane;
            const uint32_t v_addr[4] = {v_sub + sw_i[0], v_sub + sw_i[1], v_sub + sw_i[2], v_sub + sw_i[3]};
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                uint32_t b[4];
                if (n2 < 4) ldmatrix_x4_trans_off<0>(b, v_addr[n2 & 3]);
                else ldmatrix_x4_trans_off<128>(b, v_addr[n2 & 3]);
                mma16816<T>(acc[2 * n2], pa[sub], b[0], b[1]);
                mma16816<T>(acc[2 * n2 + 1], pa[sub], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    __syncthreads();                                         // all tiles consumed: the stages become the combine buffer

    // ---- fold the warps' states: four per query (PAIR = false), two per query (the two key halves of its row tile) ----
    float *acc_s = reinterpret_cast<float *>(smem);          // [4 warps][16][ACC_LD]
    float *ml_s = acc_s + 4 * 16 * C::ACC_LD;                 // [4 warps][16][2]
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        float *a0 = acc_s + (warp * 16 + g) * C::ACC_LD + n * 8 + tq * 2;
        *reinterpret_cast<float2 *>(a0) = make_float2(acc[n][0], acc[n][1]);
        *reinterpret_cast<float2 *>(a0 + 8 * C::ACC_LD) = make_float2(acc[n][2], acc[n][3]);
    }
    if (tq == 0) {
        ml_s[(warp * 16 + g) * 2] = m_run[0];
        ml_s[(warp * 16 + g) * 2 + 1] = l_run[0];
        ml_s[(warp * 16 + g + 8) * 2] = m_run[1];
        ml_s[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    {
        constexpr int TPQ = kThreads / NQ;                   // threads per query (8 or 4)
        constexpr int CPT = D / TPQ;                         // columns per thread
        constexpr int NW = PAIR ? 2 : 4;                     // states per query
        const int qi = t / TPQ, c0 = (t % TPQ) * CPT;
        // state w of query qi lives in the rows of warp (PAIR ? 2 w + row tile : w), row qi % 16
        const int wfirst = PAIR ? (qi >> 4) : 0, wstep = PAIR ? 2 : 1, qr = qi & 15;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, ml_s[((wfirst + w * wstep) * 16 + qr) * 2]);
        float wgt[NW], Lsum = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = ml_s[((wfirst + w * wstep) * 16 + qr) * 2];
            wgt[w] = mw > -INFINITY ? exp2f(mw - M) : 0.f;
            // a warp that saw no key still carries its initial l = 1 with m = -inf: weight 0 drops it
            Lsum += wgt[w] * ml_s[((wfirst + w * wstep) * 16 + qr) * 2 + 1];
        }
        if (M == -INFINITY) Lsum = 1.f;                       // empty bucket: o = 0, lse = -inf
        float o[CPT];
#pragma unroll
        for (int c = 0; c < CPT; ++c) o[c] = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float *src = acc_s + ((wfirst + w * wstep) * 16 + qr) * C::ACC_LD + c0;
#pragma unroll
            for (int c = 0; c < CPT; c += 4) {
                float4 v4 = *reinterpret_cast<const float4 *>(src + c);
                o[c] += wgt[w] * v4.x;
                o[c + 1] += wgt[w] * v4.y;
                o[c + 2] += wgt[w] * v4.z;
                o[c + 3] += wgt[w] * v4.w;
            }
        }
        if (qi < nq) {
            if (nkc == 1) {
                const size_t row = p.perm[q_begin + qi];
                T *orow = reinterpret_cast<T *>(p.o) + row * D + c0;
                const float inv = 1.f / Lsum;
#pragma unroll
                for (int c = 0; c < CPT; c += 8) {
                    uint4 pk;
                    pk.x = pack2<T>(o[c] * inv, o[c + 1] * inv);
                    pk.y = pack2<T>(o[c + 2] * inv, o[c + 3] * inv);
                    pk.z = pack2<T>(o[c + 4] * inv, o[c + 5] * inv);
                    pk.w = pack2<T>(o[c + 6] * inv, o[c + 7] * inv);
                    *reinterpret_cast<uint4 *>(orow + c) = pk;
                }
                if ((t % TPQ) == 0) p.lse[row] = (M + log2f(Lsum)) * 0.6931471805599453f;
            } else {
                float *dst = p.partials + (size_t(q_begin + qi) * p.nkc_max + kc) * (D + 2);
#pragma unroll
                for (int c = 0; c < CPT; c += 2) *reinterpret_cast<float2 *>(dst + c0 + c) = make_float2(o[c], o[c + 1]);
                if ((t % TPQ) == 0) {
                    dst[D] = M;
                    dst[D + 1] = Lsum;
                    if (kc == 0) p.qparts[q_begin + qi] = nkc;
                }
            }
        }
    }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
attn_mma_kernel(AttnParams p)
{
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_item;
    const int n_items = min(p.counters[0], p.max_items);
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_item = atomicAdd(&p.counters[1], 1);
        __syncthreads();
        const int item = s_item;
        if (item >= n_items) break;
        const int4 it = p.items[item];
        const int nq = min(min(kMaxQ, p.q_block), p.group_off[it.x + 1] - it.y);
        if (nq > 16) run_item<T, D, true>(p, smem, it, nq);
        else run_item<T, D, false>(p, smem, it, nq);
    }
}

template <typename T, int D>
int launch_mma(const AttnParams &p, int grid, cudaStream_t st)
{
    const size_t smem = MmaCfg<D>::smem;
    FM_CUDA_OK(func_attr_cached((const void *)attn_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_mma_kernel<T, D><<<grid, kThreads, smem, st>>>(p);
    FM_LAUNCHED("attn_mma_kernel");
    return FM_OK;
}

}  // namespace

bool attn_mma_supported(int dtype, int d) { return (dtype == FM_BF16 || dtype == FM_F16) && (d == 64 || d == 128); }

int launch_attn_mma(const AttnParams &p, int dtype, int d, int grid, cudaStream_t st)
{
    if (dtype == FM_BF16) return d == 128 ? launch_mma<__nv_bfloat16, 128>(p, grid, st) : launch_mma<__nv_bfloat16, 64>(p, grid, st);
    return d == 128 ? launch_mma<__half, 128>(p, grid, st) : launch_mma<__half, 64>(p, grid, st);
}

}  // namespace fm
