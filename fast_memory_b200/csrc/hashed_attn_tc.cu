// Hashed attention on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM) for 16-bit inputs with
// head dim 128.
//
// The path is bound by what an SM can pull in and push through shared memory (every bucket row is gathered once per
// <= 32 queries: ~1 MB per work item), so the kernel spends its instructions on the gather and leaves the products to
// two single-thread MMA streams.  The KEYS sit on the M side of both products, which makes a gathered tile of 128 rows
// the A operand of both without any reshuffling:
//     S^T [128 keys x 32 q]  = K_tile [128 x d]    . Q^T        (K-major A and B: rows of K / Q are contiguous in d)
//     O^T [d = 128 x 32 q]  += V_tile^T [d x 128]  . P^T        (MN-major A and B: the contraction index - the key - is
//                                                                the ROW of the V tile and of the P tile)
// A tile row is stored as two 128-byte halves in two 16 KB column blocks with the hardware's 128-byte swizzle, which
// is at once the K-major layout of K and the MN-major layout of V.
//
// CTA = 448 threads, one per SM (3 K tiles + 3 V tiles = 192 KB of shared memory):
//   warps 0-3   softmax + epilogue: thread = key row of S^T (tcgen05.ld, one TMEM lane each).  The softmax reference m of
//               a query is fixed by the item's FIRST tile (exact maximum over its 128 keys: shuffle transpose-reduce in
//               the warp, four warps folded through shared memory, once per item); every tile then costs a TMEM load,
//               p = 2^(s - m) per score, the bf16 P^T row (64 bytes, 64-byte swizzle) for the second product, and
//               l += p per thread (summed over the CTA once per item).  No running maximum, no rescaling of O^T, no
//               barrier in the tile loop.  A later key may beat the first tile's maximum: p then exceeds 1, which the
//               floating-point range takes in its stride (bf16 and the fp32 sums reach 2^127).  An item whose
//               denominator is not finite or out of the input type's range - a later score more than ~100 (bf16) /
//               14 (fp16) powers of two above the first tile's best - is put on a list and served again by the
//               mma.sync kernel, which tracks the running maximum.
//   warps 4-7   epilogue: thread = row d of O^T.  Sums l over the CTA, reads O^T from TMEM, normalises and writes the
//               output rows (or the partials of a split bucket) through the grouping permutation - under the next
//               item's tiles.
//   warp 8      one thread issues all MMAs, whichever of the two products has its operands ready first; owns the TMEM
//               allocation (S^T twice, O^T twice: 128 columns).
//   warp 9      loads the queries of an item (through the grouping permutation) as the B operand of the first product.
//   warps 10-13 gather: 16-byte cp.async copies of the tile's K and V rows through the bucket table; a copy's
//               completion arrives on the slot's barrier by itself, so the threads never wait for data and run ahead
//               as far as free slots allow, across item boundaries.
// Items are dealt out statically (item = CTA + i * grid), so every role walks the same list on its own and the roles
// meet only at the mbarriers; Q and O^T are double-buffered so that an item's first tiles run under the epilogue of
// the one before.
// Rounding points follow the reference kernel (triton_kernel.py:248-263): P is rounded to the input dtype before
// P.V while l sums the unrounded p.  The reference refers p to a running maximum and rescales; referring it to the
// first tile's maximum changes the power of two P is rounded at, nothing else, and stays inside the tolerances of the
// parity tests.
// Every mbarrier wait is bounded; a give-up sets the fourth counter of the workspace, every role leaves its loop and
// the CTA frees its TMEM and returns.
//
// Where it stands (config 2 cut to 8 heads, B200): this kernel 0.85 - 0.93 ms against 0.41 ms of the mma.sync kernel
// (hashed_attn_mma.cu), which therefore stays the default (fm_set_attn_kernel / FASTMEM_ATTN_KERNEL=tc selects this
// one).  The reason is the shape: a bucket has at most 32 queries, so every MMA is M = 128, N = 32, K = 16, and the
// issuing thread sees ~105 cycles per such instruction whatever else runs (measured with the gather and the softmax
// switched off) - about what an N = 256 instruction costs.  16 of them per 128-key tile are ~1.7 k cycles of tensor
// pipe alone, the whole time the mma.sync kernel needs per 128 keys.  Queries on the M side would make the MMAs large
// (and four times wasted) but leave one warp per 32 queries to do the softmax, since a warp reaches only its own
// quarter of the TMEM lanes.
#include "attn_common.cuh"
#include <cstdlib>
#include "mma_utils.cuh"
#include "tc_utils.cuh"

#include <type_traits>

namespace fm {

namespace {

constexpr int kD = 128;
constexpr int kTileKeys = 128;              // keys per tile = UMMA M
constexpr int kNQ = 32;                     // queries per item = UMMA N
constexpr int kKSlots = 3;                  // K tiles in flight or in use (a slot is free again after the first product)
constexpr int kVSlots = 3;                  // V tiles (a slot is held until the second product, a softmax later)
constexpr int kSoftmaxThreads = 128;
constexpr int kEpiThreads = 128;
constexpr int kGatherWarps = 4;
constexpr int kGatherThreads = 32 * kGatherWarps;
constexpr int kMmaWarp = 8, kLoaderWarp = 9, kGatherWarp0 = 10;
constexpr int kTcAttnThreads = 32 * (kGatherWarp0 + kGatherWarps);          // 448
constexpr uint32_t kColBlock = kTileKeys * 128;                            // one 64-element column block of a tile
constexpr uint32_t kTileBytes = 2 * kColBlock;                             // K (or V) tile
constexpr uint32_t kOffV = kKSlots * kTileBytes;
constexpr uint32_t kQBlock = kNQ * 128;                                    // one column block of the query tile
constexpr uint32_t kQBytes = 2 * kQBlock;
constexpr uint32_t kPBytes = kTileKeys * 64;                               // P^T tile: 128 rows of 32 bf16
constexpr uint32_t kOffQ = (kKSlots + kVSlots) * kTileBytes;                // two query tiles
constexpr uint32_t kOffP = kOffQ + 2 * kQBytes;                            // two P^T tiles
constexpr uint32_t kTcSmem = kOffP + 2 * kPBytes;

// byte offset of 16-byte chunk c (0..15) of row j inside a K / V tile (two column blocks, 128-byte swizzle)
__device__ __forceinline__ uint32_t tile_off(int j, int c) { return uint32_t(c >> 3) * kColBlock + uint32_t(j) * 128u + (uint32_t((c & 7) ^ (j & 7)) << 4); }

// lane q ends up with the maximum over the warp's 32 lanes of v[q] (31 shuffles)
__device__ __forceinline__ float warp_transpose_max(const float (&v)[32])
{
    const int lane = threadIdx.x & 31;
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const bool up = lane & 16;
        const float keep = up ? v[i + 16] : v[i], give = up ? v[i] : v[i + 16];
        a[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 16));
    }
    float b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const bool up = lane & 8;
        const float keep = up ? a[i + 8] : a[i], give = up ? a[i] : a[i + 8];
        b[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 8));
    }
    float c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const bool up = lane & 4;
        const float keep = up ? b[i + 4] : b[i], give = up ? b[i] : b[i + 4];
        c[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 4));
    }
    float d2[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const bool up = lane & 2;
        const float keep = up ? c[i + 2] : c[i], give = up ? c[i] : c[i + 2];
        d2[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 2));
    }
    const bool up = lane & 1;
    const float keep = up ? d2[1] : d2[0], give = up ? d2[0] : d2[1];
    return fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 1));
}

// the same with a sum
__device__ __forceinline__ float warp_transpose_sum(const float (&v)[32])
{
    const int lane = threadIdx.x & 31;
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const bool up = lane & 16;
        const float keep = up ? v[i + 16] : v[i], give = up ? v[i] : v[i + 16];
        a[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
    }
    float b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const bool up = lane & 8;
        const float keep = up ? a[i + 8] : a[i], give = up ? a[i] : a[i + 8];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
    }
    float c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const bool up = lane & 4;
        const float keep = up ? b[i + 4] : b[i], give = up ? b[i] : b[i + 4];
        c[i] = keep + __shfl_xor_sync(0xffffffffu, give, 4);
    }
    float d2[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const bool up = lane & 2;
        const float keep = up ? c[i + 2] : c[i], give = up ? c[i] : c[i + 2];
        d2[i] = keep + __shfl_xor_sync(0xffffffffu, give, 2);
    }
    const bool up = lane & 1;
    const float keep = up ? d2[1] : d2[0], give = up ? d2[0] : d2[1];
    return keep + __shfl_xor_sync(0xffffffffu, give, 1);
}

struct TcShared {
    uint64_t k_full[kKSlots], k_empty[kKSlots], v_full[kVSlots], v_empty[kVSlots];
    uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2];
    uint64_t q_full[2], q_empty[2], o_full[2], o_empty[2], l_full, l_empty;
    uint32_t tmem_slot;
    int abort;
    alignas(16) float wred[4][kNQ];                          // softmax: warp maxima of an item's first tile (read as float4)
    alignas(16) float l_warp[4][kNQ];                        // the softmax warps' sums of l of the item they just finished
    alignas(16) float m_ref[kNQ];                            // its softmax reference of every query
    alignas(16) float l_inv[kNQ];                            // epilogue: 1 / l of the item at hand
};

// the warp's lane 0 polls the barrier (bounded); the verdict goes to every lane
__device__ __forceinline__ bool warp_mbar_wait(uint32_t bar, uint32_t parity, const volatile int *abort)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = tc::mbar_wait_or_abort(bar, parity, abort) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// What every role derives of a work item, each on its own.
struct TcItem {
    int gb, q_begin, kc, nkc, nq, chunk_len, n_tiles;
    int64_t kbase, tbl0;
};

__device__ __forceinline__ TcItem tc_item(const AttnParams &p, int item)
{
    TcItem I;
    const int4 it = p.items[item];
    I.gb = it.x; I.q_begin = it.y; I.kc = it.z; I.nkc = it.w;
    I.nq = min(kNQ, p.group_off[I.gb + 1] - I.q_begin);
    const int64_t kb = p.bucket_off[I.gb];
    const int64_t len = p.bucket_off[I.gb + 1] - kb;
    const int64_t k0 = int64_t(I.kc) * p.key_chunk;
    I.chunk_len = int(max(int64_t(0), min(len - k0, int64_t(p.key_chunk))));
    I.n_tiles = (I.chunk_len + kTileKeys - 1) / kTileKeys;
    I.kbase = p.bucket_kbase ? p.bucket_kbase[I.gb] : 0;
    I.tbl0 = kb + k0;
    return I;
}

// Where one of the two MMA streams stands in the CTA's list of items.
struct TcCursor {
    int item;                  // index into the item list (>= n_items: finished)
    int t;                     // next tile of the item
    TcItem I;
    int next_item;             // the following item with tiles, looked up while this one is worked on
    TcItem N;
    uint32_t tile_it, item_it; // tiles / items with tiles before this one
};

template <typename T>
__global__ void __launch_bounds__(kTcAttnThreads, 1)
attn_tc_kernel(AttnParams p, uint32_t idesc_s, uint32_t idesc_o, int4 *redo_items, int *redo_count)
{
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(16) TcShared sh;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (tc::smem_addr(smem_dyn) + 1023u) & ~1023u;
    unsigned char *base_ptr = smem_dyn + (base - tc::smem_addr(smem_dyn));
    auto bar = [](uint64_t *b) { return tc::smem_addr(b); };
    volatile int *abort_flag = &sh.abort;

    if (tid == 0) {
        for (int s = 0; s < kKSlots; ++s) { tc::mbar_init(bar(&sh.k_full[s]), kGatherThreads); tc::mbar_init(bar(&sh.k_empty[s]), 1); }
        for (int s = 0; s < kVSlots; ++s) { tc::mbar_init(bar(&sh.v_full[s]), kGatherThreads); tc::mbar_init(bar(&sh.v_empty[s]), 1); }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(bar(&sh.s_full[b]), 1);
            tc::mbar_init(bar(&sh.s_empty[b]), 4);
            tc::mbar_init(bar(&sh.p_full[b]), 4);
            tc::mbar_init(bar(&sh.p_empty[b]), 1);
            tc::mbar_init(bar(&sh.q_full[b]), 32);
            tc::mbar_init(bar(&sh.q_empty[b]), 1);
            tc::mbar_init(bar(&sh.o_full[b]), 1);
            tc::mbar_init(bar(&sh.o_empty[b]), 4);
        }
        tc::mbar_init(bar(&sh.l_full), 4);
        tc::mbar_init(bar(&sh.l_empty), 4);
        tc::mbar_fence_init();
        sh.abort = 0;
    }
    if (warp == kMmaWarp) tc::tmem_alloc(tc::smem_addr(&sh.tmem_slot), 128);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = sh.tmem_slot;
    const uint32_t tmem_s[2] = {tmem_base, tmem_base + 32u};
    const uint32_t tmem_o[2] = {tmem_base + 64u, tmem_base + 96u};

    const int n_items = min(p.counters[0], p.max_items);
    // running counts of tiles and of items with tiles (the same sequence in every role): slot / buffer and barrier
    // phase of each use
    uint32_t tile_it = 0, item_it = 0;

    if (warp < 4) {
        // ================================ softmax: thread = key row of S^T ===========================================
        // NQ = 16 or 32 columns of S^T are looked at, whichever covers the item's queries (the products always run with
        // N = 32; columns past the item's queries hold whatever the buffers held and are never read back).
        const uint32_t lane_base = uint32_t(warp * 32) << 16;
        bool ok = true;
        auto run_item = [&](const TcItem &I, auto nq_tag) -> bool {
            constexpr int NQ = decltype(nq_tag)::value;
            float l_part[NQ], m_sub[NQ];
#pragma unroll
            for (int q = 0; q < NQ; ++q) { l_part[q] = 0.f; m_sub[q] = 0.f; }
            float m_mine = -INFINITY;                                           // lane q: the reference of query q
            for (int t = 0; t < I.n_tiles; ++t) {
                const uint32_t it_g = tile_it + t, buf = it_g & 1;
                ok = warp_mbar_wait(bar(&sh.s_full[buf]), (it_g >> 1) & 1, abort_flag) && ok;
                tc::fence_after_sync();
                uint32_t raw[NQ];
                if constexpr (NQ == 32) { tc::tmem_ld_x32(tmem_s[buf] + lane_base, raw); tc::tmem_ld_wait(raw); }
                else { tc::tmem_ld_x16(tmem_s[buf] + lane_base, raw); tc::tmem_ld_wait16(raw); }
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(bar(&sh.s_empty[buf]));          // S^T may be overwritten by the tile after next
                if (t * kTileKeys + tid >= I.chunk_len) {                       // a row past the end of the last tile: p = 2^-inf = 0
#pragma unroll
                    for (int q = 0; q < NQ; ++q) raw[q] = 0xff800000u;
                }
                if (t == 0) {
                    // the item's reference: maximum of every query over the first tile's keys (scale2 > 0 keeps the order)
                    float s[32];
#pragma unroll
                    for (int q = 0; q < 32; ++q) s[q] = q < NQ ? __uint_as_float(raw[q < NQ ? q : 0]) * p.scale2 : -INFINITY;
                    sh.wred[warp][lane] = warp_transpose_max(s);
                    ok = tc::named_barrier_and(1, kSoftmaxThreads, ok);         // every thread gets the same verdict
                    if (!ok) return false;
#pragma unroll
                    for (int q = 0; q < NQ; q += 4) {
                        const float4 a = *reinterpret_cast<const float4 *>(&sh.wred[0][q]), b = *reinterpret_cast<const float4 *>(&sh.wred[1][q]);
                        const float4 c = *reinterpret_cast<const float4 *>(&sh.wred[2][q]), d4 = *reinterpret_cast<const float4 *>(&sh.wred[3][q]);
                        const float m0 = fmaxf(fmaxf(a.x, b.x), fmaxf(c.x, d4.x)), m1 = fmaxf(fmaxf(a.y, b.y), fmaxf(c.y, d4.y));
                        const float m2 = fmaxf(fmaxf(a.z, b.z), fmaxf(c.z, d4.z)), m3 = fmaxf(fmaxf(a.w, b.w), fmaxf(c.w, d4.w));
                        m_sub[q] = m0 > -INFINITY ? m0 : 0.f;
                        m_sub[q + 1] = m1 > -INFINITY ? m1 : 0.f;
                        m_sub[q + 2] = m2 > -INFINITY ? m2 : 0.f;
                        m_sub[q + 3] = m3 > -INFINITY ? m3 : 0.f;
                    }
                    m_mine = fmaxf(fmaxf(sh.wred[0][lane], sh.wred[1][lane]), fmaxf(sh.wred[2][lane], sh.wred[3][lane]));
                    tc::named_barrier(2, kSoftmaxThreads);                      // wred is free for the next item
                }
                // P^T row of this key: p = 2^(s - m), rounded to the input dtype; l sums the unrounded p
                uint32_t pk[NQ / 2];
#pragma unroll
                for (int q = 0; q < NQ; q += 2) {
                    const float p0 = fast_exp2(fmaf(__uint_as_float(raw[q]), p.scale2, -m_sub[q]));
                    const float p1 = fast_exp2(fmaf(__uint_as_float(raw[q + 1]), p.scale2, -m_sub[q + 1]));
                    l_part[q] += p0;
                    l_part[q + 1] += p1;
                    pk[q >> 1] = pack2<T>(p0, p1);
                }
                // the P buffer is free once the second product of the tile before last has read it
                ok = warp_mbar_wait(bar(&sh.p_empty[buf]), ((it_g >> 1) & 1) ^ 1, abort_flag) && ok;
                unsigned char *prow = base_ptr + kOffP + buf * kPBytes + tid * 64;
#pragma unroll
                for (int c = 0; c < NQ / 8; ++c)
                    *reinterpret_cast<uint4 *>(prow + ((c ^ ((tid >> 1) & 3)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                tc::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(bar(&sh.p_full[buf]));
            }
            // the item's sums of l and its references go to the epilogue warps
            ok = warp_mbar_wait(bar(&sh.l_empty), (item_it & 1) ^ 1, abort_flag) && ok;       // the epilogue has read the item before
            float l32[32];
#pragma unroll
            for (int q = 0; q < 32; ++q) l32[q] = q < NQ ? l_part[q < NQ ? q : 0] : 1.f;
            sh.l_warp[warp][lane] = warp_transpose_sum(l32);
            if (warp == 0) sh.m_ref[lane] = m_mine;
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar(&sh.l_full));
            return true;
        };
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const TcItem I = tc_item(p, item);
            if (I.n_tiles == 0) continue;
            const bool went = I.nq <= 16 ? run_item(I, std::integral_constant<int, 16>()) : run_item(I, std::integral_constant<int, 32>());
            if (!went) break;                                                   // (taken by all 128 threads together)
            tile_it += I.n_tiles;
            item_it += 1;
        }
        if (!ok) { atomicExch(&p.counters[3], 3); *abort_flag = 1; }
    } else if (warp < 8) {
        // ================================ epilogue: thread = row d of O^T ==============================================
        const int et = tid - kSoftmaxThreads, ew = warp - 4;
        const uint32_t lane_base = uint32_t(ew * 32) << 16;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const TcItem I = tc_item(p, item);
            const int my_q = lane < I.nq ? p.perm[I.q_begin + lane] : 0;        // output row of query `lane`
            const uint32_t ob = item_it & 1;
            float o[kNQ];
            if (I.n_tiles > 0) {
                ok = warp_mbar_wait(bar(&sh.l_full), item_it & 1, abort_flag) && ok;
                ok = warp_mbar_wait(bar(&sh.o_full[ob]), (item_it >> 1) & 1, abort_flag) && ok;
                tc::fence_after_sync();
            }
            ok = tc::named_barrier_and(3, kEpiThreads, ok);                     // every thread gets the same verdict
            if (!ok) break;
            if (ew == 0) {
                float L = 1.f, M = -INFINITY;
                if (I.n_tiles > 0) {
                    L = (sh.l_warp[0][lane] + sh.l_warp[1][lane]) + (sh.l_warp[2][lane] + sh.l_warp[3][lane]);
                    M = sh.m_ref[lane];
                }
                if (M == -INFINITY) L = 1.f;                                    // no key: o = 0, lse = -inf
                // a denominator out of range: some later score dwarfs the first tile's best - the item is served again
                const float l_max = Elem<T>::id == FM_F16 ? 16384.f : 1.0e30f;
                const bool bad = lane < I.nq && !(L <= l_max);
                if (__ballot_sync(0xffffffffu, bad) && lane == 0) redo_items[atomicAdd(redo_count, 1)] = p.items[item];
                sh.l_inv[lane] = 1.f / L;
                if (lane < I.nq) {
                    if (I.nkc == 1) p.lse[my_q] = (M + log2f(L)) * 0.6931471805599453f;
                    else {
                        float *dst = p.partials + (size_t(I.q_begin + lane) * p.nkc_max + I.kc) * (kD + 2);
                        dst[kD] = M;
                        dst[kD + 1] = L;
                        if (I.kc == 0) p.qparts[I.q_begin + lane] = I.nkc;
                    }
                }
            }
            tc::named_barrier(4, kEpiThreads);
            if (I.n_tiles > 0) {
                uint32_t o_raw[32];
                tc::tmem_ld_x32(tmem_o[ob] + lane_base, o_raw);
                tc::tmem_ld_wait(o_raw);
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    tc::mbar_arrive(bar(&sh.o_empty[ob]));                      // O^T may take the item after next
                    tc::mbar_arrive(bar(&sh.l_empty));                          // (l_warp / m_ref were read before the barrier above)
                }
#pragma unroll
                for (int q = 0; q < kNQ; ++q) o[q] = __uint_as_float(o_raw[q]);
            } else {
#pragma unroll
                for (int q = 0; q < kNQ; ++q) o[q] = 0.f;
            }
            // thread = column d of the output rows: a warp writes 64 contiguous bytes of one query's row
            if (I.nkc == 1) {
                T *og = reinterpret_cast<T *>(p.o);
#pragma unroll
                for (int q = 0; q < kNQ; ++q) {
                    const int row = __shfl_sync(0xffffffffu, my_q, q);
                    if (q < I.nq) og[size_t(row) * kD + et] = Elem<T>::from_f32(o[q] * sh.l_inv[q]);
                }
            } else {
#pragma unroll
                for (int q = 0; q < kNQ; ++q)
                    if (q < I.nq) p.partials[(size_t(I.q_begin + q) * p.nkc_max + I.kc) * (kD + 2) + et] = o[q];
            }
            tc::named_barrier(4, kEpiThreads);                                  // l_inv is free for the next item
            tile_it += I.n_tiles;
            item_it += I.n_tiles > 0 ? 1 : 0;
        }
        if (!ok) { atomicExch(&p.counters[3], 5); *abort_flag = 1; }
    } else if (warp == kMmaWarp) {
        // ================================ MMA issuer ================================================================
        // Two streams over the same list of tiles: first products (S^T = K_t . Q^T) and second products
        // (O^T += V_t^T . P_t^T).  The thread issues whichever has its operands ready; the first may run two tiles ahead
        // of the softmax (two S^T buffers), the second follows the P^T tiles.
        if (lane == 0) {
            auto look_ahead = [&](TcCursor &c) {                 // the next item with tiles after c.item (its loads are in flight
                for (c.next_item = c.item + gridDim.x; c.next_item < n_items; c.next_item += gridDim.x) {   // while this item's tiles run)
                    c.N = tc_item(p, c.next_item);
                    if (c.N.n_tiles > 0) return;
                }
            };
            auto advance = [&](TcCursor &c) {                    // to the next tile, skipping items without tiles
                if (++c.t < c.I.n_tiles) return;
                c.tile_it += c.I.n_tiles;
                c.item_it += 1;
                c.t = 0;
                c.item = c.next_item;
                c.I = c.N;
                if (c.item < n_items) look_ahead(c);
            };
            auto start = [&](TcCursor &c) {
                c.tile_it = c.item_it = 0;
                c.t = 0;
                for (c.item = blockIdx.x; c.item < n_items; c.item += gridDim.x) {
                    c.I = tc_item(p, c.item);
                    if (c.I.n_tiles > 0) break;
                }
                if (c.item < n_items) look_ahead(c);
            };
            TcCursor c1, c2;
            start(c1);
            c2 = c1;
            bool ok = true;
            uint64_t idle_since = 0;
            uint32_t spins = 0;
            while (c2.item < n_items) {
                bool did = false;
                if (c1.item < n_items) {
                    const uint32_t it_g = c1.tile_it + c1.t, buf = it_g & 1, ks = it_g % kKSlots, qb = c1.item_it & 1;
                    if (tc::mbar_test_wait(bar(&sh.k_full[ks]), (it_g / kKSlots) & 1) &&
                        tc::mbar_test_wait(bar(&sh.s_empty[buf]), ((it_g >> 1) & 1) ^ 1) &&
                        (c1.t > 0 || tc::mbar_test_wait(bar(&sh.q_full[qb]), (c1.item_it >> 1) & 1))) {
                        tc::fence_proxy_async_smem();            // the K rows were written by cp.async (generic proxy)
                        tc::fence_after_sync();
                        // one descriptor per operand and tile; a K = 16 step only moves its start address (in 16-byte units)
                        const uint64_t a0 = tc::smem_desc_sw128(base + ks * kTileBytes), b0 = tc::smem_desc_sw128(base + kOffQ + qb * kQBytes);
#pragma unroll
                        for (int cb = 0; cb < 2; ++cb)
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                tc::umma_f16(tmem_s[buf], a0 + uint64_t((cb * kColBlock + k * 32) >> 4), b0 + uint64_t((cb * kQBlock + k * 32) >> 4),
                                             idesc_s, (cb | k) != 0);
                        tc::umma_commit(bar(&sh.k_empty[ks]));   // the K slot may be refilled
                        tc::umma_commit(bar(&sh.s_full[buf]));
                        if (c1.t == c1.I.n_tiles - 1) tc::umma_commit(bar(&sh.q_empty[qb]));   // the query tile has been read for the last time
                        advance(c1);
                        did = true;
                    }
                }
                {
                    const uint32_t it_g = c2.tile_it + c2.t, buf = it_g & 1, vs = it_g % kVSlots, ob = c2.item_it & 1;
                    if (tc::mbar_test_wait(bar(&sh.p_full[buf]), (it_g >> 1) & 1) &&
                        tc::mbar_test_wait(bar(&sh.v_full[vs]), (it_g / kVSlots) & 1) &&
                        (c2.t > 0 || tc::mbar_test_wait(bar(&sh.o_empty[ob]), ((c2.item_it >> 1) & 1) ^ 1))) {
                        tc::fence_proxy_async_smem();            // the V rows were written by cp.async (generic proxy)
                        tc::fence_after_sync();
                        const uint64_t a0 = tc::smem_desc_mn_sw128(base + kOffV + vs * kTileBytes, kColBlock), b0 = tc::smem_desc_mn_sw64(base + kOffP + buf * kPBytes);
                        if (c2.t > 0) {
#pragma unroll
                            for (int ks = 0; ks < kTileKeys / 16; ++ks)
                                tc::umma_f16(tmem_o[ob], a0 + uint64_t((ks * 2048) >> 4), b0 + uint64_t((ks * 1024) >> 4), idesc_o, true);
                        } else {
#pragma unroll
                            for (int ks = 0; ks < kTileKeys / 16; ++ks)
                                tc::umma_f16(tmem_o[ob], a0 + uint64_t((ks * 2048) >> 4), b0 + uint64_t((ks * 1024) >> 4), idesc_o, ks > 0);
                        }
                        tc::umma_commit(bar(&sh.v_empty[vs]));   // the V slot may be refilled
                        tc::umma_commit(bar(&sh.p_empty[buf]));  // the P buffer may be rewritten
                        if (c2.t == c2.I.n_tiles - 1) tc::umma_commit(bar(&sh.o_full[ob]));    // the item's O^T is complete
                        advance(c2);
                        did = true;
                    }
                }
                if (did) { idle_since = 0; spins = 0; continue; }
                if ((++spins & 63u) == 0) {                      // nothing ready: bounded like every other wait
                    if (*abort_flag) { ok = false; break; }
                    const uint64_t now = tc::global_timer_ns();
                    if (idle_since == 0) idle_since = now;
                    else if (now - idle_since > tc::kWaitLimitNs) { ok = false; break; }
                }
            }
            if (!ok) { atomicExch(&p.counters[3], 2); *abort_flag = 1; }
        }
    } else if (warp == kLoaderWarp) {
        // ================================ query loader (one warp) =======================================================
        // The item's queries, through the permutation, as the K-major B operand of the first product (rows past nq are
        // zero); two buffers, so the next item's queries are in place before its first key tile.
        const T *qg = reinterpret_cast<const T *>(p.q);
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const TcItem I = tc_item(p, item);
            if (I.n_tiles == 0) continue;
            const uint32_t qb = item_it & 1;
            ok = warp_mbar_wait(bar(&sh.q_empty[qb]), ((item_it >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            const int my_row = lane < I.nq ? p.perm[I.q_begin + lane] : -1;     // lane r knows the row of query r
#pragma unroll 4
            for (int e = lane; e < kNQ * 16; e += 32) {
                const int r = e >> 4, c = e & 15;
                const int row = __shfl_sync(0xffffffffu, my_row, r);
                uint4 val = make_uint4(0, 0, 0, 0);
                if (row >= 0) val = *reinterpret_cast<const uint4 *>(qg + size_t(row) * kD + c * 8);
                *reinterpret_cast<uint4 *>(base_ptr + kOffQ + qb * kQBytes + (c >> 3) * kQBlock + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = val;
            }
            tc::fence_proxy_async_smem();
            tc::mbar_arrive(bar(&sh.q_full[qb]));
            item_it += 1;
        }
        if (!ok && lane == 0) { atomicExch(&p.counters[3], 4); *abort_flag = 1; }
    } else {
        // ================================ gather =====================================================================
        // Thread g copies chunk (g & 15) of rows (g >> 4) + 8 i, i = 0..15, of the K tile, then of the V tile.  A copy's
        // completion arrives on the slot's barrier by itself (cp.async.mbarrier.arrive), so the threads never wait for
        // data: they run ahead as far as free slots allow, across item boundaries.
        const int g = tid - 32 * kGatherWarp0;                   // 0 .. 127
        const char *kg = reinterpret_cast<const char *>(p.k);
        const char *vg = reinterpret_cast<const char *>(p.v);
        const int32_t row_max = int32_t(min(p.n_k_rows - 1, int64_t(0x7fffffff)));
        const int my_c = g & 15, my_r = g >> 4;
        constexpr int RPT = kTileKeys * 16 / kGatherThreads;     // rows per thread and tile: 16
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const TcItem I = tc_item(p, item);
            if (I.n_tiles == 0) continue;
            // table entries are fetched two tiles ahead, so that their latency never sits between two rounds of copies
            int32_t rows_a[RPT], rows_b[RPT];
            auto load_rows = [&](int32_t (&rows)[RPT], int tile) {
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    const int j = tile * kTileKeys + my_r + 8 * i;
                    rows[i] = (tile < I.n_tiles && j < I.chunk_len) ? int32_t(load_index(p.table, p.idx_bytes, I.tbl0 + j)) : -1;
                }
            };
            auto copy_tile = [&](const int32_t (&rows)[RPT], int t) -> bool {
                const uint32_t it_g = tile_it + t, ks = it_g % kKSlots, vs = it_g % kVSlots;
                const int live = I.chunk_len - t * kTileKeys;
                uint32_t off[RPT];                               // row offsets in units of 16 bytes (rows * 16 < 2^32)
                uint32_t valid = 0;
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    const int32_t row = min(max(rows[i] + int32_t(I.kbase), 0), row_max);
                    off[i] = uint32_t(row) * (kD * 2 / 16) + my_c;
                    valid |= (my_r + 8 * i < live ? 1u : 0u) << i;             // rows past the chunk's end are zero-filled
                }
                if (!warp_mbar_wait(bar(&sh.k_empty[ks]), ((it_g / kKSlots) & 1) ^ 1, abort_flag)) return false;
                const uint32_t kdst = base + ks * kTileBytes;
#pragma unroll
                for (int i = 0; i < RPT; ++i) cp_async16(kdst + tile_off(my_r + 8 * i, my_c), kg + size_t(off[i]) * 16, (valid >> i) & 1);
                tc::cp_async_arrive(bar(&sh.k_full[ks]));
                if (!warp_mbar_wait(bar(&sh.v_empty[vs]), ((it_g / kVSlots) & 1) ^ 1, abort_flag)) return false;
                const uint32_t vdst = base + kOffV + vs * kTileBytes;
#pragma unroll
                for (int i = 0; i < RPT; ++i) cp_async16(vdst + tile_off(my_r + 8 * i, my_c), vg + size_t(off[i]) * 16, (valid >> i) & 1);
                tc::cp_async_arrive(bar(&sh.v_full[vs]));
                return true;
            };
            load_rows(rows_a, 0);
            load_rows(rows_b, 1);
            for (int t = 0; t < I.n_tiles && ok; t += 2) {
                ok = copy_tile(rows_a, t);
                load_rows(rows_a, t + 2);
                if (ok && t + 1 < I.n_tiles) {
                    ok = copy_tile(rows_b, t + 1);
                    load_rows(rows_b, t + 3);
                }
            }
            tile_it += I.n_tiles;
            item_it += 1;
        }
        cp_async_commit();
        cp_async_wait<0>();                                      // nothing of this thread is in flight when the CTA ends
        if (!ok && lane == 0) { atomicExch(&p.counters[3], 1); *abort_flag = 1; }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) tc::tmem_dealloc(tmem_base, 128);
}

}  // namespace

bool attn_tc_supported(int dtype, int d) { return (dtype == FM_BF16 || dtype == FM_F16) && d == kD; }

// `redo_items` / `redo_count`: list (room for every item) and its counter (zeroed by the caller) of the items that the
// caller has to serve again with the kernel that tracks a running maximum.
int launch_attn_tc(const AttnParams &p, int dtype, int grid, int4 *redo_items, int *redo_count, cudaStream_t st)
{
    const size_t smem = kTcSmem + 1024;
    const bool bf16 = dtype == FM_BF16;
    const uint32_t idesc_s = tc::instr_desc_f16(bf16, kTileKeys, kNQ);                    // K-major A and B
    const uint32_t idesc_o = tc::instr_desc_f16(bf16, kD, kNQ, true, true);               // MN-major A and B
    if (bf16) {
        FM_CUDA_OK(func_attr_cached((const void *)attn_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attn_tc_kernel<__nv_bfloat16><<<grid, kTcAttnThreads, smem, st>>>(p, idesc_s, idesc_o, redo_items, redo_count);
    } else {
        FM_CUDA_OK(func_attr_cached((const void *)attn_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attn_tc_kernel<__half><<<grid, kTcAttnThreads, smem, st>>>(p, idesc_s, idesc_o, redo_items, redo_count);
    }
    FM_LAUNCHED("attn_tc_kernel");
    return FM_OK;
}

}  // namespace fm
