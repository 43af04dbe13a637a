// Projection Y = A K^T on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands staged
// by TMA), with the epilogue that makes the index build a single pass over the keys: instead of writing
// Y (C x N fp32, several GB) each epilogue thread owns one bucket row, compares its scores with the bucket's
// threshold and appends the groups of four keys that hold a survivor to the bucket's candidate list.  A dense-store epilogue of
// the same kernel produces the small score matrix of the key sample from which the thresholds are estimated.
//
// CTA = 320 threads: warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane) and TMEM owner,
// warps 2-5 = epilogue group 0, warps 6-9 = epilogue group 1 (TMEM lane quarter = warp % 4).
// Work unit = (segment, 128-bucket tile, key range).  Per 256-key tile: K tile -> shared memory (ring of
// 64 KB stages at d = 128), 8 UMMAs (M = 128, N = 256, K = 16) into accumulator t % 2 (256 TMEM columns each);
// epilogue group t % 2 drains it while the MMAs of the next tile fill the other one.
// Every mbarrier wait is bounded; on a give-up the CTA records a status and unwinds.
#include "tc_project.cuh"

#include <cstdlib>
#include <mutex>

namespace fm {

namespace {

constexpr int kBM = kTcBM;                  // bucket rows per tile (UMMA M)
constexpr int kBN = kTcBN;                  // keys per tile (UMMA N)
constexpr int kTcThreads = 320;

template <bool DENSE> struct TcCfg { static constexpr int STAGES = 3; };

constexpr int kGroupsPerBatch = 8;          // a batch of 32 columns is 8 groups of four columns

// Appends a group of four scores to a candidate list when any of the four reaches tau, and sets the group's bit in
// the batch mask.  Branch-free (some lane of the 32 almost always has a hit, so a divergent branch would run the body
// for every group anyway).  The epilogue looks at every one of the C x N scores, so what matters is instructions per
// score:
//  - the four scores are four consecutive registers of the TMEM load, stored as they lie (a 16-byte store wants an
//    aligned register quad; a column inside the entry would cost a register move per score).  Which keys an entry
//    holds is recorded instead in one bit per group: 64 bits per (bucket, key tile), stored once per tile;
//  - the list position is a 32-bit byte offset from the array base: predicated 64-bit pointer bumps and wide
//    multiply-adds cost several instructions each.
// Every operand is an untyped 32-bit register: the scores are floats to max / setp and bits to the store.
template <int J>
__device__ __forceinline__ void append_group(const uint4 *cand, uint32_t &off16, uint32_t step16, uint32_t &mask8, uint32_t tau_bits,
                                             uint32_t s0, uint32_t s1, uint32_t s2, uint32_t s3)
{
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 m;\n\t.reg .b64 a, o;\n\t"
                 "cvt.u64.u32 o, %0;\n\t"
                 "add.s64 a, %2, o;\n\t"
                 "max.f32 m, %4, %5, %6;\n\t"
                 "max.f32 m, m, %7;\n\t"
                 "setp.ge.f32 p, m, %3;\n\t"
                 "@p st.global.v4.b32 [a], {%4, %5, %6, %7};\n\t"
                 "@p add.u32 %0, %0, %8;\n\t"
                 "@p add.u32 %1, %1, %9;\n\t}"
                 : "+r"(off16), "+r"(mask8)
                 : "l"(cand), "r"(tau_bits), "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(step16), "n"(1 << J)
                 : "memory");
}

template <int J>
__device__ __forceinline__ void append_groups(const uint4 *cand, uint32_t &off16, uint32_t step16, uint32_t &mask8, uint32_t tau_bits,
                                              const uint32_t (&v)[32])
{
    if constexpr (J < kGroupsPerBatch) {
        append_group<J>(cand, off16, step16, mask8, tau_bits, v[4 * J], v[4 * J + 1], v[4 * J + 2], v[4 * J + 3]);
        append_groups<J + 1>(cand, off16, step16, mask8, tau_bits, v);
    }
}

}  // namespace

template <int D, bool DENSE>
__global__ void __launch_bounds__(kTcThreads, 1)
tc_project_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmK, TcParams p, uint32_t idesc)
{
    constexpr int STAGES = TcCfg<DENSE>::STAGES;
    constexpr int KB = D / 64;                               // 64-element (128-byte) k-blocks
    constexpr uint32_t A_BYTES = KB * kBM * 128;
    constexpr uint32_t STAGE_BYTES = KB * kBN * 128;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1 + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (tc::smem_addr(smem_dyn) + 1023u) & ~1023u;          // 1024-byte aligned tiles
    const uint32_t a_smem = base, k_smem = base + A_BYTES;
    const uint32_t bar0 = tc::smem_addr(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    const uint32_t a_bar = bar0 + 8u * (2 * STAGES);
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 1 + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 3 + a); };

    // ---- which unit -----------------------------------------------------------------------------------------
    const int unit = blockIdx.x;
    const int range = unit % p.n_ranges;
    const int mt_global = unit / p.n_ranges;
    int seg = 0;
    {
        int lo = 0, hi = p.n_seg;                            // largest seg with mtile0 <= mt_global
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (p.segs[mid].mtile0 <= mt_global) lo = mid; else hi = mid;
        }
        seg = lo;
    }
    const TcSeg sg = p.segs[seg];
    const int m0 = (mt_global - sg.mtile0) * kBM;            // first bucket of the tile inside the segment
    const int n_tiles_seg = (sg.n_keys + kBN - 1) / kBN;
    const int per_range = (n_tiles_seg + p.n_ranges - 1) / p.n_ranges;
    const int t_begin = min(range * per_range, n_tiles_seg), t_end = min(t_begin + per_range, n_tiles_seg);
    const int n_tiles = t_end - t_begin;
    // Tiles are visited in the order 0, H, 1, H + 1, ... (H = half the range): accumulator / epilogue group 0 sees the
    // first half of the range in ascending order and group 1 the second half, so the two candidate lists of a range
    // simply concatenate into key order.
    const int half = (n_tiles + 1) >> 1;
    auto tile_of = [&](int s) { return (s & 1) ? half + (s >> 1) : (s >> 1); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { tc::mbar_init(full_bar(s), 1); tc::mbar_init(empty_bar(s), 1); }
        tc::mbar_init(a_bar, 1);
        for (int a = 0; a < 2; ++a) { tc::mbar_init(tfull_bar(a), 1); tc::mbar_init(tempty_bar(a), 4); }
        tc::mbar_fence_init();
        s_abort = 0;
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_addr(&tmem_slot), 512);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    const uint64_t limit = p.wait_limit_ns ? p.wait_limit_ns : tc::kWaitLimitNs;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------------------------------
        if (lane == 0 && n_tiles > 0) {
            tc::prefetch_tensormap(&tmA);
            tc::prefetch_tensormap(&tmK);
            tc::mbar_arrive_expect_tx(a_bar, A_BYTES);
            for (int kb = 0; kb < KB; ++kb) tc::tma_load_2d(a_smem + kb * (kBM * 128), &tmA, kb * 64, sg.a_row0 + m0, a_bar);
            int issued = 0;                                  // tiles whose loads were started
            for (int t = 0; t < n_tiles; ++t) {
                const int s = t % STAGES;
                if (!tc::mbar_wait(empty_bar(s), ((t / STAGES) & 1) ^ 1, limit)) { atomicExch(p.status, 1); s_abort = 1; break; }
                if (*(volatile int *)&s_abort) break;
                if (t == p.skip_tile) continue;              // test hook: this tile never arrives, its consumers give up
                tc::mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
                const int key_row = sg.k_row0 + (t_begin + tile_of(t)) * kBN;
                for (int kb = 0; kb < KB; ++kb)
                    tc::tma_load_2d(k_smem + s * STAGE_BYTES + kb * (kBN * 128), &tmK, kb * 64, key_row, full_bar(s));
                issued = t + 1;
            }
            // No copy of this thread may still be in flight when the CTA's shared memory is handed on, whether the
            // consumers took the tiles or gave up before them: wait (bounded) until the last loads have landed.  A stage's
            // barrier leaves the phase of tile t only when this thread arms it again, so the parities are unambiguous.
            tc::mbar_wait(a_bar, 0, limit);
            for (int t = max(0, issued - STAGES); t < issued; ++t)
                if (t != p.skip_tile) tc::mbar_wait(full_bar(t % STAGES), (t / STAGES) & 1, limit);
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------------------------------------
        if (lane == 0 && n_tiles > 0) {
            bool ok = tc::mbar_wait(a_bar, 0, limit);
            for (int t = 0; ok && t < n_tiles; ++t) {
                const int s = t % STAGES, acc = t & 1;
                ok = tc::mbar_wait(tempty_bar(acc), ((t >> 1) & 1) ^ 1, limit) && tc::mbar_wait(full_bar(s), (t / STAGES) & 1, limit);
                if (!ok || *(volatile int *)&s_abort) { ok = false; break; }
                tc::fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kBN;
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t da = tc::smem_desc_sw128(a_smem + kb * (kBM * 128) + k * 32);
                        const uint64_t db = tc::smem_desc_sw128(k_smem + s * STAGE_BYTES + kb * (kBN * 128) + k * 32);
                        tc::umma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
                    }
                }
                tc::umma_commit(empty_bar(s));               // the stage may be refilled once these MMAs have read it
                tc::umma_commit(tfull_bar(acc));             // the accumulator is complete
            }
            if (!ok) { atomicExch(p.status, 2); s_abort = 1; }
        }
    } else {
        // ---- epilogue: group g drains accumulator g (tiles t = g, g + 2, ...); one bucket row per thread -----
        const int g = (warp - 2) >> 2;
        const int q = warp & 3;                              // TMEM lane quarter this warp may read
        const int m = q * 32 + lane;                         // row of the tile
        const bool row_ok = m0 + m < sg.n_buckets;
        const int grow = sg.out_row0 + m0 + m;               // row of this bucket in the outputs
        float tau = 0.f;
        uint32_t first16 = 0, off16 = 0, step16 = 16u;       // byte offsets into cand
        int sub_cap = 0, cursor = 0;
        bool overflow = false;
        if constexpr (!DENSE) {
            if (row_ok) {
                // one buffer per key range, shared by the two groups: group 0 fills it upward, group 1 downward
                tau = p.tau[grow];
                sub_cap = p.cap / p.n_ranges;
                uint32_t slot = uint32_t(grow) * uint32_t(p.cap) + uint32_t(range) * uint32_t(sub_cap);    // host: the arrays stay below 4 GB
                if (g) { slot += sub_cap - 1; step16 = uint32_t(-16); }
                first16 = off16 = slot * 16u;
            }
        }
        bool ok = true;
        for (int t = g; t < n_tiles; t += 2) {
            ok = tc::mbar_wait(tfull_bar(g), (t >> 1) & 1, limit) && !*(volatile int *)&s_abort;
            ok = __all_sync(0xffffffffu, ok);                // the TMEM loads below need the whole warp
            if (!ok) break;
            tc::fence_after_sync();
            const int col0 = (t_begin + tile_of(t)) * kBN;
            const bool last = col0 + kBN > sg.n_keys;        // only the segment's last tile can be partial
            uint32_t mask_lo = 0, mask_hi = 0;               // which of the tile's 64 groups of four keys were appended
            // batches of 32 columns (loading the next batch while this one is looked at was measured: no gain)
            auto batch = [&](uint32_t (&v)[32], int b) {
                const int c0 = col0 + b * 32;
                if constexpr (DENSE) {
                    // blocked layout (see dense_offset): the 32 lanes of a store instruction write 512 contiguous bytes
                    if (q * 32 < sg.n_buckets - m0 && c0 < sg.n_keys) {
                        float *blk = p.Y + dense_block_offset(sg.out_row0 + m0 + q * 32, c0, p.ldy);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *reinterpret_cast<uint4 *>(blk + j * 128 + lane * 4) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                } else {
                    if (last) {
                        const int live = sg.n_keys - c0;     // columns of this batch that exist
#pragma unroll
                        for (int e = 0; e < 32; ++e)
                            if (e >= live) v[e] = 0xff800000u;                       // -inf never passes
                    }
                    if (row_ok) {
                        if (!overflow && cursor + kGroupsPerBatch <= sub_cap) {
                            uint32_t mask8 = 0;
                            append_groups<0>(p.cand, off16, step16, mask8, __float_as_uint(tau), v);
                            if (b < 4) mask_lo |= mask8 << (8 * b); else mask_hi |= mask8 << (8 * b - 32);
                            cursor = int((off16 - first16) * (g ? uint32_t(-1) : 1u)) >> 4;
                        } else {
                            overflow = true;                 // keep counting so that the selection sees the overflow
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float m = fmaxf(fmaxf(__uint_as_float(v[j]), __uint_as_float(v[j + 1])),
                                                      fmaxf(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])));
                                cursor += m >= tau ? 1 : 0;
                            }
                        }
                    }
                }
            };
            const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + g * kBN;
#pragma unroll 1
            for (int b = 0; b < kBN / 32; ++b) {
                uint32_t v[32];
                tc::tmem_ld_x32(t_addr + b * 32, v);
                tc::tmem_ld_wait();
                batch(v, b);
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tempty_bar(g));
            if constexpr (!DENSE) {
                if (row_ok) p.cand_mask[size_t(t_begin + tile_of(t)) * p.mask_ld + grow] = make_uint2(mask_lo, mask_hi);   // coalesced: 32 rows
            }
        }
        if (!ok && lane == 0) { atomicExch(p.status, 3); s_abort = 1; }
        if constexpr (!DENSE) {
            if (row_ok) p.cand_count[(size_t(grow) * p.n_ranges + range) * 2 + g] = overflow ? sub_cap + 1 : cursor;
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem_base, 512);
}

// ---- host ----------------------------------------------------------------------------------------------------
static std::atomic<uint64_t> g_test_wait_limit_ns{0};
static std::atomic<int> g_test_skip_tile{-1};

void tc_apply_test_hooks(TcParams &p)
{
    p.wait_limit_ns = g_test_wait_limit_ns.load(std::memory_order_relaxed);
    p.skip_tile = g_test_skip_tile.load(std::memory_order_relaxed);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static std::mutex mu;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

int make_tensor_map_2d(CUtensorMap *map, const void *base_ptr, int dtype, uint64_t rows, uint64_t d, uint64_t row_stride_bytes,
                       uint32_t box_rows)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return FM_ERR_CUDA;
    }
    cuuint64_t dims[2] = {d, rows};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dtype == FM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                    const_cast<void *>(base_ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with %d (rows %llu, d %llu, stride %llu)", (int)r, (unsigned long long)rows,
                  (unsigned long long)d, (unsigned long long)row_stride_bytes);
        return FM_ERR_CUDA;
    }
    return FM_OK;
}

template <int D, bool DENSE>
static int launch_tc(const CUtensorMap &tmA, const CUtensorMap &tmK, const TcParams &p, int units, bool bf16, cudaStream_t st)
{
    constexpr size_t smem = size_t(D / 64) * (kBM * 128 + TcCfg<DENSE>::STAGES * kBN * 128) + 1024;
    FM_CUDA_OK(func_attr_cached((const void *)tc_project_kernel<D, DENSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    TcParams q = p;
    tc_apply_test_hooks(q);
    tc_project_kernel<D, DENSE><<<units, kTcThreads, smem, st>>>(tmA, tmK, q, tc::instr_desc_f16(bf16, kBM, kBN));
    FM_LAUNCHED("tc_project_kernel");
    return FM_OK;
}

int tc_project_launch(const CUtensorMap &tmA, const CUtensorMap &tmK, const TcParams &p, int units, int d, bool dense, bool bf16,
                      cudaStream_t st)
{
    if (d == 128) return dense ? launch_tc<128, true>(tmA, tmK, p, units, bf16, st) : launch_tc<128, false>(tmA, tmK, p, units, bf16, st);
    if (d == 64) return dense ? launch_tc<64, true>(tmA, tmK, p, units, bf16, st) : launch_tc<64, false>(tmA, tmK, p, units, bf16, st);
    set_error("tensor-core projection supports head dim 64 and 128, got %d", d);
    return FM_ERR_UNSUPPORTED;
}

}  // namespace fm

namespace fm {
__global__ void unblock_scores_kernel(const float *__restrict__ blocked, int64_t ld_blocked, int64_t rows, int64_t cols,
                                      float *__restrict__ Y, int64_t ldy)
{
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * cols) return;
    const int64_t r = i / cols, c = i - r * cols;
    Y[r * ldy + c] = blocked[dense_offset(r, c, ld_blocked)];
}
}  // namespace fm

extern "C" size_t fm_project_tc_workspace_bytes(int64_t C, int64_t n_key_rows, int64_t key_step)
{
    const int64_t n_cols = (n_key_rows + key_step - 1) / key_step;
    return 256 + size_t(fm::ceil_div(C, 32) * 32) * size_t(fm::ceil_div(n_cols, 32) * 32) * 4;
}

// Dense tensor-core projection of ONE segment: Y[c, j] ~= A[c] . K[j * key_step] for j < n_cols, fp32
// accumulation in the tensor cores' own order (NOT the canonical chain: for scores that feed an index use
// fm_project).
extern "C" int fm_project_tc(const void *A, const void *K, int dtype, int64_t C, int64_t n_key_rows, int d, int64_t key_step,
                             float *Y, int64_t ldy, void *workspace, size_t workspace_bytes, fm_stream_t stream)
{
    using namespace fm;
    FM_REQUIRE(A && K && Y && workspace, "fm_project_tc: null pointer");
    FM_REQUIRE(C > 0 && n_key_rows > 0 && key_step >= 1, "fm_project_tc: bad sizes");
    FM_REQUIRE(((uintptr_t)A | (uintptr_t)K) % 16 == 0, "fm_project_tc: A and K must be 16-byte aligned");
    if ((dtype != FM_BF16 && dtype != FM_F16) || (d != 64 && d != 128)) {
        set_error("fm_project_tc: needs bf16/fp16 and head dim 64 or 128");
        return FM_ERR_UNSUPPORTED;
    }
    const int64_t n_cols = (n_key_rows + key_step - 1) / key_step;
    FM_REQUIRE(ldy >= n_cols, "fm_project_tc: ldy too small");
    if (workspace_bytes < fm_project_tc_workspace_bytes(C, n_key_rows, key_step)) {
        set_error("fm_project_tc: workspace %zu too small", workspace_bytes);
        return FM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    CUtensorMap tmA, tmK;
    int rc = make_tensor_map_2d(&tmA, A, dtype, (uint64_t)C, (uint64_t)d, (uint64_t)d * 2, kBM);
    if (rc != FM_OK) return rc;
    rc = make_tensor_map_2d(&tmK, K, dtype, (uint64_t)n_cols, (uint64_t)d, (uint64_t)d * 2 * key_step, kBN);
    if (rc != FM_OK) return rc;
    TcSeg seg = {0, (int)C, 0, (int)n_cols, 0, 0};
    char *ws = (char *)workspace;
    FM_CUDA_OK(cudaMemsetAsync(ws, 0, 256, st));
    FM_CUDA_OK(cudaMemcpyAsync(ws + 64, &seg, sizeof(seg), cudaMemcpyHostToDevice, st));
    TcParams p = {};
    p.segs = (const TcSeg *)(ws + 64);
    p.n_seg = 1;
    const int m_tiles = (int)ceil_div(C, kBM);
    const int n_tiles = (int)ceil_div(n_cols, kBN);
    p.n_ranges = (int)std::max<int64_t>(1, std::min<int64_t>(n_tiles, ceil_div(2 * sm_count(), m_tiles)));
    p.Y = (float *)(ws + 256);
    p.ldy = ceil_div(n_cols, 32) * 32;
    p.status = (int *)ws;
    rc = tc_project_launch(tmA, tmK, p, m_tiles * p.n_ranges, d, true, dtype == FM_BF16, st);
    if (rc != FM_OK) return rc;
    unblock_scores_kernel<<<(unsigned)ceil_div(C * n_cols, 256), 256, 0, st>>>(p.Y, p.ldy, C, n_cols, Y, ldy);
    FM_LAUNCHED("unblock_scores_kernel");
    return FM_OK;
}

extern "C" int fm_test_set_tc_hooks(int wait_limit_ms, int skip_tile)
{
    if (wait_limit_ms < 0 || skip_tile < -1) {
        fm::set_error("fm_test_set_tc_hooks: bad arguments");
        return FM_ERR_BAD_ARG;
    }
    fm::g_test_wait_limit_ns.store(uint64_t(wait_limit_ms) * 1000000ull, std::memory_order_relaxed);
    fm::g_test_skip_tile.store(skip_tile, std::memory_order_relaxed);
    return FM_OK;
}
