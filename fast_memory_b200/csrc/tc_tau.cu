// Thresholds of the fused index build without a score matrix: the projection of the KEY SAMPLE (every step-th key) runs
// on the tensor cores three times over, and the epilogue threads - one bucket row each - reduce the scores as they come
// out of TMEM instead of storing them:
//   sweep 0: minimum and maximum of the row's sample scores;
//   sweep 1: a histogram of 121 equal bins over [min, max]; the bin b1 that holds the r-th largest score and the rank r1
//            the score has inside that bin;
//   sweep 2: a histogram of 127 equal sub-bins of bin b1; tau = the lower edge of the sub-bin that holds the r1-th
//            largest of the bin's scores, less one sub-bin.
// tau is therefore at most the r-th largest sample score and misses it by at most about (max - min) / 7500: the candidate
// pass keeps a handful of keys more than an exact order statistic would, and nothing else depends on tau's value (the
// selection proves completeness on its own).  The sample projection is 1/step of the full one, so running it three times
// costs little; what it saves is writing the sample scores (rows x sample x 4 bytes) and reading them back twice.
//
// CTA = 320 threads as in tc_project.cu (warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-5 / 6-9 epilogue
// groups that drain the two accumulators alternately); one CTA per tile of 128 buckets sweeps all key tiles of the
// segment's sample.  The row histograms (128 rows x 128 counters, 64 KB) live in shared memory: the two threads that
// serve a row - one per group - add with shared-memory atomics, the rows of a warp interleaved word by word so that
// lane i only ever touches bank i.  The epilogue sees every score three times, so it is written for few instructions
// per score (integer and min / max instructions issue at half the rate of multiply-adds): one per score in sweep 0,
// four in sweep 1, six in sweep 2.  Every mbarrier wait is bounded; after a give-up the
// warps skip the pipeline but keep meeting at the sweep boundaries, so the CTA unwinds and frees its TMEM.
#include "tc_project.cuh"

#include <type_traits>

namespace fm {

namespace {

constexpr int kBM = kTcBM, kBN = kTcBN;
constexpr int kThreads = 320;
constexpr int kStages = 2;
constexpr int kBins = 128;
constexpr int kHistBytes = kBM * kBins * 4;                 // 64 KB
constexpr int kEpiBarrier = 1;                               // named barrier of the 256 epilogue threads

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
tc_tau_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmK, TauParams p, uint32_t idesc)
{
    constexpr int KB = D / 64;
    constexpr uint32_t A_BYTES = KB * kBM * 128;
    constexpr uint32_t STAGE_BYTES = KB * kBN * 128;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bars[2 * kStages + 1 + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (tc::smem_addr(smem_dyn) + 1023u) & ~1023u;
    const uint32_t a_smem = base, k_smem = base + A_BYTES, hist_smem = k_smem + kStages * STAGE_BYTES;
    uint32_t *hist = reinterpret_cast<uint32_t *>(smem_dyn + (hist_smem - tc::smem_addr(smem_dyn)));
    const uint32_t bar0 = tc::smem_addr(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    const uint32_t a_bar = bar0 + 8u * (2 * kStages);
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 1 + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 3 + a); };

    // ---- which bucket tile ------------------------------------------------------------------------------------
    const int mt_global = blockIdx.x;
    int seg = 0;
    {
        int lo = 0, hi = p.n_seg;
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (p.segs[mid].mtile0 <= mt_global) lo = mid; else hi = mid;
        }
        seg = lo;
    }
    const TcSeg sg = p.segs[seg];
    const int rank = sg.rank;
    const int m0 = (mt_global - sg.mtile0) * kBM;
    const int n_tiles = (sg.n_keys + kBN - 1) / kBN;
    const int n_steps = 3 * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { tc::mbar_init(full_bar(s), 1); tc::mbar_init(empty_bar(s), 1); }
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
    volatile int *abort_flag = &s_abort;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------------------------------------
        if (lane == 0 && n_tiles > 0) {
            tc::prefetch_tensormap(&tmA);
            tc::prefetch_tensormap(&tmK);
            tc::mbar_arrive_expect_tx(a_bar, A_BYTES);
            for (int kb = 0; kb < KB; ++kb) tc::tma_load_2d(a_smem + kb * (kBM * 128), &tmA, kb * 64, sg.a_row0 + m0, a_bar);
            int issued = 0;
            for (int t = 0; t < n_steps; ++t) {
                const int s = t % kStages;
                if (!tc::mbar_wait(empty_bar(s), ((t / kStages) & 1) ^ 1, limit)) { atomicExch(p.status, 1); *abort_flag = 1; break; }
                if (*abort_flag) break;
                tc::mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
                const int key_row = sg.k_row0 + (t % n_tiles) * kBN;
                for (int kb = 0; kb < KB; ++kb)
                    tc::tma_load_2d(k_smem + s * STAGE_BYTES + kb * (kBN * 128), &tmK, kb * 64, key_row, full_bar(s));
                issued = t + 1;
            }
            // no copy of this thread may be in flight when the CTA ends
            tc::mbar_wait(a_bar, 0, limit);
            for (int t = max(0, issued - kStages); t < issued; ++t) tc::mbar_wait(full_bar(t % kStages), (t / kStages) & 1, limit);
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------------------------------------------
        if (lane == 0 && n_tiles > 0) {
            bool ok = tc::mbar_wait(a_bar, 0, limit);
            for (int t = 0; ok && t < n_steps; ++t) {
                const int s = t % kStages, acc = t & 1;
                ok = tc::mbar_wait(tempty_bar(acc), ((t >> 1) & 1) ^ 1, limit) && tc::mbar_wait(full_bar(s), (t / kStages) & 1, limit);
                if (!ok || *abort_flag) { ok = false; break; }
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
                tc::umma_commit(empty_bar(s));
                tc::umma_commit(tfull_bar(acc));
            }
            if (!ok) { atomicExch(p.status, 2); *abort_flag = 1; }
        }
    } else {
        // ---- epilogue: the two threads (one per group) of TMEM lane m serve bucket row m0 + m --------------------------
        const int g = (warp - 2) >> 2;
        const int q = warp & 3;
        const int m = q * 32 + lane;
        const bool row_ok = m0 + m < sg.n_buckets;
        const int grow = sg.out_row0 + m0 + m;
        // the counters of the 32 rows of a TMEM lane quarter are interleaved word by word: counter b of row (q, lane) sits
        // at word (q * 128 + b) * 32 + lane, so lane i of a warp only ever touches bank i, whatever bins the scores fall into
        uint32_t *hrow = hist + q * kBins * 32 + lane;                             // counter b of the row: hrow[b * 32]
        const uint32_t hrow_s = hist_smem + (uint32_t(q) * kBins * 32 + uint32_t(lane)) * 4;
        float *xch = reinterpret_cast<float *>(hist);        // scratch for what the two groups tell each other (the histogram is idle then)
        bool ok = true;
        float mn = INFINITY, mx = -INFINITY;
        // The bin of a score x is the integer that x * sc + K rounds to, K = an integer + 2^23: the fused multiply-add
        // leaves that integer in the low bits of its result (one instruction; a float-to-int conversion runs at a quarter
        // of the rate, and this epilogue looks at every score three times).  kp = K - 2^23, so that bin b starts at
        // x = (b - 0.5 - kp) / sc.  Both bin functions are monotone in x, which is all the reasoning below needs.
        float sc1 = 0.f, K1 = 8388609.f, kp1 = 1.f;          // sweep 1: bins 2 .. 126 over [min, max]
        float sc2 = 0.f, K2 = 8388608.f, kp2 = 0.f;          // sweep 2: sub-bins 0 .. 126 of bin b1
        bool flat = true;                                    // all scores of the row (nearly) equal
        bool fine = false;                                   // sweep 2 refines inside bin b1
        int b1 = 0, r1 = 0;

        auto red_add1 = [&](uint32_t bits, bool pred) {      // (the bin is masked: a non-finite score must not leave the row)
            const uint32_t addr = hrow_s + ((bits & uint32_t(kBins - 1)) << 7);
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %1, 0;\n\t@p red.shared.add.u32 [%0], 1;\n\t}" ::"r"(addr), "r"(pred ? 1u : 0u));
        };
        // the bin that holds the `want`-th largest entry of the row's histogram, looking at bins top .. 0, and the rank inside
        // it; found = false when the bins hold fewer (every thread of group 0 scans its own row; uniform trip count)
        auto scan_from_top = [&](int top, int want, int &bin, int &inside) {
            int cum = 0;
            bin = 0; inside = want;
            bool found = false;
            for (int b = top; b >= 0; --b) {
                const int c = int(hrow[b * 32]);
                if (!found && cum + c >= want) { found = true; bin = b; inside = want - cum; }
                cum += c;
            }
            return found;
        };

        for (int sweep = 0; sweep < 3; ++sweep) {
            for (int tile = 0; tile < n_tiles; ++tile) {
                const int t = sweep * n_tiles + tile;
                if ((t & 1) != g) continue;
                if (ok) {
                    ok = !*abort_flag && tc::mbar_wait(tfull_bar(g), (t >> 1) & 1, limit);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok && lane == 0) { atomicExch(p.status, 3); *abort_flag = 1; }
                }
                if (!ok) continue;                           // (the sweep boundaries below are still met)
                tc::fence_after_sync();
                const int col0 = tile * kBN;
                const bool last = col0 + kBN > sg.n_keys;
                const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + g * kBN;
                const uint32_t base2 = __float_as_uint(8388608.f);
#pragma unroll 1
                for (int b = 0; b < kBN / 32; ++b) {
                    uint32_t v[32];
                    tc::tmem_ld_x32(t_addr + b * 32, v);
                    tc::tmem_ld_wait();
                    const int live = last ? sg.n_keys - (col0 + b * 32) : 32;       // columns of this batch that exist
                    if (live <= 0) break;
                    auto batch = [&](auto full_tag) {
                        constexpr bool FULL = decltype(full_tag)::value;
                        if (sweep == 0) {
                            if (FULL) {
#pragma unroll
                                for (int e = 0; e < 32; e += 2) {          // three-operand min / max: one instruction per score
                                    asm("min.f32 %0, %0, %1, %2;" : "+f"(mn) : "f"(__uint_as_float(v[e])), "f"(__uint_as_float(v[e + 1])));
                                    asm("max.f32 %0, %0, %1, %2;" : "+f"(mx) : "f"(__uint_as_float(v[e])), "f"(__uint_as_float(v[e + 1])));
                                }
                            } else {
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    if (e < live) { mn = fminf(mn, __uint_as_float(v[e])); mx = fmaxf(mx, __uint_as_float(v[e])); }
                            }
                        } else if (sweep == 1) {
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                                red_add1(__float_as_uint(fmaf(__uint_as_float(v[e]), sc1, K1)), FULL || e < live);
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                const uint32_t bits = __float_as_uint(fmaf(__uint_as_float(v[e]), sc2, K2));
                                red_add1(bits, (FULL || e < live) && bits - base2 <= uint32_t(kBins - 2));     // sub-bins 0 .. 126
                            }
                        }
                    };
                    if (live >= 32) batch(std::true_type{}); else batch(std::false_type{});
                }
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(tempty_bar(g));
            }

            // ---- sweep boundary: the 256 epilogue threads meet (also after a give-up) --------------------------------
            if (sweep == 0) {
                xch[(g * kBM + m) * 2] = mn;
                xch[(g * kBM + m) * 2 + 1] = mx;
                tc::named_barrier(kEpiBarrier, 256);
                mn = fminf(xch[m * 2], xch[(kBM + m) * 2]);
                mx = fmaxf(xch[m * 2 + 1], xch[(kBM + m) * 2 + 1]);
                // flat: the scores are all (nearly) equal or not finite - such a row passes everything.  The test also keeps
                // |min * sc1| below 2^22, which bounds the rounding of K1 by one bin in all
                flat = !(mx - mn > 3e-5f * fmaxf(fabsf(mn), fabsf(mx))) || !(mx - mn < INFINITY);
                if (!flat) {
                    // (x - min) * sc1 lies in [0, 120]; with the 4 the bin stays inside [2, 126] however K1 was rounded
                    sc1 = 120.f / (mx - mn);
                    K1 = fmaf(-mn, sc1, 4.f) + 8388608.f;
                    kp1 = K1 - 8388608.f;
                }
                tc::named_barrier(kEpiBarrier, 256);
            } else {
                tc::named_barrier(kEpiBarrier, 256);         // the row's histogram is complete
                int bin = 0, inside = 0;
                bool found = false;
                if (g == 0) found = scan_from_top(sweep == 1 ? kBins - 1 : kBins - 2, sweep == 1 ? rank : r1, bin, inside);
                tc::named_barrier(kEpiBarrier, 256);         // everybody has read the histogram
                if (sweep == 1) {
                    if (g == 0) { reinterpret_cast<int *>(xch)[m * 2] = bin; reinterpret_cast<int *>(xch)[m * 2 + 1] = inside; }
                    tc::named_barrier(kEpiBarrier, 256);
                    b1 = reinterpret_cast<int *>(xch)[m * 2];
                    r1 = reinterpret_cast<int *>(xch)[m * 2 + 1];
                    if (!flat) {
                        // sub-bins of 1/128 of a bin, counted from where bin b1 starts.  Sub-bin 127 and above may already
                        // belong to bin b1 + 1, whose scores have been counted: only 0 .. 126 are taken, and a score of bin
                        // b1 that falls outside them just goes uncounted, which can only lower tau.  When the row's scores
                        // are so close together that the offset of the sub-bins is not exact to a fraction of one
                        // (|lo2 * sc2| > 2^19), the refinement is left out (nothing is counted: K2 below 2^23).
                        const float lo2 = (float(b1) - 0.5f - kp1) / sc1;
                        sc2 = sc1 * float(kBins);
                        fine = fabsf(lo2 * sc2) < 524288.f;
                        K2 = fine ? fmaf(-lo2, sc2, 8388608.f) : 8388000.f;
                        kp2 = K2 - 8388608.f;
                        if (!fine) sc2 = 0.f;
                    }
                    tc::named_barrier(kEpiBarrier, 256);
                } else if (g == 0 && row_ok && ok) {
                    // sub-bin s starts at (s - 0.5 - kp2) / sc2; tau lies one sub-bin below (the arithmetic here is not the
                    // kernel's bin arithmetic to the last bit).  Fewer than r1 scores in the sub-bins: below sub-bin 0.
                    float tau = fine ? (float(found ? bin : 0) - 1.5f - kp2) / sc2
                                     : (float(b1) - 1.5f - kp1) / sc1;                 // coarse: one bin below bin b1
                    if (flat) tau = mn < INFINITY && mn > -INFINITY ? mn : -INFINITY;
                    if (rank > sg.n_keys) tau = -INFINITY;   // a sample smaller than the rank: everything passes
                    p.tau[grow] = tau;
                }
            }
            if (sweep < 2) {
                // clear the row for the next sweep: each of the row's two threads takes half of it
                for (int b = g * (kBins / 2); b < (g + 1) * (kBins / 2); ++b) hrow[b * 32] = 0u;
                tc::named_barrier(kEpiBarrier, 256);
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem_base, 512);
}

template <int D>
int launch_tau(const CUtensorMap &tmA, const CUtensorMap &tmK, const TauParams &p, int mtiles, bool bf16, cudaStream_t st)
{
    constexpr size_t smem = size_t(D / 64) * (kBM * 128 + kStages * kBN * 128) + kHistBytes + 1024;
    FM_CUDA_OK(func_attr_cached((const void *)tc_tau_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    TauParams q = p;
    TcParams hooks = {};
    tc_apply_test_hooks(hooks);
    q.wait_limit_ns = hooks.wait_limit_ns;
    tc_tau_kernel<D><<<mtiles, kThreads, smem, st>>>(tmA, tmK, q, tc::instr_desc_f16(bf16, kBM, kBN));
    FM_LAUNCHED("tc_tau_kernel");
    return FM_OK;
}

}  // namespace

int tc_tau_launch(const CUtensorMap &tmA, const CUtensorMap &tmK, const TauParams &p, int mtiles, int d, bool bf16, cudaStream_t st)
{
    if (d == 128) return launch_tau<128>(tmA, tmK, p, mtiles, bf16, st);
    if (d == 64) return launch_tau<64>(tmA, tmK, p, mtiles, bf16, st);
    set_error("tensor-core thresholds support head dim 64 and 128, got %d", d);
    return FM_ERR_UNSUPPORTED;
}

}  // namespace fm
