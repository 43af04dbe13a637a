/*
 * fastmem_b200 - C ABI of the B200 (sm_100a) LSH attention-memory kernels.
 *
 * Every entry point takes plain pointers and sizes, runs asynchronously on the CUDA stream it is
 * given, writes only into caller-provided buffers and returns FM_OK or a negative status.  Unless a
 * declaration says otherwise nothing is allocated inside: scratch memory is a caller-provided
 * workspace whose size comes from the matching *_workspace_bytes function.
 *
 * Vocabulary.  A memory is made of SEGMENTS (one per KV head, or per (head, sequence) for packed
 * variable-length memories).  Segment s owns key rows [seg_kb[s], seg_kb[s+1]) of the flat K / V
 * arrays [rows, d], buckets [seg_cb[s], seg_cb[s+1]) of the flat bucket space, the matching rows of
 * the packed projection matrix A [total_buckets, d], and query rows [seg_qb[s], seg_qb[s+1]).
 * The bucket table is a flat list of key rows ordered (bucket, slot); bucket b owns
 * table[bucket_off[b] .. bucket_off[b+1]).
 *
 * Each declaration cites the reference interface it stands in for
 * (tk = triton_kernel.py, mem = memory.py of notbadai/fast_memory).
 */
#ifndef FASTMEM_B200_H
#define FASTMEM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FM_ABI_VERSION 1

/* element types of q / k / v / A */
#define FM_F32 0
#define FM_BF16 1
#define FM_F16 2

/* status codes */
#define FM_OK 0
#define FM_ERR_BAD_ARG (-1)       /* null pointer, negative size, misaligned buffer              */
#define FM_ERR_UNSUPPORTED (-2)   /* head dim / dtype / size outside what the kernels were built for */
#define FM_ERR_WORKSPACE (-3)     /* workspace smaller than *_workspace_bytes                     */
#define FM_ERR_CUDA (-4)          /* a CUDA runtime call or launch failed (see fm_last_error)     */
#define FM_ERR_DEVICE (-5)        /* a kernel reported an anomaly through the status word         */

typedef void *fm_stream_t; /* a cudaStream_t */

int fm_abi_version(void);
const char *fm_status_string(int status);
/* Thread-local text describing the last non-OK status returned on this thread. */
const char *fm_last_error(void);
/* Number of kernels this library has launched in the calling process (for launch accounting). */
int64_t fm_launch_count(void);

/* ---------------------------------------------------------------------------------------------
 * Query hashing: hash[r] = argmax_c  A[c, :] . x[r, :]  over the buckets of r's segment, as a LOCAL
 * bucket number; first maximum wins; fp32 sequential-FMA projection.
 * Replaces: einsum + argmax at mem:281-283 and tk:280-281 (README.md:29).
 * x [n_rows, d] and A [total_buckets, d] share `dtype`.  seg_xb / seg_cb: DEVICE int32 prefix
 * arrays of n_seg+1 entries (pass NULL, NULL and n_seg = 1 for one segment covering everything).
 * max_seg_rows: largest number of rows in one segment (sizes the grid).
 * 16-bit inputs with d = 64 or 128 run on the tensor cores as a filter: rows whose two best scores are
 * closer than a bound on the accumulation error are re-decided with the fp32 chain, so the result is
 * the same bits as the all-fp32 path.
 * ------------------------------------------------------------------------------------------- */
size_t fm_hash_rows_workspace_bytes(int64_t n_rows, int n_seg);
int fm_hash_rows(const void *x, const void *A, int dtype, int64_t n_rows, int64_t total_buckets, int d,
                 int n_seg, const int32_t *seg_xb, const int32_t *seg_cb, int64_t max_seg_rows,
                 int32_t *hash_out, void *workspace, size_t workspace_bytes, fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Grouping: counting sort of rows by global bucket (segment bucket base + local hash).
 * Replaces: the stable sort / unique_consecutive / cumsum block of the reference wrapper, tk:75-88.
 * Out: group_off [total_buckets+1] int32 exclusive prefix of rows per bucket; perm [n_rows] int32,
 * perm[group_off[b] .. group_off[b+1]) = the rows hashed to bucket b (order inside a bucket is
 * unspecified; the attention result does not depend on it).
 * ------------------------------------------------------------------------------------------- */
size_t fm_group_rows_workspace_bytes(int64_t n_rows, int64_t total_buckets);
int fm_group_rows(const int32_t *hash, int64_t n_rows, int64_t total_buckets, int n_seg,
                  const int32_t *seg_xb, const int32_t *seg_cb, int32_t *group_off, int32_t *perm,
                  void *workspace, size_t workspace_bytes, fm_stream_t stream);

/* The same result in ONE launch (a CTA per segment: counts, scan and scatter in shared memory) for hashes that are
 * known to lie in [0, buckets of their segment) - the output of fm_hash_rows does.  Then the rows of a segment fill
 * exactly their own stretch of perm and no segment depends on another.  A hash outside its segment's buckets is
 * clamped into them (memory-safe, but not the dropping fm_group_rows does): pass untrusted hashes to fm_group_rows.
 * max_seg_rows / max_seg_buckets: the largest segment (rows, buckets); segments too large for one CTA (more than
 * 32768 rows or 12288 buckets) are handed to fm_group_rows, which is why the workspace is still passed. */
int fm_group_rows_segmented(const int32_t *hash, int64_t n_rows, int64_t total_buckets, int n_seg,
                            const int32_t *seg_xb, const int32_t *seg_cb, int64_t max_seg_rows, int64_t max_seg_buckets,
                            int32_t *group_off, int32_t *perm, void *workspace, size_t workspace_bytes,
                            fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * fm_group_rows for callers that cannot allocate device memory.  This entry point has no counterpart
 * in the reference: it exists for hosts that get their buffers handed to them and may not call
 * cudaMalloc themselves - code running inside a fixed memory plan or arena, a serving process whose
 * memory budget is pinned at start-up, a plugin that runs while the owning framework forbids new
 * allocations.  Inputs and outputs are as for fm_group_rows, but there is no workspace argument:
 * the per-bucket counts and cursors live in an array that is part of the library image
 * (2 x 65536 x 4 bytes = 512 KiB, held by every GPU that loads the library until the process exits).
 *   - total_buckets above fm_group_rows_static_max_buckets() (65536) is refused with
 *     FM_ERR_UNSUPPORTED; use fm_group_rows there.
 *   - Nothing is allocated or freed, here or in any routine it calls.
 *   - The first call on each device looks up the array's device address (a one-time, per-device
 *     set-up inside the call); make that first call before starting any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents (the call
 *     clears what it needs).  Two calls that overlap on the GPU - different streams, or threads -
 *     race on it; serialise them.
 * ------------------------------------------------------------------------------------------- */
int64_t fm_group_rows_static_max_buckets(void);
int fm_group_rows_static(const int32_t *hash, int64_t n_rows, int64_t total_buckets, int n_seg,
                         const int32_t *seg_xb, const int32_t *seg_cb, int32_t *group_off, int32_t *perm,
                         fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Hashed attention forward: every query attends to the keys listed in its bucket.
 * Replaces: torch op notbad::attention_hash_varlen and its Triton kernel, tk:16-41, 135-272 (the
 * gathers through the table, base-2 online softmax, P rounded to the q dtype before P.V), without
 * the q / o permutation copies of tk:77, 109: queries are read and outputs written through `perm`.
 *   q, o      [n_q_rows, d] in `dtype`;  k, v [n_k_rows, d] in `dtype`
 *   table     key rows, int32 (idx_bytes = 4) or int64 (idx_bytes = 8)
 *   bucket_off [total_buckets+1] int64, DEVICE
 *   bucket_kbase [total_buckets] int32 DEVICE or NULL: added to every table entry of the bucket
 *              (lets a table hold per-head indices as the reference's does)
 *   group_off, perm: from fm_group_rows
 *   lse       [n_q_rows] fp32 natural-log LSE; -inf (and o = 0) where the bucket is empty
 *   key_chunk  keys per work item; 0 lets the library choose.  Buckets longer than one chunk are
 *              split over CTAs and combined by a second kernel (needs the workspace).
 *   max_bucket_len  an upper bound of every bucket's length (it sizes the workspace).  The keys of a
 *              longer bucket beyond the bound are left out, and the third int32 of the workspace
 *              reads 1 after the launch.  Query rows that no group of group_off / perm lists are not
 *              written: start o / lse at 0 / -inf if the hashes are not known to be in range.
 *
 * Two tensor-core kernels serve 16-bit inputs with head dim 128: mma.sync (0, the default and the
 * faster of the two on every workload measured) and tcgen05 / TMEM (1).  fm_set_attn_kernel selects
 * one for the process (initial value from the environment variable FASTMEM_ATTN_KERNEL = mma | tc);
 * other shapes are unaffected.  It has no counterpart in the reference (Triton picks its own code).
 * ------------------------------------------------------------------------------------------- */
int fm_set_attn_kernel(int which);
size_t fm_hashed_attn_workspace_bytes(int64_t n_q_rows, int64_t total_buckets, int64_t max_bucket_len, int d,
                                      int64_t key_chunk);
int fm_hashed_attn_fwd(const void *q, const void *k, const void *v, int dtype, int d, int64_t n_q_rows,
                       int64_t n_k_rows, int64_t total_buckets, const void *table, int idx_bytes,
                       const int64_t *bucket_off, const int32_t *bucket_kbase, int64_t max_bucket_len,
                       const int32_t *group_off, const int32_t *perm, float sm_scale, void *o, float *lse,
                       int64_t key_chunk, void *workspace, size_t workspace_bytes, fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Hashed attention backward over the gathered rows: dq = dS K * sm_scale, dk += dS^T Q * sm_scale, dv += P^T dO with
 * P = exp(q.k * sm_scale - lse), dS = P * (dO V^T - rowsum(dO * o)).
 * Replaces: ring_attention_masked_backward, mem:166-206 (dense mask + five einsums), for the key shard described by
 * k, v, table.  q, o, d_o [n_q_rows, d] and k, v [n_k_rows, d] in `dtype`; table / bucket_off / bucket_kbase /
 * group_off / perm as in fm_hashed_attn_fwd; lse [n_q_rows] fp32 natural log: the LSE the forward result was
 * normalised with (it may cover more keys than this shard, e.g. after a merge).  dq [n_q_rows, d] fp32 is written
 * (zero where the bucket is empty); dk, dv [n_k_rows, d] fp32 are ACCUMULATED (a key sits in several buckets and in
 * several calls when shards take turns): the caller zeroes them first.
 * ------------------------------------------------------------------------------------------- */
int fm_hashed_attn_bwd(const void *q, const void *k, const void *v, int dtype, int d, int64_t n_q_rows, int64_t n_k_rows,
                       int64_t total_buckets, const void *table, int idx_bytes, const int64_t *bucket_off,
                       const int32_t *bucket_kbase, const int32_t *group_off, const int32_t *perm, float sm_scale,
                       const void *o, const float *lse, const void *d_o, float *dq, float *dk, float *dv, fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Shard filter of a globally indexed table: for every (head, bucket) row of k_hashes [C, H, Z] (int64
 * GLOBAL key indices) keep the entries in [lo, hi), rebased to the shard (index - lo), slot order kept,
 * packed (head, bucket, slot) into flat_out (room for C*H*Z entries); counts_out [H, C] int64.
 * Replaces: the mask / sum / boolean compaction / rebase of ring_attention_masked_forward, mem:128-142.
 * ------------------------------------------------------------------------------------------- */
size_t fm_shard_filter_workspace_bytes(int64_t C, int64_t H);
int fm_shard_filter(const int64_t *k_hashes, int64_t C, int64_t H, int64_t Z, int64_t lo, int64_t hi,
                    int64_t *flat_out, int64_t *counts_out, void *workspace, size_t workspace_bytes, fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * LSE merge, in place on fp32 accumulators:
 *   lse <- log(e^lse + e^blk_lse);  out <- out - sigmoid(blk_lse - lse) (out - blk_out)
 * Replaces: update_out_and_lse, mem:54-71 (the branch with existing accumulators, mem:67-69).
 * blk_out is in `blk_dtype`; blk_lse in `lse_dtype`.  A side whose LSE is -inf has weight 0.
 * ------------------------------------------------------------------------------------------- */
int fm_lse_merge(float *out, float *lse, const void *blk_out, int blk_dtype, const void *blk_lse, int lse_dtype,
                 int64_t n_rows, int d, fm_stream_t stream);

/* Merge of the partial results of `world` ranks (<= 8) over peer memory, for keys sharded over the ranks:
 * o_ptrs[w] / lse_ptrs[w] address rank w's partial (o [rows, d] in `o_dtype`, lse [rows] fp32) over its own keys for
 * all query rows, out_ptrs[w] / lse_out_ptrs[w] rank w's result buffers (fp32) - all of them addresses THIS GPU can
 * load from / store to (peer mappings of symmetric allocations; the arrays of pointers are host arrays).  The caller
 * owns rows [row0, row1): it pulls them from every rank, merges them (lse = log sum_w e^lse_w, out = the e^lse_w
 * weighted mean) and pushes the finished rows to every rank's result buffers.
 * Replaces: the ring of K / V blocks with its per-step update_out_and_lse, mem:307-338 (the keys stay where they are;
 * what travels is one pull of partial rows and one push of finished rows).  The caller orders the launches of the
 * ranks: all partials complete before, all results complete after (e.g. a small collective on the same stream). */
int fm_merge_peer_partials(const void *const *o_ptrs, const float *const *lse_ptrs, float *const *out_ptrs,
                           float *const *lse_out_ptrs, int world, int o_dtype, int64_t row0, int64_t row1, int d,
                           fm_stream_t stream);

/* The same merge out of place, for a caller that keeps its accumulator (e.g. a local-window result merged with a new
 * memory result per request, mem:332): reads (acc_out fp32, acc_lse fp32) and (blk_out in `blk_dtype`, blk_lse fp32),
 * writes the merged rows to `dst` in `dst_dtype` (FM_F32 or `blk_dtype`) and their LSE to `dst_lse`. */
int fm_lse_merge_out(const float *acc_out, const float *acc_lse, const void *blk_out, int blk_dtype, const float *blk_lse,
                     void *dst, int dst_dtype, float *dst_lse, int64_t n_rows, int d, fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Projection Y[c, j] = A[c, :] . K[j, :] in fp32 (sequential FMA over the head dim), row stride ldy.
 * Replaces: the einsum at mem:261 / tk:277 (README.md:25).  Stand-alone form, for tests and for
 * callers that want the scores themselves.
 * ------------------------------------------------------------------------------------------- */
int fm_project(const void *A, const void *K, int dtype, int64_t C, int64_t N, int d, float *Y, int64_t ldy,
               fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * The same projection on the tcgen05 tensor cores (TMA-fed, accumulators in TMEM) for bf16 / fp16 and
 * d = 64 or 128, optionally over every key_step-th key row: Y[c, j] ~ A[c, :] . K[j * key_step, :]
 * for j < ceil(n_key_rows / key_step).  The summation order is the hardware's, so these scores are
 * approximate (about 1e-6 relative): they drive threshold estimates, never an index decision.
 * Same reference lines as fm_project.  After the stream completes the first int32 of the workspace is
 * a status word (0 = ok).
 * ------------------------------------------------------------------------------------------- */
size_t fm_project_tc_workspace_bytes(int64_t C, int64_t n_key_rows, int64_t key_step);
int fm_project_tc(const void *A, const void *K, int dtype, int64_t C, int64_t n_key_rows, int d, int64_t key_step,
                  float *Y, int64_t ldy, void *workspace, size_t workspace_bytes, fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Exact top-Z of every row of Y [n_rows, N] (row stride ldy): the Z largest values, lower index wins
 * ties, indices written in ascending order plus `index_base`.
 * Replaces: torch.topk at mem:273 / tk:278 (README.md:27).  Z <= N.
 * ------------------------------------------------------------------------------------------- */
int fm_topz_select(const float *Y, int64_t n_rows, int64_t N, int64_t ldy, int64_t Z, int32_t index_base,
                   int32_t *table, int64_t ld_table, fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Index build for a whole memory: for every segment, table rows of its buckets = top-min(Z_s, N_s)
 * keys by projection, as ABSOLUTE key rows in ascending order.
 * Replaces: einsum + topk, mem:261 + 273 and tk:277-278.
 * 16-bit keys with d = 64 / 128 and buckets much smaller than the segment take the fused path: tcgen05
 * projection whose epilogue keeps only scores above a per-bucket threshold (estimated from a key sample),
 * then an exact selection that re-scores near-ties with the fp32 chain - same table bits as the all-fp32
 * path, which every other case (and flags = FM_BUILD_EXACT_ONLY) uses.  After the stream has completed,
 * the first int32 of the workspace is a status word: 0 = ok, non-zero = the fused path gave up (rebuild
 * with FM_BUILD_EXACT_ONLY).
 * seg_kb, seg_cb [n_seg+1] and seg_z [n_seg] are HOST arrays.  Bucket b of segment s is written at
 * table + table_off[s] + (b - seg_cb[s]) * min(seg_z[s], N_s)  (table_off: HOST, n_seg entries).
 * ------------------------------------------------------------------------------------------- */
#define FM_BUILD_EXACT_ONLY 1 /* flags: skip the tensor-core path, score every key with the fp32 chain */
#define FM_BUILD_SINGLE_RANGE 2 /* flags: tensor-core path with ONE key range per bucket tile: a bucket's candidate list is one
                                  buffer whatever the positions of its keys (slower when bucket tiles are fewer than SMs) */
size_t fm_index_build_workspace_bytes(int n_seg, const int64_t *seg_kb, const int64_t *seg_cb, const int64_t *seg_z,
                                      int d, int dtype, int flags);
int fm_index_build(const void *K, const void *A, int dtype, int d, int n_seg, const int64_t *seg_kb,
                   const int64_t *seg_cb, const int64_t *seg_z, const int64_t *table_off, int32_t *table, int flags,
                   void *workspace, size_t workspace_bytes, fm_stream_t stream);

/* scores[e] = A[b, :] . K[table[e], :] (canonical fp32 chain) for every entry e of every bucket b of a table built by
 * fm_index_build (table / bucket_off as produced there, total_buckets rows of A).  With the scores, the tables of
 * several key shards merge into the reference's GLOBAL table (top-Z over all shards' keys, mem:260-278) by one exact
 * row select over the shards' candidates instead of an all_to_all of the score matrix. */
int fm_table_scores(const void *K, const void *A, int dtype, int d, int64_t total_buckets, const int32_t *table,
                    const int64_t *bucket_off, float *scores, fm_stream_t stream);


/* ---------------------------------------------------------------------------------------------
 * Projection matrix by spherical k-means (distance 1 - c.x, README.md:37-45): `iters` rounds of
 * assignment (fm_hash_rows on the raw rows) and centroid update (exact integer sums of the unit rows
 * in units of 2^-40, normalised in fp64).  The reference's code has no k-means (mem:209-231 is a
 * different construction); this follows its README.
 * X [rows, d] in `dtype`; cent_f32 [total_buckets, d] fp32 in/out: initial centroids (unit rows) on
 * entry, final centroids on exit; A_out [total_buckets, d] in `dtype` = the final centroids rounded
 * to the key dtype (the form the index build and the query hash use).  seg_* are HOST arrays.
 * ------------------------------------------------------------------------------------------- */
size_t fm_kmeans_workspace_bytes(int n_seg, const int64_t *seg_xb, const int64_t *seg_cb, int d);
int fm_kmeans(const void *X, int dtype, int d, int n_seg, const int64_t *seg_xb, const int64_t *seg_cb, int iters,
              float *cent_f32, void *A_out, void *workspace, size_t workspace_bytes, fm_stream_t stream);

/* U[r, :] = X[r, :] / max(||X[r, :]||, 1e-6) in fp32 (unit-sphere projection, README.md:39; mem:215-217). */
int fm_unit_rows(const void *X, int dtype, int64_t n_rows, int d, float *U, fm_stream_t stream);

/* out[i, :] = mean over j < per_out of U[rows[i * per_out + j], :] (fp32, summed in list order): the averaging step of
 * the reference's coded centroid construction (gather + mean, mem:222-229).  U [n_rows, d]; rows hold indices in
 * [0, n_rows); out [n_out, d]. */
int fm_gather_mean(const float *U, int64_t n_rows, int d, const int32_t *rows, int64_t n_out, int64_t per_out, float *out,
                   fm_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Test hooks (no counterpart in the reference).  Every wait of the tensor-core projection kernel on a pipeline
 * barrier is bounded (two seconds); when one runs out the CTA records a status, waits for its own copies in flight,
 * frees its TMEM and returns.  fm_test_set_tc_hooks makes that path testable without any fault: wait_limit_ms
 * shortens the bound (0 = the library's), skip_tile makes the producer of every CTA leave out the load of its tile
 * number skip_tile (-1 = none), so that the consumers' waits run out.  Process-wide; reset with (0, -1).
 * ------------------------------------------------------------------------------------------- */
int fm_test_set_tc_hooks(int wait_limit_ms, int skip_tile);

#ifdef __cplusplus
}
#endif
#endif /* FASTMEM_B200_H */
