"""GPU parity of the hashed-attention path (through the C ABI) against the CPU oracle and the golden vectors."""
import math
import os

import numpy as np
import pytest
import torch

import fast_memory_b200 as fm
from oracle import oracle as O
from tests.util import TOL_LSE, TOL_O, assert_attn_close, random_case

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def _run_dropin(q, k, v, kh, cnt, qh, sm, **kw):
    return fm.attention_hash_varlen(q.to(DEV), k.to(DEV), v.to(DEV), kh.to(DEV), cnt.to(DEV), qh.to(DEV), sm, **kw)


@pytest.mark.parametrize("name", ["attn_f32_tiny", "attn_f32_ragged", "attn_f16_ragged", "attn_f32_d128",
                                  "attn_f32_empty_buckets"])
def test_matches_reference_golden(golden_dir, name):
    """Outputs of the reference's own kernel (tk:51-272) on the same inputs."""
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    dt = DT[str(z["dtype"])]
    t = lambda a: torch.from_numpy(np.asarray(a))
    q, k, v = t(z["q"]).to(dt), t(z["k"]).to(dt), t(z["v"]).to(dt)
    o, lse = _run_dropin(q, k, v, t(z["k_hashes"]), t(z["k_hash_counts"]), t(z["q_hashes"]), float(z["sm_scale"]))
    assert o.dtype == dt and lse.dtype == dt                         # reference returns LSE in q's dtype
    tol_o = 1e-4 if dt == torch.float32 else 2e-2
    assert (o.float().cpu() - t(z["o"])).abs().max() <= tol_o
    ref_lse = t(z["lse"])
    fin = ref_lse > torch.finfo(dt).min
    assert torch.equal(lse.float().cpu()[~fin], ref_lse[~fin])       # empty bucket -> finfo.min (tk:114-117)
    tol_l = 1e-3 if dt == torch.float32 else 8e-3                    # fp16 LSE carries its own rounding (tk:111)
    assert (lse.float().cpu()[fin] - ref_lse[fin]).abs().max() <= tol_l


@pytest.mark.parametrize("name", ["attn_bf16_ragged", "attn_bf16_d128", "attn_f16_native_d64"])
def test_matches_native_reference_golden(golden_dir, name):
    """Outputs of the reference's kernel compiled natively on a B200 (bf16 / fp16): O within 2e-2, the fp32 LSE the
    kernel wrote within 1e-3, the wrapper's rounded LSE within one ulp of the LSE's dtype."""
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    dt = DT[str(z["dtype"])]
    t = lambda a: torch.from_numpy(np.asarray(a))
    q, k, v = t(z["q"]).to(dt), t(z["k"]).to(dt), t(z["v"]).to(dt)
    args = (q, k, v, t(z["k_hashes"]), t(z["k_hash_counts"]), t(z["q_hashes"]), float(z["sm_scale"]))
    o, lse = _run_dropin(*args, return_fp32_lse=True)
    assert_attn_close(o, lse, t(z["o"]), t(z["lse_f32"]), dt)
    o2, lse2 = _run_dropin(*args)
    assert lse2.dtype == dt
    ref = t(z["lse"])
    fin = ref > torch.finfo(dt).min
    assert torch.equal(lse2.float().cpu()[~fin], ref[~fin])
    ulp = 2.0 ** (-7 if dt == torch.bfloat16 else -10)
    assert ((lse2.float().cpu()[fin] - ref[fin]).abs() <= ulp * ref[fin].abs().clamp_min(1.0)).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [16, 32, 64, 128, 256])
def test_random_ragged_vs_oracle(dtype, d):
    B, S, N, C, Z = 2, 150, 700, 12, 90
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=100 + d)
    o, lse = _run_dropin(q, k, v, kh, cnt, qh, d ** -0.5, return_fp32_lse=True)
    o_ref, lse_ref = O.hashed_attention(q, k, v, kh, cnt, qh, d ** -0.5)
    assert_attn_close(o, lse, o_ref, lse_ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reference_self_test_shape(dtype):
    """The reference's own large correctness shape, cut to 2 heads (tk:502): S=4*2040, N=61380, C=512, Z=1024, d=128."""
    B, S, N, C, Z, d = 2, 4 * 2040, 1023 * 60, 512, 1024, 128
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=20)
    o, lse = _run_dropin(q, k, v, kh, cnt, qh, d ** -0.5, return_fp32_lse=True)
    # oracle on a sample of queries (the full dense check is minutes of CPU)
    g = torch.Generator().manual_seed(1)
    pick = torch.randperm(S, generator=g)[:96]
    for b in range(B):
        o_ref, lse_ref = O.hashed_attention(q[b:b + 1, pick], k[b:b + 1], v[b:b + 1],
                                            kh[cnt[:b].sum():cnt[:b + 1].sum()], cnt[b:b + 1], qh[b:b + 1, pick], d ** -0.5)
        assert_attn_close(o[b:b + 1, pick], lse[b:b + 1, pick], o_ref, lse_ref, dtype)


@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 128), (torch.float16, 64)])
def test_many_groups_items_of_two_row_tiles(dtype, d):
    """More than 24 (bucket, queries) groups per SM: the tensor-core kernel then takes 17 to 32 queries of a bucket as
    one work item whose key tiles are shared by warp pairs.  8 heads x 512 buckets, ~24 queries per bucket, ragged
    bucket lengths (last tile partial)."""
    B, S, N, C, Z = 8, 512 * 24, 2048, 512, 203
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=31 + d)
    o, lse = _run_dropin(q, k, v, kh, cnt, qh, d ** -0.5, return_fp32_lse=True)
    g = torch.Generator().manual_seed(2)
    pick = torch.randperm(S, generator=g)[:64]
    for b in range(B):
        o_ref, lse_ref = O.hashed_attention(q[b:b + 1, pick], k[b:b + 1], v[b:b + 1],
                                            kh[cnt[:b].sum():cnt[:b + 1].sum()], cnt[b:b + 1], qh[b:b + 1, pick], d ** -0.5)
        assert_attn_close(o[b:b + 1, pick], lse[b:b + 1, pick], o_ref, lse_ref, dtype)


def test_many_groups_two_row_tile_items_with_split_buckets():
    """The 17-32 query items together with buckets cut into key chunks (partials folded by the combine kernel)."""
    B, S, N, C, Z, d, dtype = 1, 4096 * 24, 2048, 4096, 203, 128, torch.bfloat16
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=77)
    dev = lambda t: t.to(DEV)
    bucket_off = torch.zeros(B * C + 1, dtype=torch.int64)
    bucket_off[1:] = torch.cumsum(cnt.reshape(-1), 0)
    group_off, perm = fm.group_rows(dev(qh.reshape(-1).int()), B * C)
    o, lse = fm.hashed_attention(dev(q[0]), dev(k[0]), dev(v[0]), dev(kh), dev(bucket_off), group_off, perm,
                                 d ** -0.5, int(cnt.max()), key_chunk=64)
    o_whole, lse_whole = fm.hashed_attention(dev(q[0]), dev(k[0]), dev(v[0]), dev(kh), dev(bucket_off), group_off, perm,
                                             d ** -0.5, int(cnt.max()))
    assert (o.float() - o_whole.float()).abs().max() <= 2e-2 and (lse - lse_whole).abs().max() <= 1e-3
    pick = torch.randperm(S, generator=torch.Generator().manual_seed(3))[:128]
    o_ref, lse_ref = O.hashed_attention(q[:, pick], k, v, kh, cnt, qh[:, pick], d ** -0.5)
    assert_attn_close(o[None, pick], lse[None, pick], o_ref, lse_ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key_chunk", [64, 128, 1000])
def test_split_buckets_match_unsplit(dtype, key_chunk):
    """Few queries, long buckets: buckets are cut into key chunks and the partials combined."""
    B, S, N, C, Z, d = 1, 9, 3000, 4, 1000, 64
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=7)
    dev = lambda t: t.to(DEV)
    bucket_off = torch.zeros(B * C + 1, dtype=torch.int64)
    bucket_off[1:] = torch.cumsum(cnt.reshape(-1), 0)
    group_off, perm = fm.group_rows(dev(qh.reshape(-1).int()), B * C)
    o, lse = fm.hashed_attention(dev(q[0]), dev(k[0]), dev(v[0]), dev(kh), dev(bucket_off), group_off, perm,
                                 d ** -0.5, int(cnt.max()), key_chunk=key_chunk)
    o_ref, lse_ref = O.hashed_attention(q, k, v, kh, cnt, qh, d ** -0.5)
    assert_attn_close(o[None], lse[None], o_ref, lse_ref, dtype)


def test_edge_cases():
    d = 32
    # one query, one key; a bucket with no key; a query block boundary (17 queries in one bucket); int32 table
    q, k, v, kh, cnt, qh = random_case(1, 17, 64, 3, 5, d, torch.float32, seed=3)
    qh[:] = 1
    o, lse = _run_dropin(q, k, v, kh.int(), cnt, qh, 0.3, return_fp32_lse=True)
    o_ref, lse_ref = O.hashed_attention(q, k, v, kh, cnt, qh, 0.3)
    assert_attn_close(o, lse, o_ref, lse_ref, torch.float32)
    cnt0 = cnt.clone()
    cnt0[0, 1] = 0                                                   # the queried bucket becomes empty
    kh0 = torch.cat([kh[:cnt[0, 0]], kh[cnt[0, :2].sum():]])
    o, lse = _run_dropin(q, k, v, kh0, cnt0, qh, 0.3, return_fp32_lse=True)
    assert (o == 0).all() and torch.isinf(lse).all() and (lse < 0).all()
    o, lse = _run_dropin(q, k, v, kh0, cnt0, qh, 0.3)               # drop-in form: finfo.min (tk:114-117)
    assert (lse == torch.finfo(torch.float32).min).all()
    # no queries at all
    o, lse = _run_dropin(q[:, :0], k, v, kh, cnt, qh[:, :0], 0.3)
    assert o.shape == (1, 0, d) and lse.shape == (1, 0)


def test_deterministic():
    q, k, v, kh, cnt, qh = random_case(2, 300, 2000, 16, 300, 128, torch.bfloat16, seed=5)
    a = _run_dropin(q, k, v, kh, cnt, qh, 0.1, return_fp32_lse=True)
    for _ in range(20):                 # ~19 queries per bucket: items of 16 and of a few queries, split buckets
        b = _run_dropin(q, k, v, kh, cnt, qh, 0.1, return_fp32_lse=True)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])      # every query is computed by exactly one item


def test_ring_attention_masked_forward_matches_reference_dense(golden_dir):
    """mem:106-163 drop-in against the reference's dense statement (mem:74-103) on two key shards + merge."""
    z = np.load(os.path.join(golden_dir, "dense_ref_two_shards.npz"))
    t = lambda a: torch.from_numpy(np.asarray(a)).to(DEV)
    q, k, v = t(z["q"]), t(z["k"]), t(z["v"])
    out, lse = None, None
    for r in range(k.shape[0]):
        bo, bl = fm.ring_attention_masked_forward(t(z["k_hashes"]), t(z["q_hashes"]), q, k[r], v[r], float(z["sm_scale"]), r)
        assert (bo.cpu() - torch.from_numpy(z[f"out_rank{r}"])).abs().max() <= 1e-4
        out, lse = fm.update_out_and_lse(out, lse, bo, bl)
    assert (out.cpu() - torch.from_numpy(z["out_merged"])).abs().max() <= 1e-4
    assert (lse.cpu() - torch.from_numpy(z["lse_merged"])).abs().max() <= 1e-3


def test_shard_filter_matches_reference_statement():
    """mem:128-142: range mask, per-row counts, compaction in slot order, rebase."""
    g = torch.Generator().manual_seed(12)
    C, H, Z, ctx, W = 37, 3, 70, 500, 4
    k_hashes = torch.topk(torch.rand(C, H, W * ctx, generator=g), dim=-1, k=Z)[1]
    for rank in (0, 2, 3):
        flat, counts = fm.shard_filter(k_hashes.to(DEV), rank * ctx, (rank + 1) * ctx)
        ref_flat, ref_counts = O.shard_filter(k_hashes, rank, ctx)
        assert torch.equal(counts.cpu(), ref_counts)
        assert torch.equal(flat.cpu()[:ref_flat.numel()], ref_flat)
    flat, counts = fm.shard_filter(k_hashes.to(DEV), 10 ** 9, 10 ** 9 + 5)      # nothing in range
    assert int(counts.sum()) == 0


def test_merge_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "merge_chain.npz"))
    out, lse = None, None
    for i in range(3):
        bo = torch.from_numpy(z[f"block_out{i}"]).to(DEV)
        if i == 1:
            bo = bo.to(torch.bfloat16)
        out, lse = fm.update_out_and_lse(out, lse, bo, torch.from_numpy(z[f"block_lse{i}"]).to(DEV))
        assert (out.cpu() - torch.from_numpy(z[f"out{i}"])).abs().max() <= 2e-6
        assert (lse.cpu() - torch.from_numpy(z[f"lse{i}"])).abs().max() <= 2e-6


def test_merge_handles_empty_sides():
    o1 = torch.randn(6, 16, device=DEV)
    o2 = torch.randn(6, 16, device=DEV).bfloat16()
    l1 = torch.tensor([0.5, -math.inf, 1.0, -math.inf, 3.0, -2.0], device=DEV)
    l2 = torch.tensor([-math.inf, 0.25, 2.0, -math.inf, -1.0, -2.0], device=DEV)
    out, lse = fm.merge(o1, l1, o2, l2)
    ro, rl = O.merge_exact(o1.cpu(), l1.cpu(), o2.cpu(), l2.cpu())
    keep = torch.isfinite(rl)
    assert torch.allclose(out.cpu()[keep], ro[keep], atol=1e-6)
    assert torch.equal(torch.isinf(lse.cpu()), torch.isinf(rl)) and torch.allclose(lse.cpu()[keep], rl[keep], atol=1e-6)
    assert torch.equal(o1, o1) and out.data_ptr() != o1.data_ptr()      # merge() leaves its inputs alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_merge_out_of_place_equals_in_place(dtype):
    g = torch.Generator().manual_seed(4)
    rows, d = 1000, 128
    a = torch.randn(rows, d, generator=g).to(DEV)
    al = (torch.randn(rows, generator=g) * 3).to(DEV)
    b = torch.randn(rows, d, generator=g).to(dtype).to(DEV)
    bl = (torch.randn(rows, generator=g) * 3).to(DEV)
    al[::7] = -math.inf
    bl[::5] = -math.inf
    ref_o, ref_l = a.clone(), al.clone()
    fm.lse_merge(ref_o, ref_l, b, bl)
    o, l = fm.lse_merge_out(a, al, b, bl)
    assert torch.equal(o, ref_o) and torch.equal(l, ref_l)
    o2, l2 = fm.lse_merge_out(a, al, b, bl, out_dtype=dtype)
    assert o2.dtype == dtype and torch.equal(o2, ref_o.to(dtype)) and torch.equal(l2, ref_l)



def test_backward_matches_reference_golden(golden_dir):
    """Outputs of the reference's own backward (mem:166-206) per key shard, through the drop-in's pieces: shard filter,
    grouping, fm_hashed_attn_bwd."""
    z = np.load(os.path.join(golden_dir, "backward_two_shards.npz"))
    t = lambda a: torch.from_numpy(np.asarray(a)).to(DEV)
    q, d_out, out, lse = t(z["q"])[0], t(z["d_out"])[0], t(z["out"])[0], t(z["lse"])[0]
    k_hashes, q_hashes = t(z["k_hashes"]), t(z["q_hashes"])
    k_heads, G, S = q_hashes.shape
    C, d = k_hashes.shape[0], q.shape[-1]
    qf = q.reshape(k_heads * G * S, d).contiguous()
    hashes = (q_hashes.reshape(k_heads, G * S) + torch.arange(k_heads, device=DEV)[:, None] * C).reshape(-1).int()
    group_off, perm = fm.group_rows(hashes, k_heads * C)
    for r in range(z["k"].shape[0]):
        k, v = t(z["k"])[r, 0].contiguous(), t(z["v"])[r, 0].contiguous()
        ctx = k.shape[1]
        flat, counts = fm.shard_filter(k_hashes, r * ctx, (r + 1) * ctx)
        bucket_off = torch.zeros(k_heads * C + 1, dtype=torch.int64, device=DEV)
        bucket_off[1:] = torch.cumsum(counts.reshape(-1), 0)
        kbase = (torch.arange(k_heads, device=DEV, dtype=torch.int32) * ctx).repeat_interleave(C)
        dq, dk, dv = fm.hashed_attention_backward(qf, k.reshape(-1, d), v.reshape(-1, d), flat, bucket_off, group_off, perm,
                                                  float(z["sm_scale"]), out.reshape(-1, d).contiguous(), lse.reshape(-1).contiguous(),
                                                  d_out.reshape(-1, d).contiguous(), bucket_kbase=kbase)
        assert (dq.reshape(q.shape).cpu() - torch.from_numpy(z[f"dq_rank{r}"])[0]).abs().max() <= 2e-5
        assert (dk.reshape(k.shape).cpu() - torch.from_numpy(z[f"dk_rank{r}"])[0]).abs().max() <= 2e-5
        assert (dv.reshape(v.shape).cpu() - torch.from_numpy(z[f"dv_rank{r}"])[0]).abs().max() <= 2e-5


@pytest.mark.parametrize("dtype,d,tol", [(torch.float32, 64, 2e-4), (torch.float32, 256, 2e-4), (torch.bfloat16, 128, 4e-2),
                                         (torch.float16, 32, 1e-2),
                                         # the tensor-core kernel's other three instantiations (16-bit, d = 64 / 128)
                                         (torch.bfloat16, 64, 4e-2), (torch.float16, 128, 1e-2), (torch.float16, 64, 1e-2)])
def test_memory_query_backward_vs_oracle(dtype, d, tol):
    """Memory.query + Memory.query_backward against the dense restatement: ragged query blocks (17 and more queries in
    a bucket), buckets nobody asks for, keys that sit in several buckets, accumulation into given dk / dv."""
    g = torch.Generator().manual_seed(d)
    H, N, S, C, Z = 2, 700, 90, 6, 150
    k = (torch.randn(H, N, d, generator=g) * 0.5).to(dtype)
    v = (torch.randn(H, N, d, generator=g) * 0.5).to(dtype)
    q = (torch.randn(H, S, d, generator=g) * 0.5).to(dtype)
    d_out = torch.randn(H, S, d, generator=g).to(dtype)
    A = torch.nn.functional.normalize(torch.randn(H, C, d, generator=g), dim=-1).to(dtype)
    mem = fm.Memory.build(k.to(DEV), v.to(DEV), A=A.to(DEV), bucket_size=Z)
    sm = d ** -0.5
    o, lse = mem.query(q.to(DEV), sm)
    dq, dk, dv = mem.query_backward(q.to(DEV), sm, o, lse, d_out.to(DEV))
    table = torch.stack([mem.table_of(h).long().cpu() for h in range(H)])
    counts = torch.full((H, C), table.shape[-1])
    hashes = mem.hash_queries(q.to(DEV)).long().cpu()
    rq, rk, rv = O.hashed_attention_backward_dense(q, k, v, table, counts, hashes, sm, o.cpu(), lse.cpu(), d_out)
    scale = lambda x: max(1.0, float(x.abs().max()))
    assert (dq.cpu().double() - rq).abs().max() <= tol * scale(rq)
    assert (dk.cpu().double() - rk).abs().max() <= tol * scale(rk)
    assert (dv.cpu().double() - rv).abs().max() <= tol * scale(rv)
    # accumulation: a second call into the same buffers doubles them
    dq2, dk2, dv2 = mem.query_backward(q.to(DEV), sm, o, lse, d_out.to(DEV), dk=dk.clone(), dv=dv.clone())
    assert torch.allclose(dk2, 2 * dk, rtol=1e-4, atol=1e-5) and torch.allclose(dv2, 2 * dv, rtol=1e-4, atol=1e-5)
    assert torch.allclose(dq2, dq, rtol=1e-5, atol=1e-6)
