"""Pins the CPU oracle to vectors produced by the reference's own code (tests/golden/make_golden.py)."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
ATTN_CASES = ["attn_f32_tiny", "attn_f32_ragged", "attn_f16_ragged", "attn_f32_d128", "attn_f32_empty_buckets"]


def load_attn(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    dt = DT[str(z["dtype"])]
    t = lambda a: torch.from_numpy(np.asarray(a))
    return dict(q=t(z["q"]).to(dt), k=t(z["k"]).to(dt), v=t(z["v"]).to(dt), q_hashes=t(z["q_hashes"]),
                k_hashes=t(z["k_hashes"]), k_hash_counts=t(z["k_hash_counts"]), sm_scale=float(z["sm_scale"]),
                o=t(z["o"]), lse=t(z["lse"]), dtype=dt)


@pytest.mark.parametrize("name", ATTN_CASES)
def test_gathered_oracle_matches_reference_kernel(golden_dir, name):
    c = load_attn(golden_dir, name)
    o, lse = O.hashed_attention(c["q"], c["k"], c["v"], c["k_hashes"], c["k_hash_counts"], c["q_hashes"],
                                c["sm_scale"])
    tol_o = 2e-6 if c["dtype"] == torch.float32 else 1e-3
    assert torch.allclose(o.float(), c["o"], atol=tol_o, rtol=0)
    # the reference returns LSE in q's dtype after nan_to_num (tk:111-117)
    ref_like = O.dropin_lse(lse, c["dtype"]).float()
    tol_l = 5e-6 if c["dtype"] == torch.float32 else 4e-3
    assert torch.allclose(ref_like, c["lse"], atol=tol_l, rtol=0)


NATIVE_CASES = ["attn_bf16_ragged", "attn_bf16_d128", "attn_f16_native_d64"]


@pytest.mark.parametrize("name", NATIVE_CASES)
def test_gathered_oracle_matches_native_reference_kernel(golden_dir, name):
    """Vectors of the reference's wrapper + Triton kernel compiled natively on a B200 (``make_golden.py --native-bf16``):
    the only way to get the reference's bf16 results.  O within one bf16 / fp16 ulp of values below 0.25, the fp32 LSE
    as the kernel wrote it within 5e-6, empty buckets as o = 0 / -inf, and the wrapper's rounded LSE (tk:111) exactly."""
    c = load_attn(golden_dir, name)
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    lse_f32 = torch.from_numpy(z["lse_f32"])
    o, lse = O.hashed_attention(c["q"], c["k"], c["v"], c["k_hashes"], c["k_hash_counts"], c["q_hashes"], c["sm_scale"])
    ulp = 2.0 ** -11 if c["dtype"] == torch.bfloat16 else 2.0 ** -14
    assert (o.float() - c["o"]).abs().max() <= ulp
    fin = torch.isfinite(lse_f32)
    assert (~fin).any() and torch.equal(torch.isfinite(lse), fin)
    assert (c["o"][~fin] == 0).all() and (o[~fin] == 0).all()
    assert (lse[fin] - lse_f32[fin]).abs().max() <= 5e-6
    assert torch.equal(O.dropin_lse(lse, c["dtype"]).float(), c["lse"])


@pytest.mark.parametrize("name", ["attn_f32_tiny", "attn_f32_ragged", "attn_f32_d128", "attn_f32_empty_buckets"])
def test_dense_oracle_matches_reference_kernel(golden_dir, name):
    c = load_attn(golden_dir, name)
    B, C = c["k_hash_counts"].shape
    Z = int(c["k_hash_counts"].max())
    table = torch.zeros(B, C, max(Z, 1), dtype=torch.int64)
    off = 0
    for b in range(B):
        for cc in range(C):
            n = int(c["k_hash_counts"][b, cc])
            table[b, cc, :n] = c["k_hashes"][off:off + n]
            off += n
    o, lse = O.hashed_attention_dense(c["q"], c["k"], c["v"], table, c["k_hash_counts"], c["q_hashes"],
                                      c["sm_scale"])
    assert torch.allclose(o, c["o"], atol=2e-6, rtol=0)
    assert torch.allclose(O.dropin_lse(lse, torch.float32), c["lse"], atol=5e-6, rtol=0)


def test_empty_bucket_semantics(golden_dir):
    """Queries whose bucket holds no key: O = 0, LSE = finfo.min after nan_to_num (tk:114-117)."""
    c = load_attn(golden_dir, "attn_f32_empty_buckets")
    B, C = c["k_hash_counts"].shape
    cnt_of_q = c["k_hash_counts"][torch.arange(B)[:, None], c["q_hashes"]]
    empty = cnt_of_q == 0
    assert empty.any() and (~empty).any()
    assert (c["o"][empty] == 0).all()
    assert (c["lse"][empty] == torch.finfo(torch.float32).min).all()
    o, lse = O.hashed_attention(c["q"], c["k"], c["v"], c["k_hashes"], c["k_hash_counts"], c["q_hashes"],
                                c["sm_scale"])
    assert (o[empty] == 0).all() and torch.isinf(lse[empty]).all()


def test_merge_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "merge_chain.npz"))
    out, lse = None, None
    for i in range(3):
        bo = torch.from_numpy(z[f"block_out{i}"])
        if i == 1:
            bo = bo.to(torch.bfloat16)
        out, lse = O.update_out_and_lse(out, lse, bo, torch.from_numpy(z[f"block_lse{i}"]))
        assert torch.allclose(out, torch.from_numpy(z[f"out{i}"]), atol=1e-6, rtol=0)
        assert torch.allclose(lse, torch.from_numpy(z[f"lse{i}"]), atol=1e-6, rtol=0)
    # the fp64 statement used for -inf handling agrees with it on finite inputs
    o2, l2 = O.merge_exact(torch.from_numpy(z["out1"]), torch.from_numpy(z["lse1"]).squeeze(-1),
                           torch.from_numpy(z["block_out2"]), torch.from_numpy(z["block_lse2"]))
    assert torch.allclose(o2, torch.from_numpy(z["out2"]), atol=2e-6, rtol=0)
    assert torch.allclose(l2, torch.from_numpy(z["lse2"]).squeeze(-1), atol=2e-6, rtol=0)


def test_shard_filter_and_merge_match_reference_dense(golden_dir):
    """mem:74-103 per key shard + mem:54-71 merge == shard_filter (mem:128-142) + gathered oracle + merge."""
    z = np.load(os.path.join(golden_dir, "dense_ref_two_shards.npz"))
    q = torch.from_numpy(z["q"])
    k, v = torch.from_numpy(z["k"]), torch.from_numpy(z["v"])
    k_hashes, q_hashes = torch.from_numpy(z["k_hashes"]), torch.from_numpy(z["q_hashes"])
    sm = float(z["sm_scale"])
    W, _, k_heads, ctx, d = k.shape
    out, lse = None, None
    for r in range(W):
        flat, counts = O.shard_filter(k_hashes, r, ctx)
        qq = q.reshape(k_heads, -1, d)                                   # GQA folded (mem:134)
        o, l = O.hashed_attention(qq, k[r, 0], v[r, 0], flat, counts, q_hashes.reshape(k_heads, -1), sm)
        o = o.reshape(q.shape)
        l = l.reshape(q.shape[:-1])
        ref_o, ref_l = torch.from_numpy(z[f"out_rank{r}"]), torch.from_numpy(z[f"lse_rank{r}"])
        assert torch.allclose(o, ref_o, atol=2e-6, rtol=0)
        # the dense reference reports finfo.min-ish LSE for rows with no key in the shard; compare finite rows
        fin = torch.isfinite(l)
        assert torch.allclose(l[fin], ref_l[fin], atol=5e-6, rtol=0)
        out, lse = O.update_out_and_lse(out, lse, o, torch.where(fin, l, ref_l))
    assert torch.allclose(out, torch.from_numpy(z["out_merged"]), atol=2e-6, rtol=0)
    assert torch.allclose(lse, torch.from_numpy(z["lse_merged"]), atol=5e-6, rtol=0)


def test_compute_centroids_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "compute_centroids.npz"))
    out = O.compute_centroids(torch.from_numpy(z["kq"]), torch.from_numpy(z["centroids"]),
                              z["centroids"].shape[0], int(z["n_groups"]), int(z["centroid_topk"]))
    assert torch.allclose(out, torch.from_numpy(z["out"]), atol=1e-6, rtol=0)


def test_canonical_projection_and_topz_self_consistency():
    g = torch.Generator().manual_seed(3)
    A = torch.randn(24, 64, generator=g).bfloat16()
    K = torch.randn(3000, 64, generator=g).bfloat16()
    Y = O.project(A, K)
    assert np.array_equal(Y, O.project_numpy(A, K))                       # two statements, same bits
    assert np.abs(Y - (A.float() @ K.float().T).numpy()).max() < 1e-4     # and it is the same contraction
    for Z in (1, 7, 300, 3000):
        assert np.array_equal(O.topz(Y, Z), O.topz_numpy(Y, Z))
    Yt = np.round(Y)                                                       # massive ties: lower index wins
    assert np.array_equal(O.topz(Yt, 500), O.topz_numpy(Yt, 500))
    h = O.query_hash(A[None], K[None, :200])
    assert np.array_equal(h[0], Y[:, :200].argmax(0))


def test_kmeans_restatement_invariants():
    g = torch.Generator().manual_seed(4)
    cent = torch.nn.functional.normalize(torch.randn(8, 32, generator=g), dim=-1)
    X = (cent[torch.randint(8, (2000,), generator=g)] + 0.2 * torch.randn(2000, 32, generator=g)).bfloat16()
    A = O.spherical_kmeans(X, X[:8], 2)
    assert A.dtype == torch.bfloat16 and A.shape == (8, 32)
    assert torch.allclose(A.float().norm(dim=-1), torch.ones(8), atol=1e-2)
    # the k-means objective (mean cosine to the assigned centroid) does not get worse with iterations
    U = torch.from_numpy(O.unit_rows(X))
    obj = lambda c: float((U @ torch.nn.functional.normalize(c.float(), dim=-1).T).max(-1).values.mean())
    assert obj(A) >= obj(O.spherical_kmeans(X, X[:8], 1)) - 1e-3 >= obj(X[:8]) - 2e-3


def _padded_table(flat, counts):
    """(flat (head, bucket, slot) indices, counts [H, C]) -> table [H, C, max count] padded with 0."""
    H, C = counts.shape
    table = torch.zeros(H, C, max(int(counts.max()), 1), dtype=torch.long)
    pos = 0
    for h in range(H):
        for c in range(C):
            n = int(counts[h, c])
            table[h, c, :n] = flat[pos:pos + n]
            pos += n
    return table


def test_backward_restatement_matches_reference(golden_dir):
    """mem:166-206 run eagerly on two key shards with the merged forward result; GQA folded into the query axis."""
    z = np.load(os.path.join(golden_dir, "backward_two_shards.npz"))
    t = lambda a: torch.from_numpy(np.asarray(a))
    q, d_out, out, lse = t(z["q"])[0], t(z["d_out"])[0], t(z["out"])[0], t(z["lse"])[0]       # [Hq, S, d], [Hq, S]
    k_hashes, q_hashes = t(z["k_hashes"]), t(z["q_hashes"])
    k_heads, G, S = q_hashes.shape
    d = q.shape[-1]
    fold = lambda x: x.reshape(k_heads, G * S, *x.shape[2:])
    for r in range(z["k"].shape[0]):
        k, v = t(z["k"])[r, 0], t(z["v"])[r, 0]
        flat, counts = O.shard_filter(k_hashes, r, k.shape[1])
        dq, dk, dv = O.hashed_attention_backward_dense(fold(q), k, v, _padded_table(flat, counts), counts,
                                                       q_hashes.reshape(k_heads, G * S), float(z["sm_scale"]),
                                                       fold(out), fold(lse), fold(d_out))
        assert torch.allclose(dq.float().reshape(q.shape), t(z[f"dq_rank{r}"])[0], atol=2e-6, rtol=1e-5)
        assert torch.allclose(dk.float(), t(z[f"dk_rank{r}"])[0], atol=2e-6, rtol=1e-5)
        assert torch.allclose(dv.float(), t(z[f"dv_rank{r}"])[0], atol=2e-6, rtol=1e-5)
