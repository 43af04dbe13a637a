"""GPU parity of index build, query hashing, k-means and the Memory object against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import fast_memory_b200 as fm
from fast_memory_b200 import ops, synth
from oracle import oracle as O
from tests.util import assert_attn_close, oracle_for_sampled_queries, tables_equal_as_sets

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [16, 64, 128, 256])
def test_projection_is_bit_exact(dtype, d):
    g = torch.Generator().manual_seed(d)
    A = torch.randn(70, d, generator=g).to(dtype)
    K = torch.randn(333, d, generator=g).to(dtype)
    Y = fm.project(A.to(DEV), K.to(DEV)).cpu().numpy()
    assert np.array_equal(Y, O.project(A, K))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("C,N,d,step", [(128, 256, 128, 1), (130, 1000, 128, 1), (512, 5000, 128, 16), (70, 777, 64, 3),
                                        (1024, 40000, 128, 1)])
def test_tensor_core_projection_close_to_canonical(dtype, C, N, d, step):
    """tcgen05 / TMEM / TMA projection: same contraction as the canonical one up to summation order."""
    g = torch.Generator().manual_seed(C + N)
    A = torch.randn(C, d, generator=g).to(dtype)
    K = torch.randn(N, d, generator=g).to(dtype)
    Y = fm.ops.project_tc(A.to(DEV), K.to(DEV), key_step=step).cpu()
    ref = torch.from_numpy(O.project(A, K[::step].contiguous()))
    assert Y.shape == ref.shape
    assert (Y - ref).abs().max() <= 2e-5 * (A.float().norm(dim=-1).max() * K.float().norm(dim=-1).max())


@pytest.mark.parametrize("N,Z", [(1, 1), (100, 100), (1000, 1), (5000, 257), (70000, 2048), (4096, 4095)])
def test_topz_select_is_bit_exact(N, Z):
    g = torch.Generator().manual_seed(N + Z)
    Y = torch.randn(9, N, generator=g)
    got = fm.topz_select(Y.to(DEV), Z).cpu().numpy()
    assert np.array_equal(got, O.topz(Y, Z))
    # heavy ties (values on a coarse grid, signed zeros): lower index wins
    Yt = (torch.round(Y * 2) / 2) * torch.where(torch.rand(9, N, generator=g) < 0.5, -1.0, 1.0)
    got = fm.topz_select(Yt.to(DEV), Z, index_base=7).cpu().numpy()
    assert np.array_equal(got, O.topz(Yt, Z) + 7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_hash_rows_bit_exact_multi_segment(dtype):
    g = torch.Generator().manual_seed(11)
    d = 64
    Cs, Ss = [5, 64, 130], [70, 1, 200]
    A = torch.randn(sum(Cs), d, generator=g).to(dtype)
    X = torch.randn(sum(Ss), d, generator=g).to(dtype)
    xb = torch.tensor([0, 70, 71, 271], dtype=torch.int32)
    cb = torch.tensor([0, 5, 69, 199], dtype=torch.int32)
    h = fm.hash_rows(X.to(DEV), A.to(DEV), xb.to(DEV), cb.to(DEV), max(Ss)).cpu().numpy()
    for s in range(3):
        ref = O.query_hash(A[cb[s]:cb[s + 1]][None], X[xb[s]:xb[s + 1]][None])[0]
        assert np.array_equal(h[xb[s]:xb[s + 1]], ref)
    # duplicated centroids: the first maximum wins
    A2 = torch.cat([A[:5], A[:5]], 0)
    h2 = fm.hash_rows(X[:70].to(DEV), A2.to(DEV)).cpu().numpy()
    assert (h2 < 5).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [64, 128])
def test_hash_rows_near_ties_are_decided_by_the_fp32_chain(dtype, d):
    """Tensor-core filter + exact re-check: centroids that differ by one ulp in one coordinate give score gaps
    far below any accumulation error, and exact ties; the result must still equal the oracle bit for bit."""
    g = torch.Generator().manual_seed(d)
    base = torch.nn.functional.normalize(torch.randn(40, d, generator=g), dim=-1)
    A = base.repeat(8, 1)                                   # 320 buckets: every centroid 8 times ...
    A = A.to(dtype)
    bump = A.view(torch.int16).clone()
    sel = torch.arange(40, 320)
    bump[sel, sel % d] += ((sel // 40) % 3 - 1).to(torch.int16)      # ... some copies off by +-1 ulp in one place
    A = bump.view(dtype)
    X = (base[torch.randint(40, (3000,), generator=g)] + 0.2 * torch.randn(3000, d, generator=g)).to(dtype)
    h = fm.hash_rows(X.to(DEV), A.to(DEV)).cpu().numpy()
    assert np.array_equal(h, O.query_hash(A[None], X[None])[0])


def test_group_rows_is_a_valid_counting_sort():
    g = torch.Generator().manual_seed(2)
    C, n = 37, 5000
    h = torch.randint(C, (n,), generator=g).int()
    off, perm = fm.group_rows(h.to(DEV), C)
    off, perm = off.cpu(), perm.cpu().long()
    assert off[0] == 0 and off[-1] == n and torch.equal(off[1:] - off[:-1], torch.bincount(h.long(), minlength=C).int())
    assert torch.equal(torch.sort(perm).values, torch.arange(n))
    for c in range(C):
        assert (h[perm[off[c]:off[c + 1]]] == c).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kmeans_bit_exact(dtype):
    g = torch.Generator().manual_seed(9)
    d, C, n = 64, 16, 3000
    cent = torch.nn.functional.normalize(torch.randn(C, d, generator=g), dim=-1)
    X = (cent[torch.randint(C, (n,), generator=g)] + 0.3 * torch.randn(n, d, generator=g)).to(dtype)
    for iters in (0, 1, 3):
        A, c32 = fm.kmeans_projection(X.to(DEV), X[:C].to(DEV), iters, [0, n], [0, C])
        ref = O.spherical_kmeans(X, X[:C], iters)
        assert torch.equal(A.cpu(), ref), f"iters={iters}: {(A.cpu().float() - ref.float()).abs().max()}"
    assert np.array_equal(fm.unit_rows(X.to(DEV)).cpu().numpy(), O.unit_rows(X))


def _check_memory_tables(mem, A_cpu, k_cpu, Z):
    for h in range(mem.n_heads):
        ref = O.topz(O.project(A_cpu[h], k_cpu[h]), Z)
        ok, why = tables_equal_as_sets(mem.table_of(h).cpu().numpy(), ref)
        assert ok, f"head {h}: {why}"


def test_cfg1_end_to_end():
    """BASELINE config 1 in full: k-means A, index, hash, attention; every stage against the oracle."""
    cfg = synth.config("cfg1")
    q, k, v = synth.make(cfg, seed=0)
    sm = cfg.d ** -0.5
    mem = fm.Memory.build(k.to(DEV), v.to(DEV), n_buckets=cfg.n_buckets, bucket_size=cfg.bucket_size,
                          kmeans_iters=cfg.kmeans_iters, kmeans_init=q.to(DEV))
    A_ref = O.spherical_kmeans(k[0], q[0, :cfg.n_buckets], cfg.kmeans_iters)
    assert torch.equal(mem.A.cpu(), A_ref)
    _check_memory_tables(mem, A_ref[None], k, cfg.bucket_size)
    hashes = mem.hash_queries(q.to(DEV)).cpu()
    assert np.array_equal(hashes.numpy(), O.query_hash(A_ref[None], q))
    o, lse = mem.query(q.to(DEV), sm)
    table = torch.from_numpy(O.build_table(A_ref[None], k, cfg.bucket_size)).long()
    counts = torch.full((1, cfg.n_buckets), table.shape[-1])
    o_ref, lse_ref = O.hashed_attention_dense(q, k, v, table, counts, hashes.long(), sm)
    assert_attn_close(o, lse, o_ref, lse_ref, torch.float32)
    o_g, lse_g = O.hashed_attention(q, k, v, table.reshape(-1), counts, hashes.long(), sm)
    assert_attn_close(o, lse, o_g, lse_g, torch.float32)


@pytest.mark.parametrize("name,H,N,S", [("cfg2", 2, 16384, 1024), ("cfg3", 2, 32768, 16), ("cfg5", 1, 65536, 512)])
def test_cut_down_configs(name, H, N, S):
    """The bf16 configurations at reduced key counts / heads, same distributions, C and Z scaled with N."""
    cfg = synth.config(name)
    scale = N / (cfg.n_keys // cfg.shards)
    C, Z = max(16, int(cfg.n_buckets * scale ** 0.5) // 16 * 16), max(32, int(cfg.bucket_size * scale))
    q, k, v = synth.make(cfg, seed=3, kv_heads=H, n_keys=N, n_queries=S)
    sm = cfg.d ** -0.5
    mem = fm.Memory.build(k.to(DEV), v.to(DEV), n_buckets=C, bucket_size=Z, kmeans_iters=2)
    A = mem.A.reshape(H, C, cfg.d).cpu()
    for h in range(H):
        assert torch.equal(A[h], O.spherical_kmeans(k[h], k[h, :C], 2))
    _check_memory_tables(mem, A, k, Z)
    qd = q.to(DEV)
    hashes = mem.hash_queries(qd).cpu()
    G = cfg.q_groups
    ref_h = O.query_hash(A, q.reshape(H, G * S, cfg.d)).reshape(H * G, S)
    assert np.array_equal(hashes.numpy(), ref_h)
    o, lse = mem.query(qd, sm)
    table = torch.stack([mem.table_of(h) for h in range(H)]).cpu().long()
    counts = torch.full((H, C), table.shape[-1])
    o_ref, lse_ref = O.hashed_attention(q.reshape(H, G * S, cfg.d), k, v, table.reshape(-1), counts,
                                        hashes.reshape(H, G * S).long(), sm)
    assert_attn_close(o.reshape(H, G * S, -1), lse.reshape(H, G * S), o_ref, lse_ref, cfg.dtype)


@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 128), (torch.float16, 64)])
def test_fused_build_equals_exact_build(dtype, d):
    """Tensor-core filter + exact band re-scoring against the all-fp32 build: same table, bit for bit."""
    g = torch.Generator().manual_seed(77)
    H, N, C, Z = 2, 40000, 160, 512                       # 2 bucket tiles per head, the second one ragged
    cent = torch.nn.functional.normalize(torch.randn(64, d, generator=g), dim=-1)
    k = (cent[torch.randint(64, (H * N,), generator=g)] + 0.25 * torch.randn(H * N, d, generator=g)).reshape(H, N, d).to(dtype)
    v = torch.randn(H, N, d, generator=g).to(dtype)
    A = torch.nn.functional.normalize(torch.randn(H, C, d, generator=g), dim=-1).to(dtype)
    fused = fm.Memory.build(k.to(DEV), v.to(DEV), A=A.to(DEV), bucket_size=Z)
    exact = fm.Memory.build(k.to(DEV), v.to(DEV), A=A.to(DEV), bucket_size=Z, exact_only=True)
    assert torch.equal(fused.table, exact.table)
    ok, why = tables_equal_as_sets(fused.table_of(1).cpu().numpy(), O.topz(O.project(A[1], k[1]), Z))
    assert ok, why


def test_fused_build_with_massive_ties_uses_the_fallback():
    """Every key repeated 64 times: exact ties straddle the Z-th score and are resolved by index inside the
    band.  With 8 distinct keys repeated 4096 times the band is larger than the kernel re-scores in place and
    the buckets are rebuilt by the fallback; lower index must still win."""
    g = torch.Generator().manual_seed(78)
    N, C, Z, d = 32768, 16, 1000, 128
    base = torch.randn(512, d, generator=g).bfloat16()
    k = base.repeat(64, 1)[torch.randperm(N, generator=g)][None].contiguous()
    A = torch.randn(1, C, d, generator=g).bfloat16()
    mem = fm.Memory.build(k.to(DEV), k.to(DEV), A=A.to(DEV), bucket_size=Z)
    ok, why = tables_equal_as_sets(mem.table_of(0).cpu().numpy(), O.topz(O.project(A[0], k[0]), Z))
    assert ok, why
    k = base[:8].repeat(4096, 1)[torch.randperm(N, generator=g)][None].contiguous()
    A = torch.randn(1, C, d, generator=g).bfloat16()
    mem = fm.Memory.build(k.to(DEV), k.to(DEV), A=A.to(DEV), bucket_size=Z)
    ok, why = tables_equal_as_sets(mem.table_of(0).cpu().numpy(), O.topz(O.project(A[0], k[0]), Z))
    assert ok, why
    # with more such buckets than the fallback takes, the build reports it and the exact path still works
    A2 = torch.randn(1, 128, d, generator=g).bfloat16()
    with pytest.raises(fm.FastMemError):
        fm.Memory.build(k.to(DEV), k.to(DEV), A=A2.to(DEV), bucket_size=Z, fallback_exact=False)
    with pytest.warns(RuntimeWarning, match="exact fp32 path"):
        mem2 = fm.Memory.build(k.to(DEV), k.to(DEV), A=A2.to(DEV), bucket_size=Z)        # rebuilds by itself
    ok, why = tables_equal_as_sets(mem2.table_of(0).cpu().numpy(), O.topz(O.project(A2[0], k[0]), Z))
    assert ok, why
    mem2 = fm.Memory.build(k.to(DEV), k.to(DEV), A=A2.to(DEV), bucket_size=Z, exact_only=True)
    ok, why = tables_equal_as_sets(mem2.table_of(0).cpu().numpy(), O.topz(O.project(A2[0], k[0]), Z))
    assert ok, why


def test_fused_build_keys_sorted_by_score():
    """Keys ordered so that one bucket's best keys all sit at the end of the segment (one key range)."""
    g = torch.Generator().manual_seed(79)
    N, C, Z, d = 65536, 128, 1024, 128
    A = torch.nn.functional.normalize(torch.randn(1, C, d, generator=g), dim=-1).bfloat16()
    k = torch.randn(N, d, generator=g).bfloat16()
    order = torch.argsort(k.float() @ A[0, 5].float())            # ascending score for bucket 5
    k = k[order][None].contiguous()
    mem = fm.Memory.build(k.to(DEV), k.to(DEV), A=A.to(DEV), bucket_size=Z)
    ok, why = tables_equal_as_sets(mem.table_of(0).cpu().numpy(), O.topz(O.project(A[0], k[0]), Z))
    assert ok, why


def test_varlen_memory_matches_per_sequence_calls():
    """cfg4 layout cut down: packed keys/queries with cu_seqlens equal independent per-sequence memories."""
    cfg = synth.config("cfg4")
    seq = [3000, 700, 5000]
    H, S = 2, 64
    q, k, v, cu_q, cu_k = synth.make_varlen(cfg, seed=5, kv_heads=H, seq_keys=seq, n_queries=S)
    Cs = [synth.varlen_buckets(n) for n in seq]
    Zs = [synth.varlen_bucket_size(n) for n in seq]
    sm = cfg.d ** -0.5
    mem = fm.Memory.build(k.to(DEV), v.to(DEV), n_buckets=Cs, bucket_size=Zs, kmeans_iters=1, cu_seqlens_k=cu_k)
    o, lse = mem.query(q.to(DEV), sm, cu_seqlens_q=cu_q)
    for s, n in enumerate(seq):
        ks, vs = k[:, cu_k[s]:cu_k[s + 1]].contiguous(), v[:, cu_k[s]:cu_k[s + 1]].contiguous()
        qs = q[:, cu_q[s]:cu_q[s + 1]].contiguous()
        A = torch.stack([O.spherical_kmeans(ks[h], ks[h, :Cs[s]], 1) for h in range(H)])
        for h in range(H):
            assert torch.equal(mem.projection_of(h, s).cpu(), A[h])
            ok, why = tables_equal_as_sets(mem.table_of(h, s).cpu().numpy(), O.topz(O.project(A[h], ks[h]), Zs[s]))
            assert ok, why
        table = torch.from_numpy(O.build_table(A, ks, Zs[s])).long()
        hashes = torch.from_numpy(O.query_hash(A, qs)).long()
        o_ref, lse_ref = O.hashed_attention(qs, ks, vs, table.reshape(-1), torch.full((H, Cs[s]), table.shape[-1]), hashes, sm)
        assert_attn_close(o[:, cu_q[s]:cu_q[s + 1]], lse[:, cu_q[s]:cu_q[s + 1]], o_ref, lse_ref, cfg.dtype)
    # and the same through the single-sequence API of the drop-in
    m0 = fm.Memory.build(k[:, :seq[0]].contiguous().to(DEV), v[:, :seq[0]].contiguous().to(DEV), n_buckets=Cs[0],
                         bucket_size=Zs[0], kmeans_iters=1)
    o0, l0 = m0.query(q[:, :S].contiguous().to(DEV), sm)
    assert torch.equal(o0, o[:, :S]) and torch.equal(l0, lse[:, :S])


def test_attention_hash_dropin_with_key_range():
    """tk:275-286 with its key-range filter as an argument."""
    g = torch.Generator().manual_seed(8)
    B, S, N, C, Z, d = 2, 200, 4096, 16, 256, 64
    q = torch.randn(B, S, d, generator=g).bfloat16()
    k = torch.randn(B, N, d, generator=g).bfloat16()
    v = torch.randn(B, N, d, generator=g).bfloat16()
    cent = torch.randn(B, C, d, generator=g).bfloat16()
    o, lse = fm.attention_hash(q.to(DEV), k.to(DEV), v.to(DEV), cent.to(DEV), Z, 0.1, key_range=(1024, 3072))
    table = torch.from_numpy(O.build_table(cent, k, Z)).long()
    m = (table >= 1024) & (table < 3072)
    hashes = torch.from_numpy(O.query_hash(cent, q)).long()
    o_ref, lse_ref = O.hashed_attention(q, k, v, table[m], m.sum(-1), hashes, 0.1)
    assert (o.float().cpu() - o_ref.float()).abs().max() <= 2e-2
    assert (lse.float().cpu() - O.dropin_lse(lse_ref, torch.bfloat16).float()).abs().max() <= 4e-2   # bf16 LSE (tk:111)


def test_head_slices_and_host_pipeline_match_one_call():
    """Queries served in slices of KV heads (with GQA folding), and the pinned-host pipeline built on them."""
    cfg = synth.config("cfg3")
    q, k, v = synth.make(cfg, seed=6, kv_heads=6, n_keys=8192, n_queries=40)           # q [24, 40, 128]
    mem = fm.Memory.build(k.to(DEV), v.to(DEV), n_buckets=64, bucket_size=300, kmeans_iters=1)
    qd = q.to(DEV)
    o, lse = mem.query(qd, 0.1)
    G = cfg.q_groups
    o2, l2 = mem.query(qd[2 * G: 5 * G].contiguous(), 0.1, head_range=(2, 5))
    assert torch.equal(o2, o[2 * G: 5 * G]) and torch.equal(l2, lse[2 * G: 5 * G])
    q_host = q.pin_memory()
    o_host = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    l_host = torch.empty(q.shape[:2], dtype=torch.float32).pin_memory()
    for chunks in (1, 4):
        o_host.zero_()
        mem.query_from_host(q_host, 0.1, o_host, l_host, n_chunks=chunks)
        torch.cuda.synchronize()
        assert torch.equal(o_host, o.cpu()) and torch.equal(l_host, lse.cpu())
    # merged with a second result before the copy-out
    lo = torch.randn(q.shape, device=DEV)
    ll = torch.randn(q.shape[:2], device=DEV)
    mem.query_from_host(q_host, 0.1, o_host, l_host, n_chunks=3, local=(lo, ll))
    torch.cuda.synchronize()
    ro, rl = fm.merge(lo, ll, o, lse)
    assert (o_host.float() - ro.cpu()).abs().max() <= 2e-2 and (l_host - rl.cpu()).abs().max() <= 1e-5
    # consecutive calls that overlap one another: three different query sets, each into its own host tensors
    sets = []
    for i in range(3):
        qi = (q.float() + 0.05 * i * torch.randn(q.shape, generator=torch.Generator().manual_seed(i))).to(q.dtype)
        sets.append((qi.pin_memory(), torch.empty(q.shape, dtype=q.dtype).pin_memory(),
                     torch.empty(q.shape[:2], dtype=torch.float32).pin_memory()))
    for qi, oi, li in sets:
        mem.query_from_host(qi, 0.1, oi, li, n_chunks=2, overlap_calls=True)
    mem.finish_host_queries()
    torch.cuda.current_stream().synchronize()
    for qi, oi, li in sets:
        o_ref, l_ref = mem.query(qi.to(DEV), 0.1)
        assert torch.equal(oi, o_ref.cpu()) and torch.equal(li, l_ref.cpu())


def test_state_dict_round_trip(tmp_path):
    """The index goes through ``torch.save`` / ``torch.load`` on disk (map_location CPU, as a checkpoint is read) and
    serves the same answers; the restored table is the oracle's table."""
    cfg = synth.config("cfg1")
    q, k, v = synth.make(cfg, seed=2)
    mem = fm.Memory.build(k.to(DEV), v.to(DEV), n_buckets=32, bucket_size=100, kmeans_iters=1)
    path = tmp_path / "memory_index.pt"
    torch.save(mem.state_dict(), path)
    state = torch.load(path, map_location="cpu")
    assert state["table"].device.type == "cpu"
    m2 = fm.Memory.from_state_dict(state, k.to(DEV), v.to(DEV))
    m2.check_build()
    a, b = mem.query(q.to(DEV), 0.2), m2.query(q.to(DEV), 0.2)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    A = O.spherical_kmeans(k[0], k[0, :32], 1)
    assert np.array_equal(m2.table_of(0).cpu().numpy(), O.build_table(A[None], k, 100)[0])
    o_ref, l_ref = O.hashed_attention(q, k, v, torch.from_numpy(O.build_table(A[None], k, 100)).reshape(-1).long(),
                                      torch.full((1, 32), 100), torch.from_numpy(O.query_hash(A[None], q)).long(), 0.2)
    assert (b[0].cpu() - o_ref).abs().max() <= 1e-4 and (b[1].cpu() - l_ref).abs().max() <= 1e-3


def test_compute_centroids_code_variant(golden_dir):
    """mem:209-231 on the GPU path against the reference's own output (golden) and the oracle on a larger case."""
    z = np.load(os.path.join(golden_dir, "compute_centroids.npz"))
    kq, cent = torch.from_numpy(z["kq"]), torch.from_numpy(z["centroids"])
    out = fm.compute_centroids(kq.to(DEV), cent.to(DEV), cent.shape[0], int(z["n_groups"]), int(z["centroid_topk"]))
    assert out.shape == z["out"].shape
    assert (out.cpu().float() - torch.from_numpy(z["out"])).abs().max() <= 2e-6
    # larger, grouped heads, fp32 and bf16 (the unit rows are rounded to the input dtype first, as the reference does)
    g = torch.Generator().manual_seed(9)
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
        kq = torch.randn(8, 5000, 64, generator=g).to(dtype)
        cent = torch.nn.functional.normalize(torch.randn(48, 64, generator=g), dim=-1).to(dtype)
        out = fm.compute_centroids(kq.to(DEV), cent.to(DEV), 48, 4, 96)
        x = fm.unit_rows(kq.to(DEV)).to(dtype).cpu()                     # what the top-k ranks
        ref = O.compute_centroids(x, cent, 48, 4, 96)
        assert out.shape == (48, 2, 64) and out.dtype == dtype
        assert (out.cpu().float() - ref).abs().max() <= tol


def test_fused_build_with_keys_clustered_by_position():
    """Keys sorted by cluster: every bucket's best keys sit in one stretch of positions, which overflows the per-range
    candidate buffers; the build retries with one buffer per bucket and still needs no exact rebuild."""
    import warnings
    g = torch.Generator().manual_seed(31)
    N, C, Z, d = 65536, 128, 1024, 128
    cent = torch.nn.functional.normalize(torch.randn(C, d, generator=g), dim=-1)
    cid = torch.sort(torch.randint(C, (N,), generator=g)).values
    k = torch.nn.functional.normalize(cent[cid] + 0.1 * torch.randn(N, d, generator=g), dim=-1).bfloat16()[None].contiguous()
    A = cent.bfloat16()[None].contiguous()
    with warnings.catch_warnings(record=True) as rec:
        warnings.simplefilter("always")
        mem = fm.Memory.build(k.to(DEV), k.to(DEV), A=A.to(DEV), bucket_size=Z)
    assert not [w for w in rec if issubclass(w.category, RuntimeWarning)], "fell back to the exact path"
    ok, why = tables_equal_as_sets(mem.table_of(0).cpu().numpy(), O.topz(O.project(A[0], k[0]), Z))
    assert ok, why


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [64, 128])
def test_hash_rows_large_batch_ragged_segments(dtype, d):
    """Batches of 2048 rows or more take the tcgen05 kernel: segments whose bucket counts are not multiples of the
    128-bucket tile (columns of the next segment must not leak in), a one-row segment, row tiles that straddle
    segment ends."""
    g = torch.Generator().manual_seed(5 + d)
    Cs, Ss = [5, 64, 130, 300], [2500, 1, 3000, 129]
    A = torch.randn(sum(Cs), d, generator=g).to(dtype)
    X = torch.randn(sum(Ss), d, generator=g).to(dtype)
    xb = torch.tensor([0] + list(np.cumsum(Ss)), dtype=torch.int32)
    cb = torch.tensor([0] + list(np.cumsum(Cs)), dtype=torch.int32)
    h = fm.hash_rows(X.to(DEV), A.to(DEV), xb.to(DEV), cb.to(DEV), max(Ss)).cpu().numpy()
    for s in range(len(Cs)):
        ref = O.query_hash(A[cb[s]:cb[s + 1]][None], X[xb[s]:xb[s + 1]][None])[0]
        assert np.array_equal(h[xb[s]:xb[s + 1]], ref), f"segment {s}"


def test_append_equals_full_build():
    """Incremental growth of a memory: old table entries re-scored + the new block's own top-Z, merged exactly."""
    cfg = synth.config("cfg2")
    q, k, v = synth.make(cfg, seed=8, kv_heads=2, n_keys=24576, n_queries=500)
    C, Z = 48, 600
    kd, vd = k.to(DEV), v.to(DEV)
    full = fm.Memory.build(kd, vd, n_buckets=C, bucket_size=Z, kmeans_iters=1)
    A = full.A.reshape(2, C, cfg.d)
    mem = fm.Memory.build(kd[:, :16384].contiguous(), vd[:, :16384].contiguous(), A=A, bucket_size=Z)
    mem = mem.append(kd[:, 16384:20000].contiguous(), vd[:, 16384:20000].contiguous())
    mem = mem.append(kd[:, 20000:].contiguous(), vd[:, 20000:].contiguous())          # twice, ragged block sizes
    assert torch.equal(mem.k, kd) and torch.equal(mem.v, vd)
    ref_table = O.build_table(A.cpu(), k, Z)                         # the oracle over ALL the keys: independent of Memory.build
    for h in range(2):
        assert np.array_equal(mem.table_of(h).cpu().numpy(), ref_table[h]), f"head {h} differs from the oracle"
        assert torch.equal(mem.table_of(h), full.table_of(h)), f"head {h}"
    o1, l1 = mem.query(q.to(DEV), 0.1)
    o2, l2 = full.query(q.to(DEV), 0.1)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    # a memory smaller than its bucket size grows into it
    small = fm.Memory.build(kd[:, :300].contiguous(), vd[:, :300].contiguous(), A=A, bucket_size=Z)
    small = small.append(kd[:, 300:900].contiguous(), vd[:, 300:900].contiguous())
    ref = fm.Memory.build(kd[:, :900].contiguous(), vd[:, :900].contiguous(), A=A, bucket_size=Z)
    ref_small = O.build_table(A.cpu(), k[:, :900].contiguous(), Z)
    for h in range(2):
        assert torch.equal(small.table_of(h), ref.table_of(h))
        assert np.array_equal(small.table_of(h).cpu().numpy(), ref_small[h])
    # a grown memory persists like a built one
    m3 = fm.Memory.from_state_dict(mem.state_dict(), kd, vd)
    o3, l3 = m3.query(q.to(DEV), 0.1)
    assert torch.equal(o3, o1) and torch.equal(l3, l1)


def test_bounded_pipeline_wait_gives_up_and_the_next_call_is_fine():
    """Every mbarrier wait of the tcgen05 projection kernel is bounded.  With the test hook the producer leaves out its
    tile, the consumers' waits run out after 20 ms, the CTA records a status, frees its TMEM and returns normally (no
    trap, no fault); the next ordinary call on the same context gives the right scores."""
    from fast_memory_b200 import _lib as L
    g = torch.Generator().manual_seed(3)
    A = torch.randn(128, 128, generator=g).bfloat16().to(DEV)
    K = torch.randn(256, 128, generator=g).bfloat16().to(DEV)              # one bucket tile x one key tile: a single CTA
    lib = L.lib()
    assert lib.fm_test_set_tc_hooks(20, 0) == 0
    try:
        with pytest.raises(fm.FastMemError, match="pipeline wait gave up"):
            ops.project_tc(A, K)
    finally:
        assert lib.fm_test_set_tc_hooks(0, -1) == 0
    torch.cuda.synchronize()                                               # the context is intact
    Y = ops.project_tc(A, K)
    ref = A.float() @ K.float().T
    assert (Y - ref).abs().max() <= 1e-3 * ref.abs().max()


@pytest.mark.parametrize("n_seg,rows,C", [(1, 5000, 300), (6, 700, 64), (4, 9000, 2000), (2, 40000, 300), (2, 3000, 13000)])
def test_segmented_grouping_equals_the_general_one(n_seg, rows, C):
    """``fm_group_rows_segmented`` (one launch, a CTA per segment) against ``fm_group_rows`` on hashes that lie inside
    their segments' buckets: the same group offsets, and the same rows in every group (their order inside a group is
    free in both); segments too long or with too many buckets for one CTA take the general path inside the call.  Also with a slice of the segments, as ``Memory.query(head_range=...)`` passes them."""
    g = torch.Generator().manual_seed(n_seg * 1000 + C)
    seg_rows = [rows + 37 * s for s in range(n_seg)]
    seg_c = [C + 5 * s for s in range(n_seg)]
    xb = torch.tensor([0] + list(np.cumsum(seg_rows)), dtype=torch.int32)
    cb = torch.tensor([0] + list(np.cumsum(seg_c)), dtype=torch.int32)
    hashes = torch.cat([torch.randint(0, seg_c[s], (seg_rows[s],), generator=g) for s in range(n_seg)]).int().to(DEV)
    total = int(cb[-1])
    ref_off, ref_perm = ops.group_rows(hashes, total, xb.to(DEV), cb.to(DEV))
    off, perm = ops.group_rows(hashes, total, xb.to(DEV), cb.to(DEV), in_range=True, max_seg_rows=max(seg_rows),
                               max_seg_buckets=max(seg_c))
    assert torch.equal(off, ref_off)
    o = off.cpu().numpy()
    p, rp = perm.cpu().numpy(), ref_perm.cpu().numpy()
    for b in range(total):
        assert np.array_equal(np.sort(p[o[b]:o[b + 1]]), np.sort(rp[o[b]:o[b + 1]]))
    if n_seg >= 4:                                                          # segments 1 and 2 only
        sl_x = (xb[1:4] - xb[1]).to(DEV)
        h2 = hashes[int(xb[1]):int(xb[3])].contiguous()
        ref_off, ref_perm = ops.group_rows(h2, total, sl_x, cb[1:4].to(DEV))
        off, perm = ops.group_rows(h2, total, sl_x, cb[1:4].to(DEV), in_range=True, max_seg_rows=max(seg_rows),
                                   max_seg_buckets=max(seg_c))
        assert torch.equal(off, ref_off)
        assert torch.equal(torch.sort(perm)[0], torch.sort(ref_perm)[0])


@pytest.mark.parametrize("case", ["flat", "narrow", "outliers", "ragged_sample"])
def test_thresholds_from_the_sample_projection_edge_cases(case):
    """The thresholds come from histograms of the sample scores taken in the projection's epilogue.  Rows whose scores
    are all equal (flat), crowd a range that is tiny against their magnitude (the sub-bin refinement is left out), hold
    a few huge outliers (coarse first-level bins), or whose sample is not a multiple of the 256-key tile: the table must
    equal the oracle's whatever threshold comes out, because a low threshold only costs candidates."""
    g = torch.Generator().manual_seed({"flat": 1, "narrow": 2, "outliers": 3, "ragged_sample": 4}[case])
    N, C, Z, d = 16384, 16, 256, 128
    A = torch.nn.functional.normalize(torch.randn(1, C, d, generator=g), dim=-1)
    if case == "flat":
        k = torch.randn(1, d, generator=g).repeat(N, 1)
    elif case == "narrow":
        u = torch.nn.functional.normalize(torch.randn(d, generator=g), dim=0)
        A = torch.nn.functional.normalize(u[None, None] + 0.3 * A, dim=-1)             # every bucket scores near |u| = 4
        k = 4.0 * u[None] + 0.02 * torch.randn(N, d, generator=g)
    elif case == "outliers":
        k = torch.randn(N, d, generator=g)
        k[torch.randperm(N, generator=g)[:5]] *= 300.0
    else:
        N = 8192 + 1000 + 40
        k = torch.randn(N, d, generator=g)
    k = k.bfloat16()[None].contiguous()
    A = A.bfloat16()
    mem = fm.Memory.build(k.to(DEV), k.to(DEV), A=A.to(DEV), bucket_size=Z)
    ok, why = tables_equal_as_sets(mem.table_of(0).cpu().numpy(), O.topz(O.project(A[0], k[0]), Z))
    assert ok, why


def test_fused_build_random_shapes_and_data_equal_the_exact_build():
    """Sixteen random combinations of dtype, head dim, segment length, bucket count and size, and of key distributions
    (Gaussian, clustered, heavy-tailed norms, scores drifting with position, near-duplicate runs): the tensor-core
    filter with its sampled thresholds and exact band must give the table of the all-fp32 build (oracle-pinned above)."""
    import random
    import warnings
    rnd = random.Random(0)
    for it in range(16):
        g = torch.Generator().manual_seed(1000 + it)
        d, dt = rnd.choice([64, 128]), rnd.choice([torch.bfloat16, torch.float16])
        H, N = rnd.choice([1, 2, 3]), rnd.choice([8192, 12000, 20000, 40000, 65536])
        C, Z = rnd.choice([16, 100, 128, 300]), rnd.choice([64, 200, 512, 1024, 2000])
        Z = min(Z, N // 8)
        kind = rnd.choice(["gauss", "mixture", "heavy", "drift", "dups"])
        if kind == "gauss":
            k = torch.randn(H, N, d, generator=g)
        elif kind == "mixture":
            cent = torch.nn.functional.normalize(torch.randn(32, d, generator=g), dim=-1)
            k = cent[torch.randint(32, (H * N,), generator=g)].reshape(H, N, d) + 0.2 * torch.randn(H, N, d, generator=g)
        elif kind == "heavy":
            k = torch.randn(H, N, d, generator=g) * torch.exp(torch.randn(H, N, 1, generator=g))
        elif kind == "drift":
            k = torch.randn(H, N, d, generator=g) + torch.linspace(-2, 2, N)[None, :, None] * torch.randn(1, 1, d, generator=g)
        else:
            k = torch.randn(H, N // 16 + 1, d, generator=g).repeat_interleave(16, dim=1)[:, :N] + 0.001 * torch.randn(H, N, d, generator=g)
        k = k.to(dt).contiguous().to(DEV)
        A = torch.nn.functional.normalize(torch.randn(H, C, d, generator=g), dim=-1).to(dt).to(DEV)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")                 # (a data set that overflows the filter falls back with a warning)
            fused = fm.Memory.build(k, k, A=A, bucket_size=Z)
        exact = fm.Memory.build(k, k, A=A, bucket_size=Z, exact_only=True)
        assert torch.equal(fused.table, exact.table), (it, kind, dt, d, H, N, C, Z)
