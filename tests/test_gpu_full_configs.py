"""The benchmark configurations at their full sizes: size-independent properties of the index over every bucket,
bit-exact comparison with the oracle on a subset of buckets, oracle attention for a sample of queries."""
import numpy as np
import pytest
import torch

import fast_memory_b200 as fm
from fast_memory_b200 import synth
from oracle import oracle as O
from tests.util import TOL_LSE, TOL_O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def check_table_properties(mem):
    """Every bucket row: strictly ascending key rows, all inside the bucket's own segment."""
    for s in range(len(mem.seg_z)):
        C = mem.seg_cb[s + 1] - mem.seg_cb[s]
        t = mem.table[mem.table_off[s]: mem.table_off[s + 1]].reshape(C, -1)
        assert t.shape[1] == min(mem.seg_z[s], mem.seg_kb[s + 1] - mem.seg_kb[s])
        assert bool((t[:, 1:] > t[:, :-1]).all()), f"segment {s}: rows not strictly ascending"
        assert int(t.min()) >= mem.seg_kb[s] and int(t.max()) < mem.seg_kb[s + 1], f"segment {s}: row outside the segment"


def check_buckets_against_oracle(mem, seg, buckets):
    """Bit-exact table rows of some buckets of one segment (canonical projection + top-Z on the CPU)."""
    d = mem.d
    k_seg = mem.k.reshape(-1, d)[mem.seg_kb[seg]: mem.seg_kb[seg + 1]].cpu()
    A_seg = mem.A[mem.seg_cb[seg]: mem.seg_cb[seg + 1]].cpu()
    C = A_seg.shape[0]
    zc = min(mem.seg_z[seg], k_seg.shape[0])
    ref = O.topz(O.project(A_seg[buckets], k_seg), zc)
    got = mem.table[mem.table_off[seg]: mem.table_off[seg + 1]].reshape(C, zc)[buckets].cpu().numpy() - mem.seg_kb[seg]
    bad = np.nonzero((got != ref).any(-1))[0]
    assert len(bad) == 0, f"segment {seg}: {len(bad)} of {len(buckets)} checked buckets differ (first: bucket {buckets[bad[0]]})"


def check_sampled_queries(mem, q_flat, o_flat, lse_flat, hashes_flat, q_seg_of_row, rows, sm_scale, dtype):
    """Oracle attention for some query rows, each over the bucket the GPU hashed it to (hash checked separately)."""
    d = mem.d
    kf, vf = mem.k.reshape(-1, d), mem.v.reshape(-1, d)
    for r in rows:
        seg = q_seg_of_row(r)
        gb = mem.seg_cb[seg] + int(hashes_flat[r])
        lo, hi = int(mem.bucket_off[gb]), int(mem.bucket_off[gb + 1])
        idx = mem.table[lo:hi].long()
        kk, vv = kf[idx].cpu(), vf[idx].cpu()
        n = kk.shape[0]
        o_ref, l_ref = O.hashed_attention(q_flat[r].cpu()[None, None], kk[None], vv[None], torch.arange(n),
                                          torch.tensor([[n]]), torch.zeros(1, 1, dtype=torch.long), sm_scale)
        assert (o_flat[r].float().cpu() - o_ref[0, 0].float()).abs().max() <= TOL_O[dtype]
        assert abs(float(lse_flat[r]) - float(l_ref[0, 0])) <= TOL_LSE


def check_hashes(mem, q_flat, hashes_flat, seg, q_rows):
    A_seg = mem.A[mem.seg_cb[seg]: mem.seg_cb[seg + 1]].cpu()
    ref = O.query_hash(A_seg[None], q_flat[q_rows].cpu()[None])[0]
    assert np.array_equal(hashes_flat[q_rows].cpu().numpy(), ref)


def test_config2_full_size():
    cfg = synth.config("cfg2")
    q, k, v = synth.make(cfg, seed=0, device=DEV)
    H, N, d = k.shape
    S = q.shape[1]
    sm = d ** -0.5
    mem = fm.Memory.build(k, v, n_buckets=cfg.n_buckets, bucket_size=cfg.bucket_size, kmeans_iters=cfg.kmeans_iters, kmeans_init=q)
    check_table_properties(mem)
    # k-means projection of one head and all of its buckets against the oracle
    h = 5
    A_ref = O.spherical_kmeans(k[h].cpu(), q[h, :cfg.n_buckets].cpu(), cfg.kmeans_iters)
    assert torch.equal(mem.projection_of(h).cpu(), A_ref)
    check_buckets_against_oracle(mem, h, list(range(cfg.n_buckets)))
    check_buckets_against_oracle(mem, 31, [0, 17, 511])
    o, lse = mem.query(q, sm)
    hashes = mem.hash_queries(q)
    qf, of, lf, hf = q.reshape(-1, d), o.reshape(-1, d), lse.reshape(-1), hashes.reshape(-1)
    check_hashes(mem, qf, hf, 3, torch.arange(3 * S, 4 * S, device=DEV))
    g = torch.Generator().manual_seed(1)
    rows = torch.randint(H * S, (48,), generator=g).tolist()
    check_sampled_queries(mem, qf, of, lf, hf, lambda r: r // S, rows, sm, cfg.dtype)
    # merged with the local window like the benchmark step: the merge is associative with -inf handled
    out, l2 = fm.merge(o, lse, o, lse)
    assert (l2 - (lse + np.log(2.0))).abs().max() <= 1e-4 and (out - o.float()).abs().max() <= 1e-6


def test_config3_full_size_decode():
    cfg = synth.config("cfg3")
    q, k, v = synth.make(cfg, seed=1, device=DEV)                    # q [32, 64, 128], k [8, 1Mi, 128]
    H, N, d = k.shape
    Hq, S = q.shape[0], q.shape[1]
    G = Hq // H
    sm = d ** -0.5
    mem = fm.Memory.build(k, v, n_buckets=cfg.n_buckets, bucket_size=cfg.bucket_size, kmeans_iters=1)
    check_table_properties(mem)
    check_buckets_against_oracle(mem, 2, list(range(0, 1024, 41)))
    o, lse = mem.query(q, sm)                                         # few queries, long buckets: split over CTAs + combine
    hashes = mem.hash_queries(q)
    qf, of, lf, hf = q.reshape(-1, d), o.reshape(-1, d), lse.reshape(-1), hashes.reshape(-1)
    check_hashes(mem, qf, hf, 0, torch.arange(0, G * S, device=DEV))
    g = torch.Generator().manual_seed(2)
    rows = torch.randint(Hq * S, (24,), generator=g).tolist()
    check_sampled_queries(mem, qf, of, lf, hf, lambda r: r // (G * S), rows, sm, cfg.dtype)
    # unsplit buckets give the same answer
    o1, l1 = mem.query(q, sm, key_chunk=cfg.bucket_size)
    assert (o1.float() - o.float()).abs().max() <= 2e-2 and (l1 - lse).abs().max() <= 1e-3


def test_config4_full_size_varlen():
    cfg = synth.config("cfg4")
    q, k, v, cu_q, cu_k = synth.make_varlen(cfg, seed=2, device=DEV)
    H, d = k.shape[0], k.shape[2]
    Cs = [synth.varlen_buckets(n) for n in cfg.seq_keys]
    Zs = [synth.varlen_bucket_size(n) for n in cfg.seq_keys]
    sm = d ** -0.5
    mem = fm.Memory.build(k, v, n_buckets=Cs, bucket_size=Zs, kmeans_iters=1, cu_seqlens_k=cu_k)
    check_table_properties(mem)
    n_seq = len(cfg.seq_keys)
    small, large = int(np.argmin(cfg.seq_keys)), int(np.argmax(cfg.seq_keys))
    for seq in (small, large):
        seg = 3 * n_seq + seq                                          # head 3
        check_buckets_against_oracle(mem, seg, list(range(0, Cs[seq], 37)))
    o, lse = mem.query(q, sm, cu_seqlens_q=cu_q)
    hashes = mem.hash_queries(q, cu_seqlens_q=cu_q)
    Qt = q.shape[1]
    qf, of, lf, hf = q.reshape(-1, d), o.reshape(-1, d), lse.reshape(-1), hashes.reshape(-1)

    def seg_of(r):
        h, pos = divmod(r, Qt)
        return h * n_seq + int(np.searchsorted(cu_q, pos, side="right") - 1)

    seg = 5 * n_seq + large
    check_hashes(mem, qf, hf, seg, torch.arange(5 * Qt + cu_q[large], 5 * Qt + cu_q[large + 1], device=DEV))
    g = torch.Generator().manual_seed(3)
    rows = torch.randint(H * Qt, (32,), generator=g).tolist()
    check_sampled_queries(mem, qf, of, lf, hf, seg_of, rows, sm, cfg.dtype)


def test_config5_shards_several_workspace_groups():
    """Two heads of the ring config, all 8 key shards of a head on one device (16 segments of 524288 keys, C = 1024,
    Z = 8192): more buckets than one workspace group of the fused build holds, so the segments are built in several
    groups; properties everywhere, oracle rows in the first and in a later group."""
    cfg = synth.config("cfg5")
    q, k, v = synth.make(cfg, seed=4, device=DEV, kv_heads=2)
    H, N, d = k.shape
    L = N // cfg.shards
    cu_k = [i * L for i in range(cfg.shards + 1)]
    mem = fm.Memory.build(k, v, n_buckets=[cfg.n_buckets] * cfg.shards, bucket_size=[cfg.bucket_size] * cfg.shards,
                          kmeans_iters=1, cu_seqlens_k=cu_k)
    check_table_properties(mem)
    check_buckets_against_oracle(mem, 1, [0, 500, 1023])
    check_buckets_against_oracle(mem, 14, [3, 777])


def test_config5_full_size_queries_over_all_shards():
    """Two heads of the ring config at full size, queried: 8 shards of 524288 keys per head on one device through
    ``ShardedMemory`` (every bucket = the concatenation of its 8 per-shard tables, 65536 keys), all 16384 queries of a
    head.  The local table equals the per-shard oracle tables side by side; hashes and sampled query rows equal the
    oracle over the concatenated per-shard buckets; merging eight independent per-shard memories gives the same."""
    from fast_memory_b200.dist import ShardedMemory
    cfg = synth.config("cfg5")
    q, k, v = synth.make(cfg, seed=6, device=DEV, kv_heads=2)
    H, N, d = k.shape
    S = q.shape[1]
    L, C, Z = N // cfg.shards, cfg.n_buckets, cfg.bucket_size
    sm = d ** -0.5
    A = torch.stack([fm.kmeans_projection(k[h, :L].contiguous(), q[h, :C].contiguous(), 1, [0, L], [0, C])[0] for h in range(H)])
    mem = ShardedMemory.build(k, v, L, A=A, bucket_size=Z)
    loc = mem.local
    assert loc.max_bucket_len == cfg.shards * Z and loc.table.numel() == H * C * cfg.shards * Z
    # the table of bucket (h, c): per-shard oracle rows (canonical projection + top-Z over the shard's keys), shard by shard
    h, buckets = 1, [0, 511, 1023]
    for s_ in (0, 5):
        ref = O.topz(O.project(A[h, buckets].cpu(), k[h, s_ * L:(s_ + 1) * L].cpu()), Z) + s_ * L
        got = loc.table.reshape(H, C, cfg.shards, Z)[h, buckets, s_].cpu().numpy() - h * N
        assert np.array_equal(got, ref), f"shard {s_}"
    o, lse = mem.query(q, sm)
    assert o.dtype == torch.float32 and o.shape == (H, S, d)
    hashes = loc.hash_queries(q)
    qf, of, lf, hf = q.reshape(-1, d), o.reshape(-1, d), lse.reshape(-1), hashes.reshape(-1)
    check_hashes(loc, qf, hf, 1, torch.arange(S, S + 2048, device=DEV))
    g = torch.Generator().manual_seed(7)
    rows = torch.randint(H * S, (20,), generator=g).tolist()
    check_sampled_queries(loc, qf, of, lf, hf, lambda r: r // S, rows, sm, cfg.dtype)
    # the reference's structure: one memory per shard, partial results LSE-merged (mem:319-332)
    out, acc_l = None, None
    for s_ in range(cfg.shards):
        ms = fm.Memory.build(k[:, s_ * L:(s_ + 1) * L].contiguous(), v[:, s_ * L:(s_ + 1) * L].contiguous(), A=A, bucket_size=Z)
        bo, bl = ms.query(q, sm, q_hashes=hashes)
        out, acc_l = fm.update_out_and_lse(out, acc_l, bo, bl)
        del ms
    assert (out - o).abs().max() <= 2e-2 and (acc_l.squeeze(-1) - lse).abs().max() <= 1e-3
