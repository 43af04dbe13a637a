"""Sequence-sharded memories (BASELINE config 5 layout, cut down): one process with several local shards, and
- when the box has two or more GPUs - two NCCL ranks against the single-device result."""
import os
import socket

import numpy as np
import pytest
import torch

import fast_memory_b200 as fm
from fast_memory_b200 import synth
from fast_memory_b200.dist import ShardedMemory
from oracle import oracle as O
from tests.util import assert_attn_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(n_shards=4, H=2, shard_len=8192, S=300, C=32, seed=11):
    cfg = synth.config("cfg5")
    q, k, v = synth.make(cfg, seed=seed, kv_heads=H, n_keys=n_shards * shard_len, n_queries=S)
    A = torch.stack([O.spherical_kmeans(k[h, :shard_len], k[h, :C], 1) for h in range(H)])
    return cfg, q, k, v, A


def test_local_shards_equal_union_of_per_shard_indices():
    n_shards, H, L, S, C, Z = 4, 2, 8192, 300, 32, 256
    cfg, q, k, v, A = _case(n_shards, H, L, S, C)
    sm = cfg.d ** -0.5
    mem = ShardedMemory.build(k.to(DEV), v.to(DEV), L, A=A.to(DEV), bucket_size=Z)
    o, lse = mem.query(q.to(DEV), sm)
    # oracle: per-shard tables (local top-Z), concatenated per bucket with global key indices
    tabs = [O.build_table(A, k[:, s * L:(s + 1) * L].contiguous(), Z) + s * L for s in range(n_shards)]
    table = torch.from_numpy(np.concatenate(tabs, axis=-1)).long()                       # [H, C, n_shards * Z]
    assert np.array_equal(mem.local.table.reshape(H, C, -1).cpu().numpy() - (np.arange(H) * n_shards * L)[:, None, None],
                          table.numpy())
    hashes = torch.from_numpy(O.query_hash(A, q)).long()
    o_ref, lse_ref = O.hashed_attention(q, k, v, table.reshape(-1), torch.full((H, C), n_shards * Z), hashes, sm)
    assert_attn_close(o, lse, o_ref, lse_ref, cfg.dtype)
    # and it equals merging independent per-shard memories (the reference's per-step structure, mem:319-332)
    out, acc_l = None, None
    for s in range(n_shards):
        ms = fm.Memory.build(k[:, s * L:(s + 1) * L].contiguous().to(DEV), v[:, s * L:(s + 1) * L].contiguous().to(DEV),
                             A=A.to(DEV), bucket_size=Z)
        bo, bl = ms.query(q.to(DEV), sm)
        out, acc_l = fm.update_out_and_lse(out, acc_l, bo, bl)
    assert (out.cpu() - o.float().cpu()).abs().max() <= 2e-2
    assert (acc_l.squeeze(-1).cpu() - lse.cpu()).abs().max() <= 1e-3


def _rank_main(rank, world, port, n_shards, H, L, S, C, Z, result):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    cfg, q, k, v, A = _case(n_shards, H, L, S, C)
    per = n_shards // world
    lo, hi = rank * per * L, (rank + 1) * per * L
    dev = f"cuda:{rank}"
    mem = ShardedMemory.build(k[:, lo:hi].contiguous().to(dev), v[:, lo:hi].contiguous().to(dev), L, A=A.to(dev), bucket_size=Z)
    o, lse = mem.query(q.to(dev), cfg.d ** -0.5)
    o2, lse2 = mem.query(q.to(dev), cfg.d ** -0.5, exchange="allreduce")
    torch.cuda.synchronize()
    assert (o2 - o).abs().max() <= 1e-4 and (lse2 - lse).abs().max() <= 1e-4       # two ways to merge the same partials
    # the third: one kernel per rank over peer memory (pull the partial rows, merge, push the finished rows), twice in a
    # row (the second query reuses the exchange buffers)
    for _ in range(2):
        o4, lse4 = mem.query(q.to(dev), cfg.d ** -0.5, exchange="peer")
        torch.cuda.synchronize()
        assert (o4 - o).abs().max() <= 1e-4 and (lse4 - lse).abs().max() <= 1e-4
    # queries sequence-sharded like the keys (the reference's layout): this rank's slice in, its rows of the result out
    n = S // world
    o3, lse3 = mem.query_sharded(q[:, rank * n:(rank + 1) * n].contiguous().to(dev), cfg.d ** -0.5)
    torch.cuda.synchronize()
    assert (o3 - o[:, rank * n:(rank + 1) * n]).abs().max() <= 1e-4 and (lse3 - lse[:, rank * n:(rank + 1) * n]).abs().max() <= 1e-4
    # the reference's global index over the two ranks' keys, and all queries through it
    from fast_memory_b200 import dist as fmd
    k_hashes = fmd.build_global_table(k[:, lo:hi].contiguous().to(dev), A.to(dev), Z)
    go, gl = fmd.query_global_table(k_hashes, A.to(dev), q.to(dev), k[:, lo:hi].contiguous().to(dev),
                                    v[:, lo:hi].contiguous().to(dev), cfg.d ** -0.5)
    torch.cuda.synchronize()
    if rank == 0:
        result["o"], result["lse"] = o.cpu(), lse.cpu()
        result["k_hashes"], result["go"], result["gl"] = k_hashes.cpu(), go.cpu(), gl.cpu()
    dist.destroy_process_group()


def test_global_table_from_shard_candidates_equals_single_device_build():
    """mem:260-278 without the all_to_all of Y: per-shard top-Z with canonical scores, one exact select over the union."""
    from fast_memory_b200 import dist as fmd
    n_shards, H, L, S, C, Z = 4, 2, 8192, 300, 32, 700
    cfg, q, k, v, A = _case(n_shards, H, L, S, C)
    kd, vd, Ad = k.to(DEV), v.to(DEV), A.to(DEV)
    cands = [fmd.shard_candidates(kd[:, s * L:(s + 1) * L].contiguous(), Ad, Z, s * L) for s in range(n_shards)]
    k_hashes = fmd.merge_shard_candidates([c[0] for c in cands], [c[1] for c in cands], Z)        # [C, H, Z]
    assert k_hashes.shape == (C, H, Z) and k_hashes.dtype == torch.int64
    oracle_table = O.build_table(A, k, Z)                              # CPU oracle over the concatenated keys
    ref = fm.Memory.build(kd, vd, A=Ad, bucket_size=Z)
    for h in range(H):
        assert np.array_equal(k_hashes[:, h].cpu().numpy(), oracle_table[h]), f"head {h} differs from the oracle"
        assert torch.equal(k_hashes[:, h].cpu(), ref.table_of(h).long().cpu()), f"head {h}"
    # attending through the global table, shard by shard, equals the single memory
    sm = cfg.d ** -0.5
    o_ref, l_ref = ref.query(q.to(DEV), sm)
    out, acc_l = None, None
    for s in range(n_shards):
        hashes = ref.hash_queries(q.to(DEV)).long()[:, None, :]
        bo, bl = fm.ring_attention_masked_forward(k_hashes, hashes, q.to(DEV)[None], kd[None, :, s * L:(s + 1) * L].contiguous(),
                                                  vd[None, :, s * L:(s + 1) * L].contiguous(), sm, s)
        bl = torch.where(bl.float() <= torch.finfo(q.dtype).min, torch.full_like(bl.float(), float("-inf")), bl.float())
        out, acc_l = fm.update_out_and_lse(out, acc_l, bo, bl)
    assert (out[0].cpu() - o_ref.float().cpu()).abs().max() <= 2e-2
    assert (acc_l[0].squeeze(-1).cpu() - l_ref.cpu()).abs().max() <= 3e-2        # the drop-in rounds each shard's LSE to bf16


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_single_device():
    import torch.multiprocessing as mp
    n_shards, H, L, S, C, Z = 4, 2, 8192, 300, 32, 256
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_rank_main, args=(2, port, n_shards, H, L, S, C, Z, result), nprocs=2, join=True)
        o2, l2 = result["o"], result["lse"]
        kh, go, gl = result["k_hashes"], result["go"], result["gl"]
    cfg, q, k, v, A = _case(n_shards, H, L, S, C)
    single = ShardedMemory.build(k.to(DEV), v.to(DEV), L, A=A.to(DEV), bucket_size=Z)
    o1, l1 = single.query(q.to(DEV), cfg.d ** -0.5)
    assert (o1.float().cpu() - o2).abs().max() <= 2e-2          # bf16 partials merged in fp32 vs one bf16 pass
    assert (l1.cpu() - l2).abs().max() <= 1e-3
    # global table built by the two ranks = the table one device builds over all the keys; queries through it
    whole = fm.Memory.build(k.to(DEV), v.to(DEV), A=A.to(DEV), bucket_size=Z)
    oracle_table = O.build_table(A, k, Z)
    for h in range(H):
        assert np.array_equal(kh[:, h].numpy(), oracle_table[h]), f"head {h} differs from the oracle"
        assert torch.equal(kh[:, h], whole.table_of(h).long().cpu())
    ow, lw = whole.query(q.to(DEV), cfg.d ** -0.5)
    assert (ow.float().cpu() - go).abs().max() <= 2e-2 and (lw.cpu() - gl).abs().max() <= 3e-2
