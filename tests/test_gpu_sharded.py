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
    if rank == 0:
        result["o"], result["lse"] = o.cpu(), lse.cpu()
    dist.destroy_process_group()


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
    cfg, q, k, v, A = _case(n_shards, H, L, S, C)
    single = ShardedMemory.build(k.to(DEV), v.to(DEV), L, A=A.to(DEV), bucket_size=Z)
    o1, l1 = single.query(q.to(DEV), cfg.d ** -0.5)
    assert (o1.float().cpu() - o2).abs().max() <= 2e-2          # bf16 partials merged in fp32 vs one bf16 pass
    assert (l1.cpu() - l2).abs().max() <= 1e-3
