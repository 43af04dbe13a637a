"""Ring exchange of partial (O, LSE) results on CPU ranks (gloo): the host-side logic of the sequence-sharded
path, including what the peers see when a rank fails on the host."""
import datetime
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torch_merge(out, lse, blk_out, blk_lse):
    """In-place LSE merge in plain torch (mem:54-71 semantics with -inf as weight 0)."""
    m = torch.maximum(lse, blk_lse)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w1, w2 = torch.exp(lse - m), torch.exp(blk_lse - m)
    tot = (w1 + w2).clamp_min(1e-30)
    out.copy_(out * (w1 / tot)[:, None] + blk_out * (w2 / tot)[:, None])
    lse.copy_(torch.log(w1 + w2) + m)


def _partials(rank, rows, d):
    g = torch.Generator().manual_seed(100 + rank)
    o = torch.randn(rows, d, generator=g)
    l = torch.randn(rows, generator=g) * 2
    l[rank::7] = -math.inf                      # some queries have an empty bucket on this rank
    return o, l


def _worker(rank, world, port, rows, d, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from fast_memory_b200 import dist as fmd
    o, l = _partials(rank, rows, d)
    oc, lc, own = fmd.ring_reduce_scatter_partials(o.clone(), l.clone(), merge_fn=_torch_merge)
    assert own == (rank + 1) % world
    full_o = fmd.all_gather_chunks(oc, own)
    full_l = fmd.all_gather_chunks(lc, own)
    if rank == 0:
        result["o"], result["l"] = full_o, full_l
    # the same merge written as a MAX and a SUM all-reduce
    ao, al = fmd.allreduce_merge_partials(o.clone(), l.clone())
    fin = torch.isfinite(full_l)
    assert torch.equal(torch.isfinite(al), fin)
    assert torch.allclose(al[fin], full_l[fin], atol=1e-5) and torch.allclose(ao[fin], full_o[fin], atol=1e-5)
    assert (ao[~fin] == 0).all()
    # and as a MAX all-reduce + SUM reduce-scatter: every rank gets its own block of rows only
    n = rows // world
    so, sl = fmd.reduce_scatter_merge_partials(o.reshape(world, n, d).clone(), l.reshape(world, n).clone())
    mine = slice(rank * n, (rank + 1) * n)
    fin_m = fin[mine]
    assert torch.equal(torch.isfinite(sl), fin_m)
    assert torch.allclose(sl[fin_m], full_l[mine][fin_m], atol=1e-5) and torch.allclose(so[fin_m], full_o[mine][fin_m], atol=1e-5)
    # SendRecv misuse raises like the reference (mem:39-40, 45-46)
    c = fmd.SendRecv()
    with pytest.raises(RuntimeError, match="Wait called before commit"):
        c.wait()
    t = torch.full((3,), float(rank))
    got = c.send_recv(t)
    c.commit()
    with pytest.raises(RuntimeError, match="Commit called twice"):
        c.commit()
    c.wait()
    assert torch.equal(got, torch.full((3,), float((rank - 1) % world)))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_ring_merge_equals_merging_everything_at_once(world):
    rows, d = 6 * world, 8
    port = _free_port()
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_worker, args=(world, port, rows, d, result), nprocs=world, join=True)
        full_o, full_l = result["o"], result["l"]
    # reference: exact fp64 merge of all ranks' partials
    os_, ls_ = zip(*[_partials(r, rows, d) for r in range(world)])
    L = torch.stack(ls_).double()
    m = L.max(0).values
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w = torch.exp(L - m)
    ref_l = torch.log(w.sum(0)) + m
    ref_o = (torch.stack(os_).double() * (w / w.sum(0).clamp_min(1e-300))[..., None]).sum(0)
    fin = torch.isfinite(ref_l)
    assert torch.allclose(full_l[fin].double(), ref_l[fin], atol=1e-5)
    assert torch.equal(torch.isinf(full_l), ~fin)
    assert torch.allclose(full_o[fin].double(), ref_o[fin], atol=1e-5)


def _failing_worker(rank, world, port, seen):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from fast_memory_b200 import dist as fmd
    if rank == 1:
        # the failure is made on the host: this rank never joins the exchange
        dist.destroy_process_group()
        return
    o, l = _partials(rank, 4 * world, 4)
    try:
        fmd.ring_reduce_scatter_partials(o, l, merge_fn=_torch_merge)
        seen[rank] = "no error"
    except Exception as e:          # the peers must get an error within the group's timeout, not hang
        seen[rank] = type(e).__name__
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def test_peer_failure_surfaces_as_an_error_not_a_hang():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        seen = mgr.dict()
        mp.spawn(_failing_worker, args=(world, port, seen), nprocs=world, join=True)
        assert seen.get(0, "no error") != "no error"
