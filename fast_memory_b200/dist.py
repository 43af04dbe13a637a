"""Sequence-sharded memories: every rank indexes its own key shards, partial (O, LSE) results are merged
around a ring.

The reference rotates the K / V shards themselves around the ring (``SendRecv`` + the loop at mem:291-338) and
re-filters a global table at every step (mem:131-142).  Here the keys never move: each rank attends all
queries to its local shards in ONE pass (the table of a bucket is the concatenation of the per-shard tables,
so every bucket row is staged once), and only the partial results travel - a ring reduce-scatter of
(O, LSE) in W - 1 steps of NCCL send/recv, each received slice folded in with the LSE-merge kernel
(mem:54-71), then an all-gather of the finished slices.  Per step a rank sends rows / W x (d + 1) fp32
values, which is tiny next to the attention itself.

``SendRecv`` keeps the reference's interface (mem:13-50): ``send_recv`` queues a pair of P2P operations to
the next / from the previous rank, ``commit`` posts the batch, ``wait`` blocks on it; misuse raises the same
``RuntimeError`` messages.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib as L
from . import ops
from .memory import Memory, kmeans_projection

MergeFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor], None]


class SendRecv:
    """Batched exchange with the ring neighbours (drop-in for mem:13-50)."""

    def __init__(self, msg: str = "", group: Optional[dist.ProcessGroup] = None):
        self._pending_operations: List[dist.P2POp] = []
        self._active_requests = None
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.send_rank = (self.rank + 1) % self.world_size
        self.recv_rank = (self.rank + self.world_size - 1) % self.world_size

    def _global(self, group_rank: int) -> int:
        return group_rank if self.group is None else dist.get_global_rank(self.group, group_rank)

    def send_recv(self, tensor_to_send: torch.Tensor, recv_tensor: Optional[torch.Tensor] = None) -> torch.Tensor:
        result_tensor = torch.zeros_like(tensor_to_send) if recv_tensor is None else recv_tensor
        send_operation = dist.P2POp(dist.isend, tensor_to_send, self._global(self.send_rank), group=self.group)
        recv_operation = dist.P2POp(dist.irecv, result_tensor, self._global(self.recv_rank), group=self.group)
        # same ordering rule as the reference (mem:31-34): the higher neighbour is addressed first
        if self.send_rank > self.rank:
            self._pending_operations.extend([send_operation, recv_operation])
        else:
            self._pending_operations.extend([recv_operation, send_operation])
        return result_tensor

    def commit(self):
        if self._active_requests is not None:
            raise RuntimeError("Commit called twice")
        self._active_requests = dist.batch_isend_irecv(self._pending_operations)
        self._pending_operations = []

    def wait(self):
        if self._active_requests is None:
            raise RuntimeError("Wait called before commit")
        for request in self._active_requests:
            request.wait()
        self._active_requests = None
        assert not self._pending_operations


def _default_merge(out: torch.Tensor, lse: torch.Tensor, blk_out: torch.Tensor, blk_lse: torch.Tensor) -> None:
    ops.lse_merge(out, lse, blk_out, blk_lse)


def ring_reduce_scatter_partials(out: torch.Tensor, lse: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                                 merge_fn: MergeFn = _default_merge) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """Merge the partial results of all ranks.

    ``out`` fp32 ``[rows, d]`` and ``lse`` fp32 ``[rows]`` (rows a multiple of the world size) hold this rank's
    partial attention over ITS keys for ALL queries; they are used as scratch.  After W - 1 ring steps rank r
    holds the complete result for the rows of chunk ``(r + 1) % W``.  Returns views ``(out_chunk, lse_chunk)`` of
    that chunk and its index.
    """
    W, r = dist.get_world_size(group), dist.get_rank(group)
    rows, d = out.shape
    assert rows % W == 0 and lse.shape == (rows,) and out.dtype == torch.float32 and lse.dtype == torch.float32
    n = rows // W
    if W == 1:
        return out, lse, 0
    recv_o = torch.empty(n, d, dtype=torch.float32, device=out.device)
    recv_l = torch.empty(n, dtype=torch.float32, device=out.device)
    for s in range(W - 1):
        send_c, recv_c = (r - s) % W, (r - s - 1) % W
        comm = SendRecv("partials", group)
        comm.send_recv(out[send_c * n:(send_c + 1) * n], recv_o)
        comm.send_recv(lse[send_c * n:(send_c + 1) * n], recv_l)
        comm.commit()
        comm.wait()
        merge_fn(out[recv_c * n:(recv_c + 1) * n], lse[recv_c * n:(recv_c + 1) * n], recv_o, recv_l)
    own = (r + 1) % W
    return out[own * n:(own + 1) * n], lse[own * n:(own + 1) * n], own


def allreduce_merge_partials(o: torch.Tensor, lse: torch.Tensor, group: Optional[dist.ProcessGroup] = None
                             ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The same merge as a sum: with M = the maximum LSE of a row over the ranks (one MAX all-reduce of the LSEs), the
    complete result is ``sum_r w_r o_r / sum_r w_r`` and ``M + log sum_r w_r`` with ``w_r = exp(lse_r - M)``, so one
    SUM all-reduce of ``[w o | w]`` finishes the job and the library is free to use its fastest algorithm (in-switch
    reduction on NVSwitch) instead of W - 1 dependent send/recv + merge steps.

    ``o`` ``[rows, d]`` (any float dtype) and ``lse`` fp32 ``[rows]``: this rank's partial result over its keys for all
    queries.  Returns fp32 ``(out [rows, d], lse [rows])``, complete and identical on every rank; rows no rank has a
    key for come back as zeros and ``-inf``."""
    rows, d = o.shape
    M = lse.clone()
    dist.all_reduce(M, op=dist.ReduceOp.MAX, group=group)
    M = torch.where(torch.isinf(M), torch.zeros_like(M), M)              # all ranks empty: any finite shift
    acc = torch.empty(rows, d + 1, dtype=torch.float32, device=o.device)
    w = torch.exp(lse - M)                                               # exp(-inf) = 0 for a rank without keys
    torch.mul(o, w[:, None], out=acc[:, :d]) if o.dtype == torch.float32 else acc[:, :d].copy_(o.float() * w[:, None])
    acc[:, d] = w
    dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=group)
    den = acc[:, d]
    out = acc[:, :d] / den.clamp_min(torch.finfo(torch.float32).tiny)[:, None]
    return out, M + torch.log(den)


class PeerExchange:
    """Buffers every rank of the group can address (PyTorch symmetric memory over NVLink) for the merge of partial
    results in one kernel: this rank's partial (o, lse) and the result buffers all ranks push finished rows into.
    ``merge`` pulls the rows this rank owns from every rank, merges them and pushes them to everyone
    (``fm_merge_peer_partials``); two small all-reduces on the same stream order the ranks around it (all partials
    complete before, all results complete after).  No multicast object is bound (plain peer loads and stores)."""

    def __init__(self, rows: int, d: int, dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerExchange serves up to 8 ranks")
        self.rows, self.d, self.dtype = rows, d, dtype
        self.o = symm.empty(rows, d, dtype=dtype, device=device)
        self.lse = symm.empty(rows, dtype=torch.float32, device=device)
        self.out = symm.empty(rows, d, dtype=torch.float32, device=device)
        self.lse_out = symm.empty(rows, dtype=torch.float32, device=device)
        import ctypes
        self._ptrs, self._handles = [], []
        for t in (self.o, self.lse, self.out, self.lse_out):
            h = symm.rendezvous(t, self.group)
            self._handles.append(h)                                           # keeps the peer mappings alive
            self._ptrs.append((ctypes.c_void_p * self.world)(*[int(x) for x in h.buffer_ptrs]))
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        n = -(-rows // self.world)
        self.row0, self.row1 = min(rows, self.rank * n), min(rows, (self.rank + 1) * n)

    def merge(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Merge what the ranks have written into ``self.o`` / ``self.lse``; returns fp32 ``(out [rows, d], lse [rows])``,
        complete on every rank.  The tensors are this object's buffers: they hold the result until the next merge."""
        dev = self.o.device
        dist.all_reduce(self._flag, group=self.group)                      # every rank's partial is complete
        L.check(L.lib().fm_merge_peer_partials(self._ptrs[0], self._ptrs[1], self._ptrs[2], self._ptrs[3], self.world,
                                               L.dtype_id(self.dtype), self.row0, self.row1, self.d, L.stream_ptr(dev)),
                "fm_merge_peer_partials")
        dist.all_reduce(self._flag, group=self.group)                      # every rank's rows have been pushed
        return self.out, self.lse_out


def reduce_scatter_merge_partials(o: torch.Tensor, lse: torch.Tensor, group: Optional[dist.ProcessGroup] = None
                                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """:func:`allreduce_merge_partials` for a caller that needs only its own rows: ``o`` ``[W, n, d]`` and ``lse`` fp32
    ``[W, n]`` are this rank's partial results for the rows of every rank (block r belongs to rank r); the MAX
    all-reduce runs on the LSEs (small), the SUM on ``[w o | w]`` is a reduce-scatter, so every rank receives and
    normalises ``n`` rows instead of ``W n``.  Returns fp32 ``(out [n, d], lse [n])`` of this rank's block."""
    W, n, d = o.shape
    r = dist.get_rank(group)
    assert W == dist.get_world_size(group) and lse.shape == (W, n)
    M = lse.clone()
    dist.all_reduce(M, op=dist.ReduceOp.MAX, group=group)
    M = torch.where(torch.isinf(M), torch.zeros_like(M), M)
    acc = torch.empty(W, n, d + 1, dtype=torch.float32, device=o.device)
    w = torch.exp(lse - M)
    torch.mul(o, w[..., None], out=acc[..., :d]) if o.dtype == torch.float32 else acc[..., :d].copy_(o.float() * w[..., None])
    acc[..., d] = w
    mine = torch.empty(n, d + 1, dtype=torch.float32, device=o.device)
    dist.reduce_scatter_tensor(mine, acc.view(W * n, d + 1), op=dist.ReduceOp.SUM, group=group)
    den = mine[:, d]
    out = mine[:, :d] / den.clamp_min(torch.finfo(torch.float32).tiny)[:, None]
    return out, M[r] + torch.log(den)


def all_gather_chunks(chunk: torch.Tensor, own: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Rank r contributes the chunk it owns (index ``own = (r + 1) % W``); returns all chunks in row order."""
    W = dist.get_world_size(group)
    if W == 1:
        return chunk
    gathered = torch.empty((W * chunk.shape[0],) + tuple(chunk.shape[1:]), dtype=chunk.dtype, device=chunk.device)
    dist.all_gather_into_tensor(gathered, chunk.contiguous(), group=group)
    # slot r of the gather holds chunk (r + 1) % W: rotate by one slot to get row order
    n = chunk.shape[0]
    return torch.cat([gathered[(W - 1) * n:], gathered[:(W - 1) * n]], 0)


class ShardedMemory:
    """A memory whose keys are cut into contiguous shards, each with its own index (local top-Z per bucket),
    spread over the ranks of a process group.  All shards share the projection matrix A, so a query is hashed
    once.  ``query`` returns the attention over the union of all shards' buckets."""

    def __init__(self):
        self.local: Optional[Memory] = None
        self.group = None
        self.n_shards = self.n_local = 0
        self._peer: Optional["PeerExchange"] = None

    @classmethod
    def build(cls, k_local: torch.Tensor, v_local: torch.Tensor, shard_len: int, *, A: torch.Tensor, bucket_size: int,
              group: Optional[dist.ProcessGroup] = None, check: bool = True) -> "ShardedMemory":
        """``k_local`` / ``v_local``: this rank's shards back to back, ``[H, n_local * shard_len, d]``.
        ``A``: ``[H, C, d]`` in the key dtype, identical on every rank."""
        H, n_total, d = k_local.shape
        if n_total % shard_len:
            raise ValueError("the local key count must be a multiple of shard_len")
        n_local = n_total // shard_len
        C = A.shape[1]
        self = cls()
        self.group = group
        self.n_local = n_local
        self.n_shards = n_local * (dist.get_world_size(group) if dist.is_initialized() else 1)
        cu = [s * shard_len for s in range(n_local + 1)]
        # one segment per (head, shard), all shards of a head sharing its A
        A_rep = A[:, None].expand(H, n_local, C, d).reshape(H, n_local * C, d).contiguous()
        per_shard = Memory.build(k_local, v_local, n_buckets=[C] * n_local, bucket_size=[bucket_size] * n_local, A=A_rep,
                                 cu_seqlens_k=cu, check=check)
        z = min(bucket_size, shard_len)
        # bucket (h, c) of the local memory = the concatenation over shards of the shard buckets (h, s, c): ascending rows
        table = per_shard.table.reshape(H, n_local, C, z).permute(0, 2, 1, 3).reshape(-1).contiguous()
        mem = Memory()
        mem.k, mem.v, mem.A = per_shard.k, per_shard.v, A.reshape(H * C, d).contiguous()
        mem.n_heads, mem.n_seq, mem.d = H, 1, d
        mem.seg_kb = [h * n_total for h in range(H + 1)]
        mem.seg_cb = [h * C for h in range(H + 1)]
        mem.seg_z = [n_local * z] * H
        mem.table_off = [h * C * n_local * z for h in range(H + 1)]
        mem.seq_buckets = [C]
        mem.cu_seqlens_k = [0, n_total]
        mem.table = table
        mem.bucket_off = torch.arange(0, (H * C + 1) * n_local * z, n_local * z, dtype=torch.int64, device=k_local.device)
        mem.max_bucket_len = n_local * z
        mem._seg_cb_dev = torch.tensor(mem.seg_cb, dtype=torch.int32, device=k_local.device)
        mem.build_status = per_shard.build_status
        mem.centroids_f32 = None
        self.local = mem
        return self

    def query_partial(self, q: torch.Tensor, sm_scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """This rank's partial result over its own shards: o in q's dtype, fp32 lse."""
        return self.local.query(q, sm_scale)

    def query(self, q: torch.Tensor, sm_scale: float, gather: bool = True, merge_fn: MergeFn = _default_merge,
              exchange: str = "ring") -> Tuple[torch.Tensor, torch.Tensor]:
        """q ``[Hq, S, d]``, the same on every rank.  Returns fp32 ``(out [Hq, S, d], lse [Hq, S])`` over all
        shards of all ranks (``gather=False``: only the rows this rank ends up owning, plus their range).

        ``exchange="ring"``: the partial results go around the ring (send/recv + merge per step, then an all-gather),
        as the reference moves its blocks (mem:307-338).  ``exchange="allreduce"``: the merge written as one MAX and
        one SUM all-reduce (:func:`allreduce_merge_partials`).  ``exchange="peer"``: the attention writes its partial
        into memory the other GPUs can address and ONE kernel per rank pulls, merges and pushes the rows it owns
        (:class:`PeerExchange`; CUDA ranks of one node) - the returned tensors are then the exchange's own buffers,
        valid until the next query."""
        Hq, S, d = q.shape
        W = dist.get_world_size(self.group) if dist.is_initialized() else 1
        rows = Hq * S
        if W > 1 and exchange == "peer":
            if not gather:
                raise ValueError("exchange='peer' returns the complete result on every rank")
            px = self._peer
            if px is None or px.rows != rows or px.d != d or px.dtype != q.dtype:
                px = self._peer = PeerExchange(rows, d, q.dtype, q.device, self.group)
            self.local.query(q, sm_scale, out=px.o.view(Hq, S, d), lse_out=px.lse.view(Hq, S))
            out, l = px.merge()
            return out.view(Hq, S, d), l.view(Hq, S)
        o, lse = self.local.query(q, sm_scale)
        if W == 1:
            return o.float(), lse
        if exchange == "allreduce":
            if not gather:
                raise ValueError("exchange='allreduce' returns the complete result on every rank")
            out, l = allreduce_merge_partials(o.reshape(rows, d), lse.reshape(rows), self.group)
            return out.reshape(Hq, S, d), l.reshape(Hq, S)
        if exchange != "ring":
            raise ValueError(f"unknown exchange {exchange!r}")
        pad = (-rows) % W
        out = torch.empty(rows + pad, d, dtype=torch.float32, device=q.device)
        out[:rows].copy_(o.reshape(rows, d))
        l = torch.full((rows + pad,), float("-inf"), dtype=torch.float32, device=q.device)
        l[:rows].copy_(lse.reshape(rows))
        if pad:
            out[rows:].zero_()
        oc, lc, own = ring_reduce_scatter_partials(out, l, self.group, merge_fn)
        if not gather:
            n = (rows + pad) // W
            return oc, lc, (own * n, min((own + 1) * n, rows))
        full_o = all_gather_chunks(oc, own, self.group)[:rows].reshape(Hq, S, d)
        full_l = all_gather_chunks(lc, own, self.group)[:rows].reshape(Hq, S)
        return full_o, full_l


    def query_sharded(self, q_local: torch.Tensor, sm_scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """The reference's own layout of the ring (mem:291-338): queries are sequence-sharded like the keys, rank r
        holds ``q_local`` ``[Hq, S / W, d]`` = positions ``[r S / W, (r + 1) S / W)`` and wants the result for them.
        The query slices are all-gathered (they are small against the keys, which never move), every rank attends
        all queries to its own shards in one pass, and the partial results are merged by a MAX all-reduce of the
        LSEs and a SUM reduce-scatter of ``[w o | w]``.  Returns fp32 ``(out [Hq, S / W, d], lse [Hq, S / W])``."""
        Hq, n, d = q_local.shape
        W = dist.get_world_size(self.group) if dist.is_initialized() else 1
        if W == 1:
            o, lse = self.local.query(q_local, sm_scale)
            return o.float(), lse
        q_all = torch.empty(W, Hq, n, d, dtype=q_local.dtype, device=q_local.device)
        dist.all_gather_into_tensor(q_all, q_local.contiguous(), group=self.group)
        # the local memory hashes head h's rows with head h's A: [Hq, W n, d], rank blocks side by side
        o, lse = self.local.query(q_all.permute(1, 0, 2, 3).reshape(Hq, W * n, d), sm_scale)
        o = o.reshape(Hq, W, n, d).permute(1, 0, 2, 3).reshape(W, Hq * n, d)
        lse = lse.reshape(Hq, W, n).permute(1, 0, 2).reshape(W, Hq * n)
        out, l = reduce_scatter_merge_partials(o, lse, self.group)
        return out.reshape(Hq, n, d), l.reshape(Hq, n)


# ---------------------------------------------------------------------------------------------------
# The reference's GLOBAL index over sharded keys (mem:260-278): top-Z of a bucket over the keys of ALL ranks
# ---------------------------------------------------------------------------------------------------
def shard_candidates(k_local: torch.Tensor, A: torch.Tensor, bucket_size: int, key_offset: int
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """This shard's candidates for the global table: its own top-Z per bucket with their canonical fp32 scores.

    ``k_local`` ``[H, L, d]``, ``A`` ``[H, C, d]`` (the same on every rank).  Returns ``(scores [H, C, Zc] fp32,
    ids [H, C, Zc] int64)``, ``Zc = min(Z, L)``, ids = ``key_offset`` + index inside the shard, ascending per bucket.
    A key of the global top-Z is in the top-Z of its own shard, so the union of these candidates holds the answer."""
    H, Lk, d = k_local.shape
    C = A.shape[1]
    mem = Memory.build(k_local, k_local, A=A, bucket_size=bucket_size)
    zc = min(bucket_size, Lk)
    scores = torch.empty(H * C * zc, dtype=torch.float32, device=k_local.device)
    L.check(L.lib().fm_table_scores(L.ptr(mem.k), L.ptr(mem.A), L.dtype_id(k_local.dtype), d, H * C, L.ptr(mem.table),
                                    L.ptr(mem.bucket_off), L.ptr(scores), L.stream_ptr(k_local.device)), "fm_table_scores")
    local = mem.table.reshape(H, C, zc).long() - (torch.arange(H, device=k_local.device) * Lk)[:, None, None]
    return scores.reshape(H, C, zc), local + key_offset


def merge_shard_candidates(scores: Sequence[torch.Tensor], ids: Sequence[torch.Tensor], bucket_size: int) -> torch.Tensor:
    """Global table from the candidates of all shards, given in shard order (ascending key offsets): per bucket the
    ``bucket_size`` best of the concatenated candidates, exact fp32 comparison, the lower key index winning a tie - the
    table a single device would build over all the keys.  Returns ``k_hashes`` ``[C, H, Z]`` int64 global key indices,
    ascending per bucket (the layout mem:128 expects)."""
    Y = torch.cat(list(scores), dim=-1)                                  # [H, C, sum Zc]
    I = torch.cat(list(ids), dim=-1)
    H, C, n = Y.shape
    pos = ops.topz_select(Y.reshape(H * C, n).contiguous(), bucket_size).long()      # positions, ascending = ids ascending
    table = torch.gather(I.reshape(H * C, n), 1, pos).reshape(H, C, -1)
    return table.permute(1, 0, 2).contiguous()


def build_global_table(k_local: torch.Tensor, A: torch.Tensor, bucket_size: int,
                       group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """The index build of the reference's distributed path (mem:260-278) without moving the score matrix: every rank
    selects inside its own key shard on the index-build kernels, the ``(score, key)`` candidates - Z per bucket and rank
    instead of the shard's whole row of Y - are all-gathered, and one exact row select finishes the table on every rank.
    ``k_local`` ``[H, L, d]`` is rank r's contiguous shard ``[r L, (r + 1) L)`` of the keys."""
    W = dist.get_world_size(group) if dist.is_initialized() else 1
    r = dist.get_rank(group) if dist.is_initialized() else 0
    sc, idx = shard_candidates(k_local, A, bucket_size, r * k_local.shape[1])
    if W == 1:
        return merge_shard_candidates([sc], [idx], bucket_size)
    all_sc = torch.empty((W,) + tuple(sc.shape), dtype=sc.dtype, device=sc.device)
    all_id = torch.empty((W,) + tuple(idx.shape), dtype=idx.dtype, device=idx.device)
    dist.all_gather_into_tensor(all_sc, sc.contiguous(), group=group)
    dist.all_gather_into_tensor(all_id, idx.contiguous(), group=group)
    return merge_shard_candidates(list(all_sc), list(all_id), bucket_size)


def query_global_table(k_hashes: torch.Tensor, A: torch.Tensor, q: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                       sm_scale: float, group: Optional[dist.ProcessGroup] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """All queries against a globally indexed, key-sharded memory (the forward of mem:291-338 with the key blocks staying
    where they are): hash with the shared ``A``, attend to the table entries that fall into this rank's shard
    (:func:`fast_memory_b200.ops.ring_attention_masked_forward`), merge the ranks' partial results.
    ``q`` ``[Hq, S, d]``, ``k_local`` / ``v_local`` ``[H, L, d]``; returns fp32 ``(out [Hq, S, d], lse [Hq, S])``."""
    W = dist.get_world_size(group) if dist.is_initialized() else 1
    r = dist.get_rank(group) if dist.is_initialized() else 0
    Hq, S, d = q.shape
    H = k_local.shape[0]
    C = A.shape[1]
    seg_xb = torch.arange(0, (H + 1) * (Hq // H) * S, (Hq // H) * S, dtype=torch.int32, device=q.device)
    seg_cb = torch.arange(0, (H + 1) * C, C, dtype=torch.int32, device=q.device)
    hashes = ops.hash_rows(q.reshape(Hq * S, d), A.reshape(H * C, d).contiguous(), seg_xb, seg_cb, (Hq // H) * S)
    o, lse = ops.ring_attention_masked_forward(k_hashes, hashes.reshape(H, Hq // H, S).long(), q[None], k_local[None],
                                               v_local[None], sm_scale, r)
    # the drop-in returns the reference's convention (lse in q's dtype, finfo.min for an empty bucket): back to fp32 / -inf
    lse = lse[0].float()
    lse = torch.where(lse <= torch.finfo(q.dtype).min, torch.full_like(lse, float("-inf")), lse)
    if W == 1:
        return o[0].float(), lse
    out, l = allreduce_merge_partials(o[0].reshape(Hq * S, d), lse.reshape(Hq * S), group)
    return out.reshape(Hq, S, d), l.reshape(Hq, S)

