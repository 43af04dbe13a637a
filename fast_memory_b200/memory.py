"""The memory module: build an LSH index over past keys/values, query it, get (O, LSE) back for merging.

The reference describes this object (README.md:7) but ships it only as loose steps inside its training
code (mem:252-283 build + hash, mem:319-332 attend + merge).  :class:`Memory` packages those steps:

    mem = Memory.build(k, v, n_buckets=512, bucket_size=2048, kmeans_iters=2, kmeans_init=q)
    o, lse = mem.query(q, sm_scale)            # o in q's dtype, lse fp32 natural log
    out, lse = merge(o_local, lse_local, o, lse)

Layout.  ``k`` / ``v`` are ``[H, N, d]`` (H = KV heads) or, for packed variable-length memories,
``[H, N_total, d]`` with ``cu_seqlens_k``; one SEGMENT per (head, sequence).  Segment s owns buckets
``seg_cb[s]:seg_cb[s+1]`` of the packed projection matrix ``A [total_buckets, d]`` and a slice of the flat
bucket table of ABSOLUTE key rows (ascending inside a bucket).  Queries ``[Hq, S, d]`` with Hq a multiple
of H fold their GQA group into the query axis (as mem:134 does).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import functools
import warnings

import numpy as np
import torch

from . import _lib as L
from . import ops

IntOrSeq = Union[int, Sequence[int]]


def _per_seq(val: IntOrSeq, n_seq: int, name: str) -> List[int]:
    if isinstance(val, int):
        return [val] * n_seq
    vals = [int(x) for x in val]
    if len(vals) != n_seq:
        raise ValueError(f"{name}: expected {n_seq} entries, got {len(vals)}")
    return vals


def kmeans_projection(x: torch.Tensor, init: torch.Tensor, iters: int, seg_xb: Sequence[int],
                      seg_cb: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Spherical k-means per segment (README.md:37-45).

    x ``[rows, d]``; ``init [total_buckets, d]`` initial centroids (any scale, normalised here);
    ``seg_xb`` / ``seg_cb``: python prefix lists.  Returns (A in x's dtype, fp32 centroids).
    """
    dev = L.require_cuda(x, init)
    d = x.shape[1]
    cent = ops.unit_rows(init.to(x.dtype).contiguous())
    A = torch.empty(cent.shape, dtype=x.dtype, device=dev)
    n_seg = len(seg_xb) - 1
    xb, cb = L.host_i64(seg_xb), L.host_i64(seg_cb)
    need = L.lib().fm_kmeans_workspace_bytes(n_seg, xb, cb, d)
    ws = ops._ws.get("kmeans", need, dev)
    L.check(L.lib().fm_kmeans(L.ptr(x), L.dtype_id(x.dtype), d, n_seg, xb, cb, int(iters), L.ptr(cent), L.ptr(A),
                              L.ptr(ws), ws.numel(), L.stream_ptr(dev)), "fm_kmeans")
    return A, cent


def compute_centroids(kq: torch.Tensor, centroids: torch.Tensor, n_hashes: int, n_groups: int,
                      centroid_topk: int) -> torch.Tensor:
    """The projection-matrix construction of the reference's CODE (``compute_centroids``, mem:209-231; its README
    describes k-means instead, see :func:`kmeans_projection`): rows are put on the unit sphere (in ``kq``'s dtype, as
    mem:215-217 divides there), every centroid takes its ``centroid_topk`` nearest rows in each head, and the rows of
    the ``n_groups`` heads that share a KV head are averaged.

    ``kq`` ``[n_heads, ctx, d]``, ``centroids`` ``[n_hashes, d]`` -> ``[n_hashes, n_heads // n_groups, d]`` in ``kq``'s
    dtype.  The top-k runs on the index-build kernels (a table with ``Z = centroid_topk``; exact fp32 ranking, lower row
    wins a tie), the gather + mean in ``fm_gather_mean``."""
    dev = L.require_cuda(kq, centroids)
    H, ctx, d = kq.shape
    if H % n_groups or centroids.shape != (n_hashes, d):
        raise ValueError("compute_centroids: n_heads must be a multiple of n_groups and centroids [n_hashes, d]")
    if centroid_topk > ctx:
        raise ValueError("compute_centroids: centroid_topk exceeds the context length")
    k_heads = H // n_groups
    U = ops.unit_rows(kq.contiguous())                                   # fp32 [H, ctx, d]
    x = U.to(kq.dtype)
    A = centroids.to(kq.dtype).unsqueeze(0).expand(H, n_hashes, d).contiguous()
    mem = Memory.build(x, x, A=A, bucket_size=centroid_topk)
    # table rows of (head h, centroid z) -> the lists of (z, kv head): its n_groups heads back to back
    t = mem.table.reshape(k_heads, n_groups, n_hashes, centroid_topk).permute(2, 0, 1, 3).contiguous()
    xf = x.reshape(H * ctx, d) if x.dtype == torch.float32 else x.reshape(H * ctx, d).float()
    out = torch.empty(n_hashes * k_heads, d, dtype=torch.float32, device=dev)
    L.check(L.lib().fm_gather_mean(L.ptr(xf), xf.shape[0], d, L.ptr(t), out.shape[0], n_groups * centroid_topk, L.ptr(out),
                                   L.stream_ptr(dev)), "fm_gather_mean")
    return out.reshape(n_hashes, k_heads, d).to(kq.dtype)



class _SegmentLayout:
    """Host arrays of a memory's shape (heads x sequences): prefix arrays of key rows, buckets and table entries, as
    python lists and as the ctypes arrays the library takes.  Depends on the shape only, so it is made once per shape
    (the index build is short enough for this bookkeeping to show in its time)."""

    def __init__(self, H: int, cu: Tuple[int, ...], Cs: Tuple[int, ...], Zs: Tuple[int, ...]):
        n_seq, N_total = len(cu) - 1, cu[-1]
        self.seg_kb = [h * N_total + cu[s] for h in range(H) for s in range(n_seq)] + [H * N_total]
        self.seq_zc = [min(Zs[s], cu[s + 1] - cu[s]) for s in range(n_seq)]
        self.seg_c = np.tile(np.asarray(Cs, dtype=np.int64), H)                   # buckets of every segment
        self.seg_zc = np.tile(np.asarray(self.seq_zc, dtype=np.int64), H)         # keys per bucket of every segment
        self.seg_cb = [0] + np.cumsum(self.seg_c).tolist()
        self.seg_z = [Zs[s] for _ in range(H) for s in range(n_seq)]
        self.table_off = [0] + np.cumsum(self.seg_c * self.seg_zc).tolist()
        self.c_kb, self.c_cb = L.host_i64(self.seg_kb), L.host_i64(self.seg_cb)
        self.c_z, self.c_to = L.host_i64(self.seg_z), L.host_i64(self.table_off[:-1])
        self.ws_need = {}                                                         # (d, dtype, flags) -> build workspace bytes


@functools.lru_cache(maxsize=32)
def _segment_layout(H: int, cu: Tuple[int, ...], Cs: Tuple[int, ...], Zs: Tuple[int, ...]) -> _SegmentLayout:
    return _SegmentLayout(H, cu, Cs, Zs)


# (bucket_off, seg_cb) device tensors per (device, stream, heads, buckets per sequence, keys per bucket): see Memory.build
_PREFIX_CACHE: dict = {}

class Memory:
    """An indexed set of keys/values.  Create with :meth:`build`.

    Streams.  Every call runs on the current CUDA stream.  Scratch buffers are kept per stream, so calls on different
    streams may overlap; results are ordered like any other work on their stream.  A memory's own tensors (table, A)
    are written by :meth:`build` on the stream it ran on: make other streams wait for that stream before they query."""

    def __init__(self):
        self.k = self.v = self.A = None
        self.table = self.bucket_off = None
        self.seg_kb: List[int] = []
        self.seg_cb: List[int] = []
        self.seg_z: List[int] = []
        self.table_off: List[int] = []
        self.n_heads = self.n_seq = self.d = 0
        self.max_bucket_len = 0
        self.compacted = False             # True once key_range dropped entries: buckets are ragged, table_off is void
        self._seg_cb_dev = None
        self._q_seg_cache = {}

    # ---- construction ----------------------------------------------------------------------------
    @classmethod
    def build(cls, k: torch.Tensor, v: torch.Tensor, *, n_buckets: Optional[IntOrSeq] = None,
              bucket_size: IntOrSeq, A: Optional[torch.Tensor] = None, kmeans_iters: int = 2,
              kmeans_init: Optional[torch.Tensor] = None, cu_seqlens_k: Optional[Sequence[int]] = None,
              key_range: Optional[Tuple[int, int]] = None, check: bool = True, exact_only: bool = False,
              fallback_exact: bool = True) -> "Memory":
        """Index ``k`` / ``v``.

        :param k, v: ``[H, N, d]`` (or ``[H, N_total, d]`` with ``cu_seqlens_k``)
        :param n_buckets: C per sequence (int or one per sequence); not needed when ``A`` is given
        :param bucket_size: Z per sequence; a bucket holds ``min(Z, N_seq)`` keys
        :param A: projection matrix ``[H, C, d]`` (``[H, sum(C), d]`` packed per sequence when varlen) in k's
            dtype.  If omitted it is built by spherical k-means with ``kmeans_iters`` iterations from
            ``kmeans_init``
        :param kmeans_init: rows whose first C (per segment) seed the centroids: ``[H, >=C, d]`` (varlen:
            packed like A).  Defaults to the first C keys of each segment
        :param check: read the build's status word back (one device sync) and raise if the tensor-core path
            gave up; pass False to stay asynchronous and call :meth:`check_build` later
        :param exact_only: score every key with the fp32 chain instead of the tensor-core filter
        :param fallback_exact: with ``check``, when the tensor-core filter reports that too many buckets need the exact
            fallback (status 4: masses of equal scores, key order far from stationary) the table is rebuilt with
            ``exact_only`` and a warning instead of raising
        :param key_range: keep only table entries whose per-head key index lies in ``[lo, hi)`` (the
            filter the reference hard-codes at tk:283); uniform memories only
        """
        dev = L.require_cuda(k, v, A, kmeans_init)
        if k.dim() != 3 or v.shape != k.shape:
            raise ValueError(f"k and v must be [H, N, d] with equal shapes, got {tuple(k.shape)} {tuple(v.shape)}")
        if k.dtype != v.dtype:
            raise TypeError("k and v must share a dtype")
        H, N_total, d = k.shape
        cu = [0, N_total] if cu_seqlens_k is None else [int(x) for x in cu_seqlens_k]
        if cu[0] != 0 or cu[-1] != N_total or any(b < a for a, b in zip(cu, cu[1:])):
            raise ValueError("cu_seqlens_k must rise from 0 to the packed key count")
        n_seq = len(cu) - 1
        self = cls()
        self.k, self.v = k.contiguous(), v.contiguous()
        self.n_heads, self.n_seq, self.d = H, n_seq, d
        self.cu_seqlens_k = cu
        if A is not None and n_buckets is None:
            if n_seq != 1:
                raise ValueError("n_buckets is needed with a packed A")
            n_buckets = A.shape[1]
        if n_buckets is None:
            raise ValueError("n_buckets or A must be given")
        Cs = _per_seq(n_buckets, n_seq, "n_buckets")
        Zs = _per_seq(bucket_size, n_seq, "bucket_size")
        # segments tile the flat [H * N_total] key rows: segment (h, s) starts at h * N_total + cu[s]
        lay = _segment_layout(H, tuple(cu), tuple(Cs), tuple(Zs))
        seg_kb, seg_cb, seg_z, table_off = lay.seg_kb, lay.seg_cb, lay.seg_z, lay.table_off
        seq_zc, seg_c, seg_zc = lay.seq_zc, lay.seg_c, lay.seg_zc
        self.seg_kb, self.seg_cb, self.seg_z, self.table_off = list(seg_kb), list(seg_cb), list(seg_z), list(table_off)
        self.seq_buckets = Cs
        total_c = seg_cb[-1]
        c_per_head = total_c // H
        n_seg = H * n_seq
        kf = self.k.reshape(H * N_total, d)

        if A is None:
            if kmeans_init is None:
                init = torch.cat([kf[seg_kb[i]: seg_kb[i] + (seg_cb[i + 1] - seg_cb[i])] for i in range(n_seg)], 0)
                if init.shape[0] != total_c:
                    raise ValueError("a segment has fewer keys than buckets: pass kmeans_init")
            else:
                init = kmeans_init
                if init.dim() == 3:
                    if n_seq == 1:
                        init = init[:, :c_per_head]
                    init = init.reshape(-1, d)
                if init.shape[0] != total_c:
                    raise ValueError(f"kmeans_init must provide {total_c} rows, got {init.shape[0]}")
            A2, self.centroids_f32 = kmeans_projection(kf, init, kmeans_iters, seg_kb, seg_cb)
        else:
            if A.dtype != k.dtype:
                raise TypeError(f"A ({A.dtype}) must be in the key dtype ({k.dtype})")
            A2 = A.reshape(-1, d).contiguous()
            if A2.shape[0] != total_c:
                raise ValueError(f"A must have {total_c} rows in total, got {A2.shape[0]}")
            self.centroids_f32 = None
        self.A = A2

        table = torch.empty(max(table_off[-1], 1), dtype=torch.int32, device=dev)
        kb, cb, zz, to = lay.c_kb, lay.c_cb, lay.c_z, lay.c_to
        flags = 1 if exact_only else 0
        need = lay.ws_need.get((d, k.dtype, flags))
        if need is None:
            need = lay.ws_need[(d, k.dtype, flags)] = L.lib().fm_index_build_workspace_bytes(n_seg, kb, cb, zz, d, L.dtype_id(k.dtype), flags)
        ws = ops._ws.get("build", need, dev)
        def launch(fl):
            L.check(L.lib().fm_index_build(L.ptr(kf), L.ptr(A2), L.dtype_id(k.dtype), d, n_seg, kb, cb, zz, to,
                                           L.ptr(table), fl, L.ptr(ws), ws.numel(), L.stream_ptr(dev)), "fm_index_build")
            return ws[:4].view(torch.int32)[0].clone()           # device scalar: 0 = ok (see check_build)

        self.build_status = launch(flags)
        self.table = table
        # the prefix arrays are made on the host while the device builds the table; they depend on the shape of the memory
        # only, so memories of a shape seen before (on this stream) share them and their copies leave the build's tail
        key = (dev, torch.cuda.current_stream(dev).cuda_stream, H, tuple(Cs), tuple(seq_zc))
        hit = _PREFIX_CACHE.get(key)
        if hit is None:
            bucket_off = np.zeros(total_c + 1, dtype=np.int64)
            np.cumsum(np.repeat(seg_zc, seg_c), out=bucket_off[1:])
            hit = (torch.from_numpy(bucket_off).to(dev, non_blocking=True),
                   torch.tensor(seg_cb, dtype=torch.int32).to(dev, non_blocking=True))
            if len(_PREFIX_CACHE) >= 16:
                _PREFIX_CACHE.pop(next(iter(_PREFIX_CACHE)))
            _PREFIX_CACHE[key] = hit
        self.bucket_off, self._seg_cb_dev = hit                # (never written: compaction and append make new tensors)
        self.max_bucket_len = int(seg_zc.max()) if total_c else 0
        if check:
            if fallback_exact and not exact_only and int(self.build_status.item()) == 4:
                # first with one candidate buffer per bucket (key positions far from stationary overflow the per-range
                # buffers), then without the filter
                self.build_status = launch(2)
            if fallback_exact and not exact_only and int(self.build_status.item()) == 4:
                warnings.warn("index build: the tensor-core filter handed too many buckets to its fallback; "
                              "rebuilding the table with the exact fp32 path", RuntimeWarning)
                need_exact = L.lib().fm_index_build_workspace_bytes(n_seg, kb, cb, zz, d, L.dtype_id(k.dtype), 1)
                ws = ops._ws.get("build", need_exact, dev)
                self.build_status = launch(1)
            self.check_build()
        if key_range is not None:
            self._apply_key_range(key_range)
        return self

    def check_build(self) -> None:
        """Raise if the index build reported a failure (synchronises with the device)."""
        status = int(self.build_status.item())
        if status:
            raise L.FastMemError(f"index build failed with status {status}: rebuild with exact_only=True")

    def _apply_key_range(self, key_range):
        """Keep table entries whose per-head key index is in [lo, hi) (compaction like tk:283-286)."""
        if self.n_seq != 1:
            raise ValueError("key_range applies to uniform memories only")
        lo, hi = key_range
        N = self.k.shape[1]
        C = self.seq_buckets[0]
        z = min(self.seg_z[0], N)
        t = self.table.reshape(self.n_heads, C, z)
        local = t - (torch.arange(self.n_heads, device=t.device, dtype=torch.int32) * N)[:, None, None]
        m = torch.logical_and(local >= lo, local < hi)
        counts = m.sum(-1).reshape(-1).to(torch.int64)
        self.table = t[m].contiguous()
        if self.table.numel() == 0:
            self.table = torch.zeros(1, dtype=torch.int32, device=t.device)
        off = torch.zeros(counts.numel() + 1, dtype=torch.int64, device=t.device)
        torch.cumsum(counts, 0, out=off[1:])
        self.bucket_off = off
        # buckets are ragged from here on: the fixed-Z views (table_of, append) no longer apply
        self.compacted = True
        self.table_off = []

    # ---- views -------------------------------------------------------------------------------------
    @property
    def total_buckets(self) -> int:
        return self.seg_cb[-1]

    def table_of(self, head: int, seq: int = 0) -> torch.Tensor:
        """``[C, min(Z, N)]`` int32 table of one segment as indices LOCAL to the segment's keys."""
        if self.compacted:
            raise ValueError("table_of: key_range compacted this memory's table (ragged buckets): slice `table` with `bucket_off`")
        s = head * self.n_seq + seq
        C = self.seg_cb[s + 1] - self.seg_cb[s]
        t = self.table[self.table_off[s]: self.table_off[s + 1]].reshape(C, -1)
        return t - self.seg_kb[s]

    def projection_of(self, head: int, seq: int = 0) -> torch.Tensor:
        s = head * self.n_seq + seq
        return self.A[self.seg_cb[s]: self.seg_cb[s + 1]]

    # ---- query -------------------------------------------------------------------------------------
    def _query_segments(self, Hq: int, S_total: int, cu_q: Optional[Sequence[int]], dev):
        key = (Hq, S_total, None if cu_q is None else tuple(cu_q))
        hit = self._q_seg_cache.get(key)
        if hit is None:
            G = Hq // self.n_heads
            if cu_q is None:
                if self.n_seq != 1:
                    raise ValueError("a packed memory needs cu_seqlens_q")
                xb = [h * G * S_total for h in range(self.n_heads + 1)]
                max_rows = G * S_total
            else:
                cu = [int(x) for x in cu_q]
                if len(cu) != self.n_seq + 1 or cu[0] != 0 or cu[-1] != S_total:
                    raise ValueError("cu_seqlens_q must have one entry per sequence plus one and end at the query count")
                if G != 1:
                    raise ValueError("packed queries with grouped heads are not supported: fold the group first")
                xb = [h * S_total + cu[s] for h in range(self.n_heads) for s in range(self.n_seq)] + [Hq * S_total]
                max_rows = max(b - a for a, b in zip(cu, cu[1:]))
            hit = (torch.tensor(xb, dtype=torch.int32, device=dev), max_rows)
            self._q_seg_cache[key] = hit
        return hit

    def hash_queries(self, q: torch.Tensor, cu_seqlens_q: Optional[Sequence[int]] = None) -> torch.Tensor:
        """int32 LOCAL bucket of every query, shaped like ``q`` without its last dim (README.md:29)."""
        Hq, S, d = q.shape
        seg_xb, max_rows = self._query_segments(Hq, S, cu_seqlens_q, q.device)
        h = ops.hash_rows(q.reshape(Hq * S, d), self.A, seg_xb, self._seg_cb_dev, max_rows)
        return h.reshape(Hq, S)

    def query(self, q: torch.Tensor, sm_scale: float, cu_seqlens_q: Optional[Sequence[int]] = None,
              q_hashes: Optional[torch.Tensor] = None, key_chunk: int = 0,
              head_range: Optional[Tuple[int, int]] = None, out: Optional[torch.Tensor] = None,
              lse_out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """q ``[Hq, S, d]`` -> (o ``[Hq, S, d]`` in q's dtype, lse ``[Hq, S]`` fp32 natural log; ``-inf``
        and o = 0 where the query's bucket is empty).  ``head_range = (h0, h1)``: ``q`` holds only the queries of
        KV heads ``h0 .. h1-1`` (uniform memories; heads are independent, so a batch can be served in slices).
        ``out`` / ``lse_out``: contiguous tensors of the result's shapes and dtypes to write into (e.g. buffers other
        GPUs can address)."""
        dev = L.require_cuda(q)
        n_heads = self.n_heads if head_range is None else head_range[1] - head_range[0]
        if head_range is not None and (self.n_seq != 1 or cu_seqlens_q is not None or not 0 <= head_range[0] < head_range[1] <= self.n_heads):
            raise ValueError("head_range needs a uniform memory and 0 <= h0 < h1 <= n_heads")
        if q.dim() != 3 or q.shape[2] != self.d or q.shape[0] % n_heads:
            raise ValueError(f"q must be [Hq, S, {self.d}] with Hq a multiple of {n_heads}, got {tuple(q.shape)}")
        if q.dtype != self.k.dtype:
            raise TypeError(f"q ({q.dtype}) must be in the memory's dtype ({self.k.dtype})")
        q = q.contiguous()
        Hq, S, d = q.shape
        if head_range is None:
            seg_xb, max_rows = self._query_segments(Hq, S, cu_seqlens_q, dev)
            seg_cb = self._seg_cb_dev
        else:
            key = ("range", Hq, S, n_heads)
            hit = self._q_seg_cache.get(key)
            if hit is None:
                rows = (Hq // n_heads) * S
                hit = (torch.arange(0, (n_heads + 1) * rows, rows, dtype=torch.int32, device=dev), rows)
                self._q_seg_cache[key] = hit
            seg_xb, max_rows = hit
            seg_cb = self._seg_cb_dev[head_range[0]: head_range[1] + 1]
        qf = q.reshape(Hq * S, d)
        if q_hashes is None:
            hashes = ops.hash_rows(qf, self.A, seg_xb, seg_cb, max_rows)
        else:
            hashes = q_hashes.reshape(-1).to(torch.int32).contiguous()
        # hashes made by the hash kernel lie inside their segment's buckets: the one-launch grouping applies
        group_off, perm = ops.group_rows(hashes, self.total_buckets, seg_xb, seg_cb, in_range=q_hashes is None,
                                         max_seg_rows=max_rows, max_seg_buckets=max(self.seq_buckets))
        if out is not None or lse_out is not None:
            if out is None or lse_out is None or out.dtype != q.dtype or lse_out.dtype != torch.float32 or \
                    out.numel() != q.numel() or lse_out.numel() != Hq * S or not out.is_contiguous() or not lse_out.is_contiguous():
                raise ValueError("out / lse_out must both be given, contiguous, shaped like the result, in q's dtype / float32")
            if q_hashes is not None:                             # caller-made hashes may fall outside the buckets
                out.zero_()
                lse_out.fill_(float("-inf"))
        o, lse = ops.hashed_attention(qf, self.k.reshape(-1, d), self.v.reshape(-1, d), self.table, self.bucket_off,
                                      group_off, perm, sm_scale, self.max_bucket_len, key_chunk=key_chunk,
                                      out=None if out is None else out.view(Hq * S, d),
                                      lse=None if lse_out is None else lse_out.view(Hq * S),
                                      prefill=q_hashes is not None)       # caller-made hashes may fall outside the buckets
        return o.reshape(Hq, S, d), lse.reshape(Hq, S)

    def query_backward(self, q: torch.Tensor, sm_scale: float, out: torch.Tensor, lse: torch.Tensor, d_out: torch.Tensor,
                       cu_seqlens_q: Optional[Sequence[int]] = None, q_hashes: Optional[torch.Tensor] = None,
                       dk: Optional[torch.Tensor] = None, dv: Optional[torch.Tensor] = None
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Gradients of :meth:`query` w.r.t. q, k and v for the output gradient ``d_out`` (mem:166-206): ``out`` and
        ``lse`` are the forward result the caller ended up with (of this memory alone, or merged with other attention:
        mem:332, 354-378 pass the merged pair).  Returns fp32 ``(dq [Hq, S, d], dk [H, N, d], dv [H, N, d])``; ``dk`` /
        ``dv`` given are accumulated into.  The projection (hashing) is not differentiated, as in the reference."""
        dev = L.require_cuda(q, out, lse, d_out)
        q = q.contiguous()
        Hq, S, d = q.shape
        seg_xb, max_rows = self._query_segments(Hq, S, cu_seqlens_q, dev)
        qf = q.reshape(Hq * S, d)
        hashes = ops.hash_rows(qf, self.A, seg_xb, self._seg_cb_dev, max_rows) if q_hashes is None else \
            q_hashes.reshape(-1).to(torch.int32).contiguous()
        group_off, perm = ops.group_rows(hashes, self.total_buckets, seg_xb, self._seg_cb_dev)
        dq, dk, dv = ops.hashed_attention_backward(
            qf, self.k.reshape(-1, d), self.v.reshape(-1, d), self.table, self.bucket_off, group_off, perm, sm_scale,
            out.reshape(Hq * S, d).contiguous(), lse.reshape(Hq * S).float().contiguous(), d_out.reshape(Hq * S, d).contiguous(),
            dk=None if dk is None else dk.reshape(-1, d), dv=None if dv is None else dv.reshape(-1, d))
        return dq.reshape(Hq, S, d), dk.reshape(self.k.shape), dv.reshape(self.k.shape)

    def query_from_host(self, q_host: torch.Tensor, sm_scale: float, o_host: torch.Tensor, lse_host: torch.Tensor,
                        n_chunks: int = 4, local: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                        overlap_calls: bool = False) -> None:
        """Serve queries that live in pinned HOST memory and leave the result in pinned host memory, overlapping the
        copies with the kernels: the KV heads are cut into ``n_chunks`` slices; slice i + 1 is copied in and slice
        i - 1 copied out while slice i is attended.

        ``q_host`` ``[Hq, S, d]`` (memory dtype), ``o_host`` ``[Hq, S, d]`` (memory dtype), ``lse_host`` ``[Hq, S]`` fp32,
        all pinned.  ``local = (o_local, lse_local)``: fp32 device tensors of a second attention result over other keys
        (e.g. a local window) to LSE-merge with the memory's result before it is copied out (mem:332).
        Returns after the work is enqueued; synchronise the current stream before reading the host tensors.

        ``overlap_calls=True`` lets consecutive calls overlap as well (the next call's first copy-in runs under this
        call's kernels, this call's last copy-out under the next call's): the device queries are staged in two
        alternating buffers, and the current stream no longer waits for the copy-out - call
        :meth:`finish_host_queries` (or synchronise the device) before reading the host tensors."""
        if self.n_seq != 1:
            raise ValueError("query_from_host serves uniform memories")
        for t in (q_host, o_host, lse_host):
            if not t.is_pinned():
                raise ValueError("host tensors must be pinned")
        dev = self.k.device
        Hq, S, d = q_host.shape
        G = Hq // self.n_heads
        n_chunks = max(1, min(n_chunks, self.n_heads))
        bounds = [round(i * self.n_heads / n_chunks) for i in range(n_chunks + 1)]
        main = torch.cuda.current_stream(dev)
        if not hasattr(self, "_copy_streams"):
            self._copy_streams = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
            self._stage = [None, None]                       # device copies of the queries, used alternately
            self._stage_free = [None, None]                  # recorded when the kernels that read a stage are enqueued
            self._stage_next = 0
        s_in, s_out = self._copy_streams
        slot = self._stage_next
        self._stage_next ^= 1
        q_dev = self._stage[slot]
        if q_dev is None or q_dev.shape != q_host.shape or q_dev.dtype != q_host.dtype:
            s_in.wait_stream(main)
            with torch.cuda.stream(s_in):                    # allocated on the copy stream: reuse is ordered there
                q_dev = self._stage[slot] = torch.empty(Hq, S, d, dtype=q_host.dtype, device=dev)
        if self._stage_free[slot] is not None:
            s_in.wait_event(self._stage_free[slot])          # the kernels of two calls ago have read this stage
        if not overlap_calls:
            s_in.wait_stream(main)
        ev_in = []
        with torch.cuda.stream(s_in):
            for i in range(n_chunks):
                a, b = bounds[i] * G, bounds[i + 1] * G
                q_dev[a:b].copy_(q_host[a:b], non_blocking=True)
                e = torch.cuda.Event()
                e.record(s_in)
                ev_in.append(e)
        for i in range(n_chunks):
            a, b = bounds[i] * G, bounds[i + 1] * G
            main.wait_event(ev_in[i])
            o, lse = self.query(q_dev[a:b], sm_scale, head_range=(bounds[i], bounds[i + 1]))
            if local is not None:
                o, lse = ops.lse_merge_out(local[0][a:b], local[1][a:b], o, lse, out_dtype=q_host.dtype)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                o_host[a:b].copy_(o, non_blocking=True)
                lse_host[a:b].copy_(lse, non_blocking=True)
            o.record_stream(s_out)
            lse.record_stream(s_out)
        free = torch.cuda.Event()
        free.record(main)
        self._stage_free[slot] = free
        if not overlap_calls:
            main.wait_stream(s_out)

    def finish_host_queries(self) -> None:
        """Make the current stream wait for the copy-outs of earlier :meth:`query_from_host` calls."""
        if hasattr(self, "_copy_streams"):
            torch.cuda.current_stream(self.k.device).wait_stream(self._copy_streams[1])

    # ---- persistence ---------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return dict(A=self.A, table=self.table, bucket_off=self.bucket_off, seg_kb=self.seg_kb, seg_cb=self.seg_cb,
                    seg_z=self.seg_z, table_off=self.table_off, n_heads=self.n_heads, n_seq=self.n_seq, d=self.d,
                    max_bucket_len=self.max_bucket_len, seq_buckets=self.seq_buckets,
                    cu_seqlens_k=self.cu_seqlens_k, compacted=self.compacted)

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor) -> "Memory":
        """A memory over the old keys followed by ``k_new`` / ``v_new`` (``[H, N_new, d]``; uniform memories), with the
        same projection and bucket size, WITHOUT indexing the old keys again: a key of the new top-Z is either in the old
        table or in the top-Z of the new block, so the old entries (re-scored with the canonical chain,
        ``fm_table_scores``) and the new block's own top-Z are merged by one exact row select.  The table equals the one
        a full build over all the keys gives.  Returns a new ``Memory``; this one stays valid."""
        from .dist import merge_shard_candidates, shard_candidates
        if self.n_seq != 1 or self.compacted:
            raise ValueError("append serves uniform memories whose table was not compacted by key_range")
        dev = L.require_cuda(k_new, v_new)
        H, N, d = self.k.shape
        if k_new.dim() != 3 or k_new.shape[0] != H or k_new.shape[2] != d or v_new.shape != k_new.shape or k_new.dtype != self.k.dtype:
            raise ValueError("append: k_new / v_new must be [H, N_new, d] in the memory's dtype")
        C, Z = self.seq_buckets[0], self.seg_z[0]
        zc_old = min(Z, N)
        A3 = self.A.reshape(H, C, d)
        old_scores = torch.empty(H * C * zc_old, dtype=torch.float32, device=dev)
        L.check(L.lib().fm_table_scores(L.ptr(self.k), L.ptr(self.A), L.dtype_id(self.k.dtype), d, H * C, L.ptr(self.table),
                                        L.ptr(self.bucket_off), L.ptr(old_scores), L.stream_ptr(dev)), "fm_table_scores")
        old_ids = self.table.reshape(H, C, zc_old).long() - (torch.arange(H, device=dev) * N)[:, None, None]
        new_scores, new_ids = shard_candidates(k_new.contiguous(), A3, Z, N)
        k_hashes = merge_shard_candidates([old_scores.reshape(H, C, zc_old), new_scores], [old_ids, new_ids], Z)   # [C, H, Z']
        N2 = N + k_new.shape[1]
        zc = k_hashes.shape[2]
        out = Memory()
        out.k, out.v = torch.cat([self.k, k_new], 1), torch.cat([self.v, v_new], 1)
        out.n_heads, out.n_seq, out.d = H, 1, d
        out.cu_seqlens_k = [0, N2]
        out.seg_kb = [h * N2 for h in range(H + 1)]
        out.seg_cb, out.seg_z, out.seq_buckets = list(self.seg_cb), list(self.seg_z), list(self.seq_buckets)
        out.table_off = [h * C * zc for h in range(H + 1)]
        out.A, out.centroids_f32 = self.A, self.centroids_f32
        out.table = (k_hashes.permute(1, 0, 2) + (torch.arange(H, device=dev) * N2)[:, None, None]).to(torch.int32).reshape(-1).contiguous()
        out.bucket_off = torch.arange(0, (H * C + 1) * zc, zc, dtype=torch.int64, device=dev)
        out.max_bucket_len = zc
        out.build_status = torch.zeros((), dtype=torch.int32, device=dev)
        out._seg_cb_dev = self._seg_cb_dev
        return out

    @classmethod
    def from_state_dict(cls, state: dict, k: torch.Tensor, v: torch.Tensor) -> "Memory":
        """A memory over ``k`` / ``v`` (the keys and values the state was built from) with the saved index; the index
        tensors are moved to ``k``'s device wherever the state was loaded to."""
        dev = L.require_cuda(k, v)
        self = cls()
        for name, val in state.items():
            setattr(self, name, val.to(dev) if isinstance(val, torch.Tensor) else val)
        if self.seg_kb[-1] != k.shape[0] * k.shape[1] or k.shape[2] != self.d or v.shape != k.shape:
            raise ValueError("from_state_dict: k / v do not have the shape the index was built for")
        self.k, self.v = k.contiguous(), v.contiguous()
        self.centroids_f32 = None
        self.build_status = torch.zeros((), dtype=torch.int32, device=dev)
        self._seg_cb_dev = torch.tensor(self.seg_cb, dtype=torch.int32, device=dev)
        return self


def merge(o1: torch.Tensor, lse1: torch.Tensor, o2: torch.Tensor, lse2: torch.Tensor
          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """LSE-merge two partial attention results over disjoint key sets (mem:54-71): returns fp32
    ``(out, lse)``; ``o*`` are ``[..., d]``, ``lse*`` are ``[...]``."""
    out = o1.to(torch.float32).contiguous().clone() if o1.dtype == torch.float32 else o1.to(torch.float32).contiguous()
    lse = lse1.to(torch.float32).contiguous().clone() if lse1.dtype == torch.float32 else lse1.to(torch.float32).contiguous()
    ops.lse_merge(out, lse, o2.contiguous(), lse2.contiguous())
    return out, lse
