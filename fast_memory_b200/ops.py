"""Operators of the LSH attention-memory path, with the reference's names, arguments and error behaviour.

Drop-in functions (reference interface in brackets; tk = triton_kernel.py, mem = memory.py):

  * :func:`attention_hash_varlen`   [tk:51-119]
  * :func:`attention_hash`          [tk:275-286]
  * :func:`update_out_and_lse`      [mem:54-71]
  * :func:`ring_attention_masked_forward` [mem:106-163]

plus the thin tensor-level wrappers of the C entry points they are built from (``hash_rows``,
``group_rows``, ``hashed_attention``, ``lse_merge``, ``project``, ``topz_select``, ``unit_rows``).
Everything runs in the CUDA library; tensors must live on a CUDA device.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib as L


class _Workspace:
    """Scratch buffers that grow on demand and are reused between calls, one per (operator, device, CUDA stream).

    Kernels of one operator launched on the same stream run one after the other, so they can share a buffer; calls
    on DIFFERENT streams may overlap on the device and therefore get buffers of their own.  A buffer is allocated
    while its stream is current, so when a larger request replaces it the caching allocator hands the old block out
    again only in that stream's order, after the kernels that still use it."""

    def __init__(self):
        self._bufs = {}

    def get(self, key: str, nbytes: int, device) -> torch.Tensor:
        k = (key, device, torch.cuda.current_stream(device).cuda_stream)
        buf = self._bufs.get(k)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
            self._bufs[k] = buf
        return buf


_ws = _Workspace()


# ---------------------------------------------------------------------------------------------------
# tensor-level wrappers of the C entry points
# ---------------------------------------------------------------------------------------------------
def hash_rows(x: torch.Tensor, A: torch.Tensor, seg_xb: Optional[torch.Tensor] = None,
              seg_cb: Optional[torch.Tensor] = None, max_seg_rows: int = 0) -> torch.Tensor:
    """x ``[rows, d]``, A ``[buckets, d]`` (same dtype) -> int32 ``[rows]`` local bucket of each row."""
    dev = L.require_cuda(x, A, seg_xb, seg_cb)
    if x.dtype != A.dtype:
        raise TypeError(f"x ({x.dtype}) and A ({A.dtype}) must share a dtype")
    assert x.dim() == 2 and A.dim() == 2 and x.shape[1] == A.shape[1]
    assert x.is_contiguous() and A.is_contiguous()
    out = torch.empty(x.shape[0], dtype=torch.int32, device=dev)
    n_seg = 1 if seg_xb is None else seg_xb.numel() - 1
    ws = _ws.get("hash", L.lib().fm_hash_rows_workspace_bytes(x.shape[0], n_seg), dev)
    L.check(L.lib().fm_hash_rows(L.ptr(x), L.ptr(A), L.dtype_id(x.dtype), x.shape[0], A.shape[0], x.shape[1], n_seg,
                                 L.ptr(seg_xb), L.ptr(seg_cb), int(max_seg_rows), L.ptr(out), L.ptr(ws), ws.numel(),
                                 L.stream_ptr(dev)), "fm_hash_rows")
    return out


def group_rows(hashes: torch.Tensor, total_buckets: int, seg_xb: Optional[torch.Tensor] = None,
               seg_cb: Optional[torch.Tensor] = None, in_range: bool = False, max_seg_rows: int = 0,
               max_seg_buckets: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Counting sort of rows by global bucket -> (group_off int32 ``[buckets+1]``, perm int32 ``[rows]``).

    ``in_range=True`` (with the size of the largest segment in rows and buckets): the caller vouches that every hash
    lies inside its segment's buckets - the output of :func:`hash_rows` does - and the sort runs as ONE launch, a CTA
    per segment; hashes from elsewhere go through the general path, which drops rows whose hash is out of range."""
    dev = L.require_cuda(hashes, seg_xb, seg_cb)
    assert hashes.dtype == torch.int32 and hashes.is_contiguous()
    n = hashes.numel()
    group_off = torch.empty(total_buckets + 1, dtype=torch.int32, device=dev)
    perm = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    need = L.lib().fm_group_rows_workspace_bytes(n, total_buckets)
    ws = _ws.get("group", need, dev)
    n_seg = 1 if seg_xb is None else seg_xb.numel() - 1
    if in_range and max_seg_rows > 0 and max_seg_buckets > 0:
        L.check(L.lib().fm_group_rows_segmented(L.ptr(hashes), n, total_buckets, n_seg, L.ptr(seg_xb), L.ptr(seg_cb),
                                                int(max_seg_rows), int(max_seg_buckets), L.ptr(group_off), L.ptr(perm),
                                                L.ptr(ws), ws.numel(), L.stream_ptr(dev)), "fm_group_rows_segmented")
    else:
        L.check(L.lib().fm_group_rows(L.ptr(hashes), n, total_buckets, n_seg, L.ptr(seg_xb), L.ptr(seg_cb),
                                      L.ptr(group_off), L.ptr(perm), L.ptr(ws), ws.numel(), L.stream_ptr(dev)),
                "fm_group_rows")
    return group_off, perm[:n]


def hashed_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, table: torch.Tensor,
                     bucket_off: torch.Tensor, group_off: torch.Tensor, perm: torch.Tensor, sm_scale: float,
                     max_bucket_len: int, bucket_kbase: Optional[torch.Tensor] = None, key_chunk: int = 0,
                     out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None, prefill: bool = False
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """q ``[n_q, d]``, k/v ``[n_k, d]``; flat ``table`` (int32 or int64) cut by ``bucket_off`` (int64
    ``[buckets+1]``); queries grouped by ``group_off`` / ``perm``.  Returns o (q's dtype) and fp32
    natural-log LSE (``-inf`` where the bucket is empty).

    Rows that no group claims (a caller-made hash outside ``[0, buckets)`` is dropped by :func:`group_rows`) are not
    written by the kernel; ``prefill=True`` starts the outputs at o = 0, LSE = -inf so that such rows read as "no key".
    ``max_bucket_len`` must bound every bucket's length: the part of a longer bucket beyond it is left out."""
    dev = L.require_cuda(q, k, v, table, bucket_off, group_off, perm, bucket_kbase)
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k and v must share a dtype")
    assert q.dim() == 2 and k.dim() == 2 and v.shape == k.shape and q.shape[1] == k.shape[1]
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous() and table.is_contiguous()
    assert table.dtype in (torch.int32, torch.int64) and bucket_off.dtype == torch.int64
    assert group_off.dtype == torch.int32 and perm.dtype == torch.int32
    n_q, d = q.shape
    total_buckets = bucket_off.numel() - 1
    if out is None:
        out = torch.zeros_like(q) if prefill else torch.empty_like(q)
    if lse is None:
        lse = torch.full((n_q,), float("-inf"), dtype=torch.float32, device=dev) if prefill else \
            torch.empty(n_q, dtype=torch.float32, device=dev)
    need = L.lib().fm_hashed_attn_workspace_bytes(n_q, total_buckets, int(max_bucket_len), d, int(key_chunk))
    ws = _ws.get("attn", need, dev)
    L.check(L.lib().fm_hashed_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.dtype_id(q.dtype), d, n_q, k.shape[0],
                                       total_buckets, L.ptr(table), table.element_size(), L.ptr(bucket_off),
                                       L.ptr(bucket_kbase), int(max_bucket_len), L.ptr(group_off), L.ptr(perm),
                                       float(sm_scale), L.ptr(out), L.ptr(lse), int(key_chunk), L.ptr(ws), ws.numel(),
                                       L.stream_ptr(dev)), "fm_hashed_attn_fwd")
    return out, lse


def set_attention_kernel(which: str) -> None:
    """Which tensor-core kernel serves bf16 / fp16 queries with head dim 128: ``"mma"`` (mma.sync, the default and the
    faster one) or ``"tc"`` (tcgen05 with TMEM accumulators).  Process-wide."""
    if which not in ("mma", "tc"):
        raise ValueError("set_attention_kernel: 'mma' or 'tc'")
    L.check(L.lib().fm_set_attn_kernel(1 if which == "tc" else 0), "fm_set_attn_kernel")


def hashed_attention_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, table: torch.Tensor, bucket_off: torch.Tensor,
                              group_off: torch.Tensor, perm: torch.Tensor, sm_scale: float, out: torch.Tensor, lse: torch.Tensor,
                              d_out: torch.Tensor, bucket_kbase: Optional[torch.Tensor] = None,
                              dk: Optional[torch.Tensor] = None, dv: Optional[torch.Tensor] = None
                              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of the hashed attention over the gathered rows (mem:166-206 without the dense mask).  Same layouts as
    :func:`hashed_attention`; ``out`` / ``d_out`` ``[n_q, d]`` in q's dtype, ``lse`` fp32 ``[n_q]`` natural log (the LSE the
    forward result was normalised with).  Returns fp32 ``(dq [n_q, d], dk [n_k, d], dv [n_k, d])``; pass ``dk`` / ``dv``
    to accumulate into existing buffers (several shards or memories taking turns)."""
    dev = L.require_cuda(q, k, v, table, bucket_off, group_off, perm, out, lse, d_out, bucket_kbase, dk, dv)
    if not (q.dtype == k.dtype == v.dtype == out.dtype == d_out.dtype):
        raise TypeError("q, k, v, out and d_out must share a dtype")
    if lse.dtype != torch.float32:
        raise TypeError("lse must be float32 (natural log)")
    assert q.dim() == 2 and k.dim() == 2 and v.shape == k.shape and out.shape == q.shape and d_out.shape == q.shape
    for t in (q, k, v, table, out, lse, d_out):
        assert t.is_contiguous()
    assert table.dtype in (torch.int32, torch.int64) and bucket_off.dtype == torch.int64
    assert group_off.dtype == torch.int32 and perm.dtype == torch.int32
    n_q, d = q.shape
    dq = torch.empty(n_q, d, dtype=torch.float32, device=dev)
    if dk is None:
        dk = torch.zeros(k.shape, dtype=torch.float32, device=dev)
    if dv is None:
        dv = torch.zeros(k.shape, dtype=torch.float32, device=dev)
    assert dk.dtype == torch.float32 and dv.dtype == torch.float32 and dk.shape == k.shape and dv.shape == k.shape
    assert dk.is_contiguous() and dv.is_contiguous()
    L.check(L.lib().fm_hashed_attn_bwd(L.ptr(q), L.ptr(k), L.ptr(v), L.dtype_id(q.dtype), d, n_q, k.shape[0],
                                       bucket_off.numel() - 1, L.ptr(table), table.element_size(), L.ptr(bucket_off),
                                       L.ptr(bucket_kbase), L.ptr(group_off), L.ptr(perm), float(sm_scale), L.ptr(out),
                                       L.ptr(lse), L.ptr(d_out), L.ptr(dq), L.ptr(dk), L.ptr(dv), L.stream_ptr(dev)),
            "fm_hashed_attn_bwd")
    return dq, dk, dv


def lse_merge(out: torch.Tensor, lse: torch.Tensor, block_out: torch.Tensor, block_lse: torch.Tensor) -> None:
    """In place on fp32 ``out`` ``[rows, d]`` / ``lse`` ``[rows]``."""
    dev = L.require_cuda(out, lse, block_out, block_lse)
    if out.dtype != torch.float32 or lse.dtype != torch.float32:
        raise TypeError("the merge accumulators must be float32")
    assert out.is_contiguous() and lse.is_contiguous() and block_out.is_contiguous() and block_lse.is_contiguous()
    d = out.shape[-1]
    rows = out.numel() // d
    assert block_out.numel() == out.numel() and lse.numel() == rows and block_lse.numel() == rows
    L.check(L.lib().fm_lse_merge(L.ptr(out), L.ptr(lse), L.ptr(block_out), L.dtype_id(block_out.dtype),
                                 L.ptr(block_lse), L.dtype_id(block_lse.dtype), rows, d, L.stream_ptr(dev)),
            "fm_lse_merge")


def lse_merge_out(acc_out: torch.Tensor, acc_lse: torch.Tensor, block_out: torch.Tensor, block_lse: torch.Tensor,
                  out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                  lse_out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The merge of :func:`lse_merge` out of place: fp32 ``acc_out`` / ``acc_lse`` stay untouched, the result comes back
    in ``out_dtype`` (fp32, the default, or ``block_out``'s dtype) with its fp32 LSE - one pass instead of copy + merge
    + cast."""
    dev = L.require_cuda(acc_out, acc_lse, block_out, block_lse)
    if acc_out.dtype != torch.float32 or acc_lse.dtype != torch.float32 or block_lse.dtype != torch.float32:
        raise TypeError("the accumulator and both LSEs must be float32")
    assert acc_out.is_contiguous() and acc_lse.is_contiguous() and block_out.is_contiguous() and block_lse.is_contiguous()
    d = acc_out.shape[-1]
    rows = acc_out.numel() // d
    assert block_out.numel() == acc_out.numel() and acc_lse.numel() == rows and block_lse.numel() == rows
    out_dtype = out_dtype or torch.float32
    if out is None:
        out = torch.empty(acc_out.shape, dtype=out_dtype, device=dev)
    if lse_out is None:
        lse_out = torch.empty(acc_lse.shape, dtype=torch.float32, device=dev)
    assert out.dtype == out_dtype and out.is_contiguous() and lse_out.is_contiguous() and lse_out.dtype == torch.float32
    L.check(L.lib().fm_lse_merge_out(L.ptr(acc_out), L.ptr(acc_lse), L.ptr(block_out), L.dtype_id(block_out.dtype),
                                     L.ptr(block_lse), L.ptr(out), L.dtype_id(out_dtype), L.ptr(lse_out), rows, d,
                                     L.stream_ptr(dev)), "fm_lse_merge_out")
    return out, lse_out


def project(A: torch.Tensor, K: torch.Tensor) -> torch.Tensor:
    """fp32 ``Y[c, j] = A[c] . K[j]`` in the library's fixed summation order."""
    dev = L.require_cuda(A, K)
    assert A.dtype == K.dtype and A.is_contiguous() and K.is_contiguous() and A.shape[1] == K.shape[1]
    Y = torch.empty(A.shape[0], K.shape[0], dtype=torch.float32, device=dev)
    L.check(L.lib().fm_project(L.ptr(A), L.ptr(K), L.dtype_id(A.dtype), A.shape[0], K.shape[0], A.shape[1], L.ptr(Y),
                               K.shape[0], L.stream_ptr(dev)), "fm_project")
    return Y


def project_tc(A: torch.Tensor, K: torch.Tensor, key_step: int = 1) -> torch.Tensor:
    """Tensor-core (tcgen05) projection of every ``key_step``-th row of K: approximate fp32 scores."""
    dev = L.require_cuda(A, K)
    assert A.dtype == K.dtype and A.is_contiguous() and K.is_contiguous() and A.shape[1] == K.shape[1]
    n_cols = (K.shape[0] + key_step - 1) // key_step
    Y = torch.empty(A.shape[0], n_cols, dtype=torch.float32, device=dev)
    ws = _ws.get("project_tc", L.lib().fm_project_tc_workspace_bytes(A.shape[0], K.shape[0], int(key_step)), dev)
    L.check(L.lib().fm_project_tc(L.ptr(A), L.ptr(K), L.dtype_id(A.dtype), A.shape[0], K.shape[0], A.shape[1],
                                  int(key_step), L.ptr(Y), n_cols, L.ptr(ws), ws.numel(), L.stream_ptr(dev)),
            "fm_project_tc")
    status = int(ws[:4].view(torch.int32).item())
    if status:
        raise L.FastMemError(f"fm_project_tc: a pipeline wait gave up (status {status})")
    return Y


def topz_select(Y: torch.Tensor, Z: int, index_base: int = 0) -> torch.Tensor:
    """Rows of fp32 ``Y`` -> int32 ``[rows, Z]`` indices of the Z largest (lower index wins ties), ascending."""
    dev = L.require_cuda(Y)
    assert Y.dtype == torch.float32 and Y.dim() == 2 and Y.is_contiguous()
    Z = min(int(Z), Y.shape[1])
    out = torch.empty(Y.shape[0], Z, dtype=torch.int32, device=dev)
    L.check(L.lib().fm_topz_select(L.ptr(Y), Y.shape[0], Y.shape[1], Y.shape[1], Z, int(index_base), L.ptr(out), Z,
                                   L.stream_ptr(dev)), "fm_topz_select")
    return out


@torch.library.custom_op("fast_memory_b200::shard_filter", mutates_args=())
def shard_filter(k_hashes: torch.Tensor, lo: int, hi: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``k_hashes`` ``[C, H, Z]`` int64 global key indices -> (flat int64 indices of the entries in ``[lo, hi)``
    rebased by ``lo`` and packed (head, bucket, slot); counts ``[H, C]`` int64).  The flat tensor keeps its full
    ``C*H*Z`` capacity (only the first ``counts.sum()`` entries are meaningful), which avoids reading the total
    back from the device.  Registered as an operator so that a traced caller (the reference compiles this step,
    mem:106) sees one opaque node."""
    dev = L.require_cuda(k_hashes)
    assert k_hashes.dim() == 3 and k_hashes.dtype == torch.int64
    k_hashes = k_hashes.contiguous()
    C, H, Z = k_hashes.shape
    flat = torch.zeros(C * H * Z, dtype=torch.int64, device=dev)      # the unused tail reads 0, not leftovers
    counts = torch.empty(H, C, dtype=torch.int64, device=dev)
    ws = _ws.get("shard_filter", L.lib().fm_shard_filter_workspace_bytes(C, H), dev)
    L.check(L.lib().fm_shard_filter(L.ptr(k_hashes), C, H, Z, int(lo), int(hi), L.ptr(flat), L.ptr(counts), L.ptr(ws),
                                    ws.numel(), L.stream_ptr(dev)), "fm_shard_filter")
    return flat, counts


@shard_filter.register_fake
def _(k_hashes, lo, hi):
    C, H, Z = k_hashes.shape
    return k_hashes.new_empty(C * H * Z), k_hashes.new_empty(H, C)


def unit_rows(X: torch.Tensor) -> torch.Tensor:
    dev = L.require_cuda(X)
    X2 = X.reshape(-1, X.shape[-1]).contiguous()
    U = torch.empty(X2.shape, dtype=torch.float32, device=dev)
    L.check(L.lib().fm_unit_rows(L.ptr(X2), L.dtype_id(X.dtype), X2.shape[0], X2.shape[1], L.ptr(U), L.stream_ptr(dev)),
            "fm_unit_rows")
    return U.reshape(X.shape)


# ---------------------------------------------------------------------------------------------------
# drop-in operators
# ---------------------------------------------------------------------------------------------------
_kbase_cache = {}


def _uniform_kbase(B: int, C: int, N: int, device) -> torch.Tensor:
    key = (B, C, N, device)
    t = _kbase_cache.get(key)
    if t is None:
        t = (torch.arange(B * C, device=device, dtype=torch.int64) // C * N).to(torch.int32)
        _kbase_cache[key] = t
    return t


def _grouping(q_hashes: torch.Tensor, k_hash_counts: torch.Tensor, S: int, N: int):
    """(bucket_off, group_off, perm, kbase) of a uniform batch: ``q_hashes`` ``[B, S]``, ``k_hash_counts`` ``[B, C]``."""
    B, C = k_hash_counts.shape
    dev = q_hashes.device
    bucket_off = torch.zeros(B * C + 1, dtype=torch.int64, device=dev)
    bucket_off[1:] = torch.cumsum(k_hash_counts.reshape(-1).to(torch.int64), 0)
    hashes = q_hashes.reshape(-1).to(torch.int32)
    seg_xb = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
    seg_cb = torch.arange(0, (B + 1) * C, C, dtype=torch.int32, device=dev)
    group_off, perm = group_rows(hashes, B * C, seg_xb, seg_cb)
    return bucket_off, group_off, perm, _uniform_kbase(B, C, N, dev)


def _index_table(k_hashes: torch.Tensor) -> torch.Tensor:
    return (k_hashes if k_hashes.dtype in (torch.int32, torch.int64) else k_hashes.to(torch.int64)).contiguous()


@torch.library.custom_op("fast_memory_b200::hashed_attention_grouped", mutates_args=())
def _hashed_attention_grouped_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_hashes: torch.Tensor,
                                 k_hash_counts: torch.Tensor, q_hashes: torch.Tensor, sm_scale: float,
                                 max_bucket_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The operator behind :func:`attention_hash_varlen`, taking that function's own arguments: grouping of the
    queries by bucket and the attention, both in the library.  Returns o ``[B, S, d]`` in the original query order
    and fp32 natural-log LSE ``[B, S]``."""
    B, S, d = q.shape
    N = k.shape[1]
    bucket_off, group_off, perm, kbase = _grouping(q_hashes, k_hash_counts, S, N)
    o, lse = hashed_attention(q.reshape(B * S, d), k.reshape(B * N, d), v.reshape(B * N, d), _index_table(k_hashes),
                              bucket_off, group_off, perm, sm_scale, max_bucket_len, bucket_kbase=kbase, prefill=True)
    return o.reshape(B, S, d), lse.reshape(B, S)


@_hashed_attention_grouped_op.register_fake
def _(q, k, v, k_hashes, k_hash_counts, q_hashes, sm_scale, max_bucket_len):
    return torch.empty_like(q), q.new_empty(q.shape[:-1], dtype=torch.float32)


@torch.library.custom_op("fast_memory_b200::hashed_attention_grouped_backward", mutates_args=())
def _hashed_attention_grouped_bwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_hashes: torch.Tensor,
                                     k_hash_counts: torch.Tensor, q_hashes: torch.Tensor, o: torch.Tensor,
                                     lse: torch.Tensor, d_o: torch.Tensor, sm_scale: float
                                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of ``hashed_attention_grouped`` with respect to q, k and v for the output gradient ``d_o`` (the
    gathered-row form of mem:166-206), in the dtypes of q, k and v."""
    B, S, d = q.shape
    N = k.shape[1]
    bucket_off, group_off, perm, kbase = _grouping(q_hashes, k_hash_counts, S, N)
    dq, dk, dv = hashed_attention_backward(q.reshape(B * S, d), k.reshape(B * N, d), v.reshape(B * N, d),
                                           _index_table(k_hashes), bucket_off, group_off, perm, sm_scale,
                                           o.reshape(B * S, d).contiguous(), lse.reshape(B * S).contiguous(),
                                           d_o.reshape(B * S, d).contiguous(), bucket_kbase=kbase)
    return dq.reshape(q.shape).to(q.dtype), dk.reshape(k.shape).to(k.dtype), dv.reshape(v.shape).to(v.dtype)


@_hashed_attention_grouped_bwd_op.register_fake
def _(q, k, v, k_hashes, k_hash_counts, q_hashes, o, lse, d_o, sm_scale):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _grouped_setup_context(ctx, inputs, output):
    q, k, v, k_hashes, k_hash_counts, q_hashes, sm_scale, _ = inputs
    o, lse = output
    ctx.save_for_backward(q, k, v, k_hashes, k_hash_counts, q_hashes, o, lse)
    ctx.sm_scale = sm_scale


def _grouped_backward(ctx, grad_o, grad_lse):
    # The reference registers a backward that returns no gradient at all (tk:44-48) and differentiates its dense
    # restatement instead (mem:166-206).  Here the operator itself is differentiable in q, k and v through o; the LSE
    # output is treated as a constant (a caller that merges partial results differentiates the merged pair through
    # Memory.query_backward, as mem:354-378 does).
    q, k, v, k_hashes, k_hash_counts, q_hashes, o, lse = ctx.saved_tensors
    if grad_o is None:
        return (None,) * 8
    dq, dk, dv = _hashed_attention_grouped_bwd_op(q, k, v, k_hashes, k_hash_counts, q_hashes, o, lse,
                                                  grad_o.contiguous(), ctx.sm_scale)
    return dq, dk, dv, None, None, None, None, None


_hashed_attention_grouped_op.register_autograd(_grouped_backward, setup_context=_grouped_setup_context)


@torch.library.custom_op("fast_memory_b200::attention_hash_varlen", mutates_args=())
def _attention_hash_varlen_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                              k_hashes: torch.Tensor, k_hash_counts: torch.Tensor, k_hash_offset: torch.Tensor,
                              q_hashes_z: torch.Tensor, q_hashes_count: torch.Tensor, q_hashes_offset: torch.Tensor,
                              sm_scale: float, q_seq_len: int, kv_seq_len: int,
                              d_head: int, n_buckets: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Drop-in for the reference's registered operator ``notbad::attention_hash_varlen`` (tk:16-41): the same fourteen
    arguments with the same meaning and the same outputs.

    ``q`` ``[B, S, d]`` holds the queries ALREADY sorted by bucket inside each batch row (tk:75-78); group g - one per
    non-empty (row, bucket) pair, in sorted order - is bucket ``q_hashes_z[g]`` with ``q_hashes_count[g]`` queries
    starting at flat position ``q_hashes_offset[g]`` (its batch row is ``offset // q_seq_len``, tk:181);
    ``k_hash_offset`` ``[B, C]`` is the exclusive prefix sum of ``k_hash_counts`` over the flattened table (tk:86-88).
    Returns o in q's dtype in the sorted order and the fp32 LSE in BASE 2 (``m + log2 l``, tk:222), ``-inf`` for a
    bucket without keys - what the reference kernel writes; its wrapper converts afterwards (tk:111)."""
    B, S, d = q.shape
    N, C = kv_seq_len, n_buckets
    dev = q.device
    gb = (q_hashes_offset // q_seq_len) * C + q_hashes_z
    n_per_bucket = torch.zeros(B * C, dtype=torch.int64, device=dev)
    n_per_bucket.index_put_((gb,), q_hashes_count.to(torch.int64))
    group_off = torch.zeros(B * C + 1, dtype=torch.int32, device=dev)
    group_off[1:] = torch.cumsum(n_per_bucket, 0)
    perm = torch.arange(B * S, dtype=torch.int32, device=dev)                # the queries come sorted
    flat_counts = k_hash_counts.reshape(-1)
    bucket_off = torch.cat([k_hash_offset.reshape(-1).to(torch.int64),
                            (k_hash_offset.reshape(-1)[-1:] + flat_counts[-1:]).to(torch.int64)])
    max_len = int(flat_counts.max().item()) if flat_counts.numel() else 0
    o, lse = hashed_attention(q.reshape(B * S, d), k.reshape(B * N, d), v.reshape(B * N, d), _index_table(k_hashes),
                              bucket_off, group_off, perm, sm_scale, max_len, bucket_kbase=_uniform_kbase(B, C, N, dev))
    return o.reshape(B, S, d), (lse * (1.0 / math.log(2))).reshape(B, S)


@_attention_hash_varlen_op.register_fake
def _(q, k, v, k_hashes, k_hash_counts, k_hash_offset, q_hashes_z, q_hashes_count, q_hashes_offset,
      sm_scale, q_seq_len, kv_seq_len, d_head, n_buckets):
    return torch.empty_like(q), q.new_empty(q.shape[:-1], dtype=torch.float32)


def _attention_hash_varlen_backward(ctx, grad_o, grad_lse):
    # as the reference registers it (tk:44-48): no gradient flows through this operator
    return (None,) * 14


_attention_hash_varlen_op.register_autograd(_attention_hash_varlen_backward)


def attention_hash_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                          k_hashes: torch.Tensor, k_hash_counts: torch.Tensor,
                          q_hashes: torch.Tensor,
                          sm_scale: float, *, return_fp32_lse: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Hashed attention forward (drop-in for tk:51-119).

    :param q: ``[batch_size, q_seq_len, d_head]``
    :param k: ``[batch_size, kv_seq_len, d_head]``
    :param v: ``[batch_size, kv_seq_len, d_head]``
    :param k_hashes: flat key indices, ``[sum(k_hash_counts)]``, ordered (batch, bucket, slot)
    :param k_hash_counts: ``[batch_size, C]``
    :param q_hashes: ``[batch_size, q_seq_len]`` bucket of every query
    :param sm_scale: softmax scale

    Returns ``(o, lse)`` with o in q's dtype.  As in the reference, lse is returned in q's dtype after
    ``nan_to_num`` (empty bucket -> ``finfo.min``; tk:111-117); ``return_fp32_lse=True`` returns the
    un-rounded fp32 natural-log LSE with ``-inf`` for empty buckets instead.
    """
    batch_size, q_seq_len, d_head = q.shape
    _, kv_seq_len, _ = k.shape
    _, n_buckets = k_hash_counts.shape
    assert k.shape[0] == batch_size
    assert k_hash_counts.shape[0] == batch_size
    assert q_hashes.shape[0] == batch_size
    assert q_hashes.shape[1] == q_seq_len, f'{q_hashes.shape} != {q_seq_len}'
    assert d_head == k.shape[-1] == v.shape[-1]
    assert q.is_contiguous()
    assert k.is_contiguous()
    assert v.is_contiguous()
    assert k.stride() == v.stride()
    L.require_cuda(q, k, v, k_hashes, k_hash_counts, q_hashes)
    if q.numel() == 0:
        lse_dtype = torch.float32 if return_fp32_lse else q.dtype
        return torch.empty_like(q), q.new_empty(q.shape[:-1], dtype=lse_dtype)
    # the longest bucket sizes the work split; like the reference wrapper (unique_consecutive, tk:81)
    # this reads one number back from the device
    max_len = int(k_hash_counts.max().item()) if k_hash_counts.numel() else 0
    o, lse = _hashed_attention_grouped_op(q, k, v, k_hashes, k_hash_counts, q_hashes, float(sm_scale), max_len)
    if return_fp32_lse:
        return o, lse
    lse = (lse * (1.0 / math.log(2))).to(q.dtype) * math.log(2)
    lse = torch.nan_to_num(lse, nan=0.0, posinf=torch.finfo(lse.dtype).max, neginf=torch.finfo(lse.dtype).min)
    return o, lse


def attention_hash(q, k, v, centroids, bucket_size, sm_scale, key_range: Optional[Tuple[int, int]] = None):
    """Single-device build + hash + attend (drop-in for tk:275-286).

    q ``[B, S, d]``, k/v ``[B, N, d]``, centroids ``[B, C, d]``.  The reference hard-codes a key-index
    filter ``[8192, 65536)`` (tk:283); here it is the optional ``key_range``.
    """
    from .memory import Memory
    mem = Memory.build(k, v, A=centroids, bucket_size=bucket_size, key_range=key_range)
    o, lse = mem.query(q, sm_scale)
    lse = (lse * (1.0 / math.log(2))).to(q.dtype) * math.log(2)
    lse = torch.nan_to_num(lse, nan=0.0, posinf=torch.finfo(lse.dtype).max, neginf=torch.finfo(lse.dtype).min)
    return o, lse


def update_out_and_lse(out: Optional[torch.Tensor], lse: Optional[torch.Tensor],
                       block_out: torch.Tensor, block_lse: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge a block's (out, lse) into fp32 accumulators (drop-in for mem:54-71).

    First call (``out is None``): returns ``block_out`` in fp32 and ``block_lse`` with a trailing
    singleton dimension.  Unlike the reference the lse accumulator is always fp32 (the reference keeps
    the dtype of the first block's lse).  Later calls update ``out`` / ``lse`` in place and return them.
    """
    if out is None:
        return block_out.to(torch.float32).contiguous(), block_lse.to(torch.float32).unsqueeze(dim=-1).contiguous()
    assert lse is not None and lse.shape[-1] == 1
    lse_merge(out, lse, block_out.contiguous(), block_lse.contiguous())
    return out, lse


def ring_attention_masked_forward(k_hashes, q_hashes, q, k, v, sm_scale, rank):
    """Attention of all queries against ONE key shard of a globally indexed memory (drop-in for
    mem:106-163).

    :param k_hashes: ``[n_buckets, k_heads, bucket_size]`` GLOBAL key indices
    :param q_hashes: ``[k_heads, n_groups, seq_len]``
    :param q: ``[1, n_heads, seq_len, d]``;  k, v: ``[1, k_heads, context_len, d]`` (the visiting shard)
    :param rank: which shard is visiting: only table entries in ``[rank*ctx, (rank+1)*ctx)`` take part
    Returns ``(out [1, n_heads, seq_len, d], lse [1, n_heads, seq_len])`` in q's dtype.
    """
    batch_size, n_heads, seq_len, d_head = q.shape
    _, k_heads, context_len, _ = k.shape
    assert batch_size == 1
    assert k_hashes.shape[1] == k_heads
    assert q_hashes.shape[0] == k_heads
    assert q_hashes.shape[1] == n_heads // k_heads
    assert q_hashes.shape[2] == seq_len
    q_hashes = q_hashes.reshape(k_heads, -1)
    assert k_hashes.numel() > 0, k_hashes.shape
    flat, counts = shard_filter(k_hashes, rank * context_len, (rank + 1) * context_len)
    out, lse = attention_hash_varlen(q.reshape(k_heads, -1, d_head), k.reshape(k_heads, -1, d_head),
                                     v.reshape(k_heads, -1, d_head), flat, counts, q_hashes, sm_scale)
    return out.reshape(batch_size, n_heads, seq_len, d_head), lse.reshape(batch_size, n_heads, seq_len)
