"""TEST INFRASTRUCTURE ONLY - CPU oracle for the LSH attention-memory hot path.

A CPU restatement (torch/numpy + the small C library ``fm_oracle.c``) of the reference's algorithm for
this path.  It is the checker used by ``tests/``, by the smoke test and by the CPU-baseline leg of the
benchmark.  The product package never imports it.

Pinning: the functions below are checked in ``tests/test_oracle_golden.py`` against vectors produced by
running the reference's own code (its Triton kernel under the Triton CPU interpreter, and the pure-torch
functions of ``memory.py``) - see ``tests/golden/make_golden.py``.  Parts for which the reference holds no
runnable code (spherical k-means, which only its README specifies) are **parity unpinned** and say so.

Reference citations are ``file:line`` within the reference project (``triton_kernel.py`` = tk,
``memory.py`` = mem).
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import Optional, Tuple

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfm_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``fm_oracle.c`` with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "fm_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libfm_oracle.so"])
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        fp = ctypes.POINTER(ctypes.c_float)
        ip = ctypes.POINTER(ctypes.c_int32)
        i64 = ctypes.c_int64
        for name in ("fmo_project", "fmo_project_fast"):
            getattr(L, name).argtypes = [fp, fp, i64, i64, i64, fp]
            getattr(L, name).restype = None
        L.fmo_argmax_hash.argtypes = [fp, fp, i64, i64, i64, ip]
        L.fmo_argmax_hash.restype = None
        L.fmo_topz.argtypes = [fp, i64, i64, i64, ip]
        L.fmo_topz.restype = None
        L.fmo_unit_rows.argtypes = [fp, i64, i64, fp]
        L.fmo_unit_rows.restype = None
        L.fmo_num_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def _f32(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        x = x.detach().to("cpu", torch.float32).numpy()
    return np.ascontiguousarray(x, dtype=np.float32)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _ip(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))


# --------------------------------------------------------------------------------------------------
# Index build: projection + top-Z  (README.md:25-27; mem:261, 273; tk:277-278)
# --------------------------------------------------------------------------------------------------
def project(A, K) -> np.ndarray:
    """Canonical fp32 projection ``Y[c, j] = sum_i A[c, i] * K[j, i]`` as a sequential FMA chain over i."""
    A, K = _f32(A), _f32(K)
    C, d = A.shape
    N = K.shape[0]
    Y = np.empty((C, N), np.float32)
    lib().fmo_project_fast(_fp(A), _fp(K), C, N, d, _fp(Y))
    return Y


def project_numpy(A, K) -> np.ndarray:
    """Independent numpy statement of :func:`project` for inputs whose products are exact in fp32
    (16-bit inputs): fp32 multiply then fp32 add equals the fused operation."""
    A, K = _f32(A), _f32(K)
    Y = np.zeros((A.shape[0], K.shape[0]), np.float32)
    for i in range(A.shape[1]):
        Y = Y + A[:, i:i + 1] * K[None, :, i]
    return Y


def topz(Y, Z: int) -> np.ndarray:
    """Per row: indices of the Z largest values, lower index wins ties, ascending index order."""
    Y = _f32(Y)
    R, N = Y.shape
    Z = min(int(Z), N)
    out = np.empty((R, Z), np.int32)
    lib().fmo_topz(_fp(Y), R, N, Z, _ip(out))
    return out


def topz_numpy(Y, Z: int) -> np.ndarray:
    """Independent statement of :func:`topz`: stable descending sort, first Z, then ascending."""
    Y = _f32(Y) + np.float32(0.0)
    Z = min(int(Z), Y.shape[1])
    order = np.argsort(-Y, axis=1, kind="stable")[:, :Z]
    return np.sort(order, axis=1).astype(np.int32)


def build_table(A, K, Z: int) -> np.ndarray:
    """A ``[H, C, d]``, K ``[H, N, d]`` -> table ``[H, C, min(Z, N)]`` int32 of per-head key indices."""
    H = K.shape[0]
    return np.stack([topz(project(A[h], K[h]), Z) for h in range(H)], 0)


def query_hash(A, q) -> np.ndarray:
    """A ``[H, C, d]``, q ``[H, S, d]`` -> ``[H, S]`` int32 bucket of each query: argmax of the canonical
    projection, first maximum wins (README.md:29; mem:281-283; tk:280-281)."""
    H, S, d = q.shape
    out = np.empty((H, S), np.int32)
    for h in range(H):
        a, x = _f32(A[h]), _f32(q[h])
        lib().fmo_argmax_hash(_fp(a), _fp(x), a.shape[0], S, d, _ip(out[h]))
    return out


# --------------------------------------------------------------------------------------------------
# Hashed attention  (tk:51-119 wrapper, tk:135-272 kernel)
# --------------------------------------------------------------------------------------------------
def _round_to(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return x.to(dtype).to(torch.float32)


def hashed_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     k_hashes: torch.Tensor, k_hash_counts: torch.Tensor, q_hashes: torch.Tensor,
                     sm_scale: float, block_k: int = 128, k_row_base: Optional[torch.Tensor] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gathered-per-bucket restatement of the reference kernel.

    q ``[B, S, d]``, k/v ``[B, N, d]``, ``k_hashes`` flat table ordered (batch, bucket, slot),
    ``k_hash_counts`` ``[B, C]``, ``q_hashes`` ``[B, S]``.  Returns ``o`` in q's dtype and the
    natural-log LSE in fp32 (the reference wrapper would next cast it to q's dtype, tk:111).

    Rounding points follow the kernel: scores accumulate in fp32 (tk:248), are scaled by
    ``sm_scale * log2(e)`` (tk:195, 249), the softmax runs in base 2 over key blocks of ``block_k``
    (tk:252-257), P is rounded to q's dtype before P.V while the denominator sums unrounded
    p (tk:254, 262-263); ``lse2 = m + log2(l)``, ``o = acc / l`` (tk:222-223); an empty bucket gives
    o = 0, lse = -inf (tk:204-206 with zero key blocks).
    """
    B, S, d = q.shape
    C = k_hash_counts.shape[1]
    counts = k_hash_counts.reshape(-1).to(torch.int64)
    offs = torch.zeros(B * C + 1, dtype=torch.int64)
    offs[1:] = torch.cumsum(counts, 0)
    scale2 = float(sm_scale) * 1.44269504
    qf, kf, vf = q.float(), k.float(), v.float()
    o = torch.zeros(B, S, d, dtype=torch.float32)
    lse2 = torch.full((B, S), -float("inf"), dtype=torch.float32)
    k_hashes = k_hashes.to(torch.int64)
    for b in range(B):
        qh = q_hashes[b].to(torch.int64)
        for c in torch.unique(qh).tolist():
            rows = torch.nonzero(qh == c).flatten()
            idx = k_hashes[offs[b * C + c]: offs[b * C + c + 1]]
            n = idx.numel()
            qb = qf[b, rows]
            m = torch.full((rows.numel(),), -float("inf"))
            l = torch.ones(rows.numel())
            acc = torch.zeros(rows.numel(), d)
            for j0 in range(0, n, block_k):
                ii = idx[j0:j0 + block_k]
                s = (qb @ kf[b, ii].T) * scale2
                m_new = torch.maximum(m, s.max(-1).values)
                p = torch.exp2(s - m_new[:, None])
                alpha = torch.exp2(m - m_new)
                l = l * alpha + p.sum(-1)
                acc = acc * alpha[:, None] + _round_to(p, q.dtype) @ vf[b, ii]
                m = m_new
            o[b, rows] = acc / l[:, None]
            lse2[b, rows] = m + torch.log2(l)
    return o.to(q.dtype), lse2 * math.log(2)


def dropin_lse(lse_nat_fp32: torch.Tensor, q_dtype: torch.dtype) -> torch.Tensor:
    """What the reference wrapper returns for LSE: base-2 value cast to q's dtype, times ln 2,
    then nan_to_num (tk:111-117)."""
    lse2 = (lse_nat_fp32 / math.log(2)).to(q_dtype) * math.log(2)
    fi = torch.finfo(q_dtype)
    return torch.nan_to_num(lse2, nan=0.0, posinf=fi.max, neginf=fi.min)


def hashed_attention_dense(q, k, v, table: torch.Tensor, counts: torch.Tensor, q_hashes: torch.Tensor,
                           sm_scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense-mask statement for small shapes, in the manner of mem:74-103 / tk:328-351: scatter each
    query's bucket into a boolean ``[B, S, N+1]`` mask (column N absorbs unused slots), masked softmax
    in fp64.  ``table`` is ``[B, C, Z]`` with only the first ``counts[b, c]`` slots of a row valid."""
    B, S, d = q.shape
    N = k.shape[1]
    Z = table.shape[2]
    rows = table.to(torch.int64)[torch.arange(B)[:, None], q_hashes.to(torch.int64)]      # B S Z
    valid = torch.arange(Z)[None, None, :] < counts.to(torch.int64)[torch.arange(B)[:, None],
                                                                    q_hashes.to(torch.int64)][..., None]
    rows = torch.where(valid, rows, torch.full_like(rows, N))
    mask = torch.zeros(B, S, N + 1, dtype=torch.bool)
    mask.scatter_(-1, rows, valid)
    mask = mask[..., :N]
    scores = torch.einsum("bid,bjd->bij", q.double(), k.double()) * sm_scale
    scores = scores.masked_fill(~mask, -float("inf"))
    mx = scores.max(-1, keepdim=True).values
    mx = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
    e = torch.exp(scores - mx)
    ssum = e.sum(-1, keepdim=True)
    lse = (torch.log(ssum) + mx).squeeze(-1)
    p = torch.where(ssum > 0, e / ssum.clamp_min(1e-300), torch.zeros_like(e))
    out = torch.einsum("bij,bjd->bid", p, v.double())
    return out.float(), lse.float()


# --------------------------------------------------------------------------------------------------
# LSE merge  (mem:54-71)
# --------------------------------------------------------------------------------------------------
def update_out_and_lse(out: Optional[torch.Tensor], lse: Optional[torch.Tensor],
                       block_out: torch.Tensor, block_lse: torch.Tensor):
    """``lse <- log(e^lse + e^blk)``; ``out <- out - sigmoid(blk - lse) (out - blk_out)`` (mem:67-69).
    First call returns the block cast to fp32 with a trailing singleton on lse (mem:61-65)."""
    block_out = block_out.to(torch.float32)
    block_lse = block_lse.unsqueeze(-1)
    if out is None:
        return block_out, block_lse
    d = block_lse - lse
    out = out - torch.sigmoid(d) * (out - block_out)
    lse = lse - torch.nn.functional.logsigmoid(-d)
    return out, lse


def merge_exact(o1, l1, o2, l2):
    """fp64 statement of the same merge that also handles -inf on either side (weight 0)."""
    o1, o2, l1, l2 = o1.double(), o2.double(), l1.double(), l2.double()
    m = torch.maximum(l1, l2)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w1, w2 = torch.exp(l1 - m), torch.exp(l2 - m)
    tot = w1 + w2
    lse = torch.log(tot) + m
    safe = tot.clamp_min(1e-300)
    out = (o1 * (w1 / safe)[..., None] + o2 * (w2 / safe)[..., None])
    return out.float(), lse.float()


# --------------------------------------------------------------------------------------------------
# Shard filter  (mem:128-142)
# --------------------------------------------------------------------------------------------------
def shard_filter(k_hashes: torch.Tensor, rank: int, context_len: int):
    """``k_hashes`` ``[C, H, Z]`` of GLOBAL key indices -> (flat local indices ordered (head, bucket,
    slot), counts ``[H, C]``) for the shard ``[rank*ctx, (rank+1)*ctx)``."""
    t = k_hashes.permute(1, 0, 2)
    m = torch.logical_and(rank * context_len <= t, t < (rank + 1) * context_len)
    return t[m] - rank * context_len, m.to(torch.long).sum(-1)


# --------------------------------------------------------------------------------------------------
# Projection matrix: spherical k-means  (README.md:37-45).  PARITY UNPINNED: the reference has no code
# for this (its code path, mem:209-231, is a different construction - see compute_centroids below).
# --------------------------------------------------------------------------------------------------
KMEANS_FIX_SHIFT = 40      # unit vectors are summed as integers in units of 2**-40


def unit_rows(X) -> np.ndarray:
    """x / max(||x||, 1e-6) in fp32, with ||x||^2 a sequential FMA chain (clamp as in mem:215-217)."""
    X = _f32(X)
    U = np.empty_like(X)
    lib().fmo_unit_rows(_fp(X), X.shape[0], X.shape[1], _fp(U))
    return U


def kmeans_step(X, cent_T, prev_fp32) -> Tuple[np.ndarray, np.ndarray]:
    """One spherical k-means iteration.  ``cent_T``: the centroids as stored in the key dtype (what the
    hash sees); ``prev_fp32``: fp32 centroids kept for empty clusters.  Returns (new fp32 centroids,
    assignment).  Sums are exact integer sums of unit vectors quantised to 2**-40; the norm is a
    sequential fp64 sum of squares; the result is the fp64 quotient rounded to fp32."""
    Xf = _f32(X)
    C, d = cent_T.shape
    assign = np.empty(Xf.shape[0], np.int32)
    a = _f32(cent_T)
    lib().fmo_argmax_hash(_fp(a), _fp(Xf), C, Xf.shape[0], d, _ip(assign))
    u = unit_rows(Xf)
    fix = np.rint(u.astype(np.float64) * float(2 ** KMEANS_FIX_SHIFT)).astype(np.int64)
    sums = np.zeros((C, d), np.int64)
    np.add.at(sums, assign, fix)
    cnt = np.bincount(assign, minlength=C)
    s = sums.astype(np.float64) * float(2.0 ** -KMEANS_FIX_SHIFT)
    n2 = np.zeros(C, np.float64)
    for i in range(d):
        n2 = n2 + s[:, i] * s[:, i]
    nrm = np.sqrt(n2)
    new = np.array(prev_fp32, dtype=np.float32, copy=True)
    ok = (cnt > 0) & (nrm > 0)
    new[ok] = (s[ok] / nrm[ok, None]).astype(np.float32)
    return new, assign


def spherical_kmeans(X: torch.Tensor, init: torch.Tensor, iters: int) -> torch.Tensor:
    """Centroids of spherical k-means (distance ``1 - c.x``, README.md:41) after ``iters`` iterations,
    returned in X's dtype (the reference keeps centroids in the key dtype, mem:493).  ``init`` rows are
    normalised first; assignment = first maximum of the canonical projection of the raw rows (a positive
    scaling of x does not change the argmax)."""
    c = unit_rows(init)
    for _ in range(iters):
        cT = torch.from_numpy(c).to(X.dtype)
        c, _ = kmeans_step(X, cT, c)
    return torch.from_numpy(c).to(X.dtype)


def compute_centroids(kq: torch.Tensor, centroids: torch.Tensor, n_hashes: int, n_groups: int,
                      centroid_topk: int) -> torch.Tensor:
    """The construction the reference CODE uses (mem:209-231): normalise kq, take each centroid's
    ``centroid_topk`` nearest rows per head, average them over groups x topk."""
    n_heads, ctx, d = kq.shape
    k_heads = n_heads // n_groups
    x = kq.float()
    x = x / torch.norm(x, p=2, dim=-1, keepdim=True).clamp(min=1e-6)
    b = torch.einsum("zd,hid->zhi", centroids.float(), x)
    b = torch.topk(b, k=centroid_topk, dim=-1, largest=True)[1]
    g = x[torch.arange(n_heads)[None, :, None], b]
    g = g.reshape(n_hashes, k_heads, n_groups * centroid_topk, d)
    return g.mean(dim=2)


# --------------------------------------------------------------------------------------------------
# Backward of the hashed attention (mem:166-206)
# --------------------------------------------------------------------------------------------------
def hashed_attention_backward_dense(q, k, v, table, counts, q_hashes, sm_scale: float, out, lse, d_out):
    """The reference's backward (``ring_attention_masked_backward``, mem:166-206) for one key shard, in fp64: rebuild
    the dense mask from the table (mem:174-180), P = exp(S - lse) (mem:190-194), dV, dP, D, dS, dQ, dK (mem:195-205).

    q, out, d_out ``[H, S, d]``; k, v ``[H, N, d]``; table ``[H, C, Zmax]`` key indices with ``counts [H, C]`` valid slots
    per bucket; q_hashes ``[H, S]``; lse ``[H, S]`` natural log.  Returns float64 ``(dq, dk, dv)``."""
    H, S, d = q.shape
    N = k.shape[1]
    mask = torch.zeros(H, S, N, dtype=torch.bool)
    for h in range(H):
        for s_ in range(S):
            b = int(q_hashes[h, s_])
            mask[h, s_, table[h, b, :int(counts[h, b])].long()] = True
    qd, kd, vd, od, gd = q.double(), k.double(), v.double(), out.double(), d_out.double()
    scores = torch.einsum("hid,hjd->hij", qd, kd) * sm_scale
    P = torch.exp(scores - lse.double()[..., None])
    P = torch.where(mask & torch.isfinite(lse)[..., None], P, torch.zeros_like(P))
    dV = torch.einsum("hij,hid->hjd", P, gd)
    dP = torch.einsum("hid,hjd->hij", gd, vd)
    D = (gd * od).sum(-1, keepdim=True)
    dS = P * (dP - D)
    dQ = torch.einsum("hij,hjd->hid", dS, kd) * sm_scale
    dK = torch.einsum("hij,hid->hjd", dS, qd) * sm_scale
    return dQ, dK, dV


# --------------------------------------------------------------------------------------------------
# Dense local-window attention with LSE (stands in for the undefined ``attention_forward``, mem:302)
# --------------------------------------------------------------------------------------------------
def local_window_attention(q, k, v, sm_scale: float, window: int):
    """q ``[H, S, d]`` attends causally to the last ``window`` of k/v ``[H, S, d]`` (same positions)."""
    S = q.shape[1]
    s = torch.einsum("hid,hjd->hij", q.double(), k.double()) * sm_scale
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    mask = (j <= i) & (j > i - window)
    s = s.masked_fill(~mask, -float("inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("hij,hjd->hid", torch.softmax(s, -1), v.double())
    return o.float(), lse.float()
