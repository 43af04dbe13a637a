"""The reference's own GPU kernel as a comparator and as the source of bf16 golden vectors.

notbadai/fast_memory ships one GPU kernel: the Triton ``_attn_fwd`` behind ``attention_hash_varlen``
(triton_kernel.py:16-41, 51-119, 135-272).  Triton JIT-compiles it for whatever device is present, so on a
B200 it is the kernel this library has to beat, and it is the only way to get results of the reference in
bf16 (Triton's CPU interpreter does not handle bf16).

``install(src)`` copies the two reference modules UNMODIFIED into ``baseline/_ref/`` (git-ignored) together
with a stub of the third-party ``labml`` logger they import; ``load()`` imports them from there.  Nothing in
the library depends on this module: the benchmark and the GPU tests use it when ``baseline/_ref`` exists and
skip the comparator otherwise.
"""
from __future__ import annotations

import math
import os
import shutil
import sys
from typing import Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_FILES = ("triton_kernel.py", "memory.py")

_LABML_STUB = '''"""Stand-in for the third-party ``labml`` logger imported by the reference modules."""


class _Section:
    def __init__(self, *args, **kwargs):
        self.success = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _Text:
    danger = success = title = key = value = meta = None


class _Monit:
    section = _Section


class _Logger:
    Text = _Text

    @staticmethod
    def log(*args, **kwargs):
        pass

    @staticmethod
    def inspect(*args, **kwargs):
        pass


class _Tracker:
    @staticmethod
    def add(*args, **kwargs):
        pass

    @staticmethod
    def save(*args, **kwargs):
        pass


monit, logger, tracker = _Monit(), _Logger(), _Tracker()
'''


def default_source() -> str:
    """Where a reference checkout is looked for: ``$FASTMEM_REFERENCE_DIR``, else a ``reference`` folder beside
    this repository."""
    return os.environ.get("FASTMEM_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def install(src: Optional[str] = None) -> bool:
    """Copy the reference modules into ``baseline/_ref``.  Returns False when no checkout is found."""
    src = src or default_source()
    if not all(os.path.exists(os.path.join(src, f)) for f in REF_FILES):
        return False
    os.makedirs(os.path.join(REF_DIR, "labml"), exist_ok=True)
    for f in REF_FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(REF_DIR, f))
    with open(os.path.join(REF_DIR, "labml", "__init__.py"), "w") as fh:
        fh.write(_LABML_STUB)
    return True


def available() -> bool:
    return all(os.path.exists(os.path.join(REF_DIR, f)) for f in REF_FILES)


def load():
    """Import the reference's ``triton_kernel`` module from ``baseline/_ref`` (needs a GPU for its kernel)."""
    if not available():
        raise RuntimeError("baseline/_ref is empty: run baseline.ref_gpu.install(<reference checkout>) first")
    # Triton compiles a small host launcher with the C compiler; the image's default wrapper is known to fail
    if os.path.exists("/usr/bin/gcc") and "CC" not in os.environ:
        os.environ["CC"] = "/usr/bin/gcc"
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import triton_kernel
    return triton_kernel


def sorted_operands(q, q_hashes, k_hash_counts):
    """The operands the reference's registered operator takes (triton_kernel.py:17-22), made from the wrapper's
    arguments the way its wrapper makes them (a stable sort of the query hashes per batch row, one entry per
    non-empty (row, bucket) group, exclusive prefix sums): ``(q_sorted, order, group_bucket, group_count,
    group_offset, k_hash_offset)``.  ``order`` un-sorts the operator's outputs."""
    import torch
    B, S, _ = q.shape
    C = k_hash_counts.shape[1]
    z, order = torch.sort(q_hashes, dim=1, stable=True)
    rows = torch.arange(B, device=q.device)[:, None]
    q_sorted = q[rows, order].contiguous()
    gb, cnt = torch.unique_consecutive(z + rows * C, return_counts=True)
    off = torch.cumsum(cnt, 0) - cnt
    flat = k_hash_counts.reshape(-1)
    k_off = (torch.cumsum(flat, 0) - flat).reshape(k_hash_counts.shape)
    return q_sorted, order, gb % C, cnt, off, k_off


def reference_forward_fp32_lse(tk, q, k, v, k_hashes, k_hash_counts, q_hashes, sm_scale) -> Tuple:
    """``(o, lse)`` of the reference kernel in the original query order with the LSE as the kernel wrote it (fp32),
    converted from base 2 to natural log: the wrapper rounds it to q's dtype first (triton_kernel.py:111), which
    hides differences below a bf16 ulp."""
    import torch
    B, S, d = q.shape
    qs, order, gz, gc, go, k_off = sorted_operands(q, q_hashes, k_hash_counts)
    o_s, lse2 = torch.ops.notbad.attention_hash_varlen(qs, k, v, k_hashes, k_hash_counts, k_off, gz, gc, go,
                                                       sm_scale=sm_scale, q_seq_len=S, kv_seq_len=k.shape[1],
                                                       d_head=d, n_buckets=k_hash_counts.shape[1])
    rows = torch.arange(B, device=q.device)[:, None]
    o = torch.empty_like(o_s)
    o[rows, order] = o_s
    lse = torch.empty_like(lse2)
    lse[rows, order] = lse2 * math.log(2)
    return o, lse
