"""ctypes binding of ``libfastmem_b200.so`` (declared in ``include/fastmem_b200.h``).

There is no fallback: if the CUDA library is missing, importing the ops fails with a message saying how
to build it, and every entry point raises when a call returns a non-OK status.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FASTMEM_B200_LIB") or os.path.join(_HERE, "libfastmem_b200.so")      # another build of the library

F32, BF16, F16 = 0, 1, 2
_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


class FastMemError(RuntimeError):
    pass


def dtype_id(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"fast_memory_b200 supports float32, bfloat16 and float16 tensors, got {dt}") from None


_SIGNATURES = {
    "fm_abi_version": (c_int, []),
    "fm_status_string": (c_char_p, [c_int]),
    "fm_last_error": (c_char_p, []),
    "fm_launch_count": (c_int64, []),
    "fm_hash_rows_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "fm_hash_rows": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int64,
                             c_void_p, c_void_p, c_size_t, c_void_p]),
    "fm_group_rows_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "fm_group_rows": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_size_t, c_void_p]),
    "fm_group_rows_segmented": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p,
                                        c_void_p, c_void_p, c_size_t, c_void_p]),
    "fm_group_rows_static_max_buckets": (c_int64, []),
    "fm_group_rows_static": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p]),
    "fm_hashed_attn_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_int64]),
    "fm_set_attn_kernel": (c_int, [c_int]),
    "fm_test_set_tc_hooks": (c_int, [c_int, c_int]),
    "fm_hashed_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p,
                                   c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_float, c_void_p,
                                   c_void_p, c_int64, c_void_p, c_size_t, c_void_p]),
    "fm_shard_filter_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "fm_shard_filter": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                c_size_t, c_void_p]),
    "fm_hashed_attn_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p]),
    "fm_lse_merge": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_void_p]),
    "fm_lse_merge_out": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int,
                                 c_void_p]),
    "fm_merge_peer_partials": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_void_p]),
    "fm_project": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_int64, c_void_p]),
    "fm_project_tc_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "fm_project_tc": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int64, c_void_p, c_int64, c_void_p,
                              c_size_t, c_void_p]),
    "fm_topz_select": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int32, c_void_p, c_int64, c_void_p]),
    "fm_index_build_workspace_bytes": (c_size_t, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]),
    "fm_index_build": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "fm_kmeans_workspace_bytes": (c_size_t, [c_int, c_void_p, c_void_p, c_int]),
    "fm_kmeans": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                          c_size_t, c_void_p]),
    "fm_unit_rows": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p]),
    "fm_table_scores": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fm_gather_mean": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built (``python -m fast_memory_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FastMemError(
                f"{LIB_PATH} is missing: build the CUDA library with `python -m fast_memory_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)              # AttributeError here = header and library out of step
            fn.restype = res
            fn.argtypes = args
        if L.fm_abi_version() != 1:
            raise FastMemError(f"ABI version {L.fm_abi_version()} of {LIB_PATH} does not match this package (1)")
        _lib = L
    return _lib


def exported_symbols():
    return sorted(_SIGNATURES)


def check(status: int, what: str) -> None:
    if status != 0:
        L = lib()
        raise FastMemError(f"{what}: {L.fm_status_string(status).decode()} ({status}): {L.fm_last_error().decode()}")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise FastMemError("fast_memory_b200 ops run on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors on different devices: {t.device} vs {dev}")
    return dev


def host_i64(values):
    """A ctypes int64 array (host) from a python sequence."""
    arr = (c_int64 * len(values))(*[int(v) for v in values])
    return arr


def launch_count() -> int:
    return int(lib().fm_launch_count())
