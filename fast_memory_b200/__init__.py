"""fast_memory_b200 - B200-native LSH attention memory (index build, query hashing, hashed attention, LSE merge).

The operators run in an in-tree CUDA library (``libfastmem_b200.so``, C ABI in ``include/fastmem_b200.h``);
build it with ``python -m fast_memory_b200.build``.  There is no CPU or PyTorch fallback.
"""
from ._lib import FastMemError, launch_count
from .memory import Memory, compute_centroids, kmeans_projection, merge
from .ops import (attention_hash, attention_hash_varlen, group_rows, hash_rows, hashed_attention, hashed_attention_backward, lse_merge, lse_merge_out, project,
                  ring_attention_masked_forward, set_attention_kernel, shard_filter, topz_select, unit_rows, update_out_and_lse)

__all__ = [
    "hashed_attention_backward",
    "lse_merge_out",
    "compute_centroids",
    "FastMemError", "Memory", "attention_hash", "attention_hash_varlen", "group_rows", "hash_rows", "hashed_attention",
    "kmeans_projection", "launch_count", "lse_merge", "merge", "project", "ring_attention_masked_forward", "shard_filter",
    "topz_select", "unit_rows", "update_out_and_lse", "set_attention_kernel",
]
