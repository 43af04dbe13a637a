"""CPU-only checks: the C-ABI library loads and exports what the header declares; host-side logic."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from fast_memory_b200 import _lib
    header = open(os.path.join(ROOT, "include", "fastmem_b200.h")).read()
    declared = set(re.findall(r"\b(fm_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, f"declared in the header but not exported: {missing}"
    assert set(_lib.exported_symbols()) == declared, (set(_lib.exported_symbols()) ^ declared)


def test_status_plumbing_without_a_gpu():
    from fast_memory_b200 import _lib
    L = _lib.lib()
    assert L.fm_abi_version() == 1
    assert L.fm_status_string(0) == b"ok"
    assert b"workspace" in L.fm_status_string(-3)
    # argument validation happens before any CUDA call
    rc = L.fm_hash_rows(None, None, 0, 10, 4, 64, 1, None, None, 10, None, None, 0, None)
    assert rc == -1 and b"null pointer" in L.fm_last_error()
    rc = L.fm_topz_select(None, 1, 1, 1, 1, 0, None, 1, None)
    assert rc == -1
    assert L.fm_group_rows_workspace_bytes(1000, 64) >= 2 * 64 * 4


def test_ops_refuse_cpu_tensors():
    import fast_memory_b200 as fm
    q = torch.zeros(1, 4, 16)
    with pytest.raises(fm.FastMemError):
        fm.attention_hash_varlen(q, q, q, torch.zeros(4, dtype=torch.long), torch.ones(1, 4, dtype=torch.long),
                                 torch.zeros(1, 4, dtype=torch.long), 1.0)
    with pytest.raises(fm.FastMemError):
        fm.hash_rows(torch.zeros(4, 16), torch.zeros(2, 16))
    with pytest.raises(fm.FastMemError):
        fm.Memory.build(torch.zeros(1, 8, 16), torch.zeros(1, 8, 16), n_buckets=2, bucket_size=4)


def test_update_out_and_lse_first_call_needs_no_kernel():
    """mem:61-65: the first call only casts and unsqueezes."""
    import fast_memory_b200 as fm
    bo = torch.randn(1, 2, 5, 8, dtype=torch.bfloat16)
    bl = torch.randn(1, 2, 5)
    out, lse = fm.update_out_and_lse(None, None, bo, bl)
    assert out.dtype == torch.float32 and out.shape == bo.shape
    assert lse.shape == (1, 2, 5, 1) and lse.dtype == torch.float32


def test_synth_configs():
    from fast_memory_b200 import synth
    c = synth.config("cfg1")
    q, k, v = synth.make(c, seed=1)
    assert q.shape == (1, 512, 64) and k.shape == (1, 4096, 64) and q.dtype == torch.float32
    assert torch.allclose(q.norm(dim=-1), torch.ones(512), atol=1e-5)
    q2, k2, _ = synth.make(c, seed=1)
    assert torch.equal(q, q2) and torch.equal(k, k2)
    c3 = synth.config("cfg3")
    q, k, v = synth.make(c3, kv_heads=2, n_keys=1024, n_queries=8)
    assert q.shape == (8, 8, 128) and k.shape == (2, 1024, 128) and k.dtype == torch.bfloat16
    c4 = synth.config("cfg4")
    assert len(c4.seq_keys) == 16 and all(16384 <= n <= 262144 for n in c4.seq_keys)
    assert synth.varlen_buckets(65536) == 256 and synth.varlen_bucket_size(65536) == round(65536 ** 0.7)
    q, k, v, cu_q, cu_k = synth.make_varlen(c4, kv_heads=1, seq_keys=[100, 50], n_queries=4)
    assert q.shape == (1, 8, 128) and k.shape == (1, 150, 128) and cu_k == [0, 100, 150] and cu_q == [0, 4, 8]
