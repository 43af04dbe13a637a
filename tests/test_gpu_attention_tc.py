"""The tcgen05 / TMEM form of the hashed attention (``fm_set_attn_kernel(1)``): same parity bar as the default kernel,
plus the case it hands back to the kernel that tracks a running maximum."""
import numpy as np
import os
import pytest
import torch

import fast_memory_b200 as fm
from oracle import oracle as O
from tests.util import assert_attn_close, random_case

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"float16": torch.float16, "bfloat16": torch.bfloat16}


@pytest.fixture(autouse=True)
def tc_kernel():
    fm.set_attention_kernel("tc")
    yield
    fm.set_attention_kernel("mma")


def _run(q, k, v, kh, cnt, qh, sm, **kw):
    return fm.attention_hash_varlen(q.to(DEV), k.to(DEV), v.to(DEV), kh.to(DEV), cnt.to(DEV), qh.to(DEV), sm, **kw)


@pytest.mark.parametrize("name", ["attn_bf16_d128"])
def test_matches_native_reference_golden(golden_dir, name):
    """Outputs of the reference's kernel compiled natively on a B200 (bf16, head dim 128)."""
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    dt = DT[str(z["dtype"])]
    t = lambda a: torch.from_numpy(np.asarray(a))
    o, lse = _run(t(z["q"]).to(dt), t(z["k"]).to(dt), t(z["v"]).to(dt), t(z["k_hashes"]), t(z["k_hash_counts"]), t(z["q_hashes"]),
                  float(z["sm_scale"]), return_fp32_lse=True)
    assert_attn_close(o, lse, t(z["o"]), t(z["lse_f32"]), dt)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 40, 600, 4, 130), (2, 150, 700, 12, 90), (1, 200, 3000, 4, 1000), (1, 9, 3000, 4, 1000)])
def test_random_ragged_vs_oracle(dtype, shape):
    """Partial tiles, buckets with more than 32 queries (several items), few queries with long buckets (split into key
    chunks, partials combined), empty buckets."""
    B, S, N, C, Z = shape
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, 128, dtype, seed=11 + S)
    o, lse = _run(q, k, v, kh, cnt, qh, 128 ** -0.5, return_fp32_lse=True)
    o_ref, lse_ref = O.hashed_attention(q, k, v, kh, cnt, qh, 128 ** -0.5)
    assert_attn_close(o, lse, o_ref, lse_ref, dtype)


def test_many_groups_equal_the_default_kernel():
    """8 heads x 512 buckets with ~24 queries each (items of 17-32 and of up to 16 queries): the two kernels agree to
    rounding, and runs repeat bit for bit."""
    B, S, N, C, Z, d, dtype = 8, 512 * 24, 2048, 512, 203, 128, torch.bfloat16
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=31)
    a = _run(q, k, v, kh, cnt, qh, d ** -0.5, return_fp32_lse=True)
    b = _run(q, k, v, kh, cnt, qh, d ** -0.5, return_fp32_lse=True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    fm.set_attention_kernel("mma")
    c = _run(q, k, v, kh, cnt, qh, d ** -0.5, return_fp32_lse=True)
    assert (a[0].float() - c[0].float()).abs().max() <= 2e-2 and (a[1] - c[1]).abs().max() <= 1e-3


@pytest.mark.parametrize("dtype,big", [(torch.bfloat16, 40.0), (torch.float16, 6.0)])
def test_late_dominant_key_is_served_again(dtype, big):
    """The kernel refers every p to the maximum over the item's FIRST 128 keys.  A key further down whose score beats
    that by more than the number range allows (2^204 here for bf16, 2^30 for fp16) makes the item's denominator
    overflow; the item is handed to the running-maximum kernel and the result is still right."""
    g = torch.Generator().manual_seed(7)
    N, S, d = 1000, 20, 128
    q = torch.randn(1, S, d, generator=g) * 0.1
    k = torch.randn(1, N, d, generator=g) * 0.1
    q[0, :, 0] = 40.0
    k[0, 700, 0] = big
    v = torch.randn(1, N, d, generator=g)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    kh, cnt, qh = torch.arange(N), torch.tensor([[N]]), torch.zeros(1, S, dtype=torch.long)
    o, lse = _run(q, k, v, kh, cnt, qh, d ** -0.5, return_fp32_lse=True)
    o_ref, lse_ref = O.hashed_attention(q, k, v, kh, cnt, qh, d ** -0.5)
    assert_attn_close(o, lse, o_ref, lse_ref, dtype)
