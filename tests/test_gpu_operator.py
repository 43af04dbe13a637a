"""The registered operators (the reference registers ``notbad::attention_hash_varlen``, tk:16-48): schema checks,
tracing, the operator with the reference's own fourteen arguments, autograd, and - when the reference modules have
been copied into ``baseline/_ref`` - the reference's Triton kernel itself, compiled natively, on the same inputs."""
import math

import pytest
import torch

import fast_memory_b200 as fm
from baseline import ref_gpu
from fast_memory_b200 import ops
from oracle import oracle as O
from tests.util import TOL_LSE, TOL_O, assert_attn_close, random_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(dtype, B=2, S=150, N=700, C=12, Z=90, d=64, seed=5):
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=seed)
    return tuple(t.to(DEV) for t in (q, k, v, kh, cnt, qh)) + (d ** -0.5,)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_operator_with_the_reference_schema(dtype):
    """``fast_memory_b200::attention_hash_varlen`` takes the sorted queries and group lists the reference's operator
    takes (tk:17-22) and returns what its kernel writes: o in sorted order, fp32 LSE in base 2."""
    q, k, v, kh, cnt, qh, sm = _case(dtype)
    B, S, d = q.shape
    qs, order, gz, gc, go, k_off = ref_gpu.sorted_operands(q, qh, cnt)
    o_s, lse2 = torch.ops.fast_memory_b200.attention_hash_varlen(qs, k, v, kh, cnt, k_off, gz, gc, go, sm, S, k.shape[1],
                                                                 d, cnt.shape[1])
    assert o_s.dtype == dtype and lse2.dtype == torch.float32 and o_s.shape == q.shape and lse2.shape == (B, S)
    rows = torch.arange(B, device=DEV)[:, None]
    o = torch.empty_like(o_s)
    o[rows, order] = o_s
    lse = torch.empty_like(lse2)
    lse[rows, order] = lse2 * math.log(2)
    o_ref, lse_ref = O.hashed_attention(q.cpu(), k.cpu(), v.cpu(), kh.cpu(), cnt.cpu(), qh.cpu(), sm)
    assert_attn_close(o, lse, o_ref, lse_ref, dtype)
    # the function with the wrapper's arguments goes through the other operator and must agree
    o2, lse_nat = fm.attention_hash_varlen(q, k, v, kh, cnt, qh, sm, return_fp32_lse=True)
    assert (o2.float() - o.float()).abs().max() <= TOL_O[dtype]
    fin = torch.isfinite(lse_nat)
    assert torch.equal(fin, torch.isfinite(lse)) and (lse_nat[fin] - lse[fin]).abs().max() <= TOL_LSE


def test_opcheck_of_the_registered_operators():
    q, k, v, kh, cnt, qh, sm = _case(torch.bfloat16)
    B, S, d = q.shape
    qs, order, gz, gc, go, k_off = ref_gpu.sorted_operands(q, qh, cnt)
    torch.library.opcheck(torch.ops.fast_memory_b200.attention_hash_varlen.default,
                          (qs, k, v, kh, cnt, k_off, gz, gc, go, sm, S, k.shape[1], d, cnt.shape[1]))
    torch.library.opcheck(torch.ops.fast_memory_b200.hashed_attention_grouped.default,
                          (q, k, v, kh, cnt, qh, sm, int(cnt.max())),
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
    k_hashes = torch.randint(0, 512, (8, 2, 40), device=DEV)
    torch.library.opcheck(torch.ops.fast_memory_b200.shard_filter.default, (k_hashes, 128, 256))


def test_no_gradient_through_the_reference_schema_operator():
    """tk:44-48: the reference's operator takes part in autograd and hands back no gradient."""
    q, k, v, kh, cnt, qh, sm = _case(torch.float32)
    B, S, d = q.shape
    qs, order, gz, gc, go, k_off = ref_gpu.sorted_operands(q, qh, cnt)
    qs.requires_grad_(True)
    o, lse2 = torch.ops.fast_memory_b200.attention_hash_varlen(qs, k, v, kh, cnt, k_off, gz, gc, go, sm, S, k.shape[1], d,
                                                               cnt.shape[1])
    assert o.requires_grad
    o.sum().backward()
    assert qs.grad is None


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 4e-2)])
def test_autograd_of_the_grouped_operator(dtype, tol):
    """d(o)/d(q, k, v) of ``attention_hash_varlen`` through autograd against a dense fp64 restatement (every query
    attends the keys of its bucket, mem:74-103)."""
    B, S, N, C, Z, d = 2, 70, 300, 6, 40, 32
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=9)
    sm = d ** -0.5
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    o, _ = fm.attention_hash_varlen(qd, kd, vd, kh.to(DEV), cnt.to(DEV), qh.to(DEV), sm)
    g = torch.Generator().manual_seed(1)
    d_o = torch.randn(B, S, d, generator=g).to(dtype)
    o.backward(d_o.to(DEV))
    # dense restatement in fp64 on the CPU
    q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
    mask = torch.zeros(B, S, N, dtype=torch.bool)
    off = 0
    for b in range(B):
        for c in range(C):
            n = int(cnt[b, c])
            idx = kh[off:off + n]
            off += n
            rows = (qh[b] == c).nonzero().flatten()
            mask[b, rows[:, None], idx[None, :]] = True
    s = torch.einsum("bsd,bnd->bsn", q64, k64) * sm
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    p = torch.nan_to_num(p, nan=0.0)
    (torch.einsum("bsn,bnd->bsd", p, v64) * d_o.double()).sum().backward()
    for got, ref in ((qd.grad, q64.grad), (kd.grad, k64.grad), (vd.grad, v64.grad)):
        assert got.dtype == dtype
        assert (got.double().cpu() - ref).abs().max() <= tol * max(1.0, float(ref.abs().max()))


def test_ring_attention_masked_forward_under_torch_compile():
    """The reference compiles this function (``@torch.compile``, mem:106); traced with the ``aot_eager`` backend it
    gives the eager result bit for bit."""
    g = torch.Generator().manual_seed(4)
    k_heads, n_groups, S, ctx, d, C, Z, W = 2, 2, 40, 256, 32, 8, 48, 2
    q = (torch.randn(1, k_heads * n_groups, S, d, generator=g) * 0.5).bfloat16().to(DEV)
    k = (torch.randn(1, k_heads, ctx, d, generator=g) * 0.5).bfloat16().to(DEV)
    v = (torch.randn(1, k_heads, ctx, d, generator=g) * 0.5).bfloat16().to(DEV)
    k_hashes = torch.topk(torch.rand(C, k_heads, W * ctx, generator=g), dim=-1, k=Z)[1].to(DEV)
    q_hashes = torch.randint(C, (k_heads, n_groups, S), generator=g).to(DEV)
    sm = d ** -0.5
    eager = fm.ring_attention_masked_forward(k_hashes, q_hashes, q, k, v, sm, 1)
    compiled = torch.compile(fm.ring_attention_masked_forward, backend="aot_eager")(k_hashes, q_hashes, q, k, v, sm, 1)
    assert torch.equal(eager[0], compiled[0]) and torch.equal(eager[1], compiled[1])


def test_workspaces_are_per_stream():
    """Two streams serve queries against one memory at the same time: each stream has its own scratch (work list,
    counters, partials), so both results equal the single-stream result."""
    q, k, v, kh, cnt, qh, sm = _case(torch.bfloat16, B=2, S=4000, N=3000, C=40, Z=300, d=128)
    ref = fm.attention_hash_varlen(q, k, v, kh, cnt, qh, sm, return_fp32_lse=True)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for _ in range(3):
        for s in (s1, s2):
            with torch.cuda.stream(s):
                outs.append(fm.attention_hash_varlen(q, k, v, kh, cnt, qh, sm, return_fp32_lse=True))
    torch.cuda.synchronize()
    for o, lse in outs:
        assert torch.equal(o, ref[0]) and torch.equal(lse, ref[1])
    keys = [kk for kk in ops._ws._bufs if kk[0] == "attn"]
    assert len({kk[2] for kk in keys}) >= 3                      # the default stream and the two side streams


@pytest.mark.skipif(not ref_gpu.available(), reason="the reference modules are not in baseline/_ref")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_against_the_reference_triton_kernel(dtype):
    """The reference's wrapper + Triton kernel (tk:51-272), JIT-compiled for this GPU, on a reduced config-2 shape:
    O within 2e-2, fp32 LSE (as the kernel writes it, before the wrapper rounds it to q's dtype) within 1e-3."""
    tk = ref_gpu.load()
    B, S, N, C, Z, d = 2, 3000, 8192, 64, 700, 128
    q, k, v, kh, cnt, qh = random_case(B, S, N, C, Z, d, dtype, seed=41)
    q, k, v, kh, cnt, qh = (t.to(DEV) for t in (q, k, v, kh, cnt, qh))
    sm = d ** -0.5
    o_ref, lse_ref = ref_gpu.reference_forward_fp32_lse(tk, q, k, v, kh, cnt, qh, sm)
    o, lse = fm.attention_hash_varlen(q, k, v, kh, cnt, qh, sm, return_fp32_lse=True)
    assert (o.float() - o_ref.float()).abs().max() <= TOL_O[dtype]
    fin = torch.isfinite(lse_ref)
    assert torch.equal(fin, torch.isfinite(lse))
    assert (lse[fin] - lse_ref[fin]).abs().max() <= TOL_LSE
    # and the wrapper's own convention (LSE in q's dtype after nan_to_num)
    o_w, lse_w = tk.attention_hash_varlen(q, k, v, kh, cnt, qh, sm)
    o_d, lse_d = fm.attention_hash_varlen(q, k, v, kh, cnt, qh, sm)
    assert lse_d.dtype == lse_w.dtype == dtype
    assert (o_d.float() - o_w.float()).abs().max() <= TOL_O[dtype]
    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    assert ((lse_d.float() - lse_w.float()).abs() <= 2 * ulp * lse_w.float().abs().clamp_min(1.0)).all()


def test_builds_from_two_host_threads_on_two_streams():
    """Two host threads build (and query) different memories on their own streams at the same time.  The fused build
    keeps a side stream and two events per device; the enqueue of a build is serialised inside the library, the
    scratch memory is per stream, so both tables equal those of the same builds run one after the other."""
    import threading
    g = torch.Generator().manual_seed(11)
    H, N, C, Z, d = 2, 16384, 64, 256, 128
    data = []
    for _ in range(2):
        k = torch.randn(H, N, d, generator=g).bfloat16().to(DEV)
        A = torch.nn.functional.normalize(torch.randn(H, C, d, generator=g), dim=-1).bfloat16().to(DEV)
        data.append((k, A))
    ref = [fm.Memory.build(k, k, A=A, bucket_size=Z).table.clone() for k, A in data]
    torch.cuda.synchronize()
    out, errs = [None, None], []

    def work(i):
        try:
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                for _ in range(6):
                    mem = fm.Memory.build(data[i][0], data[i][0], A=data[i][1], bucket_size=Z)
                out[i] = mem.table.clone()
            s.synchronize()
        except Exception as e:                                  # noqa: BLE001 - reported by the assert below
            errs.append(e)

    th = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert not errs, errs
    assert torch.equal(out[0], ref[0]) and torch.equal(out[1], ref[1])
