"""Generate the golden vectors in this folder by running the REFERENCE's own code.

Run once where the reference checkout is available (it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/reference                       # CPU: fp32 / fp16 vectors
    python tests/golden/make_golden.py /path/to/reference --native-bf16 OUTDIR  # on a GPU: bf16 vectors

What is run, unmodified:
  * ``triton_kernel.attention_hash_varlen`` (the wrapper, tk:51-119) with the Triton kernel ``_attn_fwd``
    (tk:135-272) executed by Triton's CPU interpreter.  The only substitution is the launcher
    (tk:16-41): the custom-op/autotune wrapper needs a GPU driver, so the un-tuned JIT function is
    launched with the same arguments.
  * ``memory.update_out_and_lse`` (mem:54-71), ``memory.ring_attention_masked_forward_ref`` (mem:74-103)
    and ``memory.compute_centroids`` (mem:209-231), eager (``TORCHDYNAMO_DISABLE=1``).
A stub ``labml`` module stands in for the third-party logger the reference imports.

``--native-bf16`` runs the same wrapper with the kernel compiled natively by Triton on the GPU present (the
CPU interpreter cannot do bf16), launcher and all unmodified, on bf16 inputs generated on the CPU from the
same seeded recipe; besides the wrapper's outputs (LSE rounded to bf16, tk:111) it records the fp32 LSE the
kernel itself wrote, converted to natural log.

Inputs follow the reference's self-test generator (tk:302-322): N(0, 0.5^2) tensors, random query
hashes, table = topk of uniform noise, entries >= 0.9 N masked out.
"""
import os
import sys
import types

NATIVE = "--native-bf16" in sys.argv
if not NATIVE:
    os.environ["TRITON_INTERPRET"] = "1"
os.environ["TORCHDYNAMO_DISABLE"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _stub_labml():
    lab = types.ModuleType("labml")

    class _Sec:
        def __init__(self, *a, **k):
            self.success = True

        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    class _Text:
        danger = success = title = key = None

    monit = types.ModuleType("labml.monit")
    monit.section = _Sec
    logger = types.ModuleType("labml.logger")
    logger.log = lambda *a, **k: None
    logger.Text = _Text
    tracker = types.ModuleType("labml.tracker")
    tracker.add = lambda *a, **k: None
    lab.monit, lab.logger, lab.tracker = monit, logger, tracker
    sys.modules.update({"labml": lab, "labml.monit": monit, "labml.logger": logger, "labml.tracker": tracker})


def _load_reference(path):
    _stub_labml()
    sys.path.insert(0, path)
    import triton_kernel as tk
    import memory as mem

    def launch(q, k, v, kh, khc, kho, qz, qc, qo, sm_scale, q_seq_len, kv_seq_len, d_head, n_buckets):
        o = torch.empty_like(q)
        lse = torch.empty(q.shape[:-1], dtype=torch.float32)
        tk._attn_fwd.fn[(len(qc), 1, 1)](q, k, v, kh, khc, kho, qz, qc, qo, lse, o,
                                         sm_scale=sm_scale, q_seq_len=q_seq_len, kv_seq_len=kv_seq_len,
                                         d_head=d_head, BLOCK_K=tk._BLOCK_K, BLOCK_Q=tk._BLOCK_Q,
                                         n_buckets=n_buckets)
        return o, lse

    tk._attention_hash_varlen = launch
    return tk, mem


def _np(t):
    """Detached numpy COPY (the reference's merge mutates its accumulators in place, mem:68-69)."""
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.float().numpy().copy()
    return t.numpy().copy()


def attn_case(tk, name, B, S, N, C, Z, d, dtype, seed, keep=0.9, window=None):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, S, d, generator=g) * 0.5).to(dtype)
    k = (torch.randn(B, N, d, generator=g) * 0.5).to(dtype)
    v = (torch.randn(B, N, d, generator=g) * 0.5).to(dtype)
    q_hashes = torch.randint(C, (B, S), generator=g)
    table = torch.topk(torch.rand(B, C, N, generator=g), dim=-1, k=Z, sorted=True)[1]
    if window is None:
        mask = table < int(N * keep)
    else:                                   # tk:314-316: only a narrow key range survives -> empty buckets
        mask = torch.logical_and(window[0] <= table, table < window[1])
    counts = mask.to(torch.long).sum(-1)
    sm_scale = d ** -0.5
    o, lse = tk.attention_hash_varlen(q, k, v, table[mask], counts, q_hashes, sm_scale)
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        q=_np(q), k=_np(k), v=_np(v), q_hashes=q_hashes.numpy(),
                        k_hashes=table[mask].numpy(), k_hash_counts=counts.numpy(),
                        sm_scale=np.float64(sm_scale), dtype=str(dtype).replace("torch.", ""),
                        o=_np(o), lse=_np(lse))
    print(name, "o", tuple(o.shape), "lse range", float(lse.min()), float(lse.max()))


def merge_case(mem, name, seed):
    g = torch.Generator().manual_seed(seed)
    rows, d = 96, 32
    blocks = []
    for i in range(3):
        bo = torch.randn(1, 2, rows, d, generator=g)
        if i == 1:
            bo = bo.to(torch.bfloat16)
        bl = torch.randn(1, 2, rows, generator=g) * 3.0
        blocks.append((bo, bl))
    out, lse = None, None
    outs = {}
    for i, (bo, bl) in enumerate(blocks):
        outs[f"block_out{i}"] = _np(bo)
        outs[f"block_lse{i}"] = _np(bl)
        out, lse = mem.update_out_and_lse(out, lse, bo, bl)
        outs[f"out{i}"] = out.clone().numpy()
        outs[f"lse{i}"] = lse.clone().numpy()
    outs["block_out1_dtype"] = "bfloat16"
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **outs)
    print(name, "ok")


def dense_ref_case(mem, name, seed):
    """mem:74-103 on two key shards (rank 0 and 1) of a GLOBAL table, GQA with 2 groups."""
    g = torch.Generator().manual_seed(seed)
    k_heads, n_groups, S, ctx, d, C, Z, W = 2, 2, 40, 256, 32, 8, 48, 2
    q = torch.randn(1, k_heads * n_groups, S, d, generator=g) * 0.5
    k = torch.randn(W, 1, k_heads, ctx, d, generator=g) * 0.5
    v = torch.randn(W, 1, k_heads, ctx, d, generator=g) * 0.5
    k_hashes = torch.topk(torch.rand(C, k_heads, W * ctx, generator=g), dim=-1, k=Z)[1]    # global indices
    q_hashes = torch.randint(C, (k_heads, n_groups, S), generator=g)
    h_idx = torch.arange(k_heads)
    sm_scale = d ** -0.5
    res = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), k_hashes=k_hashes.numpy(), q_hashes=q_hashes.numpy(),
               sm_scale=np.float64(sm_scale))
    out, lse = None, None
    for r in range(W):
        bo, bl = mem.ring_attention_masked_forward_ref(k_hashes, q_hashes, h_idx, q, k[r], v[r], sm_scale, r)
        res[f"out_rank{r}"] = _np(bo)
        res[f"lse_rank{r}"] = _np(bl)
        out, lse = mem.update_out_and_lse(out, lse, bo, bl)
    res["out_merged"] = out.numpy()
    res["lse_merged"] = lse.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **res)
    print(name, "ok")


def backward_case(mem, name, seed):
    """mem:166-206 (the function under its ``torch.compile`` wrapper, run eagerly) on two key shards of a GLOBAL table
    with the MERGED forward result of both shards, GQA with 2 groups."""
    g = torch.Generator().manual_seed(seed)
    k_heads, n_groups, S, ctx, d, C, Z, W = 2, 2, 24, 128, 32, 8, 40, 2
    q = torch.randn(1, k_heads * n_groups, S, d, generator=g) * 0.5
    k = torch.randn(W, 1, k_heads, ctx, d, generator=g) * 0.5
    v = torch.randn(W, 1, k_heads, ctx, d, generator=g) * 0.5
    d_out = torch.randn(1, k_heads * n_groups, S, d, generator=g)
    k_hashes = torch.topk(torch.rand(C, k_heads, W * ctx, generator=g), dim=-1, k=Z)[1]    # global indices
    q_hashes = torch.randint(C, (k_heads, n_groups, S), generator=g)
    h_idx = torch.arange(k_heads)
    sm_scale = d ** -0.5
    out, lse = None, None
    for r in range(W):
        bo, bl = mem.ring_attention_masked_forward_ref(k_hashes, q_hashes, h_idx, q, k[r], v[r], sm_scale, r)
        out, lse = mem.update_out_and_lse(out, lse, bo, bl)
    bwd = mem.ring_attention_masked_backward
    bwd = getattr(bwd, "_torchdynamo_orig_callable", bwd)
    res = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), d_out=d_out.numpy(), k_hashes=k_hashes.numpy(), q_hashes=q_hashes.numpy(),
               sm_scale=np.float64(sm_scale), out=_np(out), lse=_np(lse.squeeze(-1)))
    for r in range(W):
        dq, dk, dv = bwd(k_hashes, q_hashes, h_idx, d_out, q, k[r], v[r], out, lse.squeeze(-1), sm_scale, r)
        res[f"dq_rank{r}"], res[f"dk_rank{r}"], res[f"dv_rank{r}"] = _np(dq), _np(dk), _np(dv)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **res)
    print(name, "ok")


def centroids_case(mem, name, seed):
    g = torch.Generator().manual_seed(seed)
    n_heads, n_groups, ctx, d, C, topk = 4, 2, 300, 32, 8, 12
    kq = torch.randn(n_heads, ctx, d, generator=g)
    cent = torch.randn(C, d, generator=g)
    cent = cent / cent.norm(dim=-1, keepdim=True)
    mem.consts = types.SimpleNamespace(centroid_topk=topk)
    out = mem.compute_centroids(kq, cent, C, n_groups)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), kq=kq.numpy(), centroids=cent.numpy(),
                        n_groups=n_groups, centroid_topk=topk, out=out.numpy())
    print(name, tuple(out.shape))


def native_attn_case(tk, out_dir, name, B, S, N, C, Z, d, dtype, seed, keep=0.9):
    """The reference wrapper and kernel, natively compiled, on a GPU.  Inputs are drawn on the CPU."""
    import math
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, S, d, generator=g) * 0.5).to(dtype)
    k = (torch.randn(B, N, d, generator=g) * 0.5).to(dtype)
    v = (torch.randn(B, N, d, generator=g) * 0.5).to(dtype)
    q_hashes = torch.randint(C, (B, S), generator=g)
    table = torch.topk(torch.rand(B, C, N, generator=g), dim=-1, k=Z, sorted=True)[1]
    mask = table < int(N * keep)
    mask[:, C // 2] = False                  # one bucket without keys in every batch row
    counts = mask.to(torch.long).sum(-1)
    sm_scale = d ** -0.5
    dev = "cuda"
    seen = {}
    launch = tk._attention_hash_varlen

    def spy(*a, **kw):                        # the fp32 base-2 LSE as the kernel wrote it, in sorted order
        o, lse = launch(*a, **kw)
        seen["lse2"] = lse.clone()
        return o, lse

    tk._attention_hash_varlen = spy
    o, lse = tk.attention_hash_varlen(q.to(dev), k.to(dev), v.to(dev), table[mask].to(dev), counts.to(dev),
                                      q_hashes.to(dev), sm_scale)
    tk._attention_hash_varlen = launch
    order = torch.sort(q_hashes, dim=1, stable=True)[1]
    lse_f32 = torch.empty(B, S)
    lse_f32[torch.arange(B)[:, None], order] = seen["lse2"].cpu() * math.log(2)
    np.savez_compressed(os.path.join(out_dir, name + ".npz"),
                        q=_np(q), k=_np(k), v=_np(v), q_hashes=q_hashes.numpy(),
                        k_hashes=table[mask].numpy(), k_hash_counts=counts.numpy(),
                        sm_scale=np.float64(sm_scale), dtype=str(dtype).replace("torch.", ""),
                        o=_np(o.cpu()), lse=_np(lse.cpu()), lse_f32=lse_f32.numpy(),
                        device=torch.cuda.get_device_name(0))
    print(name, "o", tuple(o.shape), "lse range", float(lse_f32[torch.isfinite(lse_f32)].min()), float(lse_f32.max()))


def main_native(ref, out_dir):
    _stub_labml()
    sys.path.insert(0, ref)
    import triton_kernel as tk
    os.makedirs(out_dir, exist_ok=True)
    native_attn_case(tk, out_dir, "attn_bf16_ragged", 2, 300, 1024, 16, 100, 64, torch.bfloat16, seed=25)
    native_attn_case(tk, out_dir, "attn_bf16_d128", 2, 200, 2048, 8, 300, 128, torch.bfloat16, seed=26)
    native_attn_case(tk, out_dir, "attn_f16_native_d64", 1, 150, 1024, 8, 200, 64, torch.float16, seed=27)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference [--native-bf16 OUTDIR]")
    ref = sys.argv[1]
    if NATIVE:
        return main_native(ref, sys.argv[sys.argv.index("--native-bf16") + 1])
    tk, mem = _load_reference(ref)
    # the reference self-test's small shape (tk:500) and cut-down versions of its large one (tk:502)
    attn_case(tk, "attn_f32_tiny", 1, 24, 1024, 8, 16, 16, torch.float32, seed=20)
    attn_case(tk, "attn_f32_ragged", 2, 300, 1024, 16, 100, 32, torch.float32, seed=21)
    attn_case(tk, "attn_f16_ragged", 2, 300, 1024, 16, 100, 32, torch.float16, seed=22)
    attn_case(tk, "attn_f32_d128", 1, 70, 512, 4, 150, 128, torch.float32, seed=23)
    attn_case(tk, "attn_f32_empty_buckets", 2, 64, 1024, 32, 40, 32, torch.float32, seed=24, window=(700, 730))
    merge_case(mem, "merge_chain", seed=30)
    dense_ref_case(mem, "dense_ref_two_shards", seed=40)
    centroids_case(mem, "compute_centroids", seed=50)
    backward_case(mem, "backward_two_shards", seed=60)


if __name__ == "__main__":
    main()
