"""Helpers shared by the GPU parity tests: the checker side always runs on CPU through ``oracle``."""
import numpy as np
import torch

from oracle import oracle as O

TOL_O = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}   # abs tolerance on O
TOL_LSE = 1e-3                                                              # abs tolerance on fp32 LSE


def random_case(B, S, N, C, Z, d, dtype, seed, keep=0.9, scale=0.5):
    """Inputs in the manner of the reference self-test (tk:302-322), generated on CPU."""
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, S, d, generator=g) * scale).to(dtype)
    k = (torch.randn(B, N, d, generator=g) * scale).to(dtype)
    v = (torch.randn(B, N, d, generator=g) * scale).to(dtype)
    q_hashes = torch.randint(C, (B, S), generator=g)
    table = torch.topk(torch.rand(B, C, N, generator=g), dim=-1, k=Z, sorted=True)[1]
    mask = table < int(N * keep)
    return q, k, v, table[mask], mask.long().sum(-1), q_hashes


def assert_attn_close(o, lse, o_ref, lse_ref, dtype):
    o, lse, o_ref, lse_ref = o.float().cpu(), lse.float().cpu(), o_ref.float().cpu(), lse_ref.float().cpu()
    assert torch.isfinite(o).all()
    err_o = (o - o_ref).abs().max().item()
    assert err_o <= TOL_O[dtype], f"O max abs err {err_o}"
    inf_ref = torch.isinf(lse_ref)
    assert torch.equal(torch.isinf(lse), inf_ref), "empty-bucket rows differ"
    if (~inf_ref).any():
        err_l = (lse[~inf_ref] - lse_ref[~inf_ref]).abs().max().item()
        assert err_l <= TOL_LSE, f"LSE max abs err {err_l}"


def oracle_for_sampled_queries(mem, q, hashes, sm_scale, rows):
    """Oracle O / LSE for a sample of query rows of a (possibly huge) memory: gathers each query's bucket
    from the device table and evaluates it on CPU.  ``rows``: list of (head, position)."""
    d = q.shape[-1]
    Hq, S = q.shape[0], q.shape[1]
    G = Hq // mem.n_heads
    kf, vf = mem.k.reshape(-1, d), mem.v.reshape(-1, d)
    outs, lses = [], []
    for (h, s) in rows:
        seg = h // G if mem.n_seq == 1 else None
        assert seg is not None
        gb = mem.seg_cb[seg] + int(hashes[h, s])
        lo, hi = int(mem.bucket_off[gb]), int(mem.bucket_off[gb + 1])
        idx = mem.table[lo:hi].long()
        kk, vv = kf[idx].cpu(), vf[idx].cpu()
        n = kk.shape[0]
        o, l = O.hashed_attention(q[h, s].cpu()[None, None], kk[None], vv[None], torch.arange(n),
                                  torch.tensor([[n]]), torch.zeros(1, 1, dtype=torch.long), sm_scale)
        outs.append(o[0, 0])
        lses.append(l[0, 0])
    return torch.stack(outs), torch.stack(lses)


def tables_equal_as_sets(t_gpu, t_ref):
    """Both [C, Z] with ascending rows -> plain equality; helper reports the first differing bucket."""
    a, b = np.asarray(t_gpu), np.asarray(t_ref)
    if a.shape != b.shape:
        return False, f"shape {a.shape} vs {b.shape}"
    if np.array_equal(a, b):
        return True, ""
    bad = np.nonzero((a != b).any(-1))[0]
    c = int(bad[0])
    return False, f"{len(bad)} buckets differ; bucket {c}: only-gpu {sorted(set(a[c]) - set(b[c]))[:5]} only-ref {sorted(set(b[c]) - set(a[c]))[:5]}"
