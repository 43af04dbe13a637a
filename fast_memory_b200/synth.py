"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Keys are unit directions drawn from a mixture of ``n_clusters`` centres on the sphere (centre + N(0, sigma^2 I),
renormalised) times a log-normal norm; values are N(0, 1); queries come from the same mixture with unit
norm scale.  These stand in for real model activations: the reference names no dataset.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional

import torch


@dataclasses.dataclass
class Config:
    name: str
    kv_heads: int
    q_groups: int            # query heads per KV head
    d: int
    dtype: torch.dtype
    n_keys: int              # keys per KV head (per sequence list for varlen: see seq_keys)
    n_queries: int           # queries per query head
    n_clusters: int
    sigma: float
    norm_sigma: float
    n_buckets: int
    bucket_size: int
    kmeans_iters: int = 2
    local_window: int = 0    # cfg2: causal local-window attention merged with the memory output
    seq_keys: Optional[List[int]] = None      # cfg4: keys per sequence
    shards: int = 1          # cfg5: logical key shards


def config(name: str, seed: int = 0) -> Config:
    bf16, f32 = torch.bfloat16, torch.float32
    if name == "cfg1":
        return Config("cfg1", 1, 1, 64, f32, 4096, 512, 64, 0.3, 0.25, 64, 256)
    if name == "cfg2":
        return Config("cfg2", 32, 1, 128, bf16, 131072, 8192, 512, 0.25, 0.3, 512, 2048, local_window=4096)
    if name == "cfg3":
        return Config("cfg3", 8, 4, 128, bf16, 1048576, 64, 1024, 0.25, 0.3, 1024, 8192)
    if name == "cfg4":
        g = torch.Generator().manual_seed(1000 + seed)
        seq = torch.randint(16384, 262144 + 1, (16,), generator=g).tolist()
        return Config("cfg4", 8, 1, 128, bf16, sum(seq), 1024, 256, 0.3, 0.3, 0, 0, seq_keys=seq)
    if name == "cfg5":
        return Config("cfg5", 8, 1, 128, bf16, 4194304, 16384, 4096, 0.25, 0.3, 1024, 8192, shards=8)
    raise ValueError(f"unknown config {name}")


def varlen_buckets(n: int) -> int:
    """cfg4: C = round(sqrt(N)) to a multiple of 16."""
    return max(16, int(round(n ** 0.5 / 16.0)) * 16)


def varlen_bucket_size(n: int) -> int:
    """cfg4: Z = round(N^0.7)."""
    return int(round(n ** 0.7))


def mixture(n: int, centres: torch.Tensor, sigma: float, gen: torch.Generator, chunk: int = 1 << 20) -> torch.Tensor:
    """n unit vectors: a random centre plus N(0, sigma^2 I), renormalised.  fp32, on centres' device."""
    dev = centres.device
    out = torch.empty(n, centres.shape[1], dtype=torch.float32, device=dev)
    for i in range(0, n, chunk):
        m = min(chunk, n - i)
        which = torch.randint(centres.shape[0], (m,), generator=gen, device=dev)
        x = centres[which] + sigma * torch.randn(m, centres.shape[1], generator=gen, device=dev)
        out[i:i + m] = torch.nn.functional.normalize(x, dim=-1)
    return out


def make_head(n_keys: int, n_queries: int, d: int, n_clusters: int, sigma: float, norm_sigma: float, dtype,
              gen: torch.Generator, device):
    centres = torch.nn.functional.normalize(torch.randn(n_clusters, d, generator=gen, device=device), dim=-1)
    k = mixture(n_keys, centres, sigma, gen)
    k *= torch.exp(norm_sigma * torch.randn(n_keys, 1, generator=gen, device=device))
    v = torch.randn(n_keys, d, generator=gen, device=device)
    q = mixture(n_queries, centres, sigma, gen)
    return q.to(dtype), k.to(dtype), v.to(dtype)


def make(cfg: Config, seed: int = 0, device="cpu", kv_heads: Optional[int] = None, n_keys: Optional[int] = None,
         n_queries: Optional[int] = None):
    """(q [Hq, S, d], k [H, N, d], v [H, N, d]) for a uniform config (cfg1, 2, 3, 5); optional size
    overrides make cut-down cases with the same distribution."""
    H = kv_heads or cfg.kv_heads
    N = n_keys or cfg.n_keys
    S = n_queries or cfg.n_queries
    gen = torch.Generator(device=device).manual_seed(seed)
    qs, ks, vs = [], [], []
    for _ in range(H):
        q, k, v = make_head(N, S * cfg.q_groups, cfg.d, cfg.n_clusters, cfg.sigma, cfg.norm_sigma, cfg.dtype, gen, device)
        qs.append(q.reshape(cfg.q_groups, S, cfg.d))
        ks.append(k)
        vs.append(v)
    return torch.cat(qs, 0), torch.stack(ks, 0), torch.stack(vs, 0)


def make_varlen(cfg: Config, seed: int = 0, device="cpu", kv_heads: Optional[int] = None,
                seq_keys: Optional[List[int]] = None, n_queries: Optional[int] = None):
    """Packed (q [H, S_total, d], k, v [H, N_total, d], cu_seqlens_q, cu_seqlens_k) for cfg4."""
    H = kv_heads or cfg.kv_heads
    seq = seq_keys or cfg.seq_keys
    S = n_queries or cfg.n_queries
    gen = torch.Generator(device=device).manual_seed(seed)
    cu_k, cu_q = [0], [0]
    for n in seq:
        cu_k.append(cu_k[-1] + n)
        cu_q.append(cu_q[-1] + S)
    q = torch.empty(H, cu_q[-1], cfg.d, dtype=cfg.dtype, device=device)
    k = torch.empty(H, cu_k[-1], cfg.d, dtype=cfg.dtype, device=device)
    v = torch.empty_like(k)
    for h in range(H):
        for s, n in enumerate(seq):
            qq, kk, vv = make_head(n, S, cfg.d, cfg.n_clusters, cfg.sigma, cfg.norm_sigma, cfg.dtype, gen, device)
            q[h, cu_q[s]:cu_q[s + 1]] = qq
            k[h, cu_k[s]:cu_k[s + 1]] = kk
            v[h, cu_k[s]:cu_k[s + 1]] = vv
    return q, k, v, cu_q, cu_k
