"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations.  Tensors are generated per unit (per sequence, per
batch entry, per (batch, head)) from `base_seed * 1_000_000 + unit_id`, so any
sharding over ranks reproduces the same global tensors.
"""
from __future__ import annotations

import math

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


def unit_normal(shape, base_seed: int, unit: int, std: float = 1.0) -> torch.Tensor:
    return torch.randn(*shape, generator=_gen(base_seed * 1_000_000 + unit)) * std


def cache_latent_inputs(B, H, Sq, Skv, d_qk, std=0.5, seed=1, dtype=torch.float32,
                        batch_ids=None, head_ids=None):
    """Q [B,H,Sq,d_qk], K_lat [B,Skv,d_qk] for the listed batch entries / heads."""
    batch_ids = list(range(B)) if batch_ids is None else list(batch_ids)
    head_ids = list(range(H)) if head_ids is None else list(head_ids)
    Q = torch.stack([torch.stack([unit_normal((Sq, d_qk), seed, 1000 + b * H + h, std)
                                  for h in head_ids]) for b in batch_ids])
    K = torch.stack([unit_normal((Skv, d_qk), seed, 500_000 + b, std) for b in batch_ids])
    return Q.to(dtype), K.to(dtype)


def xavier_uniform(d_in, d_out, seed, unit):
    bound = math.sqrt(6.0 / (d_in + d_out))
    return (torch.rand(d_in, d_out, generator=_gen(seed * 1_000_000 + unit)) * 2 - 1) * bound


def on_the_fly_inputs(B, H, Sq, Skv, d_model, d_lat, seed=2, dtype=torch.bfloat16):
    Q = torch.stack([torch.stack([unit_normal((Sq, d_lat), seed, 1000 + b * H + h)
                                  for h in range(H)]) for b in range(B)])
    K = torch.stack([torch.stack([unit_normal((Skv, d_model), seed, 200_000 + b * H + h)
                                  for h in range(H)]) for b in range(B)])
    V = torch.stack([torch.stack([unit_normal((Skv, d_model), seed, 400_000 + b * H + h)
                                  for h in range(H)]) for b in range(B)])
    WK = xavier_uniform(d_model, d_lat, seed, 900_001)
    WV = xavier_uniform(d_model, d_lat, seed, 900_002)
    return tuple(t.to(dtype) for t in (Q, K, V, WK, WV))


def paged_decode_inputs(B, H, seqlens, d_qk, page_size, seed=3, std=0.1, dtype=torch.bfloat16,
                        seq_ids=None, shuffle_pages=True):
    """Q [n,H,d_qk], pool [pages,page_size,d_qk], page_table [n,max_pages], seqlens [n]
    for the listed sequences (default: all B).  Page ids are a seeded random
    permutation of the local pool."""
    seq_ids = list(range(B)) if seq_ids is None else list(seq_ids)
    lens = [int(seqlens[b]) for b in seq_ids]
    pages_per = [(s + page_size - 1) // page_size for s in lens]
    max_pages = max(pages_per) if pages_per else 0
    n_pages = sum(pages_per)
    perm = (torch.randperm(n_pages, generator=_gen(seed * 1_000_000 + 7)) if shuffle_pages
            else torch.arange(n_pages))
    pool = torch.zeros(max(n_pages, 1), page_size, d_qk, dtype=dtype)
    table = torch.zeros(len(seq_ids), max(max_pages, 1), dtype=torch.int32)
    Qs, cursor = [], 0
    for n, b in enumerate(seq_ids):
        Qs.append(unit_normal((H, d_qk), seed, 1000 + b, std))
        rows = unit_normal((pages_per[n] * page_size, d_qk), seed, 500_000 + b, std).to(dtype)
        ids = perm[cursor:cursor + pages_per[n]]
        cursor += pages_per[n]
        pool[ids] = rows.view(pages_per[n], page_size, d_qk)
        table[n, :pages_per[n]] = ids.to(torch.int32)
    Q = torch.stack(Qs).to(dtype) if Qs else torch.zeros(0, H, d_qk, dtype=dtype)
    return Q, pool, table, torch.tensor(lens, dtype=torch.int32)
