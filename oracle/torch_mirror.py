"""Independent torch mirror of the oracle's math (default fp64), differentiable.

TEST INFRASTRUCTURE ONLY.  It exists so that the C oracle is checked by a
second, structurally different implementation (dense matmuls + masks instead of
row loops) and so that the backward oracle is checked by torch.autograd.
The math is the naive three-pass softmax attention of the reference's
csrc/attention/vanallia_attn.cu:33-82 with the DMLA conventions on top.
"""
from __future__ import annotations

import math

import torch


def _mask(Sq: int, Skv: int, causal: bool, device) -> torch.Tensor:
    """True where key j is visible to query i (bottom-right aligned)."""
    if not causal:
        return torch.ones(Sq, Skv, dtype=torch.bool, device=device)
    i = torch.arange(Sq, device=device)[:, None]
    j = torch.arange(Skv, device=device)[None, :]
    return j <= i + (Skv - Sq)


def attention(Q, Kl, Vl, scale, mask):
    """Q[...,Sq,d] Kl[...,Skv,d] Vl[...,Skv,dv] -> O, m, l (empty rows: -inf,0,0)."""
    S = torch.matmul(Q, Kl.transpose(-1, -2)) * scale
    S = S.masked_fill(~mask, -math.inf)
    m = S.max(dim=-1).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    E = torch.exp(S - m_safe[..., None])
    E = E.masked_fill(~mask, 0.0)
    l = E.sum(dim=-1)
    l_safe = torch.where(l > 0, l, torch.ones_like(l))
    O = torch.matmul(E / l_safe[..., None], Vl)
    return O, m, l


def fwd_cache_latent(Q, K_lat, d_v, scale, causal=True, dtype=torch.float64):
    Q, K_lat = Q.to(dtype), K_lat.to(dtype)
    Sq, Skv = Q.shape[2], K_lat.shape[1]
    Kl = K_lat[:, None]                       # shared by all heads
    return attention(Q, Kl, Kl[..., :d_v], scale, _mask(Sq, Skv, causal, Q.device))


def fwd_on_the_fly(Q, K, V, WK, WV, scale, causal=True, dtype=torch.float64):
    Q, K, V, WK, WV = (t.to(dtype) for t in (Q, K, V, WK, WV))
    Kl, Vl = K @ WK, V @ WV
    Sq, Skv = Q.shape[2], K.shape[2]
    return attention(Q, Kl, Vl, scale, _mask(Sq, Skv, causal, Q.device))


def gather_pages(kv_pool, page_table, b, n_tokens):
    """Rows of sequence b in logical order: pool[table[b, t // ps], t % ps]."""
    ps = kv_pool.shape[1]
    t = torch.arange(n_tokens, device=kv_pool.device)
    rows = page_table[b, t // ps].long() * ps + (t % ps)
    return kv_pool.reshape(-1, kv_pool.shape[-1]).index_select(0, rows)


def decode_paged(Q, kv_pool, page_table, seqlens, d_v, scale, kv_begin=0, kv_end=-1,
                 dtype=torch.float64):
    """Q[B,H,d_qk] -> O[B,H,d_v], m,l[B,H] over tokens [kv_begin, min(kv_end, seqlen))."""
    B, H, _ = Q.shape
    O = torch.zeros(B, H, d_v, dtype=dtype)
    m = torch.full((B, H), -math.inf, dtype=dtype)
    l = torch.zeros(B, H, dtype=dtype)
    for b in range(B):
        hi = int(seqlens[b])
        if kv_end >= 0:
            hi = min(hi, kv_end)
        lo = max(kv_begin, 0)
        if hi <= lo:
            continue
        rows = gather_pages(kv_pool, page_table, b, hi)[lo:].to(dtype)
        mask = torch.ones(1, hi - lo, dtype=torch.bool)
        o, mm, ll = attention(Q[b].to(dtype)[:, None, :], rows[None], rows[None, :, :d_v],
                              scale, mask)
        O[b], m[b], l[b] = o[:, 0], mm[:, 0], ll[:, 0]
    return O, m, l


def merge_partials(O_p, m_p, l_p):
    """LSE merge of partials over disjoint key sets (leading dim = parts)."""
    has = l_p > 0
    m_eff = torch.where(has, m_p, torch.full_like(m_p, -math.inf))
    m = m_eff.max(dim=0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.where(has, l_p * torch.exp(m_eff - m_safe), torch.zeros_like(l_p))
    l = w.sum(dim=0)
    l_safe = torch.where(l > 0, l, torch.ones_like(l))
    O = (w[..., None] * O_p).sum(dim=0) / l_safe[..., None]
    return O, m, l


def bwd_on_the_fly_autograd(Q, K, V, WK, WV, dO, scale, causal=True, dtype=torch.float64):
    """Gradients of the on-the-fly forward by torch.autograd."""
    ts = [t.detach().to(dtype).requires_grad_(True) for t in (Q, K, V, WK, WV)]
    O, _, _ = fwd_on_the_fly(*ts, scale, causal, dtype)
    return torch.autograd.grad(O, ts, dO.to(dtype))


def bwd_cache_latent_autograd(Q, K_lat, d_v, dO, scale, causal=True, dtype=torch.float64):
    ts = [t.detach().to(dtype).requires_grad_(True) for t in (Q, K_lat)]
    O, _, _ = fwd_cache_latent(ts[0], ts[1], d_v, scale, causal, dtype)
    return torch.autograd.grad(O, ts, dO.to(dtype))
