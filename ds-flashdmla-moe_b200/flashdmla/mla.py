"""The steps either side of the decode kernel inside an MLA block: latent down-projection of
the new token into the paged cache, and the "absorbed" query / output projections that let
the kernel work on the 576-wide latent rows while the caller keeps standard multi-head shapes
(the reference's "drop-in for standard MHA shapes", README.md:16).

    c_t   = h_t W_DKV                      latent, d_lat = 512        \\ one cache row
    k^R_t = rope(h_t W_KR)                 shared RoPE key, d_rope = 64 /  [c_t | k^R_t]  (576)
    q_h   = h_t W_Q[h] = [q^N_h | q^R_h]   d_nope + d_rope per head
    score_h(t, j) = q^N_h . (c_j W_UK[h]) + rope(q^R_h) . k^R_j
                  = (q^N_h W_UK[h]^T) . c_j + rope(q^R_h) . k^R_j      <- absorbed: Q' = [q^N W_UK^T | rope(q^R)]
    out_h = (sum_j p_hj c_j) W_UV[h]                                   <- kernel returns sum_j p c_j (512 wide)

The two absorbed projections - one small GEMM per head, directly before and after the attention
kernel - run on the library's own tensor-core GEMM (`flashdmla.gemm.absorb_query`, which also
writes the RoPE tail of Q', and `flashdmla.gemm.project_out`; CUDA bf16 tensors only, like the
attention kernel between them); the dense projections with the model-wide weights (`W_Q`, `W_DKV`, `W_KR`, `W_O`) are plain
library GEMMs.  The attention itself is `PagedLatentCache.decode`.  `reference_decode` restates
the same block with explicit per-head keys and values in fp32 for the tests.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

from .cache import PagedLatentCache


def rope(x: torch.Tensor, pos: torch.Tensor, base: float = 10000.0) -> torch.Tensor:
    """Rotary embedding of the last dimension (pairs (2i, 2i+1)); pos broadcasts against x[..., 0]."""
    d = x.shape[-1]
    inv = base ** (-torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d)
    ang = pos.to(torch.float32)[..., None] * inv
    c, s = torch.cos(ang), torch.sin(ang)
    xf = x.to(torch.float32)
    x0, x1 = xf[..., 0::2], xf[..., 1::2]
    out = torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), dim=-1).flatten(-2)
    return out.to(x.dtype)


class AbsorbedMLA:
    """Weights of one MLA attention block and its decode step over a PagedLatentCache."""

    def __init__(self, d_model: int, n_heads: int, d_lat: int = 512, d_rope: int = 64, d_nope: int = 128,
                 d_vhead: int = 128, dtype=torch.bfloat16, device="cuda", seed: int = 0):
        g = torch.Generator().manual_seed(seed)

        def w(*shape, fan_in):
            return (torch.randn(*shape, generator=g) / math.sqrt(fan_in)).to(dtype).to(device)
        self.H, self.d_lat, self.d_rope, self.d_nope, self.d_vhead = n_heads, d_lat, d_rope, d_nope, d_vhead
        self.W_DKV = w(d_model, d_lat, fan_in=d_model)
        self.W_KR = w(d_model, d_rope, fan_in=d_model)
        self.W_Q = w(d_model, n_heads * (d_nope + d_rope), fan_in=d_model)
        self.W_UK = w(n_heads, d_lat, d_nope, fan_in=d_lat)
        self.W_UV = w(n_heads, d_lat, d_vhead, fan_in=d_lat)
        self.W_O = w(n_heads * d_vhead, d_model, fan_in=n_heads * d_vhead)
        self.scale = 1.0 / math.sqrt(d_nope + d_rope)

    # ---- the step before the kernel: what is written into the cache ---------------------
    def cache_rows(self, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """h [n, t, d_model], pos [n, t] -> cache rows [n, t, d_lat + d_rope]."""
        return torch.cat((h @ self.W_DKV, rope(h @ self.W_KR, pos)), dim=-1)

    # ---- the absorbed query -------------------------------------------------------------
    def absorbed_query(self, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """h [n, d_model], pos [n] -> Q' [n, H, d_lat + d_rope]."""
        n = h.shape[0]
        q = (h @ self.W_Q).view(n, self.H, self.d_nope + self.d_rope)
        from . import gemm
        return gemm.absorb_query(q.contiguous(), self.W_UK, pos, self.d_nope)      # CUDA bf16 only, like the attention

    def absorbed_query_torch(self, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """The same Q' written with torch operators, any device and dtype: what the tests of the algebra compare with."""
        n = h.shape[0]
        q = (h @ self.W_Q).view(n, self.H, self.d_nope + self.d_rope)
        q_lat = torch.einsum("nhd,hld->nhl", q[..., : self.d_nope], self.W_UK)
        q_rope = rope(q[..., self.d_nope:], pos[:, None].expand(n, self.H))
        return torch.cat((q_lat, q_rope), dim=-1).contiguous()

    def decode(self, cache: PagedLatentCache, slots: Sequence[int], h: torch.Tensor) -> torch.Tensor:
        """Append the new token of every listed sequence and attend: h [n, d_model] -> [n, d_model]."""
        pos = torch.tensor([cache.length(s) for s in slots], device=h.device)
        cache.append(slots, self.cache_rows(h[:, None, :], pos[:, None]))
        o_lat, _, _ = cache.decode(self.absorbed_query(h, pos), slots, self.d_lat, self.scale)
        from . import gemm
        o = gemm.project_out(o_lat.contiguous(), self.W_UV)
        return o.reshape(h.shape[0], self.H * self.d_vhead) @ self.W_O

    # ---- the same block without absorption, fp32, for tests --------------------------------
    def reference_decode(self, rows: torch.Tensor, h: torch.Tensor, pos: int) -> torch.Tensor:
        """rows [T, d_lat + d_rope]: the sequence's cache rows including the new token; h [d_model]."""
        f = lambda t: t.to(torch.float32)
        c, kr = f(rows[:, : self.d_lat]), f(rows[:, self.d_lat:])
        q = f(h @ self.W_Q).view(self.H, self.d_nope + self.d_rope)
        qr = f(rope(q[:, self.d_nope:].to(h.dtype), torch.full((self.H,), pos, device=h.device)))
        k_nope = torch.einsum("tl,hld->htd", c, f(self.W_UK))                 # per-head keys [H, T, d_nope]
        v = torch.einsum("tl,hlv->htv", c, f(self.W_UV))                      # per-head values
        s = (torch.einsum("hd,htd->ht", q[:, : self.d_nope], k_nope) + qr @ kr.T) * self.scale
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("ht,htv->hv", p, v)
        return o.reshape(-1) @ f(self.W_O)
