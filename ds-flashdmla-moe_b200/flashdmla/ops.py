"""Flash-DMLA operators: autograd.Function wrappers with MHA-shaped signatures.

This is the Python surface the reference advertises as python/ops.py
(README.md:16,24-25,54-56: "custom autograd.Function wrappers", "drop-in
interface compatible with standard MHA shapes", two execution modes, row
statistics m and l saved for backward).  PyTorch is used only for device
memory and streams; all arithmetic happens in libflashdmla.so.

Every operator requires CUDA tensors and raises otherwise: there is no CPU or
eager fallback.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import FlashDMLAError, check


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.F32
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    raise FlashDMLAError(f"unsupported dtype {t.dtype}: float32 and bfloat16 only")


def _need_cuda(*ts: torch.Tensor) -> None:
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise FlashDMLAError("Flash-DMLA operators need CUDA tensors (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise FlashDMLAError("all tensors must live on the same GPU")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _same_dtype(*ts: torch.Tensor) -> None:
    for t in ts[1:]:
        if t.dtype != ts[0].dtype:
            raise FlashDMLAError("all floating-point inputs must share one dtype")


# --------------------------------------------------------------------------- #
# cache-latent mode
# --------------------------------------------------------------------------- #
class FlashDMLACacheLatentFn(torch.autograd.Function):
    """O, m, l = attention(Q, K_lat) with V = K_lat[..., :d_v].

    Q [B,H,Sq,d_qk], K_lat [B,Skv,d_qk] (shared by all heads) ->
    O [B,H,Sq,d_v], m,l [B,H,Sq] fp32 (non-differentiable).
    """

    @staticmethod
    def forward(ctx, Q, K_lat, d_v, scale, causal):
        _need_cuda(Q, K_lat)
        _same_dtype(Q, K_lat)
        if Q.dim() != 4 or K_lat.dim() != 3 or Q.shape[0] != K_lat.shape[0] or Q.shape[3] != K_lat.shape[2]:
            raise FlashDMLAError("expected Q [B,H,Sq,d_qk] and K_lat [B,Skv,d_qk]")
        Q, K_lat = Q.contiguous(), K_lat.contiguous()
        B, H, Sq, d_qk = Q.shape
        Skv = K_lat.shape[1]
        if scale is None:
            scale = 1.0 / math.sqrt(d_qk)
        O = torch.empty(B, H, Sq, d_v, dtype=Q.dtype, device=Q.device)
        m = torch.empty(B, H, Sq, dtype=torch.float32, device=Q.device)
        l = torch.empty(B, H, Sq, dtype=torch.float32, device=Q.device)
        with torch.cuda.device(Q.device):
            check(_lib.lib().fdmla_fwd_cache_latent(
                _ptr(Q), _ptr(K_lat), _ptr(O), _ptr(m), _ptr(l), B, H, Sq, Skv, d_qk, int(d_v),
                float(scale), int(bool(causal)), _dtype_code(Q), _stream(Q)), "fdmla_fwd_cache_latent")
        ctx.save_for_backward(Q, K_lat, O, m, l)
        ctx.scale, ctx.causal, ctx.d_v = float(scale), bool(causal), int(d_v)
        ctx.mark_non_differentiable(m, l)
        return O, m, l

    @staticmethod
    def backward(ctx, dO, _dm, _dl):
        Q, K_lat, O, m, l = ctx.saved_tensors
        B, H, Sq, d_qk = Q.shape
        Skv = K_lat.shape[1]
        dO = dO.contiguous().to(Q.dtype)
        dQ = torch.empty_like(Q)
        dK = torch.empty_like(K_lat)
        code = _dtype_code(Q)
        with torch.cuda.device(Q.device):
            L = _lib.lib()
            nbytes = L.fdmla_bwd_cache_latent_workspace_bytes(B, H, Sq, Skv, d_qk, ctx.d_v, code)
            ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=Q.device)
            check(L.fdmla_bwd_cache_latent(
                _ptr(Q), _ptr(K_lat), _ptr(O), _ptr(m), _ptr(l), _ptr(dO), _ptr(dQ), _ptr(dK),
                _ptr(ws), ws.numel(), B, H, Sq, Skv, d_qk, ctx.d_v, ctx.scale, int(ctx.causal),
                code, _stream(Q)), "fdmla_bwd_cache_latent")
        return dQ, dK, None, None, None


def flash_dmla_cache_latent(Q, K_lat, d_v, scale=None, causal=True):
    return FlashDMLACacheLatentFn.apply(Q, K_lat, d_v, scale, causal)


# --------------------------------------------------------------------------- #
# on-the-fly mode
# --------------------------------------------------------------------------- #
class FlashDMLAOnTheFlyFn(torch.autograd.Function):
    """O, m, l = attention(Q, K WK, V WV); WK, WV learnable.

    Q [B,H,Sq,d_lat], K,V [B,H,Skv,d_model], WK,WV [d_model,d_lat] ->
    O [B,H,Sq,d_lat], m,l [B,H,Sq] fp32.  backward(dO) -> dQ,dK,dV,dWK,dWV.
    """

    @staticmethod
    def forward(ctx, Q, K, V, WK, WV, scale, causal):
        _need_cuda(Q, K, V, WK, WV)
        _same_dtype(Q, K, V, WK, WV)
        if Q.dim() != 4 or K.dim() != 4 or K.shape != V.shape or WK.shape != WV.shape:
            raise FlashDMLAError("expected Q [B,H,Sq,d_lat], K,V [B,H,Skv,d_model], WK,WV [d_model,d_lat]")
        if K.shape[:2] != Q.shape[:2] or WK.shape[0] != K.shape[3] or WK.shape[1] != Q.shape[3]:
            raise FlashDMLAError("shape mismatch between Q, K/V and WK/WV")
        Q, K, V, WK, WV = (t.contiguous() for t in (Q, K, V, WK, WV))
        B, H, Sq, d_lat = Q.shape
        Skv, d_model = K.shape[2], K.shape[3]
        if scale is None:
            scale = 1.0 / math.sqrt(d_lat)
        code = _dtype_code(Q)
        O = torch.empty_like(Q)
        m = torch.empty(B, H, Sq, dtype=torch.float32, device=Q.device)
        l = torch.empty(B, H, Sq, dtype=torch.float32, device=Q.device)
        with torch.cuda.device(Q.device):
            L = _lib.lib()
            nbytes = L.fdmla_fwd_on_the_fly_workspace_bytes(B, H, Skv, d_lat, code)
            ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=Q.device)
            check(L.fdmla_fwd_on_the_fly(
                _ptr(Q), _ptr(K), _ptr(V), _ptr(WK), _ptr(WV), _ptr(O), _ptr(m), _ptr(l), _ptr(ws),
                ws.numel(), B, H, Sq, Skv, d_model, d_lat, float(scale), int(bool(causal)), code,
                _stream(Q)), "fdmla_fwd_on_the_fly")
        ctx.save_for_backward(Q, K, V, WK, WV, O, m, l)
        ctx.scale, ctx.causal = float(scale), bool(causal)
        ctx.mark_non_differentiable(m, l)
        return O, m, l

    @staticmethod
    def backward(ctx, dO, _dm, _dl):
        Q, K, V, WK, WV, O, m, l = ctx.saved_tensors
        B, H, Sq, d_lat = Q.shape
        Skv, d_model = K.shape[2], K.shape[3]
        dO = dO.contiguous().to(Q.dtype)
        dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
        dWK, dWV = torch.empty_like(WK), torch.empty_like(WV)
        code = _dtype_code(Q)
        with torch.cuda.device(Q.device):
            L = _lib.lib()
            nbytes = L.fdmla_bwd_on_the_fly_workspace_bytes(B, H, Sq, Skv, d_model, d_lat, code)
            ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=Q.device)
            check(L.fdmla_bwd_on_the_fly(
                _ptr(Q), _ptr(K), _ptr(V), _ptr(WK), _ptr(WV), _ptr(O), _ptr(m), _ptr(l), _ptr(dO),
                _ptr(dQ), _ptr(dK), _ptr(dV), _ptr(dWK), _ptr(dWV), _ptr(ws), ws.numel(), B, H, Sq,
                Skv, d_model, d_lat, ctx.scale, int(ctx.causal), code, _stream(Q)),
                "fdmla_bwd_on_the_fly")
        return dQ, dK, dV, dWK, dWV, None, None


def flash_dmla_on_the_fly(Q, K, V, WK, WV, scale=None, causal=True):
    return FlashDMLAOnTheFlyFn.apply(Q, K, V, WK, WV, scale, causal)


# --------------------------------------------------------------------------- #
# paged decode
# --------------------------------------------------------------------------- #
class DecodeWorkspace:
    """Caller-owned scratch for split-KV partials, reused across decode steps."""

    def __init__(self):
        self.O_part = self.m_part = self.l_part = None

    def get(self, splits: int, B: int, H: int, d_v: int, device) -> Tuple[torch.Tensor, ...]:
        need = splits * B * H
        if self.O_part is None or self.O_part.device != device or self.m_part.numel() < need \
                or self.O_part.numel() < need * d_v:
            self.O_part = torch.empty(need * d_v, dtype=torch.float32, device=device)
            self.m_part = torch.empty(need, dtype=torch.float32, device=device)
            self.l_part = torch.empty(need, dtype=torch.float32, device=device)
        return self.O_part, self.m_part, self.l_part


def suggest_splits(B: int, H: int, max_seqlen: int, d_qk: int, d_v: int, page_size: int,
                   dtype: torch.dtype = torch.bfloat16) -> int:
    code = _lib.F32 if dtype == torch.float32 else _lib.BF16
    return int(_lib.lib().fdmla_decode_suggest_splits(B, H, int(max_seqlen), d_qk, d_v, page_size, code))


def flash_dmla_paged_decode(Q, kv_pool, page_table, seqlens, d_v, scale=None, num_splits=None,
                            kv_begin=0, kv_end=-1, workspace: Optional[DecodeWorkspace] = None,
                            max_seqlen: Optional[int] = None, partial_only=False, out=None):
    """One decode step over a paged latent KV cache.

    Q [B,H,d_qk] or [B,H,1,d_qk]; kv_pool [num_pages,page_size,d_qk];
    page_table [B,max_pages] int32; seqlens [B] int32.
    Returns O [B,H,(1,)d_v] (Q's dtype), m, l [B,H,(1)] fp32.  With
    partial_only=True returns the fp32 partials (O_part [S,B,H,d_v], m_part,
    l_part [S,B,H]) of the attended window [kv_begin, kv_end) instead.
    out = (O, m, l) or, with partial_only, (O_part, m_part, l_part): contiguous
    tensors of those shapes to write into instead of fresh ones (a caller that
    keeps its results in one staging or message buffer passes views of it).
    """
    _need_cuda(Q, kv_pool, page_table, seqlens)
    _same_dtype(Q, kv_pool)
    squeeze = Q.dim() == 4
    if squeeze:
        if Q.shape[2] != 1:
            raise FlashDMLAError("decode takes one query token per sequence")
        Q = Q[:, :, 0, :]
    if page_table.dtype != torch.int32 or seqlens.dtype != torch.int32:
        raise FlashDMLAError("page_table and seqlens must be int32")
    Q, kv_pool = Q.contiguous(), kv_pool.contiguous()
    page_table, seqlens = page_table.contiguous(), seqlens.contiguous()
    B, H, d_qk = Q.shape
    num_pages, page_size, d_pool = kv_pool.shape
    if d_pool != d_qk or page_table.shape[0] != B or seqlens.shape[0] != B:
        raise FlashDMLAError("shape mismatch between Q, kv_pool, page_table and seqlens")
    max_pages = page_table.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(d_qk)
    code = _dtype_code(Q)
    if num_splits is None:
        span = max_seqlen if max_seqlen is not None else max_pages * page_size
        if kv_end >= 0:
            span = min(span, kv_end)
        span = max(span - max(kv_begin, 0), 1)
        num_splits = suggest_splits(B, H, span, d_qk, d_v, page_size, Q.dtype)
    num_splits = max(1, int(num_splits))
    dev = Q.device
    O_part = m_part = l_part = None
    if out is not None:
        want = ([(num_splits, B, H, d_v), (num_splits, B, H), (num_splits, B, H)] if partial_only
                else [(B, H, d_v), (B, H), (B, H)])
        dts = [torch.float32 if partial_only else Q.dtype, torch.float32, torch.float32]
        if len(out) != 3:
            raise FlashDMLAError("out must be a triple of tensors")
        for t, shp, dt in zip(out, want, dts):
            if tuple(t.shape) != shp or t.dtype != dt or not t.is_contiguous() or t.device != dev:
                raise FlashDMLAError(f"out tensor must be contiguous {shp} {dt} on {dev}")
    if partial_only and out is not None:
        O_part, m_part, l_part = out
    elif num_splits > 1 or partial_only:
        if workspace is not None and not partial_only:
            O_part, m_part, l_part = workspace.get(num_splits, B, H, d_v, dev)
        else:
            O_part = torch.empty(num_splits * B * H * d_v, dtype=torch.float32, device=dev)
            m_part = torch.empty(num_splits * B * H, dtype=torch.float32, device=dev)
            l_part = torch.empty(num_splits * B * H, dtype=torch.float32, device=dev)
    O = m = l = None
    if not partial_only and out is not None:
        O, m, l = out
    elif not partial_only:
        O = torch.empty(B, H, d_v, dtype=Q.dtype, device=dev)
        m = torch.empty(B, H, dtype=torch.float32, device=dev)
        l = torch.empty(B, H, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(_lib.lib().fdmla_decode_paged(
            _ptr(Q), _ptr(kv_pool), _ptr(page_table), _ptr(seqlens), _ptr(O), _ptr(m), _ptr(l),
            _ptr(O_part), _ptr(m_part), _ptr(l_part), B, H, d_qk, int(d_v), page_size, max_pages,
            num_pages, num_splits, int(kv_begin), int(kv_end), float(scale), code, _stream(Q)),
            "fdmla_decode_paged")
    if partial_only:
        return (O_part.reshape(-1)[: num_splits * B * H * d_v].view(num_splits, B, H, d_v),
                m_part.reshape(-1)[: num_splits * B * H].view(num_splits, B, H),
                l_part.reshape(-1)[: num_splits * B * H].view(num_splits, B, H))
    if squeeze:
        return O[:, :, None, :], m[:, :, None], l[:, :, None]
    return O, m, l


def suggest_partial_slabs(B: int, H: int, max_tokens: int, page_size: int = 64) -> int:
    """Scratch slabs for flash_dmla_paged_decode_partial: enough that a run of tiles (the work of one CTA pair) may be
    half as long as it would be if every sequence had max_tokens keys, so ragged batches still balance; 1 when the
    batch alone fills the GPU."""
    import ctypes
    units = ctypes.c_int(0)
    max_pages = max((int(max_tokens) + page_size - 1) // page_size, 1)
    _lib.lib().fdmla_decode_plan(B, H, 576, 512, page_size, max_pages, 2, _lib.BF16, None, ctypes.byref(units))
    pairs = units.value or 74
    tiles = max((int(max_tokens) + 255) // 256, 1)
    if B >= pairs or H > 128 or H < 2:
        return 1
    run = max(-(-B * tiles // pairs), 1)
    return int(min(64, max(2, 2 * -(-tiles // run) + 1)))


def flash_dmla_paged_decode_partial(Q, kv_pool, page_table, seqlens, d_v, scale=None, num_splits=None, out=None,
                                    scratch=None, pieces_only=False):
    """Attention of Q [B,H,d_qk] over the whole of this paged cache as an fp32 partial result: O [B,H,d_v] normalised
    by its own l, m, l [B,H] - what a rank that holds one slice of every sequence sends to its peers.  out: three
    contiguous fp32 tensors to write into (views of a message buffer); scratch: (O_part [S,B,H,d_v], m_part, l_part
    [S,B,H]) fp32 for num_splits = S > 1, allocated when missing.  pieces_only (S > 1): leave the pieces unmerged in
    `scratch` and return it - for a caller that merges them itself (`PeerExchange.merge_parts`); pieces with l <= 0
    hold nothing."""
    _need_cuda(Q, kv_pool, page_table, seqlens)
    _same_dtype(Q, kv_pool)
    if page_table.dtype != torch.int32 or seqlens.dtype != torch.int32:
        raise FlashDMLAError("page_table and seqlens must be int32")
    Q, kv_pool, page_table, seqlens = Q.contiguous(), kv_pool.contiguous(), page_table.contiguous(), seqlens.contiguous()
    B, H, d_qk = Q.shape
    if pieces_only and (num_splits is None or int(num_splits) < 2 or scratch is None):
        raise FlashDMLAError("pieces_only needs num_splits >= 2 and the scratch tensors that receive the pieces")
    num_pages, page_size, _ = kv_pool.shape
    max_pages = page_table.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(d_qk)
    dev = Q.device
    if num_splits is None:
        num_splits = suggest_partial_slabs(B, H, max_pages * page_size, page_size) if (d_qk, d_v) == (576, 512) else 1
    S = max(1, int(num_splits))
    if pieces_only:
        O = m = l = None
    else:
        if out is None:
            out = (torch.empty(B, H, d_v, dtype=torch.float32, device=dev), torch.empty(B, H, dtype=torch.float32, device=dev),
                   torch.empty(B, H, dtype=torch.float32, device=dev))
        O, m, l = out
        for t, n in ((O, B * H * d_v), (m, B * H), (l, B * H)):
            if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n or t.device != dev:
                raise FlashDMLAError("out must be contiguous float32 tensors of B*H*d_v, B*H and B*H elements")
    Op = mp = lp = None
    if S > 1:
        if scratch is None:
            scratch = (torch.empty(S, B, H, d_v, dtype=torch.float32, device=dev), torch.empty(S, B, H, dtype=torch.float32, device=dev),
                       torch.empty(S, B, H, dtype=torch.float32, device=dev))
        Op, mp, lp = scratch
        if Op.numel() < S * B * H * d_v or mp.numel() < S * B * H or lp.numel() < S * B * H:
            raise FlashDMLAError("scratch too small for num_splits")
    with torch.cuda.device(dev):
        check(_lib.lib().fdmla_decode_paged_partial(
            _ptr(Q), _ptr(kv_pool), _ptr(page_table), _ptr(seqlens), _ptr(O), _ptr(m), _ptr(l), _ptr(Op), _ptr(mp), _ptr(lp),
            B, H, d_qk, int(d_v), page_size, max_pages, num_pages, S, float(scale), _dtype_code(Q), _stream(Q)),
            "fdmla_decode_paged_partial")
    return scratch if pieces_only else (O, m, l)


def _part_stride(t: torch.Tensor, inner: int) -> Optional[int]:
    """Stride between parts if everything behind the leading dim is dense (inner elements), else None."""
    if t.shape[0] == 1:
        return inner
    return t.stride(0) if t[0].is_contiguous() and t.stride(0) >= inner else None


def merge_partials(O_p, m_p, l_p, out_dtype: Optional[torch.dtype] = None, out=None):
    """LSE merge over the leading dim: O_p [P,...,d_v] fp32, m_p,l_p [P,...] fp32.

    The parts need not sit back to back: any layout in which every part is dense
    in itself and the parts are a fixed number of elements apart is merged in
    place (views into an all-gathered buffer of per-rank messages, say).
    out = (O, m, l) writes into given contiguous tensors.
    """
    _need_cuda(O_p, m_p, l_p)
    if O_p.dtype != torch.float32 or m_p.dtype != torch.float32 or l_p.dtype != torch.float32:
        raise FlashDMLAError("partials must be float32")
    P, d_v = O_p.shape[0], O_p.shape[-1]
    rows = m_p[0].numel()
    so, sm, sl = _part_stride(O_p, rows * d_v), _part_stride(m_p, rows), _part_stride(l_p, rows)
    if so is None or sm is None or sl is None or sm != sl:
        O_p, m_p, l_p = O_p.contiguous(), m_p.contiguous(), l_p.contiguous()
        so, sm = rows * d_v, rows
    out_dtype = out_dtype or (out[0].dtype if out is not None else torch.float32)
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise FlashDMLAError("out_dtype must be float32 or bfloat16")
    if out is not None:
        O, m, l = out
        if (tuple(O.shape) != tuple(O_p.shape[1:]) or O.dtype != out_dtype or not O.is_contiguous()
                or m.numel() != rows or l.numel() != rows or not m.is_contiguous() or not l.is_contiguous()
                or m.dtype != torch.float32 or l.dtype != torch.float32):
            raise FlashDMLAError("out tensors do not match the merged result")
    else:
        O = torch.empty(O_p.shape[1:], dtype=out_dtype, device=O_p.device)
        m = torch.empty(m_p.shape[1:], dtype=torch.float32, device=O_p.device)
        l = torch.empty(m_p.shape[1:], dtype=torch.float32, device=O_p.device)
    code = _lib.F32 if out_dtype == torch.float32 else _lib.BF16
    with torch.cuda.device(O_p.device):
        check(_lib.lib().fdmla_merge_lse_strided(_ptr(O_p), _ptr(m_p), _ptr(l_p), _ptr(O), _ptr(m), _ptr(l),
                                                 rows, d_v, P, so, sm, code, _stream(O_p)), "fdmla_merge_lse_strided")
    return O, m, l


# --------------------------------------------------------------------------- #
# paged cache helpers (the writer side of the cache the decode consumes)
# --------------------------------------------------------------------------- #
def cache_append(new_rows, kv_pool, page_table, start_pos) -> None:
    """Write new_rows [B,n,d_qk] at logical positions start_pos[b]+t (in place)."""
    _need_cuda(new_rows, kv_pool, page_table, start_pos)
    _same_dtype(new_rows, kv_pool)
    if not kv_pool.is_contiguous():
        raise FlashDMLAError("kv_pool must be contiguous (it is written in place)")
    new_rows = new_rows.contiguous()
    B, n, d = new_rows.shape
    num_pages, page_size, _ = kv_pool.shape
    with torch.cuda.device(kv_pool.device):
        check(_lib.lib().fdmla_cache_append(
            _ptr(new_rows), _ptr(kv_pool), _ptr(page_table.contiguous()), _ptr(start_pos.contiguous()),
            B, n, d, page_size, page_table.shape[1], num_pages, _dtype_code(kv_pool),
            _stream(kv_pool)), "fdmla_cache_append")


def cache_gather(kv_pool, page_table, seqlens, n_tokens: int):
    """Dense [B,n_tokens,d_qk] copy of the first n_tokens logical rows (zeros past seqlen)."""
    _need_cuda(kv_pool, page_table, seqlens)
    kv_pool = kv_pool.contiguous()
    num_pages, page_size, d = kv_pool.shape
    B = page_table.shape[0]
    out = torch.empty(B, n_tokens, d, dtype=kv_pool.dtype, device=kv_pool.device)
    with torch.cuda.device(kv_pool.device):
        check(_lib.lib().fdmla_cache_gather(
            _ptr(kv_pool), _ptr(page_table.contiguous()), _ptr(seqlens.contiguous()), _ptr(out), B,
            int(n_tokens), d, page_size, page_table.shape[1], num_pages, _dtype_code(kv_pool),
            _stream(kv_pool)), "fdmla_cache_gather")
    return out
