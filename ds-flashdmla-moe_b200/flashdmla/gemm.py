"""Batched bf16 GEMMs on the tensor-core kernel of the library (fdmla_gemm_batched) and the three uses the
attention path has for them: the absorbed query and output projections of an MLA block (the reference's "drop-in
for standard MHA shapes", README.md:16) and the expert MLPs of the MoE layer over padded packing (README.md:17-20).
No CPU fallback: every function needs CUDA bf16 tensors.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import FlashDMLAError, check, lib


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need(*ts):
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise FlashDMLAError("the GEMM kernel needs contiguous CUDA bf16 tensors (there is no CPU fallback)")


def gemm_batched(A2: torch.Tensor, B2d: torch.Tensor, C2: torch.Tensor, batch: int, M: int, N: int, K: int, *,
                 a_brow: int = 0, a_bcol: int = 0, b_brow: int = 0, b_bcol: int = 0, b_k_major: bool = False,
                 c_brow: int = 0, c_bcol: int = 0, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[b] = A[b] B[b] over windows of the 2-D tensors A2, B2d, C2 (see fdmla_gemm_batched in flashdmla.h).
    gate: a tensor with B2d's geometry; then C = silu(A B) * (A gate)."""
    _need(A2, B2d, C2, gate)
    if A2.dim() != 2 or B2d.dim() != 2 or C2.dim() != 2:
        raise FlashDMLAError("gemm_batched takes 2-D tensors")
    with torch.cuda.device(A2.device):
        check(lib().fdmla_gemm_batched(_ptr(A2), _ptr(B2d), _ptr(gate), _ptr(C2), batch, M, N, K,
                                       A2.shape[0], A2.shape[1], a_brow, a_bcol, B2d.shape[0], B2d.shape[1], b_brow, b_bcol,
                                       int(bool(b_k_major)), C2.shape[1], c_brow, c_bcol, int(gate is not None),
                                       _stream(A2)), "fdmla_gemm_batched")
    return C2


def absorb_query(q: torch.Tensor, W_UK: torch.Tensor, pos: torch.Tensor, d_nope: int, rope_base: float = 10000.0) -> torch.Tensor:
    """q [n, H, d_nope + d_rope], W_UK [H, d_lat, d_nope], pos [n] int32 -> Q' [n, H, d_lat + d_rope]:
    Q'[..., :d_lat] = q[..., :d_nope] W_UK[h]^T (one GEMM per head, batch across the columns of q) and
    Q'[..., d_lat:] = rope(q[..., d_nope:], pos), written by the same pair of launches into one tensor."""
    _need(q, W_UK)
    n, H, dq = q.shape
    d_lat, d_rope = W_UK.shape[1], dq - d_nope
    out = torch.empty(n, H, d_lat + d_rope, dtype=q.dtype, device=q.device)
    gemm_batched(q.view(n, H * dq), W_UK.view(H * d_lat, d_nope), out.view(n, H * (d_lat + d_rope)), H, n, d_lat, d_nope,
                 a_bcol=dq, b_brow=d_lat, b_k_major=True, c_bcol=d_lat + d_rope)
    pos = pos.to(device=q.device, dtype=torch.int32).contiguous()
    with torch.cuda.device(q.device):
        check(lib().fdmla_rope_rows(q.data_ptr() + 2 * d_nope, dq, out.data_ptr() + 2 * d_lat, d_lat + d_rope, _ptr(pos),
                                    n * H, H, d_rope, float(rope_base), _stream(q)), "fdmla_rope_rows")
    return out


def project_out(o_lat: torch.Tensor, W_UV: torch.Tensor) -> torch.Tensor:
    """o_lat [n, H, d_lat], W_UV [H, d_lat, d_v] -> [n, H, d_v] (one GEMM per head)."""
    _need(o_lat, W_UV)
    n, H, d_lat = o_lat.shape
    d_v = W_UV.shape[2]
    out = torch.empty(n, H, d_v, dtype=o_lat.dtype, device=o_lat.device)
    gemm_batched(o_lat.view(n, H * d_lat), W_UV.view(H * d_lat, d_v), out.view(n, H * d_v), H, n, d_v, d_lat,
                 a_bcol=d_lat, b_brow=d_lat, c_bcol=d_v)
    return out


def expert_mlp(xb: torch.Tensor, W1: torch.Tensor, W3: torch.Tensor, W2: torch.Tensor) -> torch.Tensor:
    """xb [E, rows, d], W1, W3 [E, d, d_ff], W2 [E, d_ff, d] -> (silu(xb W1) * (xb W3)) W2, two launches: the gate is
    applied in the first GEMM's epilogue."""
    _need(xb, W1, W3, W2)
    E, rows, d = xb.shape
    f = W1.shape[2]
    h = torch.empty(E, rows, f, dtype=xb.dtype, device=xb.device)
    gemm_batched(xb.view(E * rows, d), W1.view(E * d, f), h.view(E * rows, f), E, rows, f, d,
                 a_brow=rows, b_brow=d, c_brow=rows, gate=W3.view(E * d, f))
    y = torch.empty(E, rows, d, dtype=xb.dtype, device=xb.device)
    gemm_batched(h.view(E * rows, f), W2.view(E * f, d), y.view(E * rows, d), E, rows, d, f,
                 a_brow=rows, b_brow=f, c_brow=rows)
    return y


def gemm_grouped(A2: torch.Tensor, B2d: torch.Tensor, C2: torch.Tensor, row_offsets: torch.Tensor, N: int, K: int, *,
                 b_brow: int, b_k_major: bool = False, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[rows of group g] = A[rows of group g] B[g] with the groups' row ranges read on the device (row_offsets: int32
    [groups + 1]); see fdmla_gemm_grouped in flashdmla.h."""
    _need(A2, B2d, C2, gate)
    if row_offsets.dtype != torch.int32 or not row_offsets.is_cuda or not row_offsets.is_contiguous():
        raise FlashDMLAError("row_offsets must be a contiguous CUDA int32 tensor")
    with torch.cuda.device(A2.device):
        check(lib().fdmla_gemm_grouped(_ptr(A2), _ptr(B2d), _ptr(gate), _ptr(C2), _ptr(row_offsets), row_offsets.numel() - 1,
                                       A2.shape[0], N, K, A2.shape[1], B2d.shape[0], B2d.shape[1], b_brow, int(bool(b_k_major)),
                                       C2.shape[1], int(gate is not None), _stream(A2)), "fdmla_gemm_grouped")
    return C2


def expert_mlp_grouped(xp: torch.Tensor, row_offsets: torch.Tensor, W1: torch.Tensor, W3: torch.Tensor, W2: torch.Tensor) -> torch.Tensor:
    """xp [rows, d] packed by expert (expert e owns rows row_offsets[e] .. row_offsets[e + 1]), W1, W3 [E, d, d_ff],
    W2 [E, d_ff, d] -> [rows, d]; rows past row_offsets[E] are left unwritten.  Nothing is read back to the host."""
    _need(xp, W1, W3, W2)
    rows, d = xp.shape
    E, _, f = W1.shape
    h = torch.empty(rows, f, dtype=xp.dtype, device=xp.device)
    gemm_grouped(xp, W1.view(E * d, f), h, row_offsets, f, d, b_brow=d, gate=W3.view(E * d, f))
    y = torch.empty(rows, d, dtype=xp.dtype, device=xp.device)
    gemm_grouped(h, W2.view(E * f, d), y, row_offsets, d, f, b_brow=f)
    return y
