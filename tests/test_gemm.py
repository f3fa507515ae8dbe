"""The batched tensor-core GEMM (fdmla_gemm_batched) and the RoPE tail kernel against plain fp32 matrix products of
the same bf16 inputs: both operand layouts, batches down the rows and across the columns, ragged row counts, the
gated epilogue, and the three uses (absorbed query, absorbed output projection, expert MLP)."""
import math

import pytest
import torch


def _rand(shape, seed, std=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * std).to(torch.bfloat16)


def _close(got, want, what, rel=1.5e-2):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs().max().item()
    scale = want.abs().max().item()
    fro = ((got - want).norm() / want.norm()).item()
    print(f"[parity] {what}: max-abs {err:.3e} (max |C| {scale:.3g}), rel-Fro {fro:.3e}")
    assert err <= rel * max(scale, 1e-6) and fro <= 5e-3, f"{what}: max-abs {err:.3e} of {scale:.3g}, rel-Fro {fro:.3e}"


def test_gemm_argument_validation_needs_no_gpu():
    from flashdmla import _lib
    L = _lib.lib()
    # empty problems are a no-op, null pointers and windows outside their tensors are refused
    assert L.fdmla_gemm_batched(None, None, None, None, 0, 8, 64, 64, 8, 64, 0, 0, 64, 64, 0, 0, 1, 64, 0, 0, 0, None) == 0
    assert L.fdmla_gemm_batched(None, None, None, None, 1, 8, 64, 64, 8, 64, 0, 0, 64, 64, 0, 0, 1, 64, 0, 0, 0, None) == -1
    assert L.fdmla_gemm_batched(1, 1, None, 1, 2, 8, 64, 64, 8, 64, 8, 0, 64, 64, 0, 0, 1, 64, 0, 0, 0, None) == -1   # A window past a_rows
    assert L.fdmla_gemm_batched(1, 1, None, 1, 1, 8, 64, 64, 8, 64, 0, 0, 64, 64, 0, 0, 1, 64, 0, 0, 1, None) == -1   # gated without B2
    assert L.fdmla_gemm_grouped(None, None, None, None, None, 0, 128, 64, 64, 64, 64, 64, 64, 1, 64, 0, None) == 0
    assert L.fdmla_gemm_grouped(None, None, None, None, None, 2, 128, 64, 64, 64, 64, 64, 64, 1, 64, 0, None) == -1
    assert L.fdmla_gemm_grouped(1, 1, None, 1, 1, 2, 128, 64, 64, 64, 64, 64, 64, 1, 64, 0, None) == -1     # B window of group 1 past b_rows
    assert L.fdmla_rope_rows(None, 64, None, 64, None, 0, 1, 64, 10000.0, None) == 0
    assert L.fdmla_rope_rows(None, 64, None, 64, None, 4, 1, 64, 10000.0, None) == -1


@pytest.mark.gpu
@pytest.mark.parametrize("k_major", [True, False])
@pytest.mark.parametrize("shape", [(1, 128, 256, 64), (3, 200, 512, 192), (2, 77, 64, 128), (5, 640, 320, 1024), (1, 1, 128, 4096)])
def test_gemm_batched_down_the_rows(shape, k_major, cuda):
    from flashdmla import gemm
    batch, M, N, K = shape
    A = _rand((batch, M, K), 1, 0.5)
    B = _rand((batch, N, K) if k_major else (batch, K, N), 2, 0.5)
    want = torch.matmul(A.float(), B.float().transpose(1, 2) if k_major else B.float())
    C = torch.full((batch, M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    gemm.gemm_batched(A.to(cuda).view(batch * M, K), B.to(cuda).view(-1, B.shape[2]), C.view(batch * M, N), batch, M, N, K,
                      a_brow=M, b_brow=B.shape[1], b_k_major=k_major, c_brow=M)
    torch.cuda.synchronize()
    _close(C, want, f"gemm {shape} k_major={k_major}")


@pytest.mark.gpu
def test_gemm_gated_epilogue_and_expert_mlp(cuda):
    import flashdmla
    from flashdmla import gemm
    E, rows, d, f = 6, 150, 256, 384
    xb, W1, W3, W2 = _rand((E, rows, d), 3, 0.5), _rand((E, d, f), 4, 0.08), _rand((E, d, f), 5, 0.08), _rand((E, f, d), 6, 0.08)
    h_want = torch.nn.functional.silu(xb.float() @ W1.float()) * (xb.float() @ W3.float())
    h = torch.empty(E, rows, f, dtype=torch.bfloat16, device=cuda)
    gemm.gemm_batched(xb.to(cuda).view(E * rows, d), W1.to(cuda).view(E * d, f), h.view(E * rows, f), E, rows, f, d,
                      a_brow=rows, b_brow=d, c_brow=rows, gate=W3.to(cuda).view(E * d, f))
    _close(h, h_want, "gated GEMM")
    y = gemm.expert_mlp(xb.to(cuda), W1.to(cuda), W3.to(cuda), W2.to(cuda))
    y_want = h_want.to(torch.bfloat16).float() @ W2.float()
    _close(y, y_want, "expert MLP")
    # K-major gated: the same weights stored transposed
    h2 = torch.empty_like(h)
    gemm.gemm_batched(xb.to(cuda).view(E * rows, d), W1.transpose(1, 2).contiguous().to(cuda).view(E * f, d), h2.view(E * rows, f),
                      E, rows, f, d, a_brow=rows, b_brow=f, b_k_major=True, c_brow=rows,
                      gate=W3.transpose(1, 2).contiguous().to(cuda).view(E * f, d))
    _close(h2, h_want, "gated GEMM, K-major weights")
    assert flashdmla.device_error_flag() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 128, 200])
def test_absorbed_projections(n, cuda):
    from flashdmla import gemm
    from flashdmla.mla import rope
    H, d_lat, d_nope, d_rope, d_v = 16, 512, 128, 64, 128
    q = _rand((n, H, d_nope + d_rope), 7, 0.5)
    W_UK, W_UV = _rand((H, d_lat, d_nope), 8, 0.05), _rand((H, d_lat, d_v), 9, 0.05)
    pos = torch.randint(0, 5000, (n,), generator=torch.Generator().manual_seed(10), dtype=torch.int32)
    Q = gemm.absorb_query(q.to(cuda), W_UK.to(cuda), pos.to(cuda), d_nope)
    want_lat = torch.einsum("nhd,hld->nhl", q[..., :d_nope].float(), W_UK.float())
    want_rope = rope(q[..., d_nope:], pos[:, None].expand(n, H)).float()
    _close(Q[..., :d_lat], want_lat, "absorbed query")
    _close(Q[..., d_lat:], want_rope, "RoPE tail", rel=1e-2)
    o_lat = _rand((n, H, d_lat), 11, 0.5)
    o = gemm.project_out(o_lat.to(cuda), W_UV.to(cuda))
    _close(o, torch.einsum("nhl,hlv->nhv", o_lat.float(), W_UV.float()), "absorbed output projection")


@pytest.mark.gpu
def test_gemm_grouped_ragged_rows(cuda):
    """Groups of 0, 1, 127, 128, 129 and 300 rows, their ranges read on the device; rows past the last group stay untouched."""
    from flashdmla import gemm
    counts = [0, 1, 127, 128, 129, 0, 300, 5]
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    rows, E, d, f = int(offs[-1]) + 40, len(counts), 192, 256
    A, W1, W3 = _rand((rows, d), 21, 0.5), _rand((E, d, f), 22, 0.08), _rand((E, d, f), 23, 0.08)
    C = torch.full((rows, f), 7.0, dtype=torch.bfloat16, device=cuda)
    gemm.gemm_grouped(A.to(cuda), W1.to(cuda).view(E * d, f), C, offs.to(cuda), f, d, b_brow=d, gate=W3.to(cuda).view(E * d, f))
    torch.cuda.synchronize()
    want = torch.full((rows, f), 7.0)
    for e in range(E):
        lo, hi = int(offs[e]), int(offs[e + 1])
        want[lo:hi] = torch.nn.functional.silu(A[lo:hi].float() @ W1[e].float()) * (A[lo:hi].float() @ W3[e].float())
    _close(C[: int(offs[-1])], want[: int(offs[-1])], "grouped gated GEMM")
    assert (C[int(offs[-1]):].float() == 7.0).all()
    # K-major weights, ungated
    W2 = _rand((E, 64, f), 24, 0.08)                      # [E, N=64, K=f]
    C2 = torch.zeros(rows, 64, dtype=torch.bfloat16, device=cuda)
    gemm.gemm_grouped(C, W2.to(cuda).view(E * 64, f), C2, offs.to(cuda), 64, f, b_brow=64, b_k_major=True)
    want2 = torch.zeros(rows, 64)
    for e in range(E):
        lo, hi = int(offs[e]), int(offs[e + 1])
        want2[lo:hi] = C[lo:hi].float().cpu() @ W2[e].float().T
    _close(C2[: int(offs[-1])], want2[: int(offs[-1])], "grouped GEMM, K-major weights")
