"""Cross-check against the reference's own kernels, run unmodified on the GPU.

oracle/_ref/libref_attn.so is compiled from the reference checkout's
csrc/attention/{vanallia_attn,fa_fwd,fa2_fwd}.cu (recipe: oracle/Makefile, target
`ref`).  Per (batch, head) the reference launchers solve the non-causal
single-head problem; the new kernels must agree with them, and so must the
oracle.  csrc/attention/fa2_bwd.cu is never built or launched: its first phase
does not terminate (fa2_bwd.cu:66-148)."""
import ctypes
import math

import numpy as np
import pytest
import torch

from helpers import max_abs
from oracle import dmla_oracle as orc

pytestmark = pytest.mark.gpu

FA2_MANGLED = "_Z11fa2_forwardPKfS0_S0_PfiiiifiP11CUstream_st"


@pytest.fixture(scope="module")
def ref(cuda):
    path = orc.ref_lib_path()
    if path is None:
        pytest.skip("oracle/_ref/libref_attn.so was not built (no reference checkout at build time)")
    lib = ctypes.CDLL(path)
    sig = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    fns = {"vanilla": lib.vanilla_attn_forward, "fa1": lib.fa1_forward, "fa2": getattr(lib, FA2_MANGLED)}
    for f in fns.values():
        f.argtypes, f.restype = sig, None
    return fns


def _run_ref(fn, Q, K, V, scale, warps=4):
    O = torch.full((Q.shape[0], V.shape[1]), float("nan"), device=Q.device)
    fn(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), Q.shape[0], K.shape[0], Q.shape[1], V.shape[1],
       ctypes.c_float(scale), warps, None)
    torch.cuda.synchronize()
    return O


def _fa1_can_run(Nq, Nk, d, dv):
    """fa1_forward ignores Nk (fa_fwd.cu:163) and never opts in to more than 48 KB of shared memory
    (fa_fwd.cu:174-175); with one warp per block its tiles are 16 rows."""
    return Nq == Nk and 4 * (16 * d + 16 * dv + 16 * 16 + 64) <= 48 * 1024


@pytest.mark.parametrize("B,H,Sq,Skv,dq,dv", [(2, 3, 40, 56, 160, 128), (1, 2, 64, 64, 64, 64)])
def test_cache_latent_noncausal_matches_reference_kernels(ref, cuda, B, H, Sq, Skv, dq, dv):
    import flashdmla
    g = torch.Generator().manual_seed(8)
    Q = (torch.randn(B, H, Sq, dq, generator=g) * 0.5).to(cuda)
    K = (torch.randn(B, Skv, dq, generator=g) * 0.5).to(cuda)
    sc = 1 / math.sqrt(dq)
    O, m, l = flashdmla.flash_dmla_cache_latent(Q, K, dv, sc, causal=False)
    Oo, _, _ = orc.fwd_cache_latent(Q, K, dv, sc, causal=False)
    for b in range(B):
        Vb = K[b, :, :dv].contiguous()
        for h in range(H):
            Ov = _run_ref(ref["vanilla"], Q[b, h].contiguous(), K[b].contiguous(), Vb, sc)
            Of = _run_ref(ref["fa2"], Q[b, h].contiguous(), K[b].contiguous(), Vb, sc)
            assert max_abs(O[b, h], Ov) <= 2e-5, "new kernel vs vanilla_attn_forward"
            assert max_abs(Oo[b, h], Ov) <= 2e-5, "oracle vs vanilla_attn_forward"
            assert max_abs(O[b, h], Of) <= 5e-3, "new kernel vs fa2_forward (fp16 QK^T)"
            if _fa1_can_run(Sq, Skv, dq, dv):
                O1 = _run_ref(ref["fa1"], Q[b, h].contiguous(), K[b].contiguous(), Vb, sc, warps=1)
                assert max_abs(O[b, h], O1) <= 2e-5, "new kernel vs fa1_forward"
                assert max_abs(Oo[b, h], O1) <= 2e-5, "oracle vs fa1_forward"


def test_tensor_core_kernel_meets_the_reference_kernels_directly(ref, cuda):
    """bf16 inputs at 64/64 take the tcgen05 kernel; the reference kernels get the same values in fp32 (a bf16
    value is an fp32 value).  fa2_forward rounds Q and K to fp16 (fa2_fwd.cu:58,71), which is exact for bf16 values
    of this magnitude, so all three reference forwards solve exactly the problem the new kernel solves and the
    difference is the new kernel's bf16 P and bf16 output: the target tolerance O max-abs <= 1e-2."""
    import flashdmla
    B, H, S, d = 1, 2, 64, 64
    g = torch.Generator().manual_seed(18)
    Q = (torch.randn(B, H, S, d, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
    K = (torch.randn(B, S, d, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
    sc = 1 / math.sqrt(d)
    O, m, l = flashdmla.flash_dmla_cache_latent(Q, K, d, sc, causal=False)
    assert flashdmla.last_kernel() == "tcgen05"
    Kf = K[0].float().contiguous()
    worst = 0.0
    for h in range(H):
        Qf = Q[0, h].float().contiguous()
        for name, warps in (("vanilla", 4), ("fa1", 1), ("fa2", 4)):
            Or = _run_ref(ref[name], Qf, Kf, Kf, sc, warps=warps)
            err = max_abs(O[0, h], Or)
            worst = max(worst, err)
            assert err <= 1e-2, f"tcgen05 kernel vs {name}: max-abs {err:.3e}"
    print(f"tcgen05 64/64 bf16 vs reference kernels: worst max-abs {worst:.3e}")
