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
    fns = {"vanilla": lib.vanilla_attn_forward, "fa2": getattr(lib, FA2_MANGLED)}
    for f in fns.values():
        f.argtypes, f.restype = sig, None
    return fns


def _run_ref(fn, Q, K, V, scale):
    O = torch.full((Q.shape[0], V.shape[1]), float("nan"), device=Q.device)
    fn(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), Q.shape[0], K.shape[0], Q.shape[1], V.shape[1],
       ctypes.c_float(scale), 4, None)
    torch.cuda.synchronize()
    return O


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
