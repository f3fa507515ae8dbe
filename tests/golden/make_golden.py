"""Record outputs of the reference's own forward kernels as golden vectors.

Run on a machine with a GPU after `make -C oracle ref` has compiled the
reference's csrc/attention/{vanallia_attn,fa_fwd,fa2_fwd}.cu unchanged into
oracle/_ref/libref_attn.so:

    python tests/golden/make_golden.py [out_dir]        # default: tests/golden

Each case stores the seeded inputs and the O the reference kernels produced
(vanilla_attn_forward, fa1_forward, fa2_forward) in ref_attn_golden.npz.
csrc/attention/fa2_bwd.cu is never built or launched (it does not terminate).
"""
from __future__ import annotations

import ctypes
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.path.join(ROOT, "oracle", "_ref", "libref_attn.so")

# (name, Nq, Nk, d, dv, std) - shapes the shipped launchers accept: d % 16 == 0
# for fa2_forward, Nq == Nk and small shared-memory footprint for fa1_forward.
CASES = [
    ("sq64_d32", 64, 64, 32, 32, 1.0),
    ("sq96_d64_dv48", 96, 96, 64, 48, 0.5),
    ("sq37_d16", 37, 37, 16, 24, 1.0),
    ("nq20_nk150_d160_dv128", 20, 150, 160, 128, 0.5),   # latent-like dims (no fa1: Nq != Nk)
    ("sq128_d64", 128, 128, 64, 64, 1.0),
]

FA2_MANGLED = "_Z11fa2_forwardPKfS0_S0_PfiiiifiP11CUstream_st"


def make_inputs(Nq, Nk, d, dv, std, seed):
    rs = np.random.RandomState(seed)
    Q = (rs.standard_normal((Nq, d)) * std).astype(np.float32)
    K = (rs.standard_normal((Nk, d)) * std).astype(np.float32)
    V = (rs.standard_normal((Nk, dv)) * std).astype(np.float32)
    return Q, K, V


def main(out_dir: str) -> None:
    lib = ctypes.CDLL(REF)
    sig = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    fns = {"vanilla": lib.vanilla_attn_forward, "fa1": lib.fa1_forward,
           "fa2": getattr(lib, FA2_MANGLED)}
    for f in fns.values():
        f.argtypes, f.restype = sig, None
    out = {}
    for idx, (name, Nq, Nk, d, dv, std) in enumerate(CASES):
        Q, K, V = make_inputs(Nq, Nk, d, dv, std, 1234 + idx)
        scale = 1.0 / np.sqrt(d)
        tq, tk, tv = (torch.from_numpy(a).cuda() for a in (Q, K, V))
        out[f"{name}/Q"], out[f"{name}/K"], out[f"{name}/V"] = Q, K, V
        out[f"{name}/scale"] = np.float32(scale)
        for kname, fn in fns.items():
            if kname == "fa1" and (Nq != Nk or 4 * (16 * d + 16 * dv + 16 * 16 + 64) > 48 * 1024):
                continue  # fa1_forward ignores Nk and never opts in to >48 KB shared memory
            O = torch.full((Nq, dv), float("nan"), device="cuda")
            warps = 1 if kname == "fa1" else 4
            fn(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), O.data_ptr(), Nq, Nk, d, dv,
               ctypes.c_float(scale), warps, None)
            torch.cuda.synchronize()
            out[f"{name}/O_{kname}"] = O.cpu().numpy()
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "ref_attn_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items() if "/O_" in k})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
