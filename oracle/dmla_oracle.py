"""ctypes front end of the CPU oracle (oracle/dmla_oracle.c).

TEST INFRASTRUCTURE ONLY.  The shipped package never imports this module; only
the tests, the smoke check and the benchmark's CPU-baseline leg do, and only as
the checker.  All arithmetic is fp32 on numpy arrays; callers convert bf16
inputs to fp32 (exactly) before calling.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libdmla_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_attn.so")
_lib = None

_f = ctypes.POINTER(ctypes.c_float)
_i = ctypes.POINTER(ctypes.c_int32)


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc (make -C oracle)."""
    src = os.path.join(_HERE, "dmla_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src))
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


def reference_dir() -> str:
    """Checkout of the reference project: $FDMLA_REFERENCE_DIR, else a directory `reference` beside this
    repository."""
    return os.environ.get("FDMLA_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build_ref(reference: str | None = None) -> str | None:
    """Compile the reference's own forward kernels where the checkout exists."""
    reference = reference or reference_dir()
    if not os.path.isdir(os.path.join(reference, "csrc", "attention")):
        return _REF_PATH if os.path.exists(_REF_PATH) else None
    subprocess.check_call(["make", "-C", _HERE, "-s", "ref", f"REFERENCE={reference}"],
                          stdout=subprocess.DEVNULL)
    return _REF_PATH


def ref_lib_path() -> str | None:
    return _REF_PATH if os.path.exists(_REF_PATH) else None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _f32(a) -> np.ndarray:
    if hasattr(a, "detach"):  # torch tensor
        a = a.detach().float().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a: np.ndarray):
    if a is None:
        return None
    if a.dtype == np.int32:
        return a.ctypes.data_as(_i)
    return a.ctypes.data_as(_f)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Undo a launcher's OMP_NUM_THREADS=1 for the timed CPU baseline; returns the thread count in use."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    L = lib()
    L.oracle_set_num_threads.restype = None
    L.oracle_set_num_threads.argtypes = [ctypes.c_int]
    L.oracle_set_num_threads(int(n))
    return num_threads()


def attn_plain(Q, K, V, scale):
    """Single-head non-causal attention: the reference launchers' problem."""
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    Nq, d = Q.shape
    Nk, dv = V.shape
    O = np.empty((Nq, dv), np.float32)
    m = np.empty((Nq,), np.float32)
    l = np.empty((Nq,), np.float32)
    lib().oracle_attn_plain(_p(Q), _p(K), _p(V), _p(O), _p(m), _p(l),
                            Nq, Nk, d, dv, ctypes.c_float(scale))
    return O, m, l


def attn_online(Q, K, V, scale, tile):
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    Nq, d = Q.shape
    Nk, dv = V.shape
    O = np.empty((Nq, dv), np.float32)
    m = np.empty((Nq,), np.float32)
    l = np.empty((Nq,), np.float32)
    lib().oracle_attn_online(_p(Q), _p(K), _p(V), _p(O), _p(m), _p(l),
                             Nq, Nk, d, dv, ctypes.c_float(scale), int(tile))
    return O, m, l


def fwd_cache_latent(Q, K_lat, d_v, scale, causal=True):
    Q, K_lat = _f32(Q), _f32(K_lat)
    B, H, Sq, d_qk = Q.shape
    Skv = K_lat.shape[1]
    O = np.empty((B, H, Sq, d_v), np.float32)
    m = np.empty((B, H, Sq), np.float32)
    l = np.empty((B, H, Sq), np.float32)
    lib().oracle_fwd_cache_latent(_p(Q), _p(K_lat), _p(O), _p(m), _p(l), B, H, Sq,
                                  Skv, d_qk, int(d_v), ctypes.c_float(scale),
                                  int(bool(causal)))
    return O, m, l


def fwd_on_the_fly(Q, K, V, WK, WV, scale, causal=True, return_latents=False, latents_bf16=False):
    Q, K, V, WK, WV = map(_f32, (Q, K, V, WK, WV))
    B, H, Sq, d_lat = Q.shape
    Skv, d_model = K.shape[2], K.shape[3]
    O = np.empty((B, H, Sq, d_lat), np.float32)
    m = np.empty((B, H, Sq), np.float32)
    l = np.empty((B, H, Sq), np.float32)
    Kl = np.empty((B, H, Skv, d_lat), np.float32) if return_latents else None
    Vl = np.empty((B, H, Skv, d_lat), np.float32) if return_latents else None
    lib().oracle_fwd_on_the_fly(_p(Q), _p(K), _p(V), _p(WK), _p(WV), _p(O), _p(m),
                                _p(l), _p(Kl), _p(Vl), B, H, Sq, Skv, d_model,
                                d_lat, ctypes.c_float(scale), int(bool(causal)),
                                int(bool(latents_bf16)))
    if return_latents:
        return O, m, l, Kl, Vl
    return O, m, l


def decode_paged(Q, kv_pool, page_table, seqlens, d_v, scale, kv_begin=0, kv_end=-1):
    Q, kv_pool = _f32(Q), _f32(kv_pool)
    page_table, seqlens = _i32(page_table), _i32(seqlens)
    if Q.ndim == 4:  # [B,H,1,d]
        Q = np.ascontiguousarray(Q[:, :, 0, :])
    B, H, d_qk = Q.shape
    page_size = kv_pool.shape[1]
    max_pages = page_table.shape[1]
    O = np.empty((B, H, d_v), np.float32)
    m = np.empty((B, H), np.float32)
    l = np.empty((B, H), np.float32)
    lib().oracle_decode_paged(_p(Q), _p(kv_pool), _p(page_table), _p(seqlens), _p(O),
                              _p(m), _p(l), B, H, d_qk, int(d_v), page_size,
                              max_pages, int(kv_begin), int(kv_end),
                              ctypes.c_float(scale))
    return O, m, l


def merge_partials(O_p, m_p, l_p):
    O_p, m_p, l_p = _f32(O_p), _f32(m_p), _f32(l_p)
    P = O_p.shape[0]
    d_v = O_p.shape[-1]
    rows = int(np.prod(m_p.shape[1:]))
    O = np.empty(O_p.shape[1:], np.float32)
    m = np.empty(m_p.shape[1:], np.float32)
    l = np.empty(m_p.shape[1:], np.float32)
    lib().oracle_merge_partials(_p(O_p), _p(m_p), _p(l_p), _p(O), _p(m), _p(l), P,
                                ctypes.c_long(rows), d_v)
    return O, m, l


def bwd_on_the_fly(Q, K, V, WK, WV, O, m, l, dO, scale, causal=True):
    Q, K, V, WK, WV, O, m, l, dO = map(_f32, (Q, K, V, WK, WV, O, m, l, dO))
    B, H, Sq, d_lat = Q.shape
    Skv, d_model = K.shape[2], K.shape[3]
    dQ = np.empty_like(Q)
    dK = np.empty_like(K)
    dV = np.empty_like(V)
    dWK = np.empty_like(WK)
    dWV = np.empty_like(WV)
    lib().oracle_bwd_on_the_fly(_p(Q), _p(K), _p(V), _p(WK), _p(WV), _p(O), _p(m),
                                _p(l), _p(dO), _p(dQ), _p(dK), _p(dV), _p(dWK),
                                _p(dWV), B, H, Sq, Skv, d_model, d_lat,
                                ctypes.c_float(scale), int(bool(causal)))
    return dQ, dK, dV, dWK, dWV


def bwd_cache_latent(Q, K_lat, O, m, l, dO, scale, causal=True):
    Q, K_lat, O, m, l, dO = map(_f32, (Q, K_lat, O, m, l, dO))
    B, H, Sq, d_qk = Q.shape
    Skv = K_lat.shape[1]
    d_v = O.shape[-1]
    dQ = np.empty_like(Q)
    dK = np.empty_like(K_lat)
    lib().oracle_bwd_cache_latent(_p(Q), _p(K_lat), _p(O), _p(m), _p(l), _p(dO),
                                  _p(dQ), _p(dK), B, H, Sq, Skv, d_qk, d_v,
                                  ctypes.c_float(scale), int(bool(causal)))
    return dQ, dK


def split_range(n: int, parts: int, r: int):
    off, ln = ctypes.c_int(), ctypes.c_int()
    lib().oracle_split_range(int(n), int(parts), int(r), ctypes.byref(off), ctypes.byref(ln))
    return off.value, ln.value
