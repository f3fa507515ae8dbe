"""ctypes binding of libflashdmla.so (the C ABI declared in include/flashdmla.h).

There is no CPU fallback: if the shared library is missing the import of the
operators fails, and every operator raises when handed a non-CUDA tensor.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FLASHDMLA_LIB names another build of the library (a development build with timeline stamps, say)
LIB_PATH = os.environ.get("FLASHDMLA_LIB") or os.path.join(_HERE, "libflashdmla.so")

F32, BF16 = 0, 1
BACKEND_AUTO, BACKEND_PORTABLE, BACKEND_TENSOR = 0, 1, 2

_vp, _i, _f, _sz, _ll = (ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t,
                         ctypes.c_longlong)

# name -> (restype, argtypes); mirrors include/flashdmla.h one to one
SIGNATURES = {
    "fdmla_version": (_i, []),
    "fdmla_status_string": (ctypes.c_char_p, [_i]),
    "fdmla_set_backend": (_i, [_i]),
    "fdmla_get_backend": (_i, []),
    "fdmla_set_single_cta": (_i, [_i]),
    "fdmla_last_kernel": (ctypes.c_char_p, []),
    "fdmla_device_error_flag": (_i, [_i]),
    "fdmla_fwd_cache_latent": (_i, [_vp] * 5 + [_i] * 6 + [_f, _i, _i, _vp]),
    "fdmla_fwd_on_the_fly_workspace_bytes": (_sz, [_i] * 5),
    "fdmla_fwd_on_the_fly": (_i, [_vp] * 9 + [_sz] + [_i] * 6 + [_f, _i, _i, _vp]),
    "fdmla_decode_paged": (_i, [_vp] * 10 + [_i] * 10 + [_f, _i, _vp]),
    "fdmla_decode_paged_partial": (_i, [_vp] * 10 + [_i] * 8 + [_f, _i, _vp]),
    "fdmla_decode_suggest_splits": (_i, [_i] * 7),
    "fdmla_decode_plan": (_i, [_i] * 8 + [_vp, _vp]),
    "fdmla_decode_paged_noalloc_max_rows": (_sz, [_i]),
    "fdmla_decode_paged_noalloc": (_i, [_vp] * 7 + [_i] * 8 + [_f, _i, _vp]),
    "fdmla_merge_lse": (_i, [_vp] * 6 + [_ll, _i, _i, _i, _vp]),
    "fdmla_merge_lse_strided": (_i, [_vp] * 6 + [_ll, _i, _i, _ll, _ll, _i, _vp]),
    "fdmla_exchange_bytes": (_sz, [_i, _ll, _i]),
    "fdmla_exchange_alloc": (_i, [_sz, _vp, _vp]),
    "fdmla_exchange_open": (_i, [_vp, _vp]),
    "fdmla_exchange_close": (_i, [_vp]),
    "fdmla_exchange_free": (_i, [_vp]),
    "fdmla_exchange_merge": (_i, [_vp, _vp, _i, _i, _ll, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "fdmla_exchange_merge_parts": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _ll, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "fdmla_gemm_batched": (_i, [_vp] * 4 + [_i] * 4 + [_ll, _ll, _i, _i, _ll, _ll, _i, _i, _i, _ll, _ll, _ll, _i, _vp]),
    "fdmla_gemm_grouped": (_i, [_vp] * 5 + [_i] * 4 + [_ll, _ll, _ll, _i, _i, _ll, _i, _vp]),
    "fdmla_rope_rows": (_i, [_vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _f, _vp]),
    "fdmla_bwd_on_the_fly_workspace_bytes": (_sz, [_i] * 7),
    "fdmla_bwd_on_the_fly": (_i, [_vp] * 15 + [_sz] + [_i] * 6 + [_f, _i, _i, _vp]),
    "fdmla_bwd_cache_latent_workspace_bytes": (_sz, [_i] * 7),
    "fdmla_bwd_cache_latent": (_i, [_vp] * 9 + [_sz] + [_i] * 6 + [_f, _i, _i, _vp]),
    "fdmla_cache_append": (_i, [_vp] * 4 + [_i] * 7 + [_vp]),
    "fdmla_cache_gather": (_i, [_vp] * 4 + [_i] * 7 + [_vp]),
    "fdmla_moe_route_topk": (_i, [_vp] * 3 + [_i] * 3 + [_vp]),
    "fdmla_moe_pack_workspace_bytes": (_sz, [_i] * 3),
    "fdmla_moe_pack": (_i, [_vp] * 5 + [_sz] + [_i] * 5 + [_vp]),
    "fdmla_moe_gather": (_i, [_vp] * 4 + [_i] * 4 + [_vp]),
    "fdmla_moe_scatter": (_i, [_vp] * 3 + [_i] * 4 + [_vp]),
    "fdmla_moe_combine": (_i, [_vp] * 5 + [_i] * 4 + [_vp]),
}

_lib = None


class FlashDMLAError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load the shared library once; raise loudly if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FlashDMLAError(
                f"{LIB_PATH} not found: build it with `python ds-flashdmla-moe_b200/build.py` "
                "(there is no CPU or eager fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().fdmla_status_string(status).decode()
        raise FlashDMLAError(f"{what} failed: {msg} (status {status})")


def set_backend(backend: int) -> None:
    check(lib().fdmla_set_backend(int(backend)), "fdmla_set_backend")


def set_single_cta(on: bool) -> None:
    """Keep 576/512 shapes on the single-CTA tcgen05 kernel (A/B measurements, tests)."""
    check(lib().fdmla_set_single_cta(int(bool(on))), "fdmla_set_single_cta")


def last_kernel() -> str:
    return lib().fdmla_last_kernel().decode()


def device_error_flag(reset: bool = False) -> int:
    """0 if no tensor-core kernel reported a timed-out wait or a bad page id (synchronises)."""
    return int(lib().fdmla_device_error_flag(int(reset)))
