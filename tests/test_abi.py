"""The C-ABI library loads without a GPU and exports what include/flashdmla.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "flashdmla.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fdmla_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_functions()
    for required in ("fdmla_fwd_cache_latent", "fdmla_fwd_on_the_fly", "fdmla_decode_paged",
                     "fdmla_merge_lse", "fdmla_bwd_on_the_fly"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from flashdmla import _lib
    L = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(L, name), f"{name} declared in flashdmla.h but not exported"
    # and the Python binding table covers the header one to one
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_status_strings_and_backend_switch():
    from flashdmla import _lib
    L = _lib.lib()
    assert L.fdmla_version() >= 100
    assert L.fdmla_status_string(0) == b"ok"
    assert b"invalid" in L.fdmla_status_string(-1)
    assert L.fdmla_set_backend(7) == -1
    assert L.fdmla_set_backend(_lib.BACKEND_PORTABLE) == 0
    assert L.fdmla_get_backend() == _lib.BACKEND_PORTABLE
    assert L.fdmla_set_backend(_lib.BACKEND_AUTO) == 0


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected with a status before any CUDA call is made
    (the reference's launchers return silently instead: fa2_fwd.cu:149)."""
    from flashdmla import _lib
    L = _lib.lib()
    # bad dtype
    assert L.fdmla_fwd_cache_latent(None, None, None, None, None, 1, 1, 1, 1, 16, 16, 1.0, 1, 9, None) == -1
    # null pointers with non-empty problem
    assert L.fdmla_fwd_cache_latent(None, None, None, None, None, 1, 1, 1, 1, 16, 16, 1.0, 1, 0, None) == -1
    # d_v > d_qk
    assert L.fdmla_fwd_cache_latent(None, None, None, None, None, 1, 1, 1, 1, 16, 32, 1.0, 1, 0, None) == -1
    # empty problems are a successful no-op, as in the reference (vanallia_attn.cu:95)
    assert L.fdmla_fwd_cache_latent(None, None, None, None, None, 0, 1, 1, 1, 16, 16, 1.0, 1, 0, None) == 0
    assert L.fdmla_merge_lse(None, None, None, None, None, None, 0, 16, 2, 0, None) == 0
    # the per-rank partial of the sequence-split decode: empty batch is a no-op, missing outputs and scratch are refused
    assert L.fdmla_decode_paged_partial(None, None, None, None, None, None, None, None, None, None, 0, 8, 576, 512, 64, 4, 4, 1, 0.1, 1, None) == 0
    assert L.fdmla_decode_paged_partial(None, None, None, None, None, None, None, None, None, None, 2, 8, 576, 512, 64, 4, 4, 1, 0.1, 1, None) == -1
    assert L.fdmla_decode_paged_partial(1, 1, 1, 1, 1, 1, 1, None, None, None, 2, 8, 576, 512, 64, 4, 4, 3, 0.1, 1, None) == -4
    assert L.fdmla_decode_paged(None, None, None, None, None, None, None, None, None, None,
                                1, 1, 16, 16, 0, 1, 1, 1, 0, -1, 1.0, 0, None) == -1   # page_size 0
    assert L.fdmla_fwd_on_the_fly_workspace_bytes(2, 2, 16, 8, 1) == 2 * 256 * ((2 * 2 * 16 * 8 * 2 + 255) // 256)
    assert L.fdmla_decode_suggest_splits(128, 128, 4096, 576, 512, 64, 1) >= 1


def test_operators_refuse_cpu_tensors():
    import torch
    import flashdmla
    with pytest.raises(flashdmla.FlashDMLAError):
        flashdmla.flash_dmla_cache_latent(torch.zeros(1, 1, 4, 16), torch.zeros(1, 4, 16), 16)
    with pytest.raises(flashdmla.FlashDMLAError):
        flashdmla.merge_partials(torch.zeros(2, 4, 8), torch.zeros(2, 4), torch.zeros(2, 4))
