"""flashdmla - B200-native Flash-DMLA attention backend (Python host side).

The package mirrors the reference's advertised python/ops.py surface
(README.md:54-56).  Importing it needs the compiled libflashdmla.so; there is
no CPU fallback.
"""
from ._lib import (BACKEND_AUTO, BACKEND_PORTABLE, BACKEND_TENSOR, FlashDMLAError, LIB_PATH,
                   device_error_flag, last_kernel, set_backend, set_single_cta)
from .cache import PagedLatentCache
from .mla import AbsorbedMLA, rope
from .moe import MoEFFN
from .ops import (DecodeWorkspace, FlashDMLACacheLatentFn, FlashDMLAOnTheFlyFn, cache_append,
                  cache_gather, flash_dmla_cache_latent, flash_dmla_on_the_fly,
                  flash_dmla_paged_decode, merge_partials, suggest_splits)

__all__ = [
    "PagedLatentCache", "AbsorbedMLA", "MoEFFN", "rope", "BACKEND_AUTO", "BACKEND_PORTABLE", "BACKEND_TENSOR", "FlashDMLAError", "LIB_PATH",
    "device_error_flag", "last_kernel", "set_backend", "set_single_cta", "DecodeWorkspace", "FlashDMLACacheLatentFn",
    "FlashDMLAOnTheFlyFn", "cache_append", "cache_gather", "flash_dmla_cache_latent",
    "flash_dmla_on_the_fly", "flash_dmla_paged_decode", "merge_partials", "suggest_splits",
]
