"""B200 (sm_100a) fused layer kernels of a Stable Diffusion pipeline: GroupNorm(+SiLU),
LayerNorm, GEGLU / gelu / quick_gelu / SiLU, token+position embedding, timestep embedding.

The product is ``lib/libsdfl.so`` (C ABI: ``include/sdfl.h``); this package is the thin host
side: a ctypes binding (``_capi``), tensor-level wrappers (``ops``), the reference-shaped
operator classes (``operators``) and the multi-GPU unit partitioner (``sharding``).  Importing
the package loads the library and fails if it is absent -- there is no fallback path.

The directory name contains a hyphen, so import it with
``importlib.import_module("mobile-stable-diffusion_b200")``.
"""
from . import _capi, ops, operators, sharding  # noqa: F401
from ._capi import SdflError  # noqa: F401

__all__ = ["ops", "operators", "sharding", "SdflError"]
