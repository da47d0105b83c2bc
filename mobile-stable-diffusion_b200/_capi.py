"""ctypes binding of libsdfl.so (the C ABI declared in include/sdfl.h).

The library is the product: there is no Python or CPU fallback.  If it cannot be loaded the
import of this module raises, and every wrapper raises SdflError on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libsdfl.so")

F32, F16 = 0, 1
GN_AUTO, GN_RESIDENT, GN_SPLIT, GN_REGISTER = 0, 1, 2, 3

OK = 0
ERR_INVALID_VALUE = -1
ERR_INVALID_POINTER = -2
ERR_UNSUPPORTED = -3
ERR_CUDA = -4
ERR_OVERLAP = -5
ERR_WORKSPACE = -6
ERR_DEVICE_FLAG = -7


class SdflError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        super().__init__(f"{where}: status {status} ({detail})")


_p = C.c_void_p


class GnTensor(C.Structure):
    """sdfl_gn_tensor of include/sdfl.h."""
    _fields_ = [("in_", C.c_void_p), ("out", C.c_void_p), ("gamma", C.c_void_p), ("beta", C.c_void_p),
                ("batch", C.c_int64), ("channels", C.c_int64), ("hw", C.c_int64),
                ("num_groups", C.c_int64), ("eps", C.c_float)]


_i64 = C.c_int64
_f = C.c_float
_i = C.c_int
_sz = C.c_size_t

# name -> (restype, argtypes); exactly the declarations of include/sdfl.h
SIGNATURES = {
    "sdfl_version": (C.c_char_p, []),
    "sdfl_status_string": (C.c_char_p, [_i]),
    "sdfl_last_cuda_error": (_i, []),
    "sdfl_last_cuda_error_string": (C.c_char_p, []),
    "sdfl_launch_count": (C.c_longlong, []),
    "sdfl_groupnorm_forward": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p, _sz, _p]),
    "sdfl_groupnorm_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i]),
    "sdfl_groupnorm_forward_ex": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p, _sz,
                                       _i, _i, _p]),
    "sdfl_groupnorm_workspace_bytes_ex": (_sz, [_i64, _i64, _i64, _i64, _i, _i, _i]),
    "sdfl_groupnorm_multi_workspace_bytes": (_sz, []),
    "sdfl_groupnorm_forward_multi": (_i, [_p, _i, _i, _i, _p, _sz, _p]),
    "sdfl_groupnorm_forward_multi_ex": (_i, [_p, _i, _i, _i, _p, _sz, _i, _p, C.POINTER(_i), _p]),
    "sdfl_groupnorm_forward_noalloc": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p]),
    "sdfl_groupnorm_bias_forward": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p, _sz, _p]),
    "sdfl_groupnorm_bias_forward_ex": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p, _sz, _i, _i, _p]),
    "sdfl_groupnorm_nhwc_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i]),
    "sdfl_groupnorm_nhwc_forward": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p, _sz, _p]),
    "sdfl_permute3D__0_2_1": (_i, [_p, _p, _i64, _i64, _i64, _i, _p]),
    "sdfl_permute_add": (_i, [_p, _p, _p, _i64, _i64, _i64, _i, _p]),
    "sdfl_up_sample_nearest": (_i, [_p, _p, _i64, _i64, _i64, _i64, _i, _p]),
    "sdfl_concat_buffer": (_i, [_p, _p, _p, _i64, _i64, _i64, _i, _p]),
    "sdfl_groupnorm_concat_forward": (_i, [_p, _i64, _p, _i64, _p, _p, _p, _i64, _i64, _i64, _f, _i, _i, _p, _sz, _p]),
    "sdfl_softmax": (_i, [_p, _p, _i64, _i64, _i, _p]),
    "sdfl_local_softmax": (_i, [_p, _p, _i64, _i64, _i, _p]),
    "sdfl_chunkwise_add": (_i, [_p, _p, _p, _i64, _i64, _i, _p]),
    "sdfl_groupnorm_plan": (_i, [_i64, _i64, _i64, _i64, _i, _i, _i, C.POINTER(_i64)]),
    "sdfl_layernorm_forward": (_i, [_p, _p, _p, _p, _i64, _i64, _f, _i, _p]),
    "sdfl_add_layernorm_forward": (_i, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f, _i, _p]),
    "sdfl_token_embedding": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _p, _p]),
    "sdfl_timestep_embedding": (_i, [_p, _p, _i64, _i64, _f, _i, _p]),
    "sdfl_local_reduction_mean": (_i, [_p, _p, _i64, _i64, _i, _p]),
    "sdfl_local_reduction_variance": (_i, [_p, _p, _p, _i64, _i64, _i, _p]),
    "sdfl_group_norm": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _f, _p, _i64, _i64, _i, _p]),
    "sdfl_layer_norm": (_i, [_p, _p, _p, _p, _p, _i64, _p, _i64, _f, _i, _p]),
    "sdfl_gelu_multiply": (_i, [_p, _p, _i64, _i64, _i, _p]),
    "sdfl_gelu": (_i, [_p, _p, _i64, _i, _p]),
    "sdfl_silu": (_i, [_p, _p, _i64, _i, _p]),
    "sdfl_quick_gelu": (_i, [_p, _p, _i64, _i, _p]),
    "sdfl_elemwise_add": (_i, [_p, _p, _p, _i64, _i, _p]),
    "sdfl_groupnorm_create": (_i, [C.POINTER(_p), _i64, _i64, _f, _p, _p, _i, _i64, _i64, _i]),
    "sdfl_groupnorm_op_forward": (_i, [_p, _p, _p, _i64, _i64, _i, _p]),
    "sdfl_groupnorm_destroy": (_i, [_p]),
    "sdfl_layernorm_create": (_i, [C.POINTER(_p), _i64, _f, _p, _p]),
    "sdfl_layernorm_op_forward": (_i, [_p, _p, _p, _i64, _i, _p]),
    "sdfl_layernorm_destroy": (_i, [_p]),
    "sdfl_geglu_create": (_i, [C.POINTER(_p), _i64, _i64]),
    "sdfl_geglu_weight_shape": (_i, [_p, C.POINTER(_i64)]),
    "sdfl_geglu_op_forward": (_i, [_p, _p, _p, _i64, _i, _p]),
    "sdfl_geglu_destroy": (_i, [_p]),
    "sdfl_device_status": (_i, [C.POINTER(C.c_uint), _i, _p]),
    "sdfl_selftest_bounded_wait": (_i, [C.c_longlong, _p]),
    "sdfl_host_pipeline_create": (_i, [C.POINTER(_p), _sz, _i]),
    "sdfl_host_pipeline_destroy": (_i, [_p]),
    "sdfl_groupnorm_forward_host": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i]),
    "sdfl_groupnorm_forward_host_async": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i]),
    "sdfl_host_pipeline_sync": (_i, [_p]),
    "sdfl_host_alloc": (_i, [C.POINTER(_p), _sz]),
    "sdfl_host_free": (_i, [_p]),
}


def load(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python mobile-stable-diffusion_b200/build.py` "
            "(needs nvcc); there is no fallback implementation")
    lib = C.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = load()


def check(status: int, where: str) -> None:
    if status == OK:
        return
    detail = lib.sdfl_status_string(status).decode()
    if status == ERR_CUDA:
        detail += ": " + lib.sdfl_last_cuda_error_string().decode()
    raise SdflError(status, where, detail)
