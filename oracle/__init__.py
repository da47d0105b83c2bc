"""CPU checker for the CUDA kernels -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the cpu-baseline / reference legs of
``bench.py`` may import this package; nothing in the product package does.

Two back ends behind one numpy API:

* ``port`` -- ``libsdfl_oracle.so`` built from ``sdfl_oracle.c``, the plain-C restatement of
  the reference's fused-layer kernels and embedding host functions.
* ``ref``  -- ``_ref/libsdfl_ref.so``, the reference's own ``.cl`` kernel files compiled as C++
  (``ref_harness.cpp``); present only where ``make ref`` has run against a reference checkout.
  It covers the eight device kernels, not the two embedding host functions or quick_gelu.

Half precision is defined on top of either back end the way the kernels define it: inputs are
fp16 values widened to fp32, arithmetic is fp32, the result is rounded to fp16 (RNE) once.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "libsdfl_oracle.so")
REF_PATH = os.path.join(_HERE, "_ref", "libsdfl_ref.so")

_f32p = C.POINTER(C.c_float)
_i64p = C.POINTER(C.c_int64)
_sz = C.c_size_t


def build(ref_root: str | None = None) -> None:
    """Compile the port, and the compiled reference when `ref_root` (default: the environment
    variable SDFL_REFERENCE_ROOT) names a checkout of the reference project."""
    subprocess.run(["make", "-s", "-C", _HERE, "port"], check=True)
    ref_root = ref_root or os.environ.get("SDFL_REFERENCE_ROOT")
    if ref_root and os.path.isdir(os.path.join(ref_root, "app/src/main/assets/kernel")):
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REF={ref_root}"], check=True)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(_f32p)


def _c32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


_port = None
_ref = None


def port_lib():
    global _port
    if _port is None:
        if not os.path.exists(PORT_PATH):
            build(None)
        lib = C.CDLL(PORT_PATH)
        lib.oracle_num_threads.restype = C.c_int
        lib.oracle_set_num_threads.argtypes = [C.c_int]
        lib.oracle_local_reduction_mean.argtypes = [_f32p, _f32p, _sz, _sz]
        lib.oracle_local_reduction_variance.argtypes = [_f32p, _f32p, _f32p, _sz, _sz]
        lib.oracle_group_norm.argtypes = [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz,
                                          C.c_float, C.c_int, _f32p, _f32p]
        lib.oracle_group_norm.restype = C.c_int
        lib.oracle_layer_norm.argtypes = [_f32p, _f32p, _f32p, _f32p, _sz, _sz, C.c_float,
                                          _f32p, _f32p]
        lib.oracle_layer_norm.restype = C.c_int
        lib.oracle_gelu_multiply.argtypes = [_f32p, _f32p, _sz, _sz]
        for name in ("oracle_gelu", "oracle_silu", "oracle_quick_gelu"):
            getattr(lib, name).argtypes = [_f32p, _f32p, _sz]
        lib.oracle_elemwise_add.argtypes = [_f32p, _f32p, _f32p, _sz]
        lib.oracle_chunkwise_add.argtypes = [_f32p, _f32p, _f32p, _sz, _sz]
        lib.oracle_permute3D__0_2_1.argtypes = [_f32p, _f32p, _sz, _sz, _sz]
        lib.oracle_softmax.argtypes = [_f32p, _f32p, _sz, _sz]
        lib.oracle_local_softmax.argtypes = [_f32p, _f32p, _sz, _sz]
        lib.oracle_up_sample_nearest.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _sz]
        lib.oracle_token_embedding.argtypes = [_i64p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz]
        lib.oracle_token_embedding.restype = C.c_int
        lib.oracle_timestep_embedding.argtypes = [_i64p, _f32p, _sz, _sz, C.c_float]
        _port = lib
    return _port


def have_ref() -> bool:
    return os.path.exists(REF_PATH)


def ref_lib():
    global _ref
    if _ref is None:
        lib = C.CDLL(REF_PATH)
        lib.ref_num_threads.restype = C.c_int
        lib.ref_set_num_threads.argtypes = [C.c_int]
        lib.ref_gn_local_reduction_mean.argtypes = [_f32p, _f32p, _sz, _sz]
        lib.ref_gn_local_reduction_variance.argtypes = [_f32p, _f32p, _f32p, _sz, _sz]
        lib.ref_ln_local_reduction_mean.argtypes = [_f32p, _f32p, _sz, _sz]
        lib.ref_ln_local_reduction_variance.argtypes = [_f32p, _f32p, _f32p, _sz, _sz]
        lib.ref_group_norm_forward.argtypes = [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz,
                                               C.c_float, _f32p, _f32p]
        lib.ref_group_norm_forward.restype = C.c_int
        lib.ref_group_norm_silu_batched.argtypes = [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz,
                                                    _sz, C.c_float, C.c_int]
        lib.ref_group_norm_silu_batched.restype = C.c_int
        lib.ref_layer_norm_forward.argtypes = [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _f32p, _f32p]
        lib.ref_layer_norm_forward.restype = C.c_int
        lib.ref_gelu_multiply.argtypes = [_f32p, _f32p, _sz, _sz]
        lib.ref_silu.argtypes = [_f32p, _f32p, _sz]
        lib.ref_gelu.argtypes = [_f32p, _f32p, _sz]
        lib.ref_elemwise_add.argtypes = [_f32p, _f32p, _f32p, _sz]
        lib.ref_chunkwise_add.argtypes = [_f32p, _f32p, _f32p, _sz, _sz]
        lib.ref_permute3D__0_2_1.argtypes = [_f32p, _f32p, _sz, _sz, _sz]
        lib.ref_softmax.argtypes = [_f32p, _f32p, _sz, _sz]
        lib.ref_local_softmax.argtypes = [_f32p, _f32p, _sz, _sz]
        lib.ref_up_sample_nearest.argtypes = [_f32p, _f32p, _sz, _sz, _sz]
        _ref = lib
    return _ref


def num_threads(backend: str = "port") -> int:
    return ref_lib().ref_num_threads() if backend == "ref" else port_lib().oracle_num_threads()


def set_num_threads(n: int) -> None:
    port_lib().oracle_set_num_threads(n)
    if have_ref():
        ref_lib().ref_set_num_threads(n)


# ---------------------------------------------------------------------------------------------
# fp32 entry points (numpy in, numpy out)
# ---------------------------------------------------------------------------------------------

def group_norm(x, gamma, beta, num_groups: int, eps: float, silu: bool = False,
               backend: str = "port", return_stats: bool = False):
    """x: [B, C, ...] NCHW fp32.  One reference GroupNorm::forward per image, then silu."""
    x = _c32(x)
    gamma, beta = _c32(gamma), _c32(beta)
    B, Cc = x.shape[0], x.shape[1]
    hw = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
    out = np.empty_like(x)
    mean = np.empty(B * num_groups, np.float32)
    var = np.empty(B * num_groups, np.float32)
    if backend == "ref":
        lib = ref_lib()
        per = Cc * hw
        xf, of = x.reshape(B, per), out.reshape(B, per)
        for n in range(B):
            rc = lib.ref_group_norm_forward(_fp(xf[n]), _fp(of[n]), _fp(gamma), _fp(beta), per,
                                            num_groups, Cc, eps,
                                            _fp(mean[n * num_groups:]), _fp(var[n * num_groups:]))
            if rc != 0:
                raise ValueError(f"reference GroupNorm rejects this shape (code {rc})")
            if silu:
                lib.ref_silu(_fp(of[n]), _fp(of[n]), per)
    else:
        rc = port_lib().oracle_group_norm(_fp(x), _fp(out), _fp(gamma), _fp(beta), B, Cc, hw,
                                          num_groups, eps, int(silu), _fp(mean), _fp(var))
        if rc != 0:
            raise ValueError(f"oracle_group_norm failed (code {rc})")
    if return_stats:
        return out, mean, var
    return out


def layer_norm(x, gamma, beta, eps: float = 1e-5, backend: str = "port",
               return_stats: bool = False):
    """x: [..., D] fp32 row-major."""
    x = _c32(x)
    gamma, beta = _c32(gamma), _c32(beta)
    D = x.shape[-1]
    rows = x.size // D if D else 0
    out = np.empty_like(x)
    mean = np.empty(max(rows, 1), np.float32)
    var = np.empty(max(rows, 1), np.float32)
    if backend == "ref":
        if abs(eps - 1e-5) > 1e-12:
            raise ValueError("the reference LayerNorm kernel has eps fixed at 1e-5")
        rc = ref_lib().ref_layer_norm_forward(_fp(x), _fp(out), _fp(gamma), _fp(beta), x.size, D,
                                              _fp(mean), _fp(var))
        if rc != 0:
            raise ValueError(f"reference LayerNorm rejects this shape (code {rc})")
    else:
        rc = port_lib().oracle_layer_norm(_fp(x), _fp(out), _fp(gamma), _fp(beta), rows, D, eps,
                                          _fp(mean), _fp(var))
        if rc != 0:
            raise ValueError(f"oracle_layer_norm failed (code {rc})")
    if return_stats:
        return out, mean[:rows], var[:rows]
    return out


def local_reduction_mean(x, groups: int, backend: str = "port", kind: str = "gn"):
    """Mean of each of `groups` equal contiguous slices of x (the stand-alone stats kernel)."""
    x = _c32(x).ravel()
    n = x.size // groups
    out = np.empty(groups, np.float32)
    if backend == "ref":
        fn = getattr(ref_lib(), f"ref_{kind}_local_reduction_mean")
        fn(_fp(x), _fp(out), groups, n // 64)
    else:
        port_lib().oracle_local_reduction_mean(_fp(x), _fp(out), groups, n)
    return out


def local_reduction_variance(x, mean, groups: int, backend: str = "port", kind: str = "gn"):
    x = _c32(x).ravel()
    mean = _c32(mean)
    n = x.size // groups
    out = np.empty(groups, np.float32)
    if backend == "ref":
        fn = getattr(ref_lib(), f"ref_{kind}_local_reduction_variance")
        fn(_fp(x), _fp(mean), _fp(out), groups, n // 64)
    else:
        port_lib().oracle_local_reduction_variance(_fp(x), _fp(mean), _fp(out), groups, n)
    return out


def gelu_multiply(ab, backend: str = "port"):
    """ab: [..., 2D] -> [..., D]; value half first, gate half second."""
    ab = _c32(ab)
    D = ab.shape[-1] // 2
    rows = ab.size // (2 * D) if D else 0
    out = np.empty(ab.shape[:-1] + (D,), np.float32)
    if backend == "ref":
        ref_lib().ref_gelu_multiply(_fp(ab), _fp(out), rows, D)
    else:
        port_lib().oracle_gelu_multiply(_fp(ab), _fp(out), rows, D)
    return out


def _unary(name: str, x, backend: str):
    x = _c32(x)
    out = np.empty_like(x)
    if backend == "ref":
        getattr(ref_lib(), f"ref_{name}")(_fp(x), _fp(out), x.size)
    else:
        getattr(port_lib(), f"oracle_{name}")(_fp(x), _fp(out), x.size)
    return out


def silu(x, backend: str = "port"):
    return _unary("silu", x, backend)


def gelu(x, backend: str = "port"):
    return _unary("gelu", x, backend)


def quick_gelu(x, backend: str = "port"):
    if backend == "ref":
        raise ValueError("the reference has no quick_gelu kernel")
    return _unary("quick_gelu", x, backend)


def elemwise_add(a, b, backend: str = "port"):
    a, b = _c32(a), _c32(b)
    out = np.empty_like(a)
    if backend == "ref":
        ref_lib().ref_elemwise_add(_fp(a), _fp(b), _fp(out), a.size)
    else:
        port_lib().oracle_elemwise_add(_fp(a), _fp(b), _fp(out), a.size)
    return out


def up_sample_nearest(x, scale: int = 2, backend: str = "port"):
    """[..., H, W] -> [..., H*scale, W*scale]; the compiled reference kernel takes square planes only."""
    x = _c32(x)
    H, W = x.shape[-2], x.shape[-1]
    planes = x.size // (H * W) if H * W else 0
    out = np.empty((*x.shape[:-2], H * scale, W * scale), np.float32)
    if backend == "ref":
        if H != W:
            raise ValueError("the reference's up_sample_nearest indexes square planes (up_sample.cl:9-10)")
        ref_lib().ref_up_sample_nearest(_fp(x), _fp(out), planes, H, scale)
    else:
        port_lib().oracle_up_sample_nearest(_fp(x), _fp(out), planes, H, W, scale)
    return out


def concat_buffer(a, b):
    """UNetModel::concat_buffer (UNetModel.cpp:1960-1990): two buffer copies, a then b.  For a batch
    that is the per-image concatenation along axis 1."""
    return np.ascontiguousarray(np.concatenate([_c32(a), _c32(b)], axis=1))


def softmax(x, backend: str = "port"):
    """Row softmax over the last axis, the reference's way (no maximum subtracted)."""
    x = _c32(x)
    chunk = x.shape[-1]
    rows = x.size // chunk if chunk else 0
    out = np.empty_like(x)
    fn = ref_lib().ref_softmax if backend == "ref" else port_lib().oracle_softmax
    fn(_fp(x), _fp(out), rows, chunk)
    return out


def local_softmax(x, backend: str = "port"):
    """Row softmax the text encoder's way (multi_head_attention.cl local_softmax): one work-item per
    element, halving reduction with a carry for odd row lengths; no maximum subtracted."""
    x = _c32(x)
    n = x.shape[-1]
    rows = x.size // n if n else 0
    out = np.empty_like(x)
    fn = ref_lib().ref_local_softmax if backend == "ref" else port_lib().oracle_local_softmax
    fn(_fp(x), _fp(out), rows, n)
    return out


def permute_021(src, backend: str = "port"):
    """[I, J, K] -> [I, K, J]: the reference's permute3D__0_2_1 with global size {I, J, K}."""
    src = _c32(src)
    I, J, K = src.shape
    out = np.empty((I, K, J), np.float32)
    fn = ref_lib().ref_permute3D__0_2_1 if backend == "ref" else port_lib().oracle_permute3D__0_2_1
    fn(_fp(src), _fp(out), I, J, K)
    return out


def chunkwise_add(a, chunk, chunk_size: int, backend: str = "port"):
    """out[i] = a[i] + chunk[i // chunk_size] over the flattened a."""
    a, chunk = _c32(a), _c32(chunk)
    out = np.empty_like(a)
    if backend == "ref":
        ref_lib().ref_chunkwise_add(_fp(a), _fp(chunk), _fp(out), a.size, chunk_size)
    else:
        port_lib().oracle_chunkwise_add(_fp(a), _fp(chunk), _fp(out), a.size, chunk_size)
    return out


def token_embedding(ids, table, pos):
    """ids: [B, T] int64; table: [vocab, D]; pos: [T, D] -> [B, T, D] fp32 (gather, then + pos)."""
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    table, pos = _c32(table), _c32(pos)
    B, T = ids.shape
    D = table.shape[1]
    out = np.empty((B, T, D), np.float32)
    rc = port_lib().oracle_token_embedding(ids.ctypes.data_as(_i64p), _fp(table), _fp(pos), _fp(out),
                                           B, T, D, table.shape[0])
    if rc != 0:
        raise IndexError("token id outside the embedding table")
    return out


def timestep_embedding(t, dim: int, max_period: float = 10000.0):
    """t: [B] int64 -> [B, dim] fp32, layout [cos | sin]."""
    t = np.ascontiguousarray(t, dtype=np.int64).ravel()
    out = np.zeros((t.size, dim), np.float32)
    port_lib().oracle_timestep_embedding(t.ctypes.data_as(_i64p), _fp(out), t.size, dim, max_period)
    return out


# ---------------------------------------------------------------------------------------------
# fp16 definition: widen -> fp32 arithmetic -> one RNE rounding
# ---------------------------------------------------------------------------------------------

def as_half_inputs(x) -> np.ndarray:
    """Round to fp16 and widen back: the values an fp16 kernel actually sees."""
    return np.asarray(x, dtype=np.float16).astype(np.float32)


def to_half(y) -> np.ndarray:
    return np.asarray(y, dtype=np.float32).astype(np.float16)
