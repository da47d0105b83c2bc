"""Functional wrappers over the C ABI for torch CUDA tensors.

torch is used for device memory and streams only; every operation below is one call into
libsdfl.so.  Inputs must be contiguous CUDA tensors of dtype float32 or float16; gamma / beta
are float32.  Nothing here computes on the host and nothing falls back to torch operators.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _capi
from ._capi import F16, F32, GN_AUTO, GN_REGISTER, GN_RESIDENT, GN_SPLIT, SdflError, check, lib

__all__ = [
    "groupnorm", "groupnorm_multi", "groupnorm_bias", "chunkwise_add", "groupnorm_noalloc", "groupnorm_plan", "layernorm", "add_layernorm", "gelu_multiply", "silu", "gelu", "quick_gelu",
    "elemwise_add", "token_embedding", "timestep_embedding", "local_reduction_mean",
    "local_reduction_variance", "group_norm_apply", "layer_norm_apply", "device_status",
    "selftest_bounded_wait",
    "launch_count", "HostPipeline", "GN_AUTO", "GN_RESIDENT", "GN_SPLIT", "GN_REGISTER", "groupnorm_nhwc", "permute_021", "permute_add", "softmax", "local_softmax", "up_sample_nearest", "concat_channels", "groupnorm_concat",
]


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.float16:
        return F16
    raise TypeError(f"unsupported dtype {t.dtype}: float32 or float16 only")


def _dev(t: torch.Tensor, name: str) -> int:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor (the kernels have no host fallback)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t.data_ptr()


def _f32(t: torch.Tensor, name: str) -> int:
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32")
    return _dev(t, name)


def _stream(stream) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream if hasattr(s, "cuda_stream") else int(s)


_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int, stream=None) -> torch.Tensor:
    """A scratch buffer per (device, stream), grown on demand and reused.  Launches on one stream
    run in order, so they can share a buffer; launches on different streams may overlap and get
    their own.  A buffer that is outgrown may still be in use by a kernel on its stream: it is
    handed back to torch's allocator with that stream recorded, so that it is not reused earlier."""
    handle = _stream(stream)
    key = (device.index if device.index is not None else torch.cuda.current_device(), handle)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            ws.record_stream(torch.cuda.ExternalStream(handle, device=device) if handle else
                             torch.cuda.default_stream(device))
        ws = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def launch_count() -> int:
    return int(lib.sdfl_launch_count())


def device_status(clear: bool = True, stream=None) -> int:
    v = C.c_uint(0)
    check(lib.sdfl_device_status(C.byref(v), int(clear), _stream(stream)), "sdfl_device_status")
    return int(v.value)


def selftest_bounded_wait(limit_cycles: int = 2_000_000, stream=None) -> None:
    """Enqueue the kernel whose bounded wait must run out (see sdfl_selftest_bounded_wait)."""
    check(lib.sdfl_selftest_bounded_wait(int(limit_cycles), _stream(stream)), "sdfl_selftest_bounded_wait")


def groupnorm_plan(batch: int, channels: int, hw: int, num_groups: int, dtype: torch.dtype,
                   path: int = GN_AUTO, cluster_or_splits: int = 0) -> dict:
    arr = (C.c_int64 * 8)()
    code = F16 if dtype == torch.float16 else F32
    check(lib.sdfl_groupnorm_plan(batch, channels, hw, num_groups, code, path, cluster_or_splits,
                                  arr), "sdfl_groupnorm_plan")
    keys = ("path", "cluster", "threads", "splits", "smem", "workspace", "nclusters", "chunk_vecs")
    return dict(zip(keys, (int(v) for v in arr)))


def groupnorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, num_groups: int,
              eps: float = 1e-5, silu: bool = False, out: torch.Tensor | None = None,
              path: int = GN_AUTO, cluster_or_splits: int = 0, stream=None) -> torch.Tensor:
    """GroupNorm(+SiLU) on an NCHW tensor [B, C, ...]; out may be x itself."""
    if x.dim() < 2:
        raise ValueError("x must be [batch, channels, ...]")
    _dev(x, "x")
    out = torch.empty_like(x) if out is None else out
    if out.shape != x.shape or out.dtype != x.dtype:
        raise ValueError("out must match x in shape and dtype")
    B, Cc = x.shape[0], x.shape[1]
    hw = x.numel() // (B * Cc) if B * Cc else 0
    code = _dtype_code(x)
    nbytes = lib.sdfl_groupnorm_workspace_bytes_ex(B, Cc, hw, num_groups, code, path,
                                                   cluster_or_splits)
    ws = _workspace(x.device, nbytes, stream)
    with torch.cuda.device(x.device):
        check(lib.sdfl_groupnorm_forward_ex(
            _dev(x, "x"), _dev(out, "out"), _f32(gamma, "gamma"), _f32(beta, "beta"), B, Cc, hw,
            num_groups, eps, int(silu), code, ws.data_ptr(), ws.numel(), path, cluster_or_splits,
            _stream(stream)), "sdfl_groupnorm_forward")
    return out


_multi_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _multi_workspace(device: torch.device, stream_handle: int) -> torch.Tensor:
    """Zero-filled exchange scratch of the multi-tensor GroupNorm, one per (device, stream):
    launches on different streams may overlap on the GPU and must not share it."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_handle)
    ws = _multi_workspaces.get(key)
    if ws is None:
        ws = torch.zeros(int(lib.sdfl_groupnorm_multi_workspace_bytes()), dtype=torch.uint8, device=device)
        _multi_workspaces[key] = ws
    return ws


def groupnorm_multi(xs, gammas, betas, num_groups, eps=1e-5, silu: bool = False, outs=None,
                    knobs: int = 0, trace: torch.Tensor | None = None, stream=None, plan: list | None = None):
    """GroupNorm(+SiLU) of a list of independent NCHW tensors in one launch
    (sdfl_groupnorm_forward_multi).  `num_groups` and `eps` may be scalars or per-tensor lists.
    Raises SdflError(ERR_UNSUPPORTED) when a tensor does not meet the call's requirements
    (alignment, hw * element size a multiple of 16, more than 8 tensors)."""
    n = len(xs)
    if len(gammas) != n or len(betas) != n:
        raise ValueError("xs, gammas and betas must have the same length")
    groups = list(num_groups) if isinstance(num_groups, (list, tuple)) else [num_groups] * n
    epss = list(eps) if isinstance(eps, (list, tuple)) else [eps] * n
    outs = [torch.empty_like(x) for x in xs] if outs is None else list(outs)
    if n == 0:
        return outs
    code = _dtype_code(xs[0])
    arr = (_capi.GnTensor * n)()
    for k, (x, g, b, o) in enumerate(zip(xs, gammas, betas, outs)):
        if x.dim() < 2 or _dtype_code(x) != code or o.shape != x.shape or o.dtype != x.dtype:
            raise ValueError("tensors must be [batch, channels, ...] of one dtype; outs must match")
        B, Cc = x.shape[0], x.shape[1]
        arr[k].in_ = _dev(x, "x")
        arr[k].out = _dev(o, "out")
        arr[k].gamma = _f32(g, "gamma")
        arr[k].beta = _f32(b, "beta")
        arr[k].batch, arr[k].channels = B, Cc
        arr[k].hw = x.numel() // (B * Cc) if B * Cc else 0
        arr[k].num_groups = groups[k]
        arr[k].eps = epss[k]
    sh = _stream(stream)
    ws = _multi_workspace(xs[0].device, sh)
    pl = (C.c_int * 4)()
    with torch.cuda.device(xs[0].device):
        check(lib.sdfl_groupnorm_forward_multi_ex(
            arr, n, int(silu), code, ws.data_ptr(), ws.numel(), knobs,
            0 if trace is None else trace.data_ptr(), pl, sh), "sdfl_groupnorm_forward_multi")
    if plan is not None:
        plan[:] = [int(v) for v in pl]
    return outs


def groupnorm_bias(x: torch.Tensor, channel_bias: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor,
                   num_groups: int, eps: float = 1e-5, silu: bool = False,
                   out: torch.Tensor | None = None, stream=None, path: int = GN_AUTO,
                   cluster_or_splits: int = 0) -> torch.Tensor:
    """act(GroupNorm(x + channel_bias[:, :, None, None])); channel_bias is [B, C] of x's dtype."""
    _dev(x, "x")
    out = torch.empty_like(x) if out is None else out
    B, Cc = x.shape[0], x.shape[1]
    if channel_bias.shape != (B, Cc) or channel_bias.dtype != x.dtype:
        raise ValueError("channel_bias must be [batch, channels] of x's dtype")
    hw = x.numel() // (B * Cc) if B * Cc else 0
    code = _dtype_code(x)
    ws = _workspace(x.device, lib.sdfl_groupnorm_workspace_bytes_ex(B, Cc, hw, num_groups, code, path,
                                                                    cluster_or_splits), stream)
    with torch.cuda.device(x.device):
        check(lib.sdfl_groupnorm_bias_forward_ex(
            _dev(x, "x"), _dev(channel_bias, "channel_bias"), _dev(out, "out"), _f32(gamma, "gamma"),
            _f32(beta, "beta"), B, Cc, hw, num_groups, eps, int(silu), code, ws.data_ptr(), ws.numel(),
            path, cluster_or_splits, _stream(stream)), "sdfl_groupnorm_bias_forward")
    return out


def groupnorm_nhwc(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, num_groups: int,
                   eps: float = 1e-5, silu: bool = False, out: torch.Tensor | None = None,
                   stream=None) -> torch.Tensor:
    """act(GroupNorm(x)) of an NCHW tensor, written channels-last: out is [B, H*W, C]."""
    _dev(x, "x")
    B, Cc = x.shape[0], x.shape[1]
    hw = x.numel() // (B * Cc) if B * Cc else 0
    out = torch.empty((B, hw, Cc), dtype=x.dtype, device=x.device) if out is None else out
    if out.numel() != x.numel() or out.dtype != x.dtype:
        raise ValueError("out must have x's element count and dtype")
    code = _dtype_code(x)
    ws = _workspace(x.device, lib.sdfl_groupnorm_nhwc_workspace_bytes(B, Cc, hw, num_groups, code), stream)
    with torch.cuda.device(x.device):
        check(lib.sdfl_groupnorm_nhwc_forward(
            _dev(x, "x"), _dev(out, "out"), _f32(gamma, "gamma"), _f32(beta, "beta"), B, Cc, hw,
            num_groups, eps, int(silu), code, ws.data_ptr(), ws.numel(),
            _stream(stream)), "sdfl_groupnorm_nhwc_forward")
    return out


def permute_021(src: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """[I, J, K] -> [I, K, J] (the reference's permute3D__0_2_1)."""
    if src.dim() != 3:
        raise ValueError("permute_021 takes a 3-D tensor")
    I, J, K = src.shape
    out = torch.empty((I, K, J), dtype=src.dtype, device=src.device) if out is None else out
    with torch.cuda.device(src.device):
        check(lib.sdfl_permute3D__0_2_1(_dev(src, "src"), _dev(out, "out"), I, J, K, _dtype_code(src),
                                        _stream(stream)), "sdfl_permute3D__0_2_1")
    return out


def permute_add(src: torch.Tensor, residual: torch.Tensor, out: torch.Tensor | None = None,
                stream=None) -> torch.Tensor:
    """out[i, k, j] = src[i, j, k] + residual[i, k, j]."""
    if src.dim() != 3:
        raise ValueError("permute_add takes a 3-D tensor")
    I, J, K = src.shape
    if residual.numel() != src.numel() or residual.dtype != src.dtype:
        raise ValueError("residual must have src's element count and dtype")
    out = torch.empty((I, K, J), dtype=src.dtype, device=src.device) if out is None else out
    with torch.cuda.device(src.device):
        check(lib.sdfl_permute_add(_dev(src, "src"), _dev(residual, "residual"), _dev(out, "out"), I, J, K,
                                   _dtype_code(src), _stream(stream)), "sdfl_permute_add")
    return out


def up_sample_nearest(x: torch.Tensor, scale: int = 2, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """[..., H, W] -> [..., H*scale, W*scale], every element repeated scale x scale times."""
    H, W = x.shape[-2], x.shape[-1]
    planes = x.numel() // (H * W) if H * W else 0
    out = torch.empty((*x.shape[:-2], H * scale, W * scale), dtype=x.dtype, device=x.device) if out is None else out
    with torch.cuda.device(x.device):
        check(lib.sdfl_up_sample_nearest(_dev(x, "x"), _dev(out, "out"), planes, H, W, scale, _dtype_code(x),
                                         _stream(stream)), "sdfl_up_sample_nearest")
    return out


def concat_channels(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """[B, C1, ...] and [B, C2, ...] -> [B, C1 + C2, ...] (the reference's concat_buffer per image)."""
    B = a.shape[0]
    n1, n2 = (a.numel() // B, b.numel() // B) if B else (0, 0)
    out = torch.empty((B, a.shape[1] + b.shape[1], *a.shape[2:]), dtype=a.dtype, device=a.device) if out is None else out
    with torch.cuda.device(a.device):
        check(lib.sdfl_concat_buffer(_dev(a, "a"), _dev(b, "b"), _dev(out, "out"), B, n1, n2, _dtype_code(a),
                                     _stream(stream)), "sdfl_concat_buffer")
    return out


def groupnorm_concat(a: torch.Tensor, b: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor,
                     num_groups: int, eps: float = 1e-5, silu: bool = False,
                     out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """act(GroupNorm(cat([a, b], dim=1))) without materialising the concatenation."""
    B, C1, C2 = a.shape[0], a.shape[1], b.shape[1]
    hw = a.numel() // (B * C1) if B * C1 else 0
    out = torch.empty((B, C1 + C2, *a.shape[2:]), dtype=a.dtype, device=a.device) if out is None else out
    code = _dtype_code(a)
    ws = _workspace(a.device, lib.sdfl_groupnorm_workspace_bytes(B, C1 + C2, hw, num_groups, code), stream)
    with torch.cuda.device(a.device):
        check(lib.sdfl_groupnorm_concat_forward(
            _dev(a, "a"), C1, _dev(b, "b"), C2, _dev(out, "out"), _f32(gamma, "gamma"), _f32(beta, "beta"),
            B, hw, num_groups, eps, int(silu), code, ws.data_ptr(), ws.numel(), _stream(stream)),
            "sdfl_groupnorm_concat_forward")
    return out


def softmax(x: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """Softmax over the last dimension (rows = all leading dimensions); out may be x."""
    out = torch.empty_like(x) if out is None else out
    dim = x.shape[-1] if x.dim() else 1
    rows = x.numel() // dim if dim else 0
    with torch.cuda.device(x.device):
        check(lib.sdfl_softmax(_dev(x, "x"), _dev(out, "out"), rows, dim, _dtype_code(x), _stream(stream)),
              "sdfl_softmax")
    return out


def local_softmax(x: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """The text encoder's attention softmax (the reference's local_softmax kernel): rows = all
    leading dimensions, -inf entries (the causal mask) give exact zeros; out may be x."""
    out = torch.empty_like(x) if out is None else out
    n = x.shape[-1] if x.dim() else 1
    rows = x.numel() // n if n else 0
    with torch.cuda.device(x.device):
        check(lib.sdfl_local_softmax(_dev(x, "x"), _dev(out, "out"), rows, n, _dtype_code(x), _stream(stream)),
              "sdfl_local_softmax")
    return out


def chunkwise_add(a: torch.Tensor, chunk: torch.Tensor, chunk_size: int, out: torch.Tensor | None = None,
                  stream=None) -> torch.Tensor:
    out = torch.empty_like(a) if out is None else out
    with torch.cuda.device(a.device):
        check(lib.sdfl_chunkwise_add(_dev(a, "a"), _dev(chunk, "chunk"), _dev(out, "out"), a.numel(),
                                     chunk_size, _dtype_code(a), _stream(stream)), "sdfl_chunkwise_add")
    return out


def groupnorm_noalloc(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, num_groups: int,
                      eps: float = 1e-5, silu: bool = False, out: torch.Tensor | None = None,
                      stream=None) -> torch.Tensor:
    """GroupNorm(+SiLU) through sdfl_groupnorm_forward_noalloc: the library call allocates no
    device memory (its scratch is a fixed array inside the library), for hosts that forbid
    allocation after start-up.  `out` should be supplied by such callers; problems whose scratch
    would not fit the fixed array raise SdflError(ERR_WORKSPACE).  Calls that may overlap on
    the GPU must be ordered: they share the one scratch array."""
    if x.dim() < 2:
        raise ValueError("x must be [batch, channels, ...]")
    _dev(x, "x")
    out = torch.empty_like(x) if out is None else out
    B, Cc = x.shape[0], x.shape[1]
    hw = x.numel() // (B * Cc) if B * Cc else 0
    with torch.cuda.device(x.device):
        check(lib.sdfl_groupnorm_forward_noalloc(
            _dev(x, "x"), _dev(out, "out"), _f32(gamma, "gamma"), _f32(beta, "beta"), B, Cc, hw,
            num_groups, eps, int(silu), _dtype_code(x), _stream(stream)),
            "sdfl_groupnorm_forward_noalloc")
    return out


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5,
              out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    out = torch.empty_like(x) if out is None else out
    D = x.shape[-1]
    rows = x.numel() // D if D else 0
    with torch.cuda.device(x.device):
        check(lib.sdfl_layernorm_forward(_dev(x, "x"), _dev(out, "out"), _f32(gamma, "gamma"),
                                         _f32(beta, "beta"), rows, D, eps, _dtype_code(x),
                                         _stream(stream)), "sdfl_layernorm_forward")
    return out


def add_layernorm(a: torch.Tensor, b: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor,
                  eps: float = 1e-5, sum_out: torch.Tensor | None = None,
                  out: torch.Tensor | None = None, stream=None):
    """sum = a + b (may be written over a), out = LayerNorm(sum); returns (sum, out)."""
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError("a and b must match")
    sum_out = torch.empty_like(a) if sum_out is None else sum_out
    out = torch.empty_like(a) if out is None else out
    D = a.shape[-1]
    rows = a.numel() // D if D else 0
    with torch.cuda.device(a.device):
        check(lib.sdfl_add_layernorm_forward(_dev(a, "a"), _dev(b, "b"), _dev(sum_out, "sum_out"),
                                             _dev(out, "out"), _f32(gamma, "gamma"), _f32(beta, "beta"),
                                             rows, D, eps, _dtype_code(a), _stream(stream)),
              "sdfl_add_layernorm_forward")
    return sum_out, out


def gelu_multiply(ab: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """ab [..., 2D] -> [..., D]: value half times gelu(gate half)."""
    D = ab.shape[-1] // 2
    if ab.shape[-1] != 2 * D:
        raise ValueError("last dimension must be even")
    out = torch.empty(ab.shape[:-1] + (D,), dtype=ab.dtype, device=ab.device) if out is None else out
    rows = ab.numel() // (2 * D) if D else 0
    with torch.cuda.device(ab.device):
        check(lib.sdfl_gelu_multiply(_dev(ab, "ab"), _dev(out, "out"), rows, D, _dtype_code(ab),
                                     _stream(stream)), "sdfl_gelu_multiply")
    return out


def _unary(fn_name: str, x: torch.Tensor, out, stream) -> torch.Tensor:
    out = torch.empty_like(x) if out is None else out
    with torch.cuda.device(x.device):
        check(getattr(lib, fn_name)(_dev(x, "x"), _dev(out, "out"), x.numel(), _dtype_code(x),
                                    _stream(stream)), fn_name)
    return out


def silu(x, out=None, stream=None):
    return _unary("sdfl_silu", x, out, stream)


def gelu(x, out=None, stream=None):
    return _unary("sdfl_gelu", x, out, stream)


def quick_gelu(x, out=None, stream=None):
    return _unary("sdfl_quick_gelu", x, out, stream)


def elemwise_add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, stream=None):
    out = torch.empty_like(a) if out is None else out
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError("a and b must match")
    with torch.cuda.device(a.device):
        check(lib.sdfl_elemwise_add(_dev(a, "a"), _dev(b, "b"), _dev(out, "out"), a.numel(),
                                    _dtype_code(a), _stream(stream)), "sdfl_elemwise_add")
    return out


def token_embedding(ids: torch.Tensor, table: torch.Tensor, pos: torch.Tensor,
                    out: torch.Tensor | None = None, status: torch.Tensor | None = None,
                    stream=None) -> torch.Tensor:
    """ids [B, T] int64; table [vocab, D]; pos [T, D] -> [B, T, D] = table[ids] + pos."""
    if ids.dtype != torch.int64:
        raise TypeError("ids must be int64")
    B, T = ids.shape
    vocab, D = table.shape
    if pos.shape != (T, D) or pos.dtype != table.dtype:
        raise ValueError("pos must be [T, D] with the table's dtype")
    out = torch.empty((B, T, D), dtype=table.dtype, device=table.device) if out is None else out
    st = 0 if status is None else _dev(status, "status")
    if status is not None and status.dtype != torch.int32:
        raise TypeError("status must be int32")
    with torch.cuda.device(table.device):
        check(lib.sdfl_token_embedding(_dev(ids, "ids"), _dev(table, "table"), _dev(pos, "pos"),
                                       _dev(out, "out"), B, T, D, vocab, _dtype_code(table), st,
                                       _stream(stream)), "sdfl_token_embedding")
    return out


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0,
                       dtype: torch.dtype = torch.float32, out: torch.Tensor | None = None,
                       stream=None) -> torch.Tensor:
    if t.dtype != torch.int64:
        raise TypeError("t must be int64")
    B = t.numel()
    out = torch.empty((B, dim), dtype=dtype, device=t.device) if out is None else out
    with torch.cuda.device(t.device):
        check(lib.sdfl_timestep_embedding(_dev(t, "t"), _dev(out, "out"), B, dim, max_period,
                                          _dtype_code(out), _stream(stream)),
              "sdfl_timestep_embedding")
    return out


# ---- the reference's three-launch sequence, kernel by kernel --------------------------------------

def local_reduction_mean(x: torch.Tensor, groups: int, stream=None) -> torch.Tensor:
    out = torch.empty(groups, dtype=torch.float32, device=x.device)
    n = x.numel() // groups if groups else 0
    with torch.cuda.device(x.device):
        check(lib.sdfl_local_reduction_mean(_dev(x, "x"), out.data_ptr(), groups, n, _dtype_code(x),
                                            _stream(stream)), "sdfl_local_reduction_mean")
    return out


def local_reduction_variance(x: torch.Tensor, mean: torch.Tensor, groups: int, stream=None):
    out = torch.empty(groups, dtype=torch.float32, device=x.device)
    n = x.numel() // groups if groups else 0
    with torch.cuda.device(x.device):
        check(lib.sdfl_local_reduction_variance(_dev(x, "x"), _f32(mean, "mean"), out.data_ptr(),
                                                groups, n, _dtype_code(x), _stream(stream)),
              "sdfl_local_reduction_variance")
    return out


def group_norm_apply(x, mean, var, weight, bias, group_size: int, channel_size: int, eps: float,
                     num_channels: int, out=None, stream=None):
    out = torch.empty_like(x) if out is None else out
    with torch.cuda.device(x.device):
        check(lib.sdfl_group_norm(_dev(x, "x"), _f32(mean, "mean"), _f32(var, "var"),
                                  _f32(weight, "weight"), _f32(bias, "bias"), group_size,
                                  channel_size, eps, _dev(out, "out"), x.numel(), num_channels,
                                  _dtype_code(x), _stream(stream)), "sdfl_group_norm")
    return out


def layer_norm_apply(x, mean, var, weight, bias, chunk_size: int, eps: float = 1e-5, out=None,
                     stream=None):
    out = torch.empty_like(x) if out is None else out
    with torch.cuda.device(x.device):
        check(lib.sdfl_layer_norm(_dev(x, "x"), _f32(mean, "mean"), _f32(var, "var"),
                                  _f32(weight, "weight"), _f32(bias, "bias"), chunk_size,
                                  _dev(out, "out"), x.numel(), eps, _dtype_code(x),
                                  _stream(stream)), "sdfl_layer_norm")
    return out


class HostPipeline:
    """Host-buffer GroupNorm(+SiLU): page-locked host tensors in, page-locked host tensors out.

    Owns the device staging slots and streams (sdfl_host_pipeline_create); `groupnorm` blocks
    until the output is complete on the host.
    """

    def __init__(self, max_slot_bytes: int = 32 << 20, depth: int = 4, device: int | None = None):
        self._h = C.c_void_p()
        self.device = torch.cuda.current_device() if device is None else device
        with torch.cuda.device(self.device):
            check(lib.sdfl_host_pipeline_create(C.byref(self._h), max_slot_bytes, depth),
                  "sdfl_host_pipeline_create")

    def close(self) -> None:
        if self._h:
            with torch.cuda.device(self.device):
                lib.sdfl_host_pipeline_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def groupnorm(self, h_x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, num_groups: int,
                  eps: float = 1e-5, silu: bool = False, h_out: torch.Tensor | None = None,
                  wait: bool = True):
        """wait=False only enqueues (sdfl_groupnorm_forward_host_async); call sync() before
        reading h_out."""
        if h_x.is_cuda or not h_x.is_contiguous():
            raise TypeError("h_x must be a contiguous host tensor")
        h_out = torch.empty_like(h_x, pin_memory=h_x.is_pinned()) if h_out is None else h_out
        B, Cc = h_x.shape[0], h_x.shape[1]
        hw = h_x.numel() // (B * Cc) if B * Cc else 0
        fn = lib.sdfl_groupnorm_forward_host if wait else lib.sdfl_groupnorm_forward_host_async
        with torch.cuda.device(self.device):
            check(fn(self._h, h_x.data_ptr(), h_out.data_ptr(), _f32(gamma, "gamma"), _f32(beta, "beta"),
                     B, Cc, hw, num_groups, eps, int(silu), _dtype_code(h_x)),
                  "sdfl_groupnorm_forward_host")
        return h_out

    def sync(self) -> None:
        with torch.cuda.device(self.device):
            check(lib.sdfl_host_pipeline_sync(self._h), "sdfl_host_pipeline_sync")


_ = (_capi, SdflError)
