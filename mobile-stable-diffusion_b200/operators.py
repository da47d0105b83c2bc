"""Operator classes with the reference's call shape: constructor, ``init()``, ``forward()``.

Reference interface (paths inside the reference project, app/src/main/cpp/modules/nn/):
  GroupNorm.h:15-29   GroupNorm(ctx, queue, num_groups, num_channels, eps, weight_name, bias_name,
                      kernel); void init(); cl_int forward(in, out, n_wait, wait_list, event)
  LayerNorm.h:16-28   LayerNorm(ctx, queue, dim, weight_name, bias_name, kernel); same trio
  GEGLU.h:18-36       GEGLU(ctx, queue, in_features, out_features, ...); same trio

What changes at this boundary: the OpenCL context/queue/kernel-holder arguments disappear (a
CUDA stream is given per call instead of events), weights are handed over as arrays instead of
``.npy`` file names (file loading is Android glue, util.cpp:103-147), and the batch size is
taken from the tensor shape (the reference is batch-1).  What stays: argument meaning,
``init()`` uploading and validating the weights with the reference's error messages
(GroupNorm.cpp:51-66), ``forward(input, output)`` with ``output`` possibly the same buffer,
returning 0 on success, and contract violations raising (the reference throws
std::runtime_error: GroupNorm.cpp:83-93, LayerNorm.cpp:54-63).
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops


def _to_device_f32(a, device) -> torch.Tensor:
    if isinstance(a, torch.Tensor):
        return a.detach().to(device=device, dtype=torch.float32).contiguous()
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)


class GroupNorm:
    def __init__(self, num_groups: int, num_channels: int, eps: float, weight, bias,
                 fuse_silu: bool = False, device: str | torch.device = "cuda"):
        self.num_groups = int(num_groups)
        self.num_channels = int(num_channels)
        self.eps = float(eps)
        self.fuse_silu = bool(fuse_silu)
        self.device = torch.device(device)
        self._weight_src, self._bias_src = weight, bias
        self.weightSize = self.num_channels     # GroupNorm.cpp:38
        self.bufferWeight = None
        self.bufferBias = None

    def init(self) -> None:
        if self.bufferWeight is not None and self.bufferBias is not None:
            return                                              # GroupNorm.cpp:52-54
        w = _to_device_f32(self._weight_src, self.device)
        b = _to_device_f32(self._bias_src, self.device)
        if w.numel() != b.numel():
            raise RuntimeError("weight.shape[0] != bias.shape[0]")      # GroupNorm.cpp:59-61
        if w.numel() != self.weightSize:
            raise RuntimeError("weight.shape[0] != weightSize")         # GroupNorm.cpp:63-65
        self.bufferWeight, self.bufferBias = w, b

    def forward(self, input: torch.Tensor, output: torch.Tensor, stream=None) -> int:
        if self.bufferWeight is None:
            raise RuntimeError("GroupNorm.forward before init()")
        if input.dim() < 2 or input.shape[1] != self.num_channels:
            raise RuntimeError("input_size % weight->num_vals != 0")    # GroupNorm.cpp:83-87
        ops.groupnorm(input, self.bufferWeight, self.bufferBias, self.num_groups, self.eps,
                      self.fuse_silu, out=output, stream=stream)
        return 0


class LayerNorm:
    def __init__(self, dim: int, weight, bias, eps: float = 1e-5,
                 device: str | torch.device = "cuda"):
        self.weightSize = int(dim)              # LayerNorm.cpp:35
        self.eps = float(eps)                   # constant 1e-5 in the reference (layer_norm.cl:58)
        self.device = torch.device(device)
        self._weight_src, self._bias_src = weight, bias
        self.bufferWeight = None
        self.bufferBias = None

    def init(self) -> None:
        if self.bufferWeight is not None and self.bufferBias is not None:
            return
        w = _to_device_f32(self._weight_src, self.device)
        b = _to_device_f32(self._bias_src, self.device)
        if w.numel() != b.numel():
            raise RuntimeError("weightSize != biasSize")                # LayerNorm.cpp:53-55
        if w.numel() != self.weightSize:
            raise RuntimeError("weightSize != weight->num_vals")        # LayerNorm.cpp:57-59
        self.bufferWeight, self.bufferBias = w, b

    def forward(self, input: torch.Tensor, output: torch.Tensor, stream=None) -> int:
        if self.bufferWeight is None:
            raise RuntimeError("LayerNorm.forward before init()")
        if input.numel() % self.weightSize != 0 or input.shape[-1] != self.weightSize:
            raise RuntimeError("input_size % weight->num_vals != 0")    # LayerNorm.cpp:78-82
        ops.layernorm(input, self.bufferWeight, self.bufferBias, self.eps, out=output, stream=stream)
        return 0


class GEGLU:
    """The gelu_multiply stage of GEGLU::forward (GEGLU.cpp:71-77).

    The reference's GEGLU owns a Linear(in_features -> 2*out_features) in front of the gate
    (GEGLU.cpp:32-34); dense layers are outside this library, so ``forward`` takes the
    projected tensor [rows, 2*out_features] and writes [rows, out_features].
    """

    def __init__(self, in_features: int, out_features: int):
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.weightShape = [2 * self.out_features, self.in_features]    # GEGLU.cpp:36

    def init(self) -> None:
        return

    def forward(self, projected: torch.Tensor, output: torch.Tensor, stream=None) -> int:
        if projected.shape[-1] != 2 * self.out_features:
            raise RuntimeError("projected.shape[-1] != 2 * out_features")
        ops.gelu_multiply(projected, out=output, stream=stream)
        return 0
