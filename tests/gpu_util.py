"""Helpers for the GPU parity tests: numpy <-> device tensors, guard bands, oracle in fp16."""
from __future__ import annotations

import numpy as np
import torch

import oracle

NP_DTYPE = {"float32": np.float32, "float16": np.float16}
SENTINEL = 0x5A


def to_dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


class Guarded:
    """A device tensor carved out of a larger byte buffer filled with a sentinel, so that any
    write outside the tensor is caught.  `misalign` shifts the start by that many elements
    (to exercise the paths that cannot use 16-byte accesses)."""

    def __init__(self, shape, dtype: torch.dtype, misalign: int = 0, band: int = 4096):
        esz = torch.empty((), dtype=dtype).element_size()
        n = int(np.prod(shape)) if len(shape) else 1
        self.nbytes = n * esz
        self.start = band + misalign * esz
        self.raw = torch.full((band * 2 + self.nbytes + 64,), SENTINEL, dtype=torch.uint8, device="cuda")
        self.tensor = self.raw[self.start:self.start + self.nbytes].view(dtype).view(*shape)

    def check(self) -> None:
        head = self.raw[:self.start]
        tail = self.raw[self.start + self.nbytes:]
        assert bool((head == SENTINEL).all()), "write before the start of the output buffer"
        assert bool((tail == SENTINEL).all()), "write past the end of the output buffer"


def gn_inputs(rng: np.random.Generator, shape, dtype: str, mean: float = 0.0, std: float = 1.0):
    C = shape[1]
    x = (rng.standard_normal(shape) * std + mean).astype(np.float32).astype(NP_DTYPE[dtype])
    gamma = (1.0 + 0.1 * rng.standard_normal(C)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(C)).astype(np.float32)
    return x, gamma, beta


def oracle_group_norm(x: np.ndarray, gamma, beta, G: int, eps: float, silu: bool) -> np.ndarray:
    """fp16 definition: the fp32 oracle on the widened fp16 values (result left in fp32)."""
    return oracle.group_norm(x.astype(np.float32), gamma, beta, G, eps, silu)
