"""GEGLU gate, gelu, silu, quick_gelu, elemwise_add against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from conftest import TOL, assert_bit_equal, assert_close, rng_for
from gpu_util import NP_DTYPE, Guarded, to_dev, to_np

import oracle

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz")
ACTS = {"silu": oracle.silu, "gelu": oracle.gelu, "quick_gelu": oracle.quick_gelu}


def test_golden_vectors_from_the_reference_kernels(sdfl):
    g = np.load(GOLDEN)
    x = to_dev(g["act.x"])
    assert_close(to_np(sdfl.ops.silu(x)), g["act.silu"], 1e-5, "silu")
    assert_close(to_np(sdfl.ops.gelu(x)), g["act.gelu"], 1e-5, "gelu")
    assert_bit_equal(to_np(sdfl.ops.elemwise_add(x, to_dev(g["act.other"]))), g["act.add"], "add")
    assert_close(to_np(sdfl.ops.gelu_multiply(to_dev(g["geglu_r5_d64.ab"]))), g["geglu_r5_d64.y"],
                 1e-5, "gelu_multiply")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("name", ["silu", "gelu", "quick_gelu"])
@pytest.mark.parametrize("n", [2 * 77 * 3072, 2 * 1280, 1, 7, 1025, 77 * 4096 + 3])
def test_activations_match_oracle(sdfl, name, n, dtype):
    x = (rng_for(2, n % 997).standard_normal(n) * 3).astype(np.float32).astype(NP_DTYPE[dtype])
    want = ACTS[name](x.astype(np.float32))
    out = Guarded((n,), getattr(torch, dtype))
    getattr(sdfl.ops, name)(to_dev(x), out=out.tensor)
    out.check()
    assert_close(to_np(out.tensor), want, TOL[dtype], f"{name} n={n} {dtype}")


@pytest.mark.parametrize("name", ["silu", "gelu", "quick_gelu"])
def test_activation_extremes_in_place_and_misaligned(sdfl, name):
    x = np.array([0.0, -0.0, 1e-30, -1e-30, 5.0, -5.0, 20.0, -20.0, 87.0, -87.0, 100.0, -100.0,
                  1e4, -1e4, 0.5, -0.5, 3.3, -3.3], np.float32)
    want = ACTS[name](x)
    buf = Guarded(x.shape, torch.float32, misalign=1)
    buf.tensor.copy_(to_dev(x))
    getattr(sdfl.ops, name)(buf.tensor, out=buf.tensor)
    buf.check()
    assert_close(to_np(buf.tensor), want, 1e-5, f"{name} extremes")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("rows,D", [(8192, 1280), (154, 3072), (77, 4096), (5, 64), (3, 7), (9, 1),
                                    (2, 1284)])
def test_gelu_multiply_matches_oracle(sdfl, rows, D, dtype):
    ab = (rng_for(4, rows % 100 + D).standard_normal((rows, 2 * D)) * 1.5).astype(np.float32)
    ab = ab.astype(NP_DTYPE[dtype])
    want = oracle.gelu_multiply(ab.astype(np.float32))
    out = Guarded((rows, D), getattr(torch, dtype))
    sdfl.ops.gelu_multiply(to_dev(ab), out=out.tensor)
    out.check()
    assert_close(to_np(out.tensor), want, TOL[dtype], f"geglu {rows}x{D} {dtype}")


def test_gelu_multiply_value_half_first_gate_half_second(sdfl):
    """geglu.cl:6-8: a = AB[r, j], b = AB[r, D + j]; a zero gate zeroes the output."""
    ab = np.ones((4, 16), np.float32)
    ab[:, 8:] = 0.0
    assert np.all(to_np(sdfl.ops.gelu_multiply(to_dev(ab))) == 0.0)
    ab[:, 8:] = 10.0
    ab[:, :8] = 2.0
    assert_close(to_np(sdfl.ops.gelu_multiply(to_dev(ab))), np.full((4, 8), 20.0), 1e-5, "gate")


@pytest.mark.parametrize("n", [77 * 1024, 2 * 77 * 768, 5, 1023])
def test_elemwise_add_is_bit_exact(sdfl, n):
    rng = rng_for(2, n % 991)
    a = (0.02 * rng.standard_normal(n)).astype(np.float32)
    b = (0.02 * rng.standard_normal(n)).astype(np.float32)
    assert_bit_equal(to_np(sdfl.ops.elemwise_add(to_dev(a), to_dev(b))), oracle.elemwise_add(a, b), "fp32")
    ah, bh = a.astype(np.float16), b.astype(np.float16)
    want = oracle.to_half(oracle.elemwise_add(ah.astype(np.float32), bh.astype(np.float32)))
    assert_bit_equal(to_np(sdfl.ops.elemwise_add(to_dev(ah), to_dev(bh))), want, "fp16")
    buf = to_dev(a)
    sdfl.ops.elemwise_add(buf, to_dev(b), out=buf)      # C aliases A: TextEncoder.cpp:141-143
    assert_bit_equal(to_np(buf), oracle.elemwise_add(a, b), "in place")


def test_full_size_geglu_fp16_properties(sdfl):
    """[2,4096,2560] -> [2,4096,1280] fp16 at full size: compare against gelu() * value computed
    by the library's own flat kernels (different kernel, same definition) within tolerance."""
    gen = torch.Generator(device="cuda").manual_seed(4040)
    ab = torch.randn((2, 4096, 2560), device="cuda", generator=gen).half()
    y = sdfl.ops.gelu_multiply(ab)
    gate = sdfl.ops.gelu(ab[..., 1280:].contiguous()).float()
    want = ab[..., :1280].float() * gate
    diff = (y.float() - want).abs()
    assert float((diff - 2e-3 * want.abs()).max()) <= 2e-3
    rows = oracle.gelu_multiply(ab[0, :16].cpu().numpy().astype(np.float32))
    assert_close(to_np(y[0, :16]), rows, TOL["float16"], "first rows vs oracle")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("n,chunk_size,misalign", [
    (320 * 4096, 4096, 0),        # the time-embedding add of a ResBlock: [320, 64, 64] + [320]
    (1280 * 64, 64, 0),
    (40 * 72, 72, 0),             # chunk a multiple of the vector width, vector kernel
    (40 * 72 + 5, 72, 0),         # ... with a scalar tail (the last chunk is ragged)
    (33 * 77, 77, 0),             # chunk not a multiple of the vector width: scalar kernel
    (40 * 72, 72, 1),             # unaligned buffers: scalar kernel
    (7, 3, 0), (1, 1, 0),
])
def test_chunkwise_add_is_bit_exact(sdfl, n, chunk_size, misalign, dtype):
    """chunkwise_add (util.cl:136-148): C[i] = A[i] + chunk[i / chunk_size], one rounding."""
    rng = rng_for(2, 4000 + n % 991 + chunk_size)
    nchunks = -(-n // chunk_size)
    a = rng.standard_normal(n).astype(np.float32).astype(NP_DTYPE[dtype])
    e = rng.standard_normal(nchunks).astype(np.float32).astype(NP_DTYPE[dtype])
    want = oracle.chunkwise_add(a.astype(np.float32), e.astype(np.float32), chunk_size).astype(NP_DTYPE[dtype])
    src = Guarded((n,), getattr(torch, dtype), misalign=misalign)
    src.tensor.copy_(to_dev(a))
    out = Guarded((n,), getattr(torch, dtype), misalign=misalign)
    sdfl.ops.chunkwise_add(src.tensor, to_dev(e), chunk_size, out=out.tensor)
    out.check()
    assert_bit_equal(to_np(out.tensor), want, f"chunkwise_add n={n} chunk={chunk_size} {dtype}")
    sdfl.ops.chunkwise_add(src.tensor, to_dev(e), chunk_size, out=src.tensor)     # in place, as the reference does
    src.check()
    assert_bit_equal(to_np(src.tensor), want, "chunkwise_add in place")
