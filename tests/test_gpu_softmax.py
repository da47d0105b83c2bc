"""Row softmax of the attention scores (util.cl:150-187) against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from conftest import TOL, assert_close, rng_for
from gpu_util import Guarded, to_dev, to_np

pytestmark = pytest.mark.gpu

# (rows, keys): cross-attention rows of 77, self-attention rows of 64 .. 4096, ragged and long rows
SHAPES = [(8 * 64, 77), (8 * 64, 64), (8 * 32, 256), (64, 1024), (48, 4096), (5, 100), (3, 1), (7, 333),
          (4, 8192), (2, 20000),
          (130, 77), (257, 33), (300, 255), (129, 3)]      # short odd rows, a few more than a multiple of 64


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("rows,keys", SHAPES)
def test_softmax_matches_the_reference_kernel(sdfl, rows, keys, dtype):
    rng = rng_for(8, rows + keys)
    x = (rng.standard_normal((rows, keys)) * 3.0).astype(np.float32).astype(dtype)
    want = oracle.softmax(x.astype(np.float32))
    out = Guarded((rows, keys), getattr(torch, dtype))
    sdfl.ops.softmax(to_dev(x), out=out.tensor)
    out.check()
    assert_close(to_np(out.tensor), want, TOL[dtype], f"softmax {rows}x{keys} {dtype}")
    buf = to_dev(x)                                  # in place, as nn/CrossAttention.cpp:365-366
    sdfl.ops.softmax(buf, out=buf)
    assert_close(to_np(buf), want, TOL[dtype], f"softmax in place {rows}x{keys} {dtype}")


def test_softmax_rows_sum_to_one_and_survive_large_scores(sdfl):
    """Where the reference overflows (scores above 88) the result here is still a distribution."""
    x = torch.full((4, 77), 200.0, device="cuda")
    x[:, 3] = 210.0
    y = sdfl.ops.softmax(x)
    assert torch.isfinite(y).all()
    np.testing.assert_allclose(to_np(y).sum(-1), 1.0, rtol=1e-6)
    assert float(y[0, 3]) > 0.99
    big = torch.randn((1024, 4096), device="cuda", dtype=torch.float16) * 4
    s = sdfl.ops.softmax(big).float().sum(-1)
    assert float((s - 1).abs().max()) < 2e-3


def test_softmax_misaligned_and_errors(sdfl):
    rng = rng_for(8, 77)
    x = (rng.standard_normal(4 * 64 + 1) * 2).astype(np.float32)
    dx = to_dev(x)[1:].view(4, 64)                   # 4-byte aligned rows only
    want = oracle.softmax(x[1:].reshape(4, 64))
    assert_close(to_np(sdfl.ops.softmax(dx)), want, 1e-5, "misaligned softmax")
    assert sdfl.ops.softmax(torch.zeros((0, 77), device="cuda")).shape == (0, 77)


@pytest.mark.parametrize("dtype", ["float32", "float16"])
def test_local_softmax_of_the_text_encoder(sdfl, dtype):
    """sdfl_local_softmax against the reference's local_softmax kernel (multi_head_attention.cl:28-54) on
    what the text encoder feeds it: [heads * 77, 77] scores with the causal mask, in place
    (nn/MultiHeadAttention.cpp:213-225); sdfl_softmax on the same rows agrees."""
    heads = 12
    rng = rng_for(2, 77)
    x = (rng.standard_normal((heads, 77, 77)) * 3.0).astype(np.float32).astype(dtype)
    x = x + np.triu(np.full((77, 77), -np.inf, np.float32), 1).astype(dtype)
    want = oracle.local_softmax(x.astype(np.float32))
    buf = to_dev(x)
    sdfl.ops.local_softmax(buf, out=buf)
    got = to_np(buf)
    assert_close(got, want, TOL[dtype], f"local_softmax {dtype}")
    iu = np.triu_indices(77, 1)
    assert np.all(got[:, iu[0], iu[1]] == 0)                       # masked scores: exact zeros
    again = to_np(sdfl.ops.softmax(to_dev(x).view(heads * 77, 77)))
    assert np.array_equal(again.reshape(got.shape), got)
