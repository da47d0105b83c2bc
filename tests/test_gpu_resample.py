"""up_sample_nearest, concat_buffer and the concat fused into GroupNorm's loads."""
import numpy as np
import pytest
import torch

import oracle
from conftest import TOL, assert_bit_equal, assert_close, rng_for
from gpu_util import Guarded, gn_inputs, oracle_group_norm, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape,scale", [((2, 1280, 8, 8), 2), ((1, 640, 32, 32), 2), ((3, 5, 7, 9), 2),
                                         ((2, 4, 6, 6), 3), ((1, 2, 1, 1), 2), ((1, 3, 5, 3), 2)])
def test_up_sample_nearest_is_a_bit_exact_copy(sdfl, shape, scale, dtype):
    x = rng_for(9, sum(shape)).standard_normal(shape).astype(np.float32).astype(dtype)
    want = oracle.up_sample_nearest(x.astype(np.float32), scale).astype(dtype)
    out = Guarded((*shape[:2], shape[2] * scale, shape[3] * scale), getattr(torch, dtype))
    sdfl.ops.up_sample_nearest(to_dev(x), scale, out=out.tensor)
    out.check()
    assert_bit_equal(to_np(out.tensor), want, f"upsample {shape} x{scale} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("B,C1,C2,H", [(2, 320, 320, 16), (1, 640, 320, 8), (3, 5, 7, 3), (2, 1, 1, 1)])
def test_concat_buffer_per_image(sdfl, B, C1, C2, H, dtype):
    rng = rng_for(9, B + C1 + C2 + H)
    a = rng.standard_normal((B, C1, H, H)).astype(np.float32).astype(dtype)
    b = rng.standard_normal((B, C2, H, H)).astype(np.float32).astype(dtype)
    out = Guarded((B, C1 + C2, H, H), getattr(torch, dtype))
    sdfl.ops.concat_channels(to_dev(a), to_dev(b), out=out.tensor)
    out.check()
    assert_bit_equal(to_np(out.tensor), oracle.concat_buffer(a, b).astype(dtype), "concat")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("B,C1,C2,H,G", [
    (2, 320, 320, 32, 32),      # boundary between groups (640 channels, 20 per group)
    (2, 640, 320, 32, 32),      # 960 channels, 30 per group: group 21 takes channels from both tensors
    (2, 1280, 1280, 8, 32),
    (1, 640, 320, 64, 32),      # 32 slabs of 240 / 480 KB: the cluster kernel, two bulk copies per chunk at the seam
    (1, 128, 128, 256, 32),     # 2 / 4 MB slabs, several chunks per share
    (2, 6, 10, 5, 4),           # hw * element size not a multiple of 16: concat kernel + in-place norm
])
def test_groupnorm_of_a_concatenation_without_materialising_it(sdfl, B, C1, C2, H, G, dtype):
    """concat_buffer (UNetModel.cpp:1960-1990) + GroupNorm + silu of a ResBlock in an output block."""
    rng = rng_for(9, 300 + C1 + C2 + H)
    x, gamma, beta = gn_inputs(rng, (B, C1 + C2, H, H), dtype)
    a, b = np.ascontiguousarray(x[:, :C1]), np.ascontiguousarray(x[:, C1:])
    for silu in (True, False):
        want = oracle_group_norm(x, gamma, beta, G, 1e-5, silu)
        out = Guarded(x.shape, getattr(torch, dtype))
        sdfl.ops.groupnorm_concat(to_dev(a), to_dev(b), to_dev(gamma), to_dev(beta), G, 1e-5, silu, out=out.tensor)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"GN(concat) {B}x({C1}+{C2})x{H} silu={silu}")
    assert sdfl.ops.device_status() == 0


def test_fused_concat_equals_concat_then_norm_bit_for_bit(sdfl):
    rng = rng_for(9, 4321)
    x, gamma, beta = gn_inputs(rng, (2, 960, 32, 32), "float16")
    a, b = to_dev(np.ascontiguousarray(x[:, :640])), to_dev(np.ascontiguousarray(x[:, 640:]))
    dg, db = to_dev(gamma), to_dev(beta)
    fused = sdfl.ops.groupnorm_concat(a, b, dg, db, 32, 1e-5, True)
    two = sdfl.ops.groupnorm(sdfl.ops.concat_channels(a, b), dg, db, 32, 1e-5, True)
    assert_bit_equal(to_np(fused), to_np(two), "fused concat vs concat + norm")
