"""The transposes around the transformer of a SpatialTransformer block, stand-alone and fused:
permute3D__0_2_1, permute + residual add, and GroupNorm with a channels-last store."""
import numpy as np
import pytest
import torch

import oracle
from conftest import TOL, assert_bit_equal, assert_close, rng_for
from gpu_util import Guarded, gn_inputs, oracle_group_norm, to_dev, to_np

pytestmark = pytest.mark.gpu

SHAPES_3D = [(1, 320, 4096), (2, 4096, 320), (2, 64, 64),
             (3, 72, 200), (2, 8, 8), (1, 136, 264),        # multiples of 8 but not of the 64 x 64 tile
             (3, 5, 7), (1, 1, 9), (2, 33, 64), (1, 130, 66),
             (70000, 2, 2)]


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape", SHAPES_3D)
def test_permute_is_a_bit_exact_copy(sdfl, shape, dtype):
    rng = rng_for(7, sum(shape))
    x = rng.standard_normal(shape).astype(np.float32).astype(dtype)
    want = oracle.permute_021(x.astype(np.float32)).astype(dtype)
    out = Guarded((shape[0], shape[2], shape[1]), getattr(torch, dtype))
    sdfl.ops.permute_021(to_dev(x), out=out.tensor)
    out.check()
    assert_bit_equal(to_np(out.tensor), want, f"permute {shape} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape", SHAPES_3D[:10])
def test_permute_fused_with_the_residual_add(sdfl, shape, dtype):
    """permute3D__0_2_1 then elemwise_add (SpatialTransformer.cpp:154-171): one rounded add per element."""
    rng = rng_for(7, 50 + sum(shape))
    x = rng.standard_normal(shape).astype(np.float32).astype(dtype)
    r = rng.standard_normal((shape[0], shape[2], shape[1])).astype(np.float32).astype(dtype)
    want = oracle.elemwise_add(oracle.permute_021(x.astype(np.float32)), r.astype(np.float32)).astype(dtype)
    out = Guarded(r.shape, getattr(torch, dtype))
    sdfl.ops.permute_add(to_dev(x), to_dev(r), out=out.tensor)
    out.check()
    assert_bit_equal(to_np(out.tensor), want, f"permute+add {shape} {dtype}")
    acc = to_dev(r)                                    # residual accumulated in place
    sdfl.ops.permute_add(to_dev(x), acc, out=acc)
    assert_bit_equal(to_np(acc), want, f"permute+add in place {shape} {dtype}")


def test_permute_misaligned_views_take_the_scalar_tiles(sdfl):
    rng = rng_for(7, 999)
    x = rng.standard_normal(2 * 6 * 10 + 1).astype(np.float16)
    dx = to_dev(x)[1:].view(2, 6, 10)                  # 2-byte aligned only
    want = x[1:].reshape(2, 6, 10).transpose(0, 2, 1)
    got = sdfl.ops.permute_021(dx.contiguous() if not dx.is_contiguous() else dx)
    assert_bit_equal(to_np(got), np.ascontiguousarray(want), "misaligned permute")


def test_permute_errors(sdfl):
    x = torch.zeros((2, 4, 6), device="cuda")
    with pytest.raises(sdfl.SdflError):
        sdfl.ops.permute_021(x, out=x.view(2, 6, 4))   # in place
    assert sdfl.ops.permute_021(torch.zeros((0, 4, 6), device="cuda")).shape == (0, 6, 4)


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape,G", [
    ((2, 320, 64, 64), 32), ((2, 640, 32, 32), 32), ((2, 1280, 16, 16), 32), ((2, 1280, 8, 8), 32),
    ((1, 12, 6, 6), 3),          # vectors straddle channels
    ((2, 6, 5, 8), 2),           # odd channels per group: scalar channels-last stores
    ((1, 64, 128, 128), 32),     # fp32 slabs of 128 KB; still one CTA per slab
    ((1, 128, 256, 256), 32),    # slabs too large for one CTA: norm into the scratch, then the transpose
    ((1, 512, 40, 40), 32),      # ... with tiles that are long along the channels (C a multiple of 128, H*W not)
    ((1, 320, 40, 40), 8),       # ... and with neither a multiple of 128: square tiles, ragged edges
])
def test_groupnorm_with_channels_last_store(sdfl, shape, G, dtype):
    """GroupNorm::forward + permute3D__0_2_1{1, C, HW} (SpatialTransformer.cpp:127-140) as one call."""
    rng = rng_for(7, 200 + sum(shape))
    x, gamma, beta = gn_inputs(rng, shape, dtype)
    B, C, H, W = shape
    for silu in (False, True):
        nchw = oracle_group_norm(x, gamma, beta, G, 1e-6, silu)
        want = oracle.permute_021(nchw.reshape(B, C, H * W))
        out = Guarded((B, H * W, C), getattr(torch, dtype))
        sdfl.ops.groupnorm_nhwc(to_dev(x), to_dev(gamma), to_dev(beta), G, 1e-6, silu, out=out.tensor)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"GN channels-last {shape} silu={silu}")
    assert sdfl.ops.device_status() == 0


def test_channels_last_store_matches_norm_then_permute_bit_for_bit(sdfl):
    """The fused store moves the same rounded values as the two-kernel sequence."""
    shape, G = (2, 320, 32, 32), 32
    x, gamma, beta = gn_inputs(rng_for(7, 777), shape, "float16")
    dx, dg, db = to_dev(x), to_dev(gamma), to_dev(beta)
    fused = sdfl.ops.groupnorm_nhwc(dx, dg, db, G, 1e-6, False)
    two = sdfl.ops.permute_021(sdfl.ops.groupnorm(dx, dg, db, G, 1e-6, False,
                                                  path=sdfl.ops.GN_REGISTER).view(2, 320, 1024))
    assert_bit_equal(to_np(fused), to_np(two), "fused vs norm + permute")
