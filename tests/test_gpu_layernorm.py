"""LayerNorm CUDA kernels against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from conftest import TOL, assert_close, rng_for
from gpu_util import NP_DTYPE, Guarded, to_dev, to_np

import oracle

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz")


def ln_inputs(rng, rows, D, dtype, mean=0.0, std=1.0):
    x = (rng.standard_normal((rows, D)) * std + mean).astype(np.float32).astype(NP_DTYPE[dtype])
    gamma = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(D)).astype(np.float32)
    return x, gamma, beta


def test_golden_vectors_from_the_reference_kernels(sdfl):
    g = np.load(GOLDEN)
    for name in sorted({k.split(".")[0] for k in g.files if k.startswith("ln_")}):
        got = sdfl.ops.layernorm(to_dev(g[f"{name}.x"]), to_dev(g[f"{name}.gamma"]),
                                 to_dev(g[f"{name}.beta"]), 1e-5)
        assert_close(to_np(got), g[f"{name}.y"], 1e-5, name)


# rows x D: config 2 (CLIP, 768 and the reference's own 1024), config 4 (UNet), every register
# bucket of the row-in-registers kernel, and rows that force the block-per-row kernel.
LN_SHAPES = [(154, 768), (77, 1024), (8192, 320), (1024, 640), (256, 1280), (64, 1280),
             (5, 64), (3, 8), (7, 4096), (2, 8192), (3, 16384), (33, 100), (9, 7), (4, 1), (1, 330)]


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("rows,D", LN_SHAPES)
def test_layernorm_matches_oracle(sdfl, rows, D, dtype):
    x, gamma, beta = ln_inputs(rng_for(2, rows + D), rows, D, dtype)
    want = oracle.layer_norm(x.astype(np.float32), gamma, beta, 1e-5)
    out = Guarded((rows, D), getattr(torch, dtype))
    sdfl.ops.layernorm(to_dev(x), to_dev(gamma), to_dev(beta), 1e-5, out=out.tensor)
    out.check()
    assert_close(to_np(out.tensor), want, TOL[dtype], f"LN {rows}x{D} {dtype}")


def test_layernorm_eps_argument_in_place_and_3d(sdfl):
    x, gamma, beta = ln_inputs(rng_for(4, 1), 2 * 64, 320, "float16")
    x = x.reshape(2, 64, 320)
    want = oracle.layer_norm(x.astype(np.float32), gamma, beta, 1e-3)
    buf = to_dev(x)
    sdfl.ops.layernorm(buf, to_dev(gamma), to_dev(beta), 1e-3, out=buf)
    assert_close(to_np(buf), want, TOL["float16"], "in place, eps 1e-3")


def test_layernorm_misaligned_rows(sdfl):
    x, gamma, beta = ln_inputs(rng_for(2, 77), 16, 768, "float32")
    want = oracle.layer_norm(x, gamma, beta, 1e-5)
    xin = Guarded((16, 768), torch.float32, misalign=1)
    xin.tensor.copy_(to_dev(x))
    out = Guarded((16, 768), torch.float32, misalign=2)
    sdfl.ops.layernorm(xin.tensor, to_dev(gamma), to_dev(beta), 1e-5, out=out.tensor)
    out.check()
    assert_close(to_np(out.tensor), want, 1e-5, "misaligned")


def test_three_launch_sequence_kernel_by_kernel(sdfl):
    """The reference's call sequence: mean, variance (both inspectable, nn/LayerNorm.cpp:
    108-124), then layer_norm -- and the same for GroupNorm."""
    x, gamma, beta = ln_inputs(rng_for(2, 5), 154, 768, "float32")
    want, wmean, wvar = oracle.layer_norm(x, gamma, beta, 1e-5, return_stats=True)
    dx = to_dev(x)
    mean = sdfl.ops.local_reduction_mean(dx, 154)
    var = sdfl.ops.local_reduction_variance(dx, mean, 154)
    assert_close(to_np(mean), wmean, 1e-5, "row means")
    assert_close(to_np(var), wvar, 1e-5, "row variances")
    y = sdfl.ops.layer_norm_apply(dx, mean, var, to_dev(gamma), to_dev(beta), 768, 1e-5)
    assert_close(to_np(y), want, 1e-5, "layer_norm kernel")

    rng = rng_for(1, 5)
    xg = rng.standard_normal((2, 64, 16, 16)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(64)).astype(np.float32)
    b = (0.1 * rng.standard_normal(64)).astype(np.float32)
    wantg, gm, gv = oracle.group_norm(xg, g, b, 32, 1e-5, False, return_stats=True)
    dxg = to_dev(xg)
    mean = sdfl.ops.local_reduction_mean(dxg, 2 * 32)
    var = sdfl.ops.local_reduction_variance(dxg, mean, 2 * 32)
    assert_close(to_np(mean), gm, 1e-5, "group means")
    assert_close(to_np(var), gv, 1e-5, "group variances")
    y = sdfl.ops.group_norm_apply(dxg, mean, var, to_dev(g), to_dev(b), group_size=2 * 256,
                                  channel_size=256, eps=1e-5, num_channels=64)
    assert_close(to_np(y), wantg, 1e-5, "group_norm kernel")
    z = sdfl.ops.silu(y, out=y)                       # silu in place, nn/ResBlock.cpp:136-137
    assert_close(to_np(z), oracle.group_norm(xg, g, b, 32, 1e-5, True), 1e-5, "then silu")


def test_full_size_rows_have_zero_mean_unit_variance(sdfl):
    rows, D = 2 * 4096, 1280
    gen = torch.Generator(device="cuda").manual_seed(4004)
    x = (torch.randn((rows, D), device="cuda", generator=gen) * 2 + 1).half()
    y = sdfl.ops.layernorm(x, torch.ones(D, device="cuda"), torch.zeros(D, device="cuda"), 1e-5)
    mean = sdfl.ops.local_reduction_mean(y, rows)
    var = sdfl.ops.local_reduction_variance(y, mean, rows)
    assert float(mean.abs().max()) < 2e-3 and float((var - 1).abs().max()) < 5e-3
    assert torch.equal(y, sdfl.ops.layernorm(x, torch.ones(D, device="cuda"),
                                             torch.zeros(D, device="cuda"), 1e-5))


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("rows,D", [(8192, 320), (1024, 640), (256, 1280), (154, 768), (7, 100), (3, 16384)])
def test_add_then_layernorm_equals_the_reference_two_steps(sdfl, rows, D, dtype):
    """elemwise_add into the residual, then LayerNorm of it (BasicTransformerBlock.cpp:126-136)."""
    rng = rng_for(4, rows + D)
    a = (rng.standard_normal((rows, D)) * 1.2).astype(np.float32).astype(NP_DTYPE[dtype])
    b = (rng.standard_normal((rows, D)) * 0.7 + 0.1).astype(np.float32).astype(NP_DTYPE[dtype])
    gamma = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(D)).astype(np.float32)
    want_sum = oracle.elemwise_add(a.astype(np.float32), b.astype(np.float32)).astype(NP_DTYPE[dtype])
    want = oracle.layer_norm(want_sum.astype(np.float32), gamma, beta, 1e-5)
    da = to_dev(a)
    s, y = sdfl.ops.add_layernorm(da, to_dev(b), to_dev(gamma), to_dev(beta), 1e-5, sum_out=da)
    assert s.data_ptr() == da.data_ptr()                 # the sum went over `a`, as the reference does
    assert to_np(s).tobytes() == want_sum.tobytes(), "the residual sum must be bit exact"
    assert_close(to_np(y), want, TOL[dtype], f"add+LN {rows}x{D} {dtype}")


def test_add_layernorm_rejects_out_overlapping_the_sum(sdfl):
    a = torch.zeros((4, 64), device="cuda")
    g = torch.ones(64, device="cuda")
    with pytest.raises(sdfl.SdflError) as e:
        sdfl.ops.add_layernorm(a, torch.zeros_like(a), g, g, sum_out=a, out=a)
    assert e.value.status == sdfl._capi.ERR_OVERLAP


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape,groups,misalign", [
    ((1, 320, 64, 64), 32, 0),      # 32 groups: a cluster of CTAs per group
    ((2, 64, 16, 16), 32, 0),       # one CTA per group, vector loads
    ((2, 64, 5, 7), 32, 0),         # 35-pixel channels: element-wise kernels
    ((2, 64, 16, 16), 32, 1),       # unaligned buffers: element-wise kernels
])
def test_groupnorm_kernel_by_kernel_all_layouts(sdfl, shape, groups, misalign, dtype):
    """local_reduction_mean -> local_reduction_variance -> group_norm (group_norm.cl:1-76) at
    shapes that reach the clustered, the vector and the element-wise forms of the kernels."""
    rng = rng_for(1, 60 + sum(shape) + misalign)
    B, C = shape[:2]
    hw = int(np.prod(shape[2:]))
    x = (rng.standard_normal(shape) * 1.5 + 0.3).astype(np.float32).astype(NP_DTYPE[dtype])
    g = (1 + 0.1 * rng.standard_normal(C)).astype(np.float32)
    b = (0.1 * rng.standard_normal(C)).astype(np.float32)
    want, wmean, wvar = oracle.group_norm(x.astype(np.float32), g, b, groups, 1e-5, False, return_stats=True)
    src = Guarded(shape, getattr(torch, dtype), misalign=misalign)
    src.tensor.copy_(to_dev(x))
    mean = sdfl.ops.local_reduction_mean(src.tensor, B * groups)
    var = sdfl.ops.local_reduction_variance(src.tensor, mean, B * groups)
    assert_close(to_np(mean), wmean.reshape(-1), 1e-5, "group means")
    assert_close(to_np(var), wvar.reshape(-1), 1e-5, "group variances")
    out = Guarded(shape, getattr(torch, dtype), misalign=misalign)
    sdfl.ops.group_norm_apply(src.tensor, mean, var, to_dev(g), to_dev(b), group_size=(C // groups) * hw,
                              channel_size=hw, eps=1e-5, num_channels=C, out=out.tensor)
    out.check()
    assert_close(to_np(out.tensor), want, TOL[dtype], f"group_norm kernel {shape} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("rows,D,misalign", [(8192, 320, 0), (154, 768, 0), (33, 77, 0), (64, 320, 1)])
def test_layernorm_kernel_by_kernel_all_layouts(sdfl, rows, D, misalign, dtype):
    """local_reduction_mean -> local_reduction_variance -> layer_norm (layer_norm.cl:1-78)."""
    x, gamma, beta = ln_inputs(rng_for(2, 90 + rows + D + misalign), rows, D, dtype, mean=0.2, std=1.3)
    want, wmean, wvar = oracle.layer_norm(x.astype(np.float32), gamma, beta, 1e-5, return_stats=True)
    src = Guarded((rows, D), getattr(torch, dtype), misalign=misalign)
    src.tensor.copy_(to_dev(x))
    mean = sdfl.ops.local_reduction_mean(src.tensor, rows)
    var = sdfl.ops.local_reduction_variance(src.tensor, mean, rows)
    assert_close(to_np(mean), wmean.reshape(-1), 1e-5, "row means")
    assert_close(to_np(var), wvar.reshape(-1), 1e-5, "row variances")
    out = Guarded((rows, D), getattr(torch, dtype), misalign=misalign)
    sdfl.ops.layer_norm_apply(src.tensor, mean, var, to_dev(gamma), to_dev(beta), D, 1e-5, out=out.tensor)
    out.check()
    assert_close(to_np(out.tensor), want, TOL[dtype], f"layer_norm kernel [{rows},{D}] {dtype}")
