"""GroupNorm(+SiLU) CUDA kernels against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from conftest import TOL, assert_close, rng_for
from gpu_util import Guarded, gn_inputs, oracle_group_norm, to_dev, to_np

import oracle

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz")


def run_gn(sdfl, x, gamma, beta, G, eps, silu, **kw):
    return to_np(sdfl.ops.groupnorm(to_dev(x), to_dev(gamma), to_dev(beta), G, eps, silu, **kw))


def test_golden_vectors_from_the_reference_kernels(sdfl):
    g = np.load(GOLDEN)
    for name in sorted({k.split(".")[0] for k in g.files if k.startswith("gn_")}):
        G, silu = (int(v) for v in g[f"{name}.meta"])
        eps = float(g[f"{name}.eps"][0])
        for path in (sdfl.ops.GN_AUTO, sdfl.ops.GN_SPLIT):
            got = run_gn(sdfl, g[f"{name}.x"], g[f"{name}.gamma"], g[f"{name}.beta"], G, eps,
                         bool(silu), path=path)
            assert_close(got, g[f"{name}.y"], 1e-5, f"{name} path {path}")


def test_config1_fp32_every_path_and_cluster_size(sdfl):
    x, gamma, beta = gn_inputs(rng_for(1, 0), (1, 320, 64, 64), "float32")
    want = oracle_group_norm(x, gamma, beta, 32, 1e-5, True)
    plan = sdfl.ops.groupnorm_plan(1, 320, 4096, 32, torch.float32)
    assert plan["path"] == sdfl.ops.GN_REGISTER and plan["cluster"] == 4 and plan["workspace"] == 0
    assert_close(run_gn(sdfl, x, gamma, beta, 32, 1e-5, True), want, 1e-5, "auto")
    for cluster in (1, 2, 3, 4, 5, 7, 8, 12, 16):
        try:
            got = run_gn(sdfl, x, gamma, beta, 32, 1e-5, True, path=sdfl.ops.GN_RESIDENT,
                         cluster_or_splits=cluster)
        except sdfl.SdflError as e:
            # a 16-CTA cluster is an opt-in size: the device may not be able to host one
            assert cluster > 8 and e.status == sdfl._capi.ERR_UNSUPPORTED
            continue
        assert_close(got, want, 1e-5, f"resident cluster {cluster}")
    for splits in (0, 1, 3, 8):
        got = run_gn(sdfl, x, gamma, beta, 32, 1e-5, True, path=sdfl.ops.GN_SPLIT,
                     cluster_or_splits=splits)
        assert_close(got, want, 1e-5, f"split {splits}")
    assert sdfl.ops.device_status() == 0


UNET_SHAPES = [(320, 64), (640, 32), (1280, 16), (1280, 8), (640, 64), (960, 64), (960, 32),
               (1280, 32), (1920, 32), (1920, 16), (2560, 16), (2560, 8)]


@pytest.mark.parametrize("C,H", UNET_SHAPES)
def test_config3_unet_sweep_fp16_batch2(sdfl, C, H):
    x, gamma, beta = gn_inputs(rng_for(3, UNET_SHAPES.index((C, H))), (2, C, H, H), "float16")
    want = oracle_group_norm(x, gamma, beta, 32, 1e-5, True)
    got = run_gn(sdfl, x, gamma, beta, 32, 1e-5, True)
    assert got.dtype == np.float16
    assert_close(got, want, TOL["float16"], f"{C}@{H}")


@pytest.mark.parametrize("C,H", [(320, 64), (1280, 8), (2560, 16)])
def test_unet_shapes_fp32_eps_and_no_silu(sdfl, C, H):
    x, gamma, beta = gn_inputs(rng_for(3, 100 + C + H), (2, C, H, H), "float32")
    for eps, silu in ((1e-5, True), (1e-6, False)):      # ResBlock norm / SpatialTransformer norm
        want = oracle_group_norm(x, gamma, beta, 32, eps, silu)
        assert_close(run_gn(sdfl, x, gamma, beta, 32, eps, silu), want, 1e-5, f"{C}@{H} {eps}")


@pytest.mark.parametrize("shape", [(2, 512, 64, 64), (1, 512, 128, 128), (1, 256, 256, 256),
                                   (1, 128, 512, 512)])
def test_config5_vae_shapes_fp16(sdfl, shape):
    x, gamma, beta = gn_inputs(rng_for(5, shape[1]), shape, "float16")
    want = oracle_group_norm(x, gamma, beta, 32, 1e-6, True)
    plan = sdfl.ops.groupnorm_plan(shape[0], shape[1], shape[2] * shape[3], 32, torch.float16)
    # 128 KB slabs fit one CTA's registers, 32 slabs of 512 KB a cluster of 8 CTAs' registers
    want_path = sdfl.ops.GN_REGISTER if shape[2] <= 128 else sdfl.ops.GN_RESIDENT
    assert plan["path"] == want_path, plan
    got = run_gn(sdfl, x, gamma, beta, 32, 1e-6, True)
    assert_close(got, want, TOL["float16"], f"{shape} automatic path {plan}")
    got = run_gn(sdfl, x, gamma, beta, 32, 1e-6, True, path=sdfl.ops.GN_RESIDENT)
    assert_close(got, want, TOL["float16"], f"{shape} cluster path")
    got = run_gn(sdfl, x, gamma, beta, 32, 1e-6, True, path=sdfl.ops.GN_SPLIT)
    assert_close(got, want, TOL["float16"], f"{shape} split")
    assert sdfl.ops.device_status() == 0


def test_vae_fp32_slab_larger_than_any_cluster_can_hold(sdfl):
    shape = (1, 128, 512, 512)                 # 4 MiB per group in fp32: cannot be shared-memory resident
    x, gamma, beta = gn_inputs(rng_for(5, 99), shape, "float32")
    want = oracle_group_norm(x, gamma, beta, 32, 1e-6, True)
    assert_close(run_gn(sdfl, x, gamma, beta, 32, 1e-6, True), want, 1e-5, "fp32 4 MiB slabs, auto")
    got = run_gn(sdfl, x, gamma, beta, 32, 1e-6, True, path=sdfl.ops.GN_SPLIT)
    assert_close(got, want, 1e-5, "fp32 4 MiB slabs, split path")
    assert sdfl.ops.groupnorm_plan(1, 128, 512 * 512, 32, torch.float32, sdfl.ops.GN_SPLIT)["workspace"] > 0


RAGGED = [((3, 6, 5, 7), 3), ((2, 12, 1, 1), 4), ((1, 4, 3, 3), 4), ((2, 10, 9, 11), 5),
          ((1, 8, 2, 2), 1), ((5, 32, 1, 3), 32), ((1, 64, 33, 31), 8)]


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape,G", RAGGED)
def test_ragged_shapes_the_reference_refuses(sdfl, shape, G, dtype):
    """Group sizes that are not multiples of 64 (the reference throws) or of the vector width."""
    x, gamma, beta = gn_inputs(rng_for(1, 200 + sum(shape)), shape, dtype)
    for silu in (False, True):
        want = oracle_group_norm(x, gamma, beta, G, 1e-5, silu)
        out = Guarded(shape, getattr(torch, dtype))
        sdfl.ops.groupnorm(to_dev(x), to_dev(gamma), to_dev(beta), G, 1e-5, silu, out=out.tensor)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"{shape} G={G} silu={silu}")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
def test_misaligned_buffers_and_guard_bands(sdfl, dtype):
    shape = (2, 64, 16, 16)
    x, gamma, beta = gn_inputs(rng_for(1, 300), shape, dtype)
    want = oracle_group_norm(x, gamma, beta, 32, 1e-5, True)
    for mis_in, mis_out in ((0, 0), (1, 0), (0, 3), (1, 1)):
        xin = Guarded(shape, getattr(torch, dtype), misalign=mis_in)
        xin.tensor.copy_(to_dev(x))
        out = Guarded(shape, getattr(torch, dtype), misalign=mis_out)
        sdfl.ops.groupnorm(xin.tensor, to_dev(gamma), to_dev(beta), 32, 1e-5, True, out=out.tensor)
        out.check()
        xin.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"misalign {mis_in},{mis_out}")


@pytest.mark.parametrize("path", [1, 2])
def test_in_place_as_the_reference_callers_do(sdfl, path):
    """forward(buf, buf): nn/ResBlock.cpp:222, UNetModel.cpp:1797, Decoder.cpp:523."""
    x, gamma, beta = gn_inputs(rng_for(1, 400), (2, 320, 32, 32), "float32")
    want = oracle_group_norm(x, gamma, beta, 32, 1e-5, True)
    buf = to_dev(x)
    sdfl.ops.groupnorm(buf, to_dev(gamma), to_dev(beta), 32, 1e-5, True, out=buf, path=path)
    assert_close(to_np(buf), want, 1e-5, f"in place path {path}")


def _group_norm_float64(x, gamma, beta, G, eps, silu):
    x = x.astype(np.float64)
    B, C = x.shape[:2]
    xs = x.reshape(B, G, -1)
    y = ((xs - xs.mean(-1, keepdims=True)) / np.sqrt(xs.var(-1, keepdims=True) + eps)).reshape(x.shape)
    y = y * gamma.astype(np.float64)[None, :, None, None] + beta.astype(np.float64)[None, :, None, None]
    return y / (1 + np.exp(-y)) if silu else y


def test_large_mean_small_spread(sdfl):
    """Statistics must not cancel: mean 10, std 0.5 (an fp32 mean of such data is good to ~1e-6, and
    the division by the spread doubles that).  Two anchors, both at the fp32 tolerance of 1e-5: a
    float64 evaluation, and the oracle; the oracle's own distance from float64 on this input is
    measured beside them (the reference's kernels, which the oracle equals bit for bit, sit at about
    0.12 x the bound: the reference is inside 1e-5 here as well)."""
    x, gamma, beta = gn_inputs(rng_for(1, 500), (2, 64, 32, 32), "float32", mean=10.0, std=0.5)
    exact = _group_norm_float64(x, gamma, beta, 32, 1e-5, True)
    want = oracle_group_norm(x, gamma, beta, 32, 1e-5, True)
    bound = 1e-5 + 1e-5 * np.abs(exact)
    ref_dist = float((np.abs(want - exact) / bound).max())
    assert ref_dist < 0.5, f"oracle vs float64: {ref_dist:.3f} x bound"
    for path in (sdfl.ops.GN_RESIDENT, sdfl.ops.GN_SPLIT, sdfl.ops.GN_REGISTER):
        got = run_gn(sdfl, x, gamma, beta, 32, 1e-5, True, path=path)
        assert_close(got, exact, 1e-5, f"offset data path {path} vs float64")
        assert_close(got, want, 1e-5, f"offset data path {path} vs oracle")
        d = float((np.abs(got - exact) / bound).max())
        print(f"path {path}: {d:.3f} x bound from float64 (oracle: {ref_dist:.3f})")
    got = to_np(sdfl.ops.groupnorm_multi([to_dev(x)], [to_dev(gamma)], [to_dev(beta)], 32, 1e-5, True)[0])
    assert_close(got, exact, 1e-5, "offset data, multi-tensor launch vs float64")
    assert_close(got, want, 1e-5, "offset data, multi-tensor launch vs oracle")


def test_batch_is_independent_runs_and_results_are_deterministic(sdfl):
    x, gamma, beta = gn_inputs(rng_for(5, 600), (4, 512, 32, 32), "float16")
    dx, dg, db = to_dev(x), to_dev(gamma), to_dev(beta)
    full = sdfl.ops.groupnorm(dx, dg, db, 32, 1e-6, True)
    again = sdfl.ops.groupnorm(dx, dg, db, 32, 1e-6, True)
    assert torch.equal(full, again)
    # with the same cluster size the per-slab arithmetic does not depend on the batch at all
    kw = dict(path=sdfl.ops.GN_RESIDENT, cluster_or_splits=4)
    full4 = sdfl.ops.groupnorm(dx, dg, db, 32, 1e-6, True, **kw)
    for n in range(4):
        one = sdfl.ops.groupnorm(dx[n:n + 1].contiguous(), dg, db, 32, 1e-6, True, **kw)
        assert torch.equal(one[0], full4[n])
        # and whatever plan a single image gets, the values agree within tolerance
        auto = sdfl.ops.groupnorm(dx[n:n + 1].contiguous(), dg, db, 32, 1e-6, True)
        assert_close(to_np(auto[0]), to_np(full[n]).astype(np.float32), TOL["float16"], f"image {n}")


def test_empty_batch_and_errors(sdfl):
    g = to_dev(np.ones(32, np.float32))
    out = sdfl.ops.groupnorm(torch.empty((0, 32, 8, 8), device="cuda"), g, g, 32)
    assert out.shape == (0, 32, 8, 8)
    x = torch.zeros((1, 30, 8, 8), device="cuda")
    with pytest.raises(sdfl.SdflError) as e:
        sdfl.ops.groupnorm(x, g, g, 32)
    assert e.value.status == sdfl._capi.ERR_INVALID_VALUE
    with pytest.raises(TypeError):
        sdfl.ops.groupnorm(torch.zeros((1, 32, 8, 8)), g, g, 32)       # host tensor: no fallback


def test_full_size_vae_tensor_properties(sdfl):
    """[8,128,512,512] fp16 (1 GiB in, 1 GiB out): too big for the CPU oracle in a test, so
    check what must hold at any size: with gamma = 1, beta = 0 and no activation every
    (image, group) slab of the output has mean ~0 and variance ~1; image n of the batch equals
    the single-image run bit for bit; the SiLU variant equals silu() of the plain output."""
    B, C, H = 8, 128, 512
    gen = torch.Generator(device="cuda").manual_seed(5005)
    x = (torch.randn((B, C, H, H), device="cuda", generator=gen, dtype=torch.float32) * 1.5 + 0.5).half()
    ones = torch.ones(C, device="cuda")
    zeros = torch.zeros(C, device="cuda")
    y = sdfl.ops.groupnorm(x, ones, zeros, 32, 1e-6, False)
    mean = sdfl.ops.local_reduction_mean(y, B * 32)
    var = sdfl.ops.local_reduction_variance(y, mean, B * 32)
    assert float(mean.abs().max()) < 2e-3
    assert float((var - 1).abs().max()) < 5e-3
    one = sdfl.ops.groupnorm(x[3:4].contiguous(), ones, zeros, 32, 1e-6, False)
    d = (one[0].float() - y[3].float()).abs()          # other cluster size, same values
    assert float((d - 2e-3 * y[3].float().abs()).max()) <= 2e-3
    del one, d
    ys = sdfl.ops.groupnorm(x, ones, zeros, 32, 1e-6, True)
    ref = sdfl.ops.silu(y)
    diff = (ys.float() - ref.float()).abs()
    assert float((diff - 2e-3 * ref.float().abs()).max()) <= 2e-3
    assert sdfl.ops.device_status() == 0


def oracle_bias_group_norm(x, e, gamma, beta, G, eps, silu):
    """Reference sequence on one image at a time: chunkwise_add (util.cl:136-148) with
    chunk_size = H*W, then GroupNorm::forward, then silu; fp32 throughout."""
    B, C = x.shape[:2]
    hw = int(np.prod(x.shape[2:]))
    xs = np.stack([oracle.chunkwise_add(x[n].astype(np.float32), e[n].astype(np.float32), hw)
                   for n in range(B)])
    return oracle.group_norm(xs, gamma, beta, G, eps, silu)


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape,G", [((2, 320, 64, 64), 32), ((2, 1280, 8, 8), 32), ((2, 640, 32, 32), 32),
                                     ((1, 128, 256, 256), 32), ((3, 6, 5, 7), 3), ((2, 64, 33, 31), 8)])
def test_time_embedding_add_fused_into_the_norm(sdfl, shape, G, dtype):
    """chunkwise_add -> out_group_norm -> silu of a ResBlock (nn/ResBlock.cpp:188-231) as one call."""
    rng = rng_for(3, 700 + sum(shape))
    x, gamma, beta = gn_inputs(rng, shape, dtype)
    e = (rng.standard_normal(shape[:2]) * 0.8).astype(np.float32).astype(x.dtype)
    for silu in (True, False):
        want = oracle_bias_group_norm(x, e, gamma, beta, G, 1e-5, silu)
        out = Guarded(shape, getattr(torch, dtype))
        sdfl.ops.groupnorm_bias(to_dev(x), to_dev(e), to_dev(gamma), to_dev(beta), G, 1e-5, silu,
                                out=out.tensor)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"bias GN {shape} silu={silu}")
    # the stand-alone kernel with the reference's name and argument order
    hw = int(np.prod(shape[2:]))
    got = sdfl.ops.chunkwise_add(to_dev(x[0]), to_dev(e[0]), hw)
    want = oracle.chunkwise_add(x[0].astype(np.float32), e[0].astype(np.float32), hw)
    if dtype == "float32":
        assert to_np(got).tobytes() == want.tobytes()
    else:
        assert to_np(got).tobytes() == want.astype(np.float16).tobytes()


def ring_knob(cluster, slots, chunk_kb, consumer_warps):
    """Encoding of sdfl_groupnorm_forward_ex's `cluster_or_splits` for the cluster path."""
    return cluster | (slots << 8) | (chunk_kb << 16) | (consumer_warps << 24)


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape,G,cluster,chunk_kb", [
    ((2, 64, 64, 64), 8, 2, 16),       # whole chunks inside one channel
    ((2, 64, 64, 64), 8, 4, 32),
    ((1, 128, 128, 128), 32, 8, 16),   # several chunks per share, last ones held between the passes
    ((2, 96, 40, 40), 8, 2, 16),       # chunks straddle channel ends: per-chunk fall-back to the loop
    ((1, 32, 96, 96), 4, 3, 32),       # odd cluster size, ragged last chunk
])
def test_unrolled_chunks_with_256_consumer_threads(sdfl, shape, G, cluster, chunk_kb, dtype):
    """The variants whose full chunks are a compile-time number of vectors per thread (8 consumer
    warps, 16 or 32 KB chunks), with and without the fused per-channel addend."""
    rng = rng_for(5, 900 + sum(shape) + cluster)
    x, gamma, beta = gn_inputs(rng, shape, dtype)
    e = (rng.standard_normal(shape[:2]) * 0.8).astype(np.float32).astype(x.dtype)
    knob = ring_knob(cluster, 3, chunk_kb, 8)
    kw = dict(path=sdfl.ops.GN_RESIDENT, cluster_or_splits=knob)
    plan = sdfl.ops.groupnorm_plan(shape[0], shape[1], shape[2] * shape[3], G, getattr(torch, dtype),
                                   sdfl.ops.GN_RESIDENT, knob)
    assert plan["threads"] == 288 and plan["cluster"] == cluster
    for silu in (True, False):
        want = oracle_group_norm(x, gamma, beta, G, 1e-5, silu)
        out = Guarded(shape, getattr(torch, dtype))
        sdfl.ops.groupnorm(to_dev(x), to_dev(gamma), to_dev(beta), G, 1e-5, silu, out=out.tensor, **kw)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"unrolled {shape} c={cluster} silu={silu}")
        want = oracle_bias_group_norm(x, e, gamma, beta, G, 1e-5, silu)
        out = Guarded(shape, getattr(torch, dtype))
        sdfl.ops.groupnorm_bias(to_dev(x), to_dev(e), to_dev(gamma), to_dev(beta), G, 1e-5, silu,
                                out=out.tensor, **kw)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"unrolled+bias {shape} c={cluster} silu={silu}")
    assert sdfl.ops.device_status() == 0


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape,G", [
    ((2, 320, 64, 64), 32), ((2, 1280, 8, 8), 32), ((2, 640, 32, 32), 32), ((2, 1920, 16, 16), 32),
    ((1, 960, 32, 32), 32),
    ((3, 12, 6, 6), 3),        # 4-channel groups of 36 elements: vectors straddle channels
    ((2, 8, 2, 2), 2),         # one vector per slab (fp32) / half a vector's worth of threads
    ((40, 64, 8, 8), 32),      # more slabs than CTAs in a wave
])
def test_register_path_one_cta_per_slab(sdfl, shape, G, dtype):
    """Slabs up to 192 KB held in one CTA's registers: same results as the oracle, with and
    without the fused per-channel addend, also in place."""
    rng = rng_for(6, 1100 + sum(shape))
    x, gamma, beta = gn_inputs(rng, shape, dtype)
    e = (rng.standard_normal(shape[:2]) * 0.8).astype(np.float32).astype(x.dtype)
    kw = dict(path=sdfl.ops.GN_REGISTER)
    plan = sdfl.ops.groupnorm_plan(shape[0], shape[1], shape[2] * shape[3], G, getattr(torch, dtype),
                                   sdfl.ops.GN_REGISTER, 0)
    assert plan["path"] == sdfl.ops.GN_REGISTER
    for silu in (True, False):
        want = oracle_group_norm(x, gamma, beta, G, 1e-5, silu)
        out = Guarded(shape, getattr(torch, dtype))
        sdfl.ops.groupnorm(to_dev(x), to_dev(gamma), to_dev(beta), G, 1e-5, silu, out=out.tensor, **kw)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"register {shape} silu={silu}")
        buf = to_dev(x)
        sdfl.ops.groupnorm(buf, to_dev(gamma), to_dev(beta), G, 1e-5, silu, out=buf, **kw)
        assert_close(to_np(buf), want, TOL[dtype], f"register in place {shape} silu={silu}")
        want = oracle_bias_group_norm(x, e, gamma, beta, G, 1e-5, silu)
        out = Guarded(shape, getattr(torch, dtype))
        sdfl.ops.groupnorm_bias(to_dev(x), to_dev(e), to_dev(gamma), to_dev(beta), G, 1e-5, silu,
                                out=out.tensor, **kw)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"register+bias {shape} silu={silu}")


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape,G", [
    ((2, 640, 64, 64), 32),    # 64 slabs of 160 KB (fp16): the automatic plan's cluster of 4
    ((1, 512, 64, 64), 32),    # 32 slabs of 128 KB (fp16)
    ((2, 96, 20, 20), 32),     # 150 vectors (fp16) per slab: shares of 19 vectors, the last CTA short
    ((3, 12, 6, 6), 3),        # vectors straddle channels; fewer vectors than CTAs x threads
    ((2, 8, 2, 2), 2),         # one or two vectors per slab: most CTAs of the cluster hold nothing
    ((40, 64, 8, 8), 32),      # more slabs than clusters in a wave
    ((80, 64, 8, 8), 32),      # 2560 slabs: more than the persistent grid has clusters, so clusters take a second slab
])
def test_register_path_cluster_per_slab(sdfl, shape, G, dtype):
    """A thread-block cluster of 2, 4 or 8 CTAs per slab, each CTA's share in its registers and the
    moments exchanged through distributed shared memory: same results as the oracle, with and
    without the fused per-channel addend, also in place."""
    rng = rng_for(6, 1500 + sum(shape))
    x, gamma, beta = gn_inputs(rng, shape, dtype)
    e = (rng.standard_normal(shape[:2]) * 0.8).astype(np.float32).astype(x.dtype)
    want = oracle_group_norm(x, gamma, beta, G, 1e-5, True)
    want_bias = oracle_bias_group_norm(x, e, gamma, beta, G, 1e-5, False)
    for cluster in (2, 4, 8):
        kw = dict(path=sdfl.ops.GN_REGISTER, cluster_or_splits=cluster)
        plan = sdfl.ops.groupnorm_plan(shape[0], shape[1], shape[2] * shape[3], G, getattr(torch, dtype),
                                       sdfl.ops.GN_REGISTER, cluster)
        assert plan["path"] == sdfl.ops.GN_REGISTER and plan["cluster"] == cluster
        out = Guarded(shape, getattr(torch, dtype))
        sdfl.ops.groupnorm(to_dev(x), to_dev(gamma), to_dev(beta), G, 1e-5, True, out=out.tensor, **kw)
        out.check()
        assert_close(to_np(out.tensor), want, TOL[dtype], f"register cluster {cluster} {shape}")
        buf = to_dev(x)
        sdfl.ops.groupnorm(buf, to_dev(gamma), to_dev(beta), G, 1e-5, True, out=buf, **kw)
        assert_close(to_np(buf), want, TOL[dtype], f"register cluster {cluster} in place {shape}")
        out = Guarded(shape, getattr(torch, dtype))
        sdfl.ops.groupnorm_bias(to_dev(x), to_dev(e), to_dev(gamma), to_dev(beta), G, 1e-5, False,
                                out=out.tensor, **kw)
        out.check()
        assert_close(to_np(out.tensor), want_bias, TOL[dtype], f"register cluster {cluster} + bias {shape}")
    assert sdfl.ops.device_status() == 0


def test_register_cluster_is_the_automatic_plan_for_few_medium_slabs(sdfl):
    """At most 64 slabs of 100-512 KB: a cluster per slab on the register path; results as the oracle's,
    also for the input given as two tensors to concatenate."""
    cases = [((2, 640, 64, 64), torch.float16, 4), ((2, 960, 64, 64), torch.float16, 4),
             ((1, 320, 64, 64), torch.float32, 4), ((1, 512, 128, 128), torch.float16, 8),
             ((2, 320, 64, 64), torch.float16, 1), ((8, 512, 64, 64), torch.float16, 1)]
    for shape, dt, cluster in cases:
        plan = sdfl.ops.groupnorm_plan(shape[0], shape[1], shape[2] * shape[3], 32, dt)
        assert plan["path"] == sdfl.ops.GN_REGISTER and plan["cluster"] == cluster, (shape, plan)
    # not a power of two, or beyond the portable cluster size: refused
    for bad in (3, 16):
        with pytest.raises(sdfl.SdflError):
            sdfl.ops.groupnorm_plan(2, 640, 4096, 32, torch.float16, sdfl.ops.GN_REGISTER, bad)
    rng = rng_for(6, 1601)
    a, gamma, beta = gn_inputs(rng, (2, 640, 64, 64), "float16")
    want = oracle_group_norm(a, gamma, beta, 32, 1e-5, True)
    got = sdfl.ops.groupnorm_concat(to_dev(a[:, :320]).contiguous(), to_dev(a[:, 320:]).contiguous(),
                                    to_dev(gamma), to_dev(beta), 32, 1e-5, True)
    assert_close(to_np(got), want, TOL["float16"], "concat, cluster of 4 per slab")
    assert sdfl.ops.device_status() == 0


def test_register_path_refuses_large_slabs(sdfl):
    x = torch.zeros((1, 32, 128, 128), device="cuda", dtype=torch.float32)     # 64 KB... per group 1 channel
    g, b = torch.ones(32, device="cuda"), torch.zeros(32, device="cuda")
    sdfl.ops.groupnorm(x, g, b, 32, 1e-5, False, path=sdfl.ops.GN_REGISTER)    # 64 KB slab: fine
    big = torch.zeros((1, 32, 256, 256), device="cuda", dtype=torch.float32)   # 256 KB slabs
    with pytest.raises(sdfl.SdflError):
        sdfl.ops.groupnorm(big, g, b, 32, 1e-5, False, path=sdfl.ops.GN_REGISTER)
