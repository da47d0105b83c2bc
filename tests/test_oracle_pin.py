"""Pins of the plain-C oracle beyond the golden file.

1. Against the reference's kernel source compiled as C++ (oracle/_ref), when that library is
   present: bit equality on the workload's own shapes.  Skipped where the reference is absent.
2. Against independent float64 numpy evaluations: a sanity bound (the reference kernels sit
   ~1e-6 from exact arithmetic), and the only check available for the pieces the reference has
   no compilable code for (embeddings, quick_gelu).
"""
import math

import numpy as np
import pytest

from conftest import assert_bit_equal, assert_close, rng_for

import oracle

needs_ref = pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference not built here")


def _gn_inputs(rng, B, C, H, W):
    x = rng.standard_normal((B, C, H, W)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(C)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(C)).astype(np.float32)
    return x, gamma, beta


@needs_ref
@pytest.mark.parametrize("C,H,eps,silu", [(320, 64, 1e-5, True), (640, 32, 1e-5, True),
                                          (1280, 8, 1e-6, False), (2560, 8, 1e-5, True),
                                          (512, 64, 1e-6, True)])
def test_port_equals_compiled_reference_group_norm(C, H, eps, silu):
    x, g, b = _gn_inputs(rng_for(1, C + H), 2, C, H, H)
    p = oracle.group_norm(x, g, b, 32, eps, silu, backend="port", return_stats=True)
    r = oracle.group_norm(x, g, b, 32, eps, silu, backend="ref", return_stats=True)
    for a, c, what in zip(p, r, ("y", "mean", "var")):
        assert_bit_equal(a, c, f"GN {C}@{H} {what}")


@needs_ref
@pytest.mark.parametrize("rows,D", [(154, 768), (77, 1024), (256, 320), (64, 1280)])
def test_port_equals_compiled_reference_layer_norm(rows, D):
    rng = rng_for(2, rows + D)
    x = (rng.standard_normal((rows, D)) * 1.3 + 0.2).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    b = (0.1 * rng.standard_normal(D)).astype(np.float32)
    p = oracle.layer_norm(x, g, b, 1e-5, backend="port", return_stats=True)
    r = oracle.layer_norm(x, g, b, 1e-5, backend="ref", return_stats=True)
    for a, c, what in zip(p, r, ("y", "mean", "var")):
        assert_bit_equal(a, c, f"LN {rows}x{D} {what}")


@needs_ref
def test_port_equals_compiled_reference_elementwise():
    rng = rng_for(4, 0)
    ab = (rng.standard_normal((64, 2 * 1280)) * 2).astype(np.float32)
    assert_bit_equal(oracle.gelu_multiply(ab, "port"), oracle.gelu_multiply(ab, "ref"), "geglu")
    x = (rng.standard_normal(77 * 3072) * 3).astype(np.float32)
    y = rng.standard_normal(77 * 3072).astype(np.float32)
    assert_bit_equal(oracle.silu(x, "port"), oracle.silu(x, "ref"), "silu")
    assert_bit_equal(oracle.gelu(x, "port"), oracle.gelu(x, "ref"), "gelu")
    assert_bit_equal(oracle.elemwise_add(x, y, "port"), oracle.elemwise_add(x, y, "ref"), "add")


@needs_ref
def test_reference_contract_checks_are_kept_by_the_compiled_reference():
    x, g, b = _gn_inputs(rng_for(1, 1), 1, 6, 5, 7)     # group size 70: not a multiple of 64
    with pytest.raises(ValueError):
        oracle.group_norm(x, g, b, 3, 1e-5, backend="ref")
    oracle.group_norm(x, g, b, 3, 1e-5, backend="port")    # the port defines the ragged case


def _gn_float64(x, gamma, beta, G, eps, silu):
    B, C = x.shape[:2]
    xd = x.astype(np.float64).reshape(B, G, -1)
    m = xd.mean(-1, keepdims=True)
    v = xd.var(-1, keepdims=True)
    y = ((xd - m) / np.sqrt(v + eps)).reshape(x.shape)
    shp = (1, C) + (1,) * (x.ndim - 2)
    y = y * gamma.astype(np.float64).reshape(shp) + beta.astype(np.float64).reshape(shp)
    return y / (1.0 + np.exp(-y)) if silu else y


@pytest.mark.parametrize("shape,G", [((1, 320, 64, 64), 32), ((2, 64, 8, 8), 32),
                                     ((3, 6, 5, 7), 3), ((1, 12, 1, 1), 4)])
def test_group_norm_against_float64(shape, G):
    x, g, b = _gn_inputs(rng_for(1, sum(shape)), *shape)
    for silu in (False, True):
        got = oracle.group_norm(x, g, b, G, 1e-5, silu)
        assert_close(got, _gn_float64(x, g, b, G, 1e-5, silu), 1e-5, f"GN {shape}")


def test_layer_norm_against_float64():
    rng = rng_for(2, 9)
    x = rng.standard_normal((154, 768)).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(768)).astype(np.float32)
    b = (0.1 * rng.standard_normal(768)).astype(np.float32)
    xd = x.astype(np.float64)
    want = (xd - xd.mean(-1, keepdims=True)) / np.sqrt(xd.var(-1, keepdims=True) + 1e-5) * g + b
    assert_close(oracle.layer_norm(x, g, b), want, 1e-5, "LN")


def test_activations_against_float64():
    x = (rng_for(2, 3).standard_normal(4096) * 3).astype(np.float32)
    xd = x.astype(np.float64)
    erf = np.vectorize(math.erf)
    assert_close(oracle.silu(x), xd / (1 + np.exp(-xd)), 1e-5, "silu")
    assert_close(oracle.quick_gelu(x), xd / (1 + np.exp(-1.702 * xd)), 1e-5, "quick_gelu")
    assert_close(oracle.gelu(x), xd * 0.5 * (1 + erf(xd / math.sqrt(2))), 1e-5, "gelu")
    ab = (rng_for(4, 3).standard_normal((8, 128)) * 2).astype(np.float32)
    a, gte = ab[:, :64].astype(np.float64), ab[:, 64:].astype(np.float64)
    assert_close(oracle.gelu_multiply(ab), a * (gte * 0.5 * (1 + erf(gte / math.sqrt(2)))), 1e-5,
                 "gelu_multiply")


def test_token_embedding_is_gather_plus_add():
    rng = rng_for(2, 0)
    table = (0.02 * rng.standard_normal((1000, 96))).astype(np.float32)
    pos = (0.02 * rng.standard_normal((77, 96))).astype(np.float32)
    ids = rng.integers(0, 1000, size=(2, 77), dtype=np.int64)
    got = oracle.token_embedding(ids, table, pos)
    assert_bit_equal(got, table[ids] + pos[None], "token embedding")
    ids[1, 5] = 1000
    with pytest.raises(IndexError):
        oracle.token_embedding(ids, table, pos)


def test_timestep_embedding_layout_and_values():
    t = np.array([0, 1, 981, 999], np.int64)
    got = oracle.timestep_embedding(t, 320)
    assert got.shape == (4, 320)
    assert np.all(got[0, :160] == 1.0) and np.all(got[0, 160:] == 0.0)     # cos | sin at t = 0
    i = np.arange(160, dtype=np.float64)
    freq = np.exp(-math.log(10000.0) * i / 160.0)
    # float32 rounding of freq moves the angle by up to ~6e-5 rad at t ~ 1000
    for row, tt in zip(got, t):
        assert np.abs(row[:160] - np.cos(tt * freq)).max() < 2e-4
        assert np.abs(row[160:] - np.sin(tt * freq)).max() < 2e-4


@needs_ref
def test_port_equals_compiled_reference_adjacent_kernels():
    """chunkwise_add, permute3D__0_2_1 and softmax: the kernels either side of the norms."""
    rng = rng_for(1, 4242)
    a = rng.standard_normal((320, 256)).astype(np.float32)
    e = rng.standard_normal(320).astype(np.float32)
    assert_bit_equal(oracle.chunkwise_add(a, e, 256, backend="port"),
                     oracle.chunkwise_add(a, e, 256, backend="ref"), "chunkwise_add")
    t3 = rng.standard_normal((2, 320, 64)).astype(np.float32)
    assert_bit_equal(oracle.permute_021(t3, backend="port"), oracle.permute_021(t3, backend="ref"), "permute")
    for rows, chunk in ((64, 77), (16, 4096), (40, 64), (8, 100)):
        x = (rng.standard_normal((rows, chunk)) * 3.0).astype(np.float32)
        assert_bit_equal(oracle.softmax(x, backend="port"), oracle.softmax(x, backend="ref"),
                         f"softmax {rows}x{chunk}")


@needs_ref
def test_port_equals_compiled_reference_local_softmax():
    """multi_head_attention.cl local_softmax: rows of 77 (the odd work-group size of the text encoder)
    with the causal mask, and a few other lengths for the carry logic of its reduction."""
    rng = rng_for(2, 4244)
    x = (rng.standard_normal((12, 77, 77)) * 3.0).astype(np.float32)
    x += np.triu(np.full((77, 77), -np.inf, np.float32), 1)
    assert_bit_equal(oracle.local_softmax(x, "port"), oracle.local_softmax(x, "ref"), "local_softmax 12x77x77 masked")
    for n in (1, 2, 3, 5, 6, 7, 64, 100, 255):
        x = (rng.standard_normal((9, n)) * 2.0).astype(np.float32)
        assert_bit_equal(oracle.local_softmax(x, "port"), oracle.local_softmax(x, "ref"), f"local_softmax rows of {n}")


def test_local_softmax_against_float64_and_softmax():
    rng = rng_for(2, 4245)
    x = (rng.standard_normal((8, 77, 77)) * 3.0).astype(np.float32)
    x += np.triu(np.full((77, 77), -np.inf, np.float32), 1)
    e = np.exp(x.astype(np.float64))
    want = (e / e.sum(-1, keepdims=True)).astype(np.float32)
    got = oracle.local_softmax(x)
    assert_close(got, want, 1e-5, "local_softmax vs float64")
    # the two reference softmax kernels compute the same function (different summation order)
    assert_close(got, oracle.softmax(x.reshape(-1, 77)).reshape(x.shape), 1e-5, "local_softmax vs softmax")


def test_softmax_against_float64():
    rng = rng_for(1, 4243)
    x = (rng.standard_normal((32, 77)) * 4.0).astype(np.float32)
    e = np.exp(x.astype(np.float64))
    assert_close(oracle.softmax(x), (e / e.sum(-1, keepdims=True)).astype(np.float32), 1e-5, "softmax vs float64")
