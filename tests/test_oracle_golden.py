"""The plain-C oracle against the golden vectors produced by the reference's own kernel
source (tests/golden/reference_kernels.npz, written by tests/golden/make_golden.py).
Bit equality: same operations in the same order, no contraction."""
import os

import numpy as np
import pytest

from conftest import assert_bit_equal

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def _names(golden, prefix):
    return sorted({k.split(".")[0] for k in golden.files if k.startswith(prefix)})


def test_golden_file_has_cases(golden):
    assert len(_names(golden, "gn_")) >= 4 and len(_names(golden, "ln_")) >= 3


def test_group_norm_matches_reference_kernels(golden, oracle_mod):
    for name in _names(golden, "gn_"):
        G, silu = (int(v) for v in golden[f"{name}.meta"])
        eps = float(golden[f"{name}.eps"][0])
        y, mean, var = oracle_mod.group_norm(golden[f"{name}.x"], golden[f"{name}.gamma"],
                                             golden[f"{name}.beta"], G, eps, bool(silu),
                                             return_stats=True)
        assert_bit_equal(mean, golden[f"{name}.mean"], f"{name} mean")
        assert_bit_equal(var, golden[f"{name}.var"], f"{name} var")
        assert_bit_equal(y, golden[f"{name}.y"], f"{name} y")


def test_layer_norm_matches_reference_kernels(golden, oracle_mod):
    for name in _names(golden, "ln_"):
        y, mean, var = oracle_mod.layer_norm(golden[f"{name}.x"], golden[f"{name}.gamma"],
                                             golden[f"{name}.beta"], 1e-5, return_stats=True)
        assert_bit_equal(mean, golden[f"{name}.mean"], f"{name} mean")
        assert_bit_equal(var, golden[f"{name}.var"], f"{name} var")
        assert_bit_equal(y, golden[f"{name}.y"], f"{name} y")


def test_geglu_and_activations_match_reference_kernels(golden, oracle_mod):
    assert_bit_equal(oracle_mod.gelu_multiply(golden["geglu_r5_d64.ab"]), golden["geglu_r5_d64.y"],
                     "gelu_multiply")
    x = golden["act.x"]
    assert_bit_equal(oracle_mod.silu(x), golden["act.silu"], "silu")
    assert_bit_equal(oracle_mod.gelu(x), golden["act.gelu"], "gelu")
    assert_bit_equal(oracle_mod.elemwise_add(x, golden["act.other"]), golden["act.add"], "add")
    assert_bit_equal(oracle_mod.chunkwise_add(golden["chunk.a"], golden["chunk.chunk"], 40),
                     golden["chunk.y"], "chunkwise_add")
    assert_bit_equal(oracle_mod.permute_021(golden["permute.x"]), golden["permute.y"], "permute3D__0_2_1")
    assert np.array_equal(golden["permute.y"], golden["permute.x"].transpose(0, 2, 1))
    assert_bit_equal(oracle_mod.up_sample_nearest(golden["upsample.x"], 2), golden["upsample.y"], "up_sample_nearest")
    assert np.array_equal(golden["upsample.y"], golden["upsample.x"].repeat(2, axis=1).repeat(2, axis=2))
    for name in ("softmax_r6_c77", "softmax_r3_c256"):
        assert_bit_equal(oracle_mod.softmax(golden[f"{name}.x"]), golden[f"{name}.y"], name)
        np.testing.assert_allclose(golden[f"{name}.y"].sum(-1), 1.0, rtol=1e-6)
    for name in ("local_softmax_h3_77", "local_softmax_r5_64"):
        assert_bit_equal(oracle_mod.local_softmax(golden[f"{name}.x"]), golden[f"{name}.y"], name)
        np.testing.assert_allclose(golden[f"{name}.y"].sum(-1), 1.0, rtol=1e-6)
    y = golden["local_softmax_h3_77.y"]
    assert np.all(y[:, np.triu_indices(77, 1)[0], np.triu_indices(77, 1)[1]] == 0.0)   # the causal mask
