"""Token+position embedding gather (bit exact) and timestep embedding, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import TOL, assert_bit_equal, assert_close, rng_for
from gpu_util import Guarded, to_dev, to_np

import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("vocab,D,B,T", [(49408, 768, 2, 77), (49408, 1024, 1, 77), (1000, 100, 3, 5),
                                         (17, 3, 2, 4)])
def test_token_embedding_bit_exact_fp32(sdfl, vocab, D, B, T):
    rng = rng_for(2, D)
    table = (0.02 * rng.standard_normal((vocab, D))).astype(np.float32)
    pos = (0.02 * rng.standard_normal((T, D))).astype(np.float32)
    ids = rng.integers(0, vocab, size=(B, T), dtype=np.int64)
    ids[0, 0], ids[-1, -1] = 0, vocab - 1
    want = oracle.token_embedding(ids, table, pos)
    out = Guarded((B, T, D), torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sdfl.ops.token_embedding(to_dev(ids), to_dev(table), to_dev(pos), out=out.tensor, status=status)
    out.check()
    assert_bit_equal(to_np(out.tensor), want, f"gather {vocab}x{D}")
    assert int(status.item()) == 0


def test_token_embedding_bit_exact_fp16(sdfl):
    rng = rng_for(2, 16)
    table = (0.02 * rng.standard_normal((2048, 768))).astype(np.float16)
    pos = (0.02 * rng.standard_normal((77, 768))).astype(np.float16)
    ids = rng.integers(0, 2048, size=(2, 77), dtype=np.int64)
    want = oracle.to_half(oracle.token_embedding(ids, table.astype(np.float32), pos.astype(np.float32)))
    got = sdfl.ops.token_embedding(to_dev(ids), to_dev(table), to_dev(pos))
    assert_bit_equal(to_np(got), want, "fp16 gather")


def test_token_embedding_bad_ids_never_read_outside_the_table(sdfl):
    rng = rng_for(2, 17)
    table = rng.standard_normal((50, 64)).astype(np.float32)
    pos = rng.standard_normal((4, 64)).astype(np.float32)
    ids = np.array([[0, 49, 50, -1]], np.int64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = to_np(sdfl.ops.token_embedding(to_dev(ids), to_dev(table), to_dev(pos), status=status))
    assert int(status.item()) == 1
    assert_bit_equal(got[0, :2], (table[[0, 49]] + pos[:2]), "good rows")
    assert np.all(got[0, 2:] == 0.0)


@pytest.mark.parametrize("dim", [320, 64, 2, 7])
def test_timestep_embedding_matches_host_function(sdfl, dim):
    t = np.array([981, 0, 1, 999, 500, 17], np.int64)
    want = oracle.timestep_embedding(t, dim)
    got = sdfl.ops.timestep_embedding(to_dev(t), dim)
    assert_close(to_np(got), want, 1e-5, f"timestep dim {dim}")
    got16 = sdfl.ops.timestep_embedding(to_dev(t), dim, dtype=torch.float16)
    assert_close(to_np(got16), want, TOL["float16"], f"timestep fp16 dim {dim}")


def test_timestep_embedding_every_step_of_the_schedule(sdfl):
    t = np.arange(1000, dtype=np.int64)
    want = oracle.timestep_embedding(t, 320)
    got = to_np(sdfl.ops.timestep_embedding(to_dev(t), 320))
    assert_close(got, want, 1e-5, "t = 0..999")
    # layout [cos | sin] (UNetModel.cpp:1952-1953)
    assert np.all(got[0, :160] == 1.0) and np.all(got[0, 160:] == 0.0)


def test_config4_time_path_silu_on_the_1280_vector(sdfl):
    x = rng_for(4, 0).standard_normal((2, 1280)).astype(np.float16)
    want = oracle.silu(x.astype(np.float32))
    assert_close(to_np(sdfl.ops.silu(to_dev(x))), want, TOL["float16"], "silu [2,1280]")
