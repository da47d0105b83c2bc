"""The reference-shaped operator classes (constructor / init / forward), the host-buffer
pipeline, the launch counter, and sharded execution equivalence on one device."""
import numpy as np
import pytest
import torch

from conftest import TOL, assert_close, rng_for
from gpu_util import gn_inputs, oracle_group_norm, to_dev, to_np

import oracle

pytestmark = pytest.mark.gpu


def test_groupnorm_operator_trio(sdfl):
    x, gamma, beta = gn_inputs(rng_for(1, 0), (1, 320, 64, 64), "float32")
    op = sdfl.operators.GroupNorm(32, 320, 1e-5, gamma, beta, fuse_silu=True)
    with pytest.raises(RuntimeError):
        op.forward(to_dev(x), to_dev(x))                      # before init()
    op.init()
    op.init()                                                  # idempotent, GroupNorm.cpp:52-54
    buf = to_dev(x)
    assert op.forward(buf, buf) == 0                           # in place, ResBlock.cpp:222
    assert_close(to_np(buf), oracle_group_norm(x, gamma, beta, 32, 1e-5, True), 1e-5, "operator")
    with pytest.raises(RuntimeError, match="input_size % weight->num_vals != 0"):
        op.forward(torch.zeros((1, 64, 8, 8), device="cuda"), torch.zeros((1, 64, 8, 8), device="cuda"))
    bad = sdfl.operators.GroupNorm(32, 320, 1e-5, gamma, beta[:100])
    with pytest.raises(RuntimeError, match=r"weight.shape\[0\] != bias.shape\[0\]"):
        bad.init()
    bad = sdfl.operators.GroupNorm(32, 640, 1e-5, gamma, beta)
    with pytest.raises(RuntimeError, match=r"weight.shape\[0\] != weightSize"):
        bad.init()


def test_layernorm_and_geglu_operator_trio(sdfl):
    rng = rng_for(4, 7)
    x = rng.standard_normal((2, 64, 320)).astype(np.float16)
    gamma = (1 + 0.1 * rng.standard_normal(320)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(320)).astype(np.float32)
    ln = sdfl.operators.LayerNorm(320, gamma, beta)
    ln.init()
    out = torch.empty((2, 64, 320), dtype=torch.float16, device="cuda")
    assert ln.forward(to_dev(x), out) == 0
    assert_close(to_np(out), oracle.layer_norm(x.astype(np.float32), gamma, beta), TOL["float16"], "LN op")
    with pytest.raises(RuntimeError):
        sdfl.operators.LayerNorm(320, gamma, beta[:10]).init()

    ge = sdfl.operators.GEGLU(320, 1280)
    ge.init()
    assert ge.weightShape == [2560, 320]
    ab = (rng.standard_normal((2, 64, 2560))).astype(np.float16)
    out = torch.empty((2, 64, 1280), dtype=torch.float16, device="cuda")
    assert ge.forward(to_dev(ab), out) == 0
    assert_close(to_np(out), oracle.gelu_multiply(ab.astype(np.float32)), TOL["float16"], "GEGLU op")


def test_launch_counter_counts_one_launch_for_the_fused_path(sdfl):
    x, gamma, beta = gn_inputs(rng_for(1, 2), (2, 320, 32, 32), "float16")
    dx, dg, db = to_dev(x), to_dev(gamma), to_dev(beta)
    n0 = sdfl.ops.launch_count()
    sdfl.ops.groupnorm(dx, dg, db, 32, 1e-5, True, path=sdfl.ops.GN_RESIDENT)
    assert sdfl.ops.launch_count() - n0 == 1               # the reference needs 4 launches
    n0 = sdfl.ops.launch_count()
    sdfl.ops.groupnorm(dx, dg, db, 32, 1e-5, True, path=sdfl.ops.GN_SPLIT)
    assert sdfl.ops.launch_count() - n0 == 2


@pytest.mark.parametrize("dtype", ["float32", "float16"])
def test_host_pipeline_matches_device_path_and_oracle(sdfl, dtype):
    shape = (3, 64, 48, 48)
    x, gamma, beta = gn_inputs(rng_for(5, 3), shape, dtype)
    want = oracle_group_norm(x, gamma, beta, 32, 1e-6, True)
    h_x = torch.from_numpy(x).pin_memory()
    for slot_bytes, depth in ((1 << 20, 3), (20 << 10, 2), (64 << 20, 1)):
        pipe = sdfl.ops.HostPipeline(max_slot_bytes=slot_bytes, depth=depth)
        h_y = pipe.groupnorm(h_x, to_dev(gamma), to_dev(beta), 32, 1e-6, True)
        pipe.close()
        assert not h_y.is_cuda
        assert_close(h_y.numpy(), want, TOL[dtype], f"host pipeline slot {slot_bytes}")
    dev = sdfl.ops.groupnorm(to_dev(x), to_dev(gamma), to_dev(beta), 32, 1e-6, True)
    assert_close(h_y.numpy(), to_np(dev), TOL[dtype], "host vs device path")
    small = sdfl.ops.HostPipeline(max_slot_bytes=1024, depth=2)     # a group does not fit a slot
    with pytest.raises(sdfl.SdflError) as e:
        small.groupnorm(h_x, to_dev(gamma), to_dev(beta), 32, 1e-6, True)
    assert e.value.status == sdfl._capi.ERR_WORKSPACE
    small.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_pieces_reproduce_the_whole_tensor(sdfl, world):
    """What each rank of an N-GPU run computes (its pieces, as sub-tensor calls) put together
    equals the single-call result bit for bit -- the path has no cross-unit dependence."""
    B, C, H, G = 2, 64, 16, 32
    x, gamma, beta = gn_inputs(rng_for(3, world), (B, C, H, H), "float16")
    dx, dg, db = to_dev(x), to_dev(gamma), to_dev(beta)
    whole = sdfl.ops.groupnorm(dx, dg, db, G, 1e-5, True)
    out = torch.zeros_like(whole)
    cpg = C // G
    for rank in range(world):
        pieces = sdfl.sharding.groupnorm_pieces(B, G, world, rank)
        for first, n_img, g0, ng in sdfl.sharding.merge_whole_images(pieces, G):
            c0, c1 = g0 * cpg, (g0 + ng) * cpg
            sub = dx[first:first + n_img, c0:c1].contiguous()
            y = sdfl.ops.groupnorm(sub, dg[c0:c1].contiguous(), db[c0:c1].contiguous(), ng, 1e-5, True)
            out[first:first + n_img, c0:c1] = y
    assert torch.equal(out, whole)


def test_a_wait_that_cannot_be_satisfied_ends_by_itself_and_is_reported(sdfl):
    """Failure detection without a GPU fault: the kernels' waits are bounded.  A wait on a
    barrier that nothing completes gives up after its limit, the status word says so, and the
    device keeps working."""
    assert sdfl.ops.device_status(clear=True) == 0
    import time
    t0 = time.perf_counter()
    sdfl.ops.selftest_bounded_wait(2_000_000)            # ~1 ms at ~2 GHz
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert sdfl.ops.device_status(clear=True) & 1
    assert sdfl.ops.device_status(clear=False) == 0      # cleared
    x, gamma, beta = gn_inputs(rng_for(1, 77), (1, 64, 16, 16), "float32")
    got = sdfl.ops.groupnorm(to_dev(x), to_dev(gamma), to_dev(beta), 32, 1e-5, True)
    assert_close(to_np(got), oracle_group_norm(x, gamma, beta, 32, 1e-5, True), 1e-5, "after the time-out")
    assert sdfl.ops.device_status() == 0


def test_cpp_operator_classes_against_the_oracle():
    """include/sdfl_operators.hpp (the C++ mirror of the reference's GroupNorm / LayerNorm / GEGLU
    classes) and the C operator handles under it, compiled into tests/cpp/test_operators by
    tests/cpp/build.py (__graft_entry__.build() runs it)."""
    import os
    import subprocess
    exe = os.path.join(os.path.dirname(__file__), "cpp", "test_operators")
    if not os.path.exists(exe):
        pytest.skip("tests/cpp/test_operators not built (run __graft_entry__.build())")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr


def test_c_operator_handles_through_ctypes(sdfl):
    """sdfl_groupnorm_create / _op_forward / _destroy and the LayerNorm / GEGLU handles as a non-C++
    binder sees them; the results are those of the flat entry points."""
    import ctypes as C
    lib = sdfl._capi.lib
    s = torch.cuda.current_stream().cuda_stream
    x, gamma, beta = gn_inputs(rng_for(3, 900), (2, 320, 32, 32), "float16")
    dx, dg, db = to_dev(x), to_dev(gamma), to_dev(beta)
    op = C.c_void_p()
    assert lib.sdfl_groupnorm_create(C.byref(op), 32, 320, 1e-5, dg.data_ptr(), db.data_ptr(), 1, 2, 1024, 1) == 0
    y = torch.empty_like(dx)
    assert lib.sdfl_groupnorm_op_forward(op, dx.data_ptr(), y.data_ptr(), 2, 1024, 1, s) == 0
    assert_close(to_np(y), oracle_group_norm(x, gamma, beta, 32, 1e-5, True), TOL["float16"], "GroupNorm handle")
    assert torch.equal(y, sdfl.ops.groupnorm(dx, dg, db, 32, 1e-5, True))
    assert lib.sdfl_groupnorm_op_forward(None, dx.data_ptr(), y.data_ptr(), 2, 1024, 1, s) == sdfl._capi.ERR_INVALID_POINTER
    assert lib.sdfl_groupnorm_destroy(op) == 0

    rng = rng_for(2, 901)
    xl = rng.standard_normal((154, 768)).astype(np.float32)
    gl = (1 + 0.1 * rng.standard_normal(768)).astype(np.float32)
    bl = (0.1 * rng.standard_normal(768)).astype(np.float32)
    dgl, dbl, dxl = to_dev(gl), to_dev(bl), to_dev(xl)
    ln = C.c_void_p()
    assert lib.sdfl_layernorm_create(C.byref(ln), 768, 1e-5, dgl.data_ptr(), dbl.data_ptr()) == 0
    assert lib.sdfl_layernorm_op_forward(ln, dxl.data_ptr(), dxl.data_ptr(), 154, 0, s) == 0     # in place
    assert_close(to_np(dxl), oracle.layer_norm(xl, gl, bl), 1e-5, "LayerNorm handle")
    assert lib.sdfl_layernorm_destroy(ln) == 0

    ab = rng.standard_normal((64, 2560)).astype(np.float32)
    dab = to_dev(ab)
    out = torch.empty((64, 1280), device="cuda")
    ge = C.c_void_p()
    assert lib.sdfl_geglu_create(C.byref(ge), 320, 1280) == 0
    shape = (C.c_int64 * 2)()
    assert lib.sdfl_geglu_weight_shape(ge, shape) == 0 and list(shape) == [2560, 320]
    assert lib.sdfl_geglu_op_forward(ge, dab.data_ptr(), out.data_ptr(), 64, 0, s) == 0
    assert_close(to_np(out), oracle.gelu_multiply(ab), 1e-5, "GEGLU handle")
    assert lib.sdfl_geglu_destroy(ge) == 0


def test_host_pipeline_async_queue_of_tensors(sdfl):
    """Several tensors queued without waiting, one sync at the end (what bench.py's e2e leg does)."""
    pipe = sdfl.ops.HostPipeline(max_slot_bytes=256 << 10, depth=3)
    cases = []
    for i, shape in enumerate([(2, 64, 32, 32), (1, 128, 16, 16), (3, 32, 8, 8)]):
        x, gamma, beta = gn_inputs(rng_for(5, 40 + i), shape, "float16")
        h_x = torch.from_numpy(x).pin_memory()
        h_y = torch.empty_like(h_x).pin_memory()
        pipe.groupnorm(h_x, to_dev(gamma), to_dev(beta), 32, 1e-6, True, h_out=h_y, wait=False)
        cases.append((x, gamma, beta, h_x, h_y))
    pipe.sync()
    pipe.close()
    for x, gamma, beta, _, h_y in cases:
        assert_close(h_y.numpy(), oracle_group_norm(x, gamma, beta, 32, 1e-6, True), TOL["float16"], "queued")
