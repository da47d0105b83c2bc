"""The allocation-free GroupNorm entry point (sdfl_groupnorm_forward_noalloc), through the C ABI.

It exists for callers that must not allocate device memory after start-up (hosts that own all
device memory through their own pools, plugins inside them, latency-critical threads).  Its
scratch is a fixed array inside the library, shared by every call on a device and never
cleared, so the checks here are: same bits as the ordinary split-path entry point, on two calls
in a row with different data (stale scratch from the first call must not leak into the
second), and a clean refusal when the problem needs more scratch than the array holds.

This file is collected last on purpose: if it fails under `-x`, every other test has run.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import TOL, assert_close, rng_for
from gpu_util import gn_inputs, oracle_group_norm, to_dev, to_np

pytestmark = pytest.mark.gpu


def _call_noalloc(sdfl, x, gamma, beta, out, G, eps, silu):
    cap = sdfl._capi
    B, Cc = x.shape[0], x.shape[1]
    hw = x.numel() // (B * Cc)
    code = cap.F16 if x.dtype == torch.float16 else cap.F32
    return cap.lib.sdfl_groupnorm_forward_noalloc(
        x.data_ptr(), out.data_ptr(), gamma.data_ptr(), beta.data_ptr(), B, Cc, hw, G, eps,
        int(silu), code, torch.cuda.current_stream().cuda_stream)


def _call_split(sdfl, x, gamma, beta, out, G, eps, silu):
    """The existing entry point on the same device path, with a caller-allocated workspace."""
    cap = sdfl._capi
    B, Cc = x.shape[0], x.shape[1]
    hw = x.numel() // (B * Cc)
    code = cap.F16 if x.dtype == torch.float16 else cap.F32
    nbytes = cap.lib.sdfl_groupnorm_workspace_bytes_ex(B, Cc, hw, G, code, cap.GN_SPLIT, 0)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    return cap.lib.sdfl_groupnorm_forward_ex(
        x.data_ptr(), out.data_ptr(), gamma.data_ptr(), beta.data_ptr(), B, Cc, hw, G, eps,
        int(silu), code, ws.data_ptr(), ws.numel(), cap.GN_SPLIT, 0,
        torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", ["float16", "float32"])
def test_noalloc_matches_split_entry_point_twice_in_a_row(sdfl, dtype):
    shapes = [(2, 320, 64, 64), (3, 64, 33, 31)]          # second call: other data, other sizes
    for call, shape in enumerate(shapes):
        x, gamma, beta = gn_inputs(rng_for(1, 900 + call), shape, dtype)
        dx, dg, db = to_dev(x), to_dev(gamma), to_dev(beta)
        got = torch.empty_like(dx)
        want = torch.empty_like(dx)
        assert _call_noalloc(sdfl, dx, dg, db, got, 32 if call == 0 else 8, 1e-5, True) == 0
        assert _call_split(sdfl, dx, dg, db, want, 32 if call == 0 else 8, 1e-5, True) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: differs from the split-path entry point"
        ref = oracle_group_norm(x, gamma, beta, 32 if call == 0 else 8, 1e-5, True)
        assert_close(to_np(got), ref, TOL[dtype], f"call {call} vs oracle")


def test_noalloc_call_leaves_device_memory_as_it_found_it(sdfl):
    """What the entry point is for: with the output supplied by the caller, a call changes neither
    the device's free memory nor the bytes torch's allocator holds.  Measured around the second
    call, because the driver loads a kernel's code the first time it is launched."""
    x, gamma, beta = gn_inputs(rng_for(1, 905), (2, 320, 64, 64), "float16")
    dx, dg, db = to_dev(x), to_dev(gamma), to_dev(beta)
    out = torch.empty_like(dx)
    assert _call_noalloc(sdfl, dx, dg, db, out, 32, 1e-5, True) == 0
    torch.cuda.synchronize()
    free0, allocated0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    assert _call_noalloc(sdfl, dx, dg, db, out, 32, 1e-5, True) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert torch.cuda.memory_allocated() == allocated0 and torch.cuda.memory_reserved() == reserved0


def test_noalloc_in_place_and_wrapper(sdfl):
    x, gamma, beta = gn_inputs(rng_for(1, 910), (1, 128, 16, 16), "float32")
    buf = to_dev(x)
    sdfl.ops.groupnorm_noalloc(buf, to_dev(gamma), to_dev(beta), 32, 1e-6, False, out=buf)
    assert_close(to_np(buf), oracle_group_norm(x, gamma, beta, 32, 1e-6, False), 1e-5, "in place")


def test_noalloc_refuses_what_the_fixed_scratch_cannot_hold(sdfl):
    cap = sdfl._capi
    # 512 images x 32 groups = 16384 slabs -> 128 KiB of (mean, M2) pairs: over the 64 KiB array
    x = torch.zeros((512, 32, 2, 2), device="cuda")
    out = torch.full_like(x, 7.0)
    g = torch.ones(32, device="cuda")
    assert _call_noalloc(sdfl, x, g, g, out, 32, 1e-5, False) == cap.ERR_WORKSPACE
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()), "a refused call must not touch the output"
    assert _call_noalloc(sdfl, x, g, g, out, 5, 1e-5, False) == cap.ERR_INVALID_VALUE
    assert cap.lib.sdfl_groupnorm_forward_noalloc(None, out.data_ptr(), g.data_ptr(), g.data_ptr(),
                                                  1, 32, 4, 32, 1e-5, 0, 0, None) == cap.ERR_INVALID_POINTER
    _ = (C, np)
