"""The C-ABI library loads on a machine without a GPU, exports every symbol include/sdfl.h
declares, and rejects bad arguments before touching CUDA.  No compute call is made here."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT, load_package

HEADER = os.path.join(ROOT, "include", "sdfl.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sdfl_[A-Za-z0-9_]+)\s*\(", text)))


def test_header_declares_the_reference_kernel_names():
    names = declared_symbols()
    for kernel in ("local_reduction_mean", "local_reduction_variance", "group_norm", "layer_norm",
                   "gelu_multiply", "gelu", "silu", "elemwise_add"):
        assert f"sdfl_{kernel}" in names
    assert len(names) >= 25


def test_library_exports_every_declared_symbol():
    pkg = load_package()
    lib = C.CDLL(pkg._capi.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in sdfl.h but not exported"
    assert set(pkg._capi.SIGNATURES) == set(declared_symbols())


def test_version_and_status_strings():
    lib = load_package()._capi.lib
    assert b"sm_100a" in lib.sdfl_version()
    assert lib.sdfl_status_string(0) == b"ok"
    assert lib.sdfl_status_string(-5) == b"input and output partially overlap"
    assert lib.sdfl_launch_count() >= 0


def test_argument_validation_needs_no_device():
    cap = load_package()._capi
    lib = cap.lib
    A, B = 4096, 8192                      # stand-in addresses: rejected before any use
    # channels not divisible by groups (the reference throws at nn/GroupNorm.cpp:83-87)
    assert lib.sdfl_groupnorm_forward(A, B, A, A, 1, 30, 64, 32, 1e-5, 1, 0, None, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_groupnorm_forward(A, B, A, A, 1, 32, 64, 32, 1e-5, 1, 7, None, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_groupnorm_forward(None, B, A, A, 1, 32, 64, 32, 1e-5, 1, 0, None, 0, None) == cap.ERR_INVALID_POINTER
    assert lib.sdfl_groupnorm_forward(A, A + 64, A, A, 1, 32, 64, 32, 1e-5, 1, 0, None, 0, None) == cap.ERR_OVERLAP
    assert lib.sdfl_groupnorm_forward(A, B, A, A, 0, 32, 64, 32, 1e-5, 1, 0, None, 0, None) == cap.OK   # empty batch
    assert lib.sdfl_layernorm_forward(A, B, A, A, 4, 0, 1e-5, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_layernorm_forward(A, None, A, A, 4, 64, 1e-5, 0, None) == cap.ERR_INVALID_POINTER
    assert lib.sdfl_layernorm_forward(A, B, A, A, 0, 64, 1e-5, 0, None) == cap.OK
    assert lib.sdfl_gelu_multiply(A, A + 16, 4, 64, 0, None) == cap.ERR_OVERLAP
    assert lib.sdfl_silu(A, A + 4, 64, 0, None) == cap.ERR_OVERLAP
    assert lib.sdfl_silu(A, A, 0, 0, None) == cap.OK
    assert lib.sdfl_silu(A, A, -1, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_elemwise_add(A, B, None, 8, 0, None) == cap.ERR_INVALID_POINTER
    assert lib.sdfl_token_embedding(A, A, A, B, 2, 77, 768, 0, 0, None, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_timestep_embedding(A, B, 2, 320, -1.0, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_local_reduction_mean(A, B, 4, 0, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_host_pipeline_create(None, 1024, 2) == cap.ERR_INVALID_POINTER
    # the kernels either side of the norms
    assert lib.sdfl_groupnorm_bias_forward(A, None, B, A, A, 1, 32, 64, 32, 1e-5, 1, 0, None, 0, None) == cap.ERR_INVALID_POINTER
    assert lib.sdfl_add_layernorm_forward(A, B, None, B, A, A, 4, 64, 1e-5, 0, None) == cap.ERR_INVALID_POINTER
    assert lib.sdfl_chunkwise_add(A, A, B, 64, 0, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_permute3D__0_2_1(A, A, 2, 4, 6, 0, None) == cap.ERR_OVERLAP          # a transpose cannot run in place
    assert lib.sdfl_permute3D__0_2_1(A, B, 0, 4, 6, 0, None) == cap.OK
    assert lib.sdfl_permute_add(A, None, B, 2, 4, 6, 0, None) == cap.ERR_INVALID_POINTER
    assert lib.sdfl_groupnorm_nhwc_forward(A, A, A, A, 1, 32, 64, 32, 1e-5, 0, 0, None, 0, None) == cap.ERR_OVERLAP
    assert lib.sdfl_softmax(A, B, -1, 77, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_softmax(A, A + 4, 8, 77, 0, None) == cap.ERR_OVERLAP
    assert lib.sdfl_softmax(A, A, 0, 77, 0, None) == cap.OK
    assert lib.sdfl_up_sample_nearest(A, B, 4, 8, 8, 0, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_up_sample_nearest(A, A, 4, 8, 8, 2, 0, None) == cap.ERR_OVERLAP
    assert lib.sdfl_concat_buffer(A, None, B, 1, 4, 4, 0, None) == cap.ERR_INVALID_POINTER
    assert lib.sdfl_groupnorm_concat_forward(A, 0, A, 32, B, A, A, 1, 64, 32, 1e-5, 1, 0, None, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_groupnorm_concat_forward(A, 16, None, 16, B, A, A, 1, 64, 32, 1e-5, 1, 0, None, 0, None) == cap.ERR_INVALID_POINTER


def test_workspace_query_and_plan_without_device():
    cap = load_package()._capi
    lib = cap.lib
    n = lib.sdfl_groupnorm_workspace_bytes(8, 128, 512 * 512, 32, 1)
    assert n > 0 and n % 8 == 0
    assert lib.sdfl_groupnorm_workspace_bytes(8, 130, 64, 32, 1) == 0     # invalid shape
    plan = (C.c_int64 * 8)()
    assert lib.sdfl_groupnorm_plan(2, 30, 64, 32, 0, 0, 0, plan) == cap.ERR_INVALID_VALUE


def test_forced_split_count_with_zero_low_bits_is_clamped():
    """cluster_or_splits = 65536 has no chunk count in its low 16 bits: one chunk, not a division by zero."""
    cap = load_package()._capi
    lib = cap.lib
    assert lib.sdfl_groupnorm_workspace_bytes_ex(2, 320, 4096, 32, 0, cap.GN_SPLIT, 65536) == 2 * 32 * 1 * 8
    plan = (C.c_int64 * 8)()
    assert lib.sdfl_groupnorm_plan(2, 320, 4096, 32, 0, cap.GN_SPLIT, 65536, plan) == cap.OK
    assert plan[0] == cap.GN_SPLIT and plan[3] == 1


def test_register_path_cluster_plan_without_a_device():
    """At most 64 slabs of 100-512 KB get a cluster of CTAs per slab on the register path; a forced
    cluster size must be a power of two up to 8."""
    cap = load_package()._capi
    lib = cap.lib
    plan = (C.c_int64 * 8)()
    for shape, dtype, want in [((2, 640, 4096), 1, 4), ((2, 960, 4096), 1, 4), ((1, 320, 4096), 0, 4),
                               ((1, 512, 16384), 1, 8), ((2, 320, 4096), 1, 1), ((8, 512, 4096), 1, 1)]:
        assert lib.sdfl_groupnorm_plan(*shape, 32, dtype, cap.GN_AUTO, 0, plan) == cap.OK
        assert (plan[0], plan[1], plan[5]) == (cap.GN_REGISTER, want, 0), (shape, list(plan))
    for forced in (2, 4, 8):
        assert lib.sdfl_groupnorm_plan(2, 640, 4096, 32, 1, cap.GN_REGISTER, forced, plan) == cap.OK
        assert plan[1] == forced and plan[6] == 64
    for forced in (3, 5, 16):
        assert lib.sdfl_groupnorm_plan(2, 640, 4096, 32, 1, cap.GN_REGISTER, forced, plan) == cap.ERR_UNSUPPORTED
    # a slab that fits the registers of 8 CTAs but not of one
    assert lib.sdfl_groupnorm_plan(1, 32, 256 * 256, 32, 0, cap.GN_REGISTER, 0, plan) == cap.ERR_UNSUPPORTED
    assert lib.sdfl_groupnorm_plan(1, 32, 256 * 256, 32, 0, cap.GN_REGISTER, 8, plan) == cap.OK


def test_multi_tensor_call_validates_without_a_device():
    cap = load_package()._capi
    lib = cap.lib
    assert lib.sdfl_groupnorm_multi_workspace_bytes() >= 4096
    A, B = 4096, 1 << 20
    arr = (cap.GnTensor * 2)()
    for k in range(2):
        arr[k].in_, arr[k].out, arr[k].gamma, arr[k].beta = A + k * (1 << 22), B + k * (1 << 22), A, A
        arr[k].batch, arr[k].channels, arr[k].hw, arr[k].num_groups, arr[k].eps = 1, 64, 256, 32, 1e-5
    assert lib.sdfl_groupnorm_forward_multi(None, 2, 1, 0, None, 0, None) == cap.ERR_INVALID_POINTER
    assert lib.sdfl_groupnorm_forward_multi(arr, 0, 1, 0, None, 0, None) == cap.OK
    assert lib.sdfl_groupnorm_forward_multi(arr, 2, 1, 5, None, 0, None) == cap.ERR_INVALID_VALUE
    assert lib.sdfl_groupnorm_forward_multi(arr, 2, 1, 0, A, 16, None) == cap.ERR_WORKSPACE
    arr[1].channels = 30                                    # not divisible by the groups
    assert lib.sdfl_groupnorm_forward_multi(arr, 2, 1, 0, None, 0, None) == cap.ERR_INVALID_VALUE
    arr[1].channels = 64
    arr[1].out = arr[0].out                                 # two tensors, one output buffer
    assert lib.sdfl_groupnorm_forward_multi(arr, 2, 1, 0, None, 0, None) == cap.ERR_OVERLAP
    arr[1].out = B + (1 << 22)
    arr[1].hw = 9                                           # 9 * 4 bytes: not a multiple of 16
    assert lib.sdfl_groupnorm_forward_multi(arr, 2, 1, 0, None, 0, None) == cap.ERR_UNSUPPORTED
    arr[1].batch = 0                                        # an empty tensor is skipped, the other one is valid
    arr[0].batch = 0
    assert lib.sdfl_groupnorm_forward_multi(arr, 2, 1, 0, None, 0, None) == cap.OK


def test_missing_library_is_a_loud_import_error(tmp_path):
    cap = load_package()._capi
    with pytest.raises(ImportError):
        cap.load(str(tmp_path / "libsdfl.so"))
