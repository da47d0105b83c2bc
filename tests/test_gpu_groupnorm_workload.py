"""The benchmark's own launches against the oracle: SD VAE-decoder GroupNorm(32, eps 1e-6)+SiLU, fp16,
the four shapes at batch 8 and at the shard sizes of 2, 4 and 8 GPUs (4, 2, 1 images), through

  * sdfl_groupnorm_forward with the automatic plan (one launch per tensor), and
  * sdfl_groupnorm_forward_multi (the four tensors of a step in one launch).

Every image of every run is compared with the CPU oracle, one [1, C, H, W] image at a time so that
the host side stays small; an image's oracle result is computed once and reused for all runs that
contain the image.  Inputs follow the workload's seed convention (config 5).
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import TOL, rng_for
from gpu_util import to_dev

pytestmark = pytest.mark.gpu

SHAPES = [(512, 64), (512, 128), (256, 256), (128, 512)]      # (C, H = W)
BATCHES = (8, 4, 2, 1)                                         # 1, 2, 4, 8 GPUs
GROUPS, EPS = 32, 1e-6
# plan of the one-launch-per-tensor path at batch 8: path (3 register, 1 cluster ring), cluster size
BATCH8_PLAN = {(512, 64): (3, 1), (512, 128): (1, 2), (256, 256): (1, 4), (128, 512): (1, 8)}


def image(C, H, n):
    """Image n of the [8, C, H, H] tensor: x ~ N(0, 1) rounded to fp16."""
    rng = rng_for(5, 1000 * SHAPES.index((C, H)) + n)
    return rng.standard_normal((C, H, H), dtype=np.float32).astype(np.float16)


def weights(C, H):
    rng = rng_for(5, 900 + SHAPES.index((C, H)))
    return ((1 + 0.1 * rng.standard_normal(C)).astype(np.float32),
            (0.1 * rng.standard_normal(C)).astype(np.float32))


def worst_error(got: torch.Tensor, want: np.ndarray, tol: float) -> float:
    """max |got - want| / (tol + tol |want|), evaluated on the device."""
    w = torch.from_numpy(want).cuda()
    err = (got.float() - w).abs() / (tol + tol * w.abs())
    assert bool(torch.isfinite(got).all())
    return float(err.max())


def test_config5_every_image_of_every_shard_size(sdfl):
    ops = sdfl.ops
    tol = TOL["float16"]
    xs, gs, bs = [], [], []
    for C, H in SHAPES:
        xs.append(torch.stack([to_dev(image(C, H, n)) for n in range(8)]))
        g, b = weights(C, H)
        gs.append(to_dev(g))
        bs.append(to_dev(b))

    single, multi, plans = {}, {}, {}
    for B in BATCHES:
        shard = [x[:B] for x in xs]                # images 0 .. B-1: contiguous leading slices
        single[B] = [ops.groupnorm(x, g, b, GROUPS, EPS, True) for x, g, b in zip(shard, gs, bs)]
        plan = []
        multi[B] = ops.groupnorm_multi(shard, gs, bs, GROUPS, EPS, True, plan=plan)
        plans[B] = plan
        for (C, H), x in zip(SHAPES, shard):
            p = ops.groupnorm_plan(B, C, H * H, GROUPS, torch.float16)
            assert p["path"] in (ops.GN_RESIDENT, ops.GN_REGISTER), (B, C, H, p)
            if B == 8:
                assert (p["path"], p["cluster"]) == BATCH8_PLAN[(C, H)], (C, H, p)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    # the one-launch plan at batch 8: gangs of 8 CTAs on every CTA slot, a team size per tensor so that
    # a CTA's share of a slab is 256 KB (1, 2, 4, 8 CTAs per slab for the four shapes)
    assert plans[8][0] == 8 and plans[8][2] == 0x08040201, plans[8]

    report = {}
    for k, (C, H) in enumerate(SHAPES):
        g, b = gs[k].cpu().numpy(), bs[k].cpu().numpy()
        for n in range(8):
            want = oracle.group_norm(image(C, H, n).astype(np.float32)[None], g, b, GROUPS, EPS, True)[0]
            for B in BATCHES:
                if n >= B:
                    continue
                for name, runs in (("one launch per tensor", single), ("one launch per step", multi)):
                    e = worst_error(runs[B][k][n], want, tol)
                    assert e <= 1.0, f"[{B},{C},{H},{H}] image {n}, {name}: {e:.3f} x tolerance"
                    report[(name, B)] = max(report.get((name, B), 0.0), e)
    for key in sorted(report):
        print(f"{key[0]}, batch {key[1]}: worst {report[key]:.3f} x tolerance (2e-3)")


def test_multi_fp32_mixed_shapes_and_eps(sdfl):
    """Four fp32 tensors with different group counts, eps and sizes (one with a channel shorter than a
    chunk, one whose last item does not fill every team), no activation; in place for one of them."""
    ops = sdfl.ops
    specs = [((3, 64, 32, 32), 32, 1e-5), ((2, 320, 64, 64), 32, 1e-6), ((5, 96, 24, 24), 8, 1e-5),
             ((1, 128, 8, 8), 4, 1e-3)]
    xs, gs, bs, wants = [], [], [], []
    for k, (shape, G, eps) in enumerate(specs):
        rng = rng_for(1, 700 + k)
        x = (rng.standard_normal(shape) * (1 + k) + k).astype(np.float32)
        g = (1 + 0.1 * rng.standard_normal(shape[1])).astype(np.float32)
        b = (0.1 * rng.standard_normal(shape[1])).astype(np.float32)
        xs.append(to_dev(x)); gs.append(to_dev(g)); bs.append(to_dev(b))
        wants.append(oracle.group_norm(x, g, b, G, eps, False))
    outs = [torch.empty_like(x) for x in xs]
    outs[2] = xs[2]                                  # in place
    for knobs in (0, 8 | (2 << 8) | (1 << 14), 4 | (1 << 8) | (16 << 16), 2 | (2 << 8) | (1 << 11)):
        ins = [x.clone() for x in xs]
        o = [ins[2] if k == 2 else outs[k] for k in range(4)]
        plan = []
        ops.groupnorm_multi(ins, gs, bs, [s[1] for s in specs], [s[2] for s in specs], False, outs=o,
                            knobs=knobs, plan=plan)
        for k in range(4):
            e = worst_error(o[k], wants[k], 2e-5)
            assert e <= 1.0, f"tensor {k}, knobs {knobs:#x}, plan {plan}: {e:.3f} x (2e-5)"
    assert ops.device_status() == 0


@pytest.mark.parametrize("seed", range(12))
def test_multi_random_lists_and_plans(sdfl, seed):
    """Seeded random lists of 1-8 tensors (ragged batch / group / channel / pixel counts, both dtypes,
    with and without SiLU) under random plan knobs (gang size, team rule, static or dynamic order,
    reversed upper half, chunk size, ring slots): every tensor equals the oracle's result, whatever
    the deal of slabs to gangs and teams."""
    ops = sdfl.ops
    rng = rng_for(9, seed)
    dtype = "float16" if seed % 2 else "float32"
    vec = 8 if dtype == "float16" else 4
    n = int(rng.integers(1, 9))
    silu = bool(rng.integers(0, 2))
    xs, gs, bs, groups, epss, wants = [], [], [], [], [], []
    for k in range(n):
        G = int(rng.choice([1, 2, 3, 4, 8, 32]))
        cpg = int(rng.choice([1, 2, 3, 5, 8, 16]))
        B = int(rng.integers(1, 6))
        # hw a multiple of the vector, the slab at least 512 bytes (32 vectors); up to ~1 MB slabs
        hw = vec * int(rng.choice([4, 9, 32, 50, 128, 333, 1024, 4096]))
        while cpg * hw < 32 * vec:
            hw *= 2
        if B * G * cpg * hw > (1 << 21):
            B = 1
        shape = (B, G * cpg, hw)
        x = (rng.standard_normal(shape) * float(rng.uniform(0.5, 3)) + float(rng.uniform(-2, 2))).astype(np.float32)
        x = x.astype(np.float16) if dtype == "float16" else x
        g = (1 + 0.2 * rng.standard_normal(shape[1])).astype(np.float32)
        b = (0.2 * rng.standard_normal(shape[1])).astype(np.float32)
        eps = float(rng.choice([1e-6, 1e-5, 1e-3]))
        xs.append(to_dev(x)); gs.append(to_dev(g)); bs.append(to_dev(b)); groups.append(G); epss.append(eps)
        wants.append(oracle.group_norm(x.astype(np.float32), g, b, G, eps, silu))
    tol = TOL[dtype]
    for trial in range(4):
        K = int(rng.choice([0, 1, 2, 3, 4, 6, 8, 12, 16]))
        knobs = (K | (int(rng.integers(0, 3)) << 8) | (int(rng.integers(0, 2)) << 11) |
                 (int(rng.integers(0, 4)) << 12) | (int(rng.integers(0, 3)) << 14) |
                 (int(rng.choice([0, 16, 32])) << 16) | (int(rng.choice([0, 2, 3, 4])) << 24))
        if (knobs >> 16) & 0xff in (0, 32) and (knobs >> 24) & 0xf == 4:
            knobs &= ~(0xf << 24)                # 4 slots of 32 KB: larger than the ring may be
        outs = [torch.full_like(x, float("nan")) for x in xs]
        plan = []
        try:
            ops.groupnorm_multi(xs, gs, bs, groups, epss, silu, outs=outs, knobs=knobs, plan=plan)
        except sdfl.SdflError as e:
            # a forced gang size that no team rule can serve for these slabs is refused, not run
            assert e.status == sdfl._capi.ERR_UNSUPPORTED and K > 0, (seed, trial, hex(knobs), e)
            continue
        for k in range(n):
            e = worst_error(outs[k], wants[k], tol)
            assert e <= 1.0, (f"seed {seed} trial {trial} tensor {k} {tuple(xs[k].shape)} G={groups[k]} "
                              f"knobs {knobs:#x} plan {plan}: {e:.3f} x ({tol})")
    assert ops.device_status() == 0


def test_multi_repeated_launches_share_the_library_scratch(sdfl):
    """Back-to-back launches on one stream through the library's own scratch (workspace NULL) and
    through a caller's zero-filled workspace give the same bits every time."""
    cap = sdfl._capi
    lib = cap.lib
    import ctypes as C
    rng = rng_for(5, 800)
    x = to_dev(rng.standard_normal((2, 256, 64, 64), dtype=np.float32).astype(np.float16))
    g = to_dev((1 + 0.1 * rng.standard_normal(256)).astype(np.float32))
    b = to_dev((0.1 * rng.standard_normal(256)).astype(np.float32))
    arr = (cap.GnTensor * 1)()
    outs = []
    ws = torch.zeros(int(lib.sdfl_groupnorm_multi_workspace_bytes()), dtype=torch.uint8, device="cuda")
    for i in range(6):
        y = torch.empty_like(x)
        arr[0].in_, arr[0].out, arr[0].gamma, arr[0].beta = x.data_ptr(), y.data_ptr(), g.data_ptr(), b.data_ptr()
        arr[0].batch, arr[0].channels, arr[0].hw, arr[0].num_groups, arr[0].eps = 2, 256, 4096, 32, 1e-6
        wsp, wsn = (None, 0) if i % 2 == 0 else (ws.data_ptr(), ws.numel())
        rc = lib.sdfl_groupnorm_forward_multi(arr, 1, 1, cap.F16, wsp, wsn, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        outs.append(y)
    torch.cuda.synchronize()
    for y in outs[1:]:
        assert torch.equal(y, outs[0])
    want = oracle.group_norm(x.float().cpu().numpy(), g.cpu().numpy(), b.cpu().numpy(), 32, 1e-6, True)
    assert worst_error(outs[0], want, TOL["float16"]) <= 1.0
    assert sdfl.ops.device_status() == 0


def test_multi_refuses_what_it_cannot_run(sdfl):
    ops = sdfl.ops
    g = torch.ones(32, device="cuda")
    ok = torch.zeros((1, 32, 16, 16), device="cuda")
    odd = torch.zeros((1, 32, 3, 3), device="cuda")                 # hw * 4 bytes is not a multiple of 16
    with pytest.raises(sdfl.SdflError) as e:
        ops.groupnorm_multi([ok, odd], [g, g], [g, g], 32)
    assert e.value.status == sdfl._capi.ERR_UNSUPPORTED
    with pytest.raises(sdfl.SdflError) as e:
        ops.groupnorm_multi([ok, ok], [g, g], [g, g], 32, outs=[ok, ok])      # two tensors writing one buffer
    assert e.value.status == sdfl._capi.ERR_OVERLAP
    with pytest.raises(sdfl.SdflError) as e:
        ops.groupnorm_multi([ok] * 9, [g] * 9, [g] * 9, 32, outs=[torch.empty_like(ok) for _ in range(9)])
    assert e.value.status == sdfl._capi.ERR_UNSUPPORTED
    assert ops.groupnorm_multi([], [], [], 32) == []
