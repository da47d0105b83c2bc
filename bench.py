"""Benchmark of the fused-layer hot path on B200: achieved HBM GB/s of GroupNorm+SiLU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the scaling target is quoted on): SD VAE-decoder GroupNorm(32 groups,
eps 1e-6) + fused SiLU, fp16, batch 8, shapes [8,512,64,64], [8,512,128,128], [8,256,256,256],
[8,128,512,512]; x ~ N(0,1), gamma ~ N(1,0.1), beta ~ N(0,0.1), synthetic and seeded.  One step
= one pass over all four tensors (four kernel launches per GPU).  With N GPUs the batch is
split by image (8/N images per GPU), no inter-GPU traffic: total work is fixed ("strong").

Printed (rank 0, one JSON line): `value` = algorithmic bytes (2*N*2 + 2*C*4 per tensor) of all
ranks / device time of K steps (CUDA events, max over ranks), inputs resident in HBM; `e2e` =
same bytes / wall time through the host-buffer C-ABI call (pinned host tensors in and out,
H2D and D2H copies inside the timed region); `roofline` for the one kernel the step consists
of; `cpu_baseline` = the reference's kernels on this machine's host cores (N = 1 only).

--impl reference times the reference's own CPU implementation of the same workload
(oracle/_ref: its .cl kernel files compiled as C++, all host threads), each step a bounded
sample (one image of every shape).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fused GroupNorm+SiLU achieved HBM bandwidth (VAE decoder, fp16, batch 8)"
UNIT = "GB/s"
SHAPES = [(512, 64), (512, 128), (256, 256), (128, 512)]     # (C, H=W), batch 8 each
BATCH = 8
GROUPS = 32
EPS = 1e-6
L2_BYTES = 126 * 1024 * 1024
PEAK_FALLBACK_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the step's kernel divided by its
# algorithmic bytes, from an ncu capture of the same kernel on a smaller batch of the same four
# shapes (inputs larger than L2, within the size an ncu capture may have).  Traffic grows in
# proportion to the slabs processed, so the per-launch figure reported is this ratio times the
# launch's algorithmic bytes; None until a capture exists.
NCU_TRAFFIC_RATIO_MULTI = 0.934
NCU_TRAFFIC_SOURCE = ("ncu capture of the same kernel and plan on the 4-GPU shard of the step (batch 2, 486.55 MB: "
                      "268.3 MB read + 186.0 MB written), scaled by algorithmic bytes; measured for that launch only")


def algorithmic_bytes(batch: int, C: int, H: int, esz: int = 2) -> int:
    return 2 * batch * C * H * H * esz + 2 * C * 4


def measured_peak() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return PEAK_FALLBACK_GBS, "fallback"


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML while work runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch_device: int, period: float = 0.02):
        self.samples: list[tuple[float, int, int]] = []
        self.max_mhz = None
        self.period = period
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_device).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self._nv = pynvml
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception as e:      # no NVML: report that instead of clocks
            self.error = f"{type(e).__name__}: {e}"

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self, t0: float, t1: float, label: str) -> dict:
        if self._h is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": getattr(self, "error", "")}
        inside = [(m, r) for (t, m, r) in self.samples if t0 <= t <= t1]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0,
                    "window": label}
        bits = 0
        for _, r in inside:
            bits |= r
        reasons = [name for bit, name in self.REASONS.items() if bits & bit]
        return {"sm_mhz": statistics.median(m for m, _ in inside), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(inside), "window": label}


# ---------------------------------------------------------------------------------------------
# reference arm / cpu baseline
# ---------------------------------------------------------------------------------------------
def cpu_reference_step(oracle, data, backend: str) -> int:
    """One bounded sample of the workload on the host: the first `ng` groups of ONE image of
    every shape through the reference's call sequence (three GroupNorm launches, then silu).
    Returns the number of elements processed."""
    done = 0
    for x, gamma, beta, ng in data:
        oracle.group_norm(x, gamma, beta, ng, EPS, True, backend=backend)
        done += x.size
    return done


def cpu_reference_data(np, groups_used: int = GROUPS):
    """One image of each shape (its first `groups_used` of 32 groups), as the fp32 values an
    fp16 tensor holds: the reference computes in fp32 only."""
    rng = np.random.Generator(np.random.PCG64(5000))
    data = []
    for C, H in SHAPES:
        c_used = C // GROUPS * groups_used
        x = rng.standard_normal((1, c_used, H, H), dtype=np.float32).astype(np.float16).astype(np.float32)
        gamma = (1 + 0.1 * rng.standard_normal(c_used)).astype(np.float32)
        beta = (0.1 * rng.standard_normal(c_used)).astype(np.float32)
        data.append((x, gamma, beta, groups_used))
    return data


def time_cpu_reference(steps: int, warmup: int, budget_s: float, exact_steps: bool) -> dict:
    """Times the reference's CPU implementation.  With exact_steps the sample per step is
    shrunk (fewer groups per image) until `steps` steps fit the budget; otherwise full
    one-image samples are repeated until the budget is used."""
    import numpy as np
    import oracle
    backend = "ref" if oracle.have_ref() else "port"
    kind = "reference" if backend == "ref" else "port"
    # all the cores this process may run on, whatever OMP_NUM_THREADS says (torchrun exports 1)
    oracle.set_num_threads(len(os.sched_getaffinity(0)))
    cores = oracle.num_threads(backend)
    groups_used = GROUPS
    data = cpu_reference_data(np, groups_used)
    t0 = time.perf_counter()
    cpu_reference_step(oracle, data, backend)                 # warm-up and calibration
    t1 = time.perf_counter() - t0
    if exact_steps:
        while groups_used > 1 and t1 * (groups_used / GROUPS) * (steps + warmup) > budget_s:
            groups_used //= 2
        if groups_used != GROUPS:
            data = cpu_reference_data(np, groups_used)
    for _ in range(max(warmup - 1, 0) if groups_used == GROUPS else warmup):
        cpu_reference_step(oracle, data, backend)
    t0 = time.perf_counter()
    elems = 0
    done_steps = 0
    for _ in range(steps):
        elems += cpu_reference_step(oracle, data, backend)
        done_steps += 1
        if not exact_steps and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    # same metric as the GPU line: algorithmic bytes of the fp16 workload (2 B in + 2 B out per
    # element) per second
    gbs = elems * 4 / dt / 1e9
    return {"value": gbs, "unit": UNIT, "cores": cores, "kind": kind, "steps": done_steps,
            "ms_per_step": dt / done_steps * 1e3,
            "sample": (f"per step: groups 0..{groups_used - 1} of ONE image of each of the four shapes "
                       f"({elems // done_steps} elements = {groups_used}/{GROUPS * BATCH} of a workload "
                       f"step), fp32 arithmetic on fp16-rounded values, the reference's call sequence "
                       f"(3 GroupNorm launches + silu, 6 passes over the tensor), {cores} OpenMP "
                       f"threads; GB/s counts the fp16 workload's algorithmic bytes"),
            "opencl_cpu_runtime": probe_opencl()}


def probe_opencl() -> str:
    """Is an OpenCL CPU runtime (e.g. PoCL) installed?  Only asks the ICD loader for platforms."""
    import ctypes
    try:
        cl = ctypes.CDLL("libOpenCL.so.1")
    except OSError:
        return "unavailable on this box (no libOpenCL.so.1)"
    n = ctypes.c_uint(0)
    try:
        rc = cl.clGetPlatformIDs(0, None, ctypes.byref(n))
    except Exception as e:
        return f"unavailable on this box ({e})"
    if rc != 0 or n.value == 0:
        return "unavailable on this box (ICD loader reports no platform)"
    return f"{n.value} OpenCL platform(s) present (not used: kernels run as compiled C++)"


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = time_cpu_reference(args.steps, max(args.warmup, 1), budget_s=150.0, exact_steps=True)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": r["steps"], "warmup": max(args.warmup, 1),
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "SD VAE decoder GroupNorm(32, eps 1e-6)+SiLU, batch 8, four shapes "
                               "(bounded sample: one image of each shape per step)"},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "opencl_cpu_runtime": r["opencl_cpu_runtime"],
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(torch, local_rank: int) -> dict:
    """Pin this process to the CPUs of the NUMA node its GPU hangs off, so that the page-locked
    host buffers allocated afterwards (first touch) are local to the GPU's PCIe root.  Returns
    what was found; leaves the affinity alone when the topology cannot be read."""
    info = {"numa_node": None, "cpus": len(os.sched_getaffinity(0))}
    try:
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev = torch.cuda.get_device_properties(local_rank).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        node = int(open(path).read().strip())
        if node < 0:
            return info
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            info.update({"numa_node": node, "cpus": len(cpus)})
    except Exception as e:                      # no sysfs / no permission: report and carry on
        info["error"] = f"{type(e).__name__}: {e}"
    return info


def run_ours(args) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # convenience: relaunch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
               str(29500 + os.getpid() % 1000), os.path.abspath(__file__), *sys.argv[1:]]
        raise SystemExit(subprocess.call(cmd))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    pkg = importlib.import_module("mobile-stable-diffusion_b200")
    ops, sharding = pkg.ops, pkg.sharding

    lo, hi = sharding.partition(BATCH, world, rank)          # images of this rank
    b_local = hi - lo
    K, W = args.steps, max(args.warmup, 3)
    R = max(args.blocks, 1)

    # ring of buffer sets so that a buffer is reused only after > 4x L2 of other traffic
    step_bytes = sum(algorithmic_bytes(b_local, C, H) for C, H in SHAPES)
    ring = max(1, -(-4 * L2_BYTES // max(step_bytes, 1)))
    while K % ring != 0:             # a block of K steps walks the ring a whole number of times
        ring += 1
    gen = torch.Generator(device=dev).manual_seed(5000 + rank)
    sets = []
    for _ in range(ring):
        tensors = []
        for C, H in SHAPES:
            x = torch.randn((b_local, C, H, H), device=dev, generator=gen, dtype=torch.float32).half()
            gamma = 1 + 0.1 * torch.randn(C, device=dev, generator=gen)
            beta = 0.1 * torch.randn(C, device=dev, generator=gen)
            tensors.append((x, gamma, beta, torch.empty_like(x)))
        sets.append(tensors)

    multi_plan: list = []

    def step_multi(tensors):         # the step as ONE launch over its four tensors
        ops.groupnorm_multi([t[0] for t in tensors], [t[1] for t in tensors], [t[2] for t in tensors],
                            GROUPS, EPS, True, outs=[t[3] for t in tensors], plan=multi_plan)

    def step_chain(tensors):         # the step as four launches, one per tensor
        for x, gamma, beta, y in tensors:
            ops.groupnorm(x, gamma, beta, GROUPS, EPS, True, out=y)

    step = step_chain if args.chain else step_multi
    launches_per_step = len(SHAPES) if args.chain else 1
    stream = torch.cuda.Stream(device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def capture(fn):
        """One CUDA graph of a block: K steps back to back, step i on buffer set i mod ring."""
        for s in sets:                      # first calls: attribute set-up, plan cache, workspace
            fn(s)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(K):
                fn(sets[i % ring])
        return g

    def timed_blocks(graph, blocks):
        """`blocks` replays of the K-step graph, each between its own pair of events; returns the
        event pairs (this rank)."""
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(blocks)]
        for a, b in evs:
            a.record(stream)
            graph.replay()
            b.record(stream)
        return evs

    with torch.cuda.stream(stream):
        graphs = capture(step)
        for _ in range(-(-W // K)):         # at least W untimed steps
            graphs.replay()
        stream.synchronize()

        sampler = ClockSampler(local_rank, period=0.005)
        sampler.start()
        barrier()
        t_begin = time.perf_counter()
        evs = timed_blocks(graphs, R)
        barrier()
        t_end = time.perf_counter()
        block_ms = [a.elapsed_time(b) for a, b in evs]
        clocks = sampler.summary(t_begin, t_end, f"timed region ({R} blocks of {K} steps)")

        # the other way of launching the step, same buffers, outside the headline region
        other = step_multi if args.chain else step_chain
        other_graphs = capture(other)
        for _ in range(-(-W // K)):
            other_graphs.replay()
        barrier()
        other_evs = timed_blocks(other_graphs, min(R, 7))
        barrier()
        other_ms = [a.elapsed_time(b) for a, b in other_evs]
        del other_graphs

    def max_over_ranks(values):
        t = torch.tensor(values, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    block_ms = max_over_ranks(block_ms)              # a block is as slow as its slowest rank
    other_ms = max_over_ranks(other_ms)
    ms_med = statistics.median(block_ms)
    total_bytes = sum(algorithmic_bytes(BATCH, C, H) for C, H in SHAPES) if BATCH % world == 0 else None
    if total_bytes is None:
        tb = torch.tensor([step_bytes], device=dev, dtype=torch.float64)
        dist.all_reduce(tb)
        total_bytes = float(tb.item())
    to_gbs = lambda ms: total_bytes * K / (ms * 1e-3) / 1e9
    value = to_gbs(ms_med)

    # ---- parity of what was just timed: one image per shape of the step's own output vs the oracle ----
    parity = None
    if rank == 0 and not args.no_parity_check:
        import oracle
        with torch.cuda.stream(stream):
            graphs.replay()                  # the timed graph once more: its step 0 wrote sets[0]
            stream.synchronize()
        worst = 0.0
        for (C, H), (x, gamma, beta, y) in zip(SHAPES, sets[0]):
            want = oracle.group_norm(x[:1].float().cpu().numpy(), gamma.cpu().numpy(), beta.cpu().numpy(),
                                     GROUPS, EPS, True)
            got = y[:1].float().cpu().numpy().astype(np.float64)
            worst = max(worst, float((np.abs(got - want) / (2e-3 + 2e-3 * np.abs(want))).max()))
        parity = {"max_err_over_tol": round(worst, 4), "tolerance": 2e-3, "images": len(SHAPES),
                  "what": "image 0 of each of the four tensors as written by the timed step, against the "
                          "CPU oracle (the reference's kernels restated in C)"}

    # ---- per-shape device times of single launches (L2 flushed between launches; not the headline) ----
    per_shape = []
    with torch.cuda.stream(stream):
        flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
        reps = 5
        for (C, H), (x, gamma, beta, y) in zip(SHAPES, sets[0]):
            times = []
            for _ in range(reps):
                flush.fill_(1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                ops.groupnorm(x, gamma, beta, GROUPS, EPS, True, out=y)
                b.record(stream)
                stream.synchronize()
                times.append(a.elapsed_time(b))
            tmed = statistics.median(times)
            nbytes = algorithmic_bytes(b_local, C, H)
            plan = ops.groupnorm_plan(b_local, C, H * H, GROUPS, torch.float16)
            per_shape.append({"shape": [b_local, C, H, H], "us": round(tmed * 1e3, 2),
                              "gbs": round(nbytes / (tmed * 1e-3) / 1e9, 1),
                              "path": {1: "cluster ring", 2: "split", 3: "register"}.get(plan["path"], plan["path"]), "cluster": plan["cluster"],
                              "nclusters": plan["nclusters"], "threads": plan["threads"]})
        del flush

    # ---- end to end through the host-buffer C-ABI call ------------------------------------------
    numa = bind_to_gpu_numa_node(torch, local_rank)      # before the page-locked buffers are allocated
    e2e_steps = max(2, min(K, 5))
    pipe = ops.HostPipeline(max_slot_bytes=16 << 20, depth=6, device=local_rank)
    host = []
    for (C, H), (x, gamma, beta, y) in zip(SHAPES, sets[0]):
        h_in = torch.empty(x.shape, dtype=torch.float16, pin_memory=True)
        h_in.copy_(x)
        host.append((h_in, torch.empty(x.shape, dtype=torch.float16, pin_memory=True), gamma, beta))

    def e2e_step():
        for h_in, h_out, gamma, beta in host:            # queue the four tensors, then one wait
            pipe.groupnorm(h_in, gamma, beta, GROUPS, EPS, True, h_out=h_out, wait=False)
        pipe.sync()
        return float(host[-1][1][-1, -1, -1, -1])        # the step's result is read on the host

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    # copies alone (same buffers, same slots' worth of bytes, both directions at once): what PCIe and
    # the host memory give this rank while all ranks copy together
    copy_streams = [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)]
    d_stage = [torch.empty_like(sets[0][k][0]) for k in range(len(SHAPES))]
    barrier()
    t0 = time.perf_counter()
    for _ in range(2):
        with torch.cuda.stream(copy_streams[0]):
            for k, (h_in, _, _, _) in enumerate(host):
                d_stage[k].copy_(h_in, non_blocking=True)
        with torch.cuda.stream(copy_streams[1]):
            for k, (_, h_out, _, _) in enumerate(host):
                h_out.copy_(sets[0][k][3], non_blocking=True)
        torch.cuda.synchronize(dev)
    copy_s = (time.perf_counter() - t0) / 2
    del d_stage
    te = max_over_ranks([e2e_s, copy_s])
    e2e_value = total_bytes * e2e_steps / te[0] / 1e9
    # the host path runs groups in smaller calls (other plans): same values within fp16 tolerance
    with torch.cuda.stream(stream):
        step(sets[0])
        stream.synchronize()
    e2e_step()
    ok = all(bool(((h_out.to(dev).float() - t[3].float()).abs() - 2e-3 * t[3].float().abs()).max() <= 2e-3)
             for (_, h_out, _, _), t in zip(host, sets[0]))
    pipe.close()
    half_bytes = sum(b_local * C * H * H * 2 for C, H in SHAPES)
    hb = torch.tensor([half_bytes], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(hb)
    sampler.stop()

    if rank == 0:
        peak, peak_kind = measured_peak()
        per_gpu = value / world
        if args.chain:
            kernel = ("gn_resident_kernel<__half, silu> / gn_register_kernel (one launch per tensor): " +
                      ", ".join(f"[{p['shape'][0]},{p['shape'][1]},{p['shape'][2]},{p['shape'][3]}] {p['path']}"
                                + (f" cluster {p['cluster']} x {p['nclusters']}"
                                   if p["path"] == "cluster ring" or p["cluster"] > 1 else "")
                                for p in per_shape))
        else:
            teams = [(multi_plan[2] >> (8 * k)) & 0xff for k in range(len(SHAPES))] if multi_plan else []
            kernel = (f"gn_multi_kernel<__half, silu, 8 vectors/thread> (the step's one launch): {multi_plan[1]} CTAs "
                      f"in gangs of {multi_plan[0]}, CTAs per slab {teams} for the four tensors")
        # DRAM traffic per launch: from the ncu capture of the same kernel on the 4-image shard
        # (profiles/), scaled by the algorithmic bytes; only the plan of that capture is measured
        traffic_ratio = None if args.chain else NCU_TRAFFIC_RATIO_MULTI
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": round(ms_med / K, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 arithmetic on f16 storage",
            "data": "synthetic",
            "config": {"workload": "SD VAE decoder GroupNorm(32, eps 1e-6)+SiLU fp16, batch 8: "
                                   "[8,512,64,64] [8,512,128,128] [8,256,256,256] [8,128,512,512]",
                       "sharding": f"{BATCH // world if BATCH % world == 0 else 'ragged'} images per GPU, no collective",
                       "l2": f"in+out per step per GPU {step_bytes / 1e6:.0f} MB, ring of {ring} buffer "
                             f"set(s): a buffer is reused after >= {ring * step_bytes / 1e6:.0f} MB of other traffic (L2 126 MB)",
                       "launch": f"one CUDA graph per block of {K} steps ({K * launches_per_step} kernel nodes)"},
            "timing": {"blocks": R, "steps_per_block": K,
                       "block_ms": {"min": round(min(block_ms), 4), "median": round(ms_med, 4), "max": round(max(block_ms), 4)},
                       "how": "every block (one replay of the K-step graph) between its own CUDA events on the launching stream, "
                              "max over ranks per block, median over blocks; value and ms_per_step are the median block's"},
            "elements_per_s": round(value * 1e9 / 4, 0),
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "steps": e2e_steps,
                    "h2d_bytes_per_step": int(hb.item()), "d2h_bytes_per_step": int(hb.item()),
                    "matches_device_path": bool(ok), "host_numa": numa,
                    "copies_alone": {"gbs_both_directions": round(2 * hb.item() / te[1] / 1e9, 2),
                                     "what": "the same bytes copied in and out at once with no kernel, all ranks "
                                             "together (max over ranks): the ceiling PCIe and host memory set"}},
            "gpu_launches": K * R * launches_per_step * world,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": kernel,
                         "achieved": round(per_gpu, 1), "peak": peak, "unit": UNIT,
                         "frac": round(per_gpu / peak, 4), "peak_source": f"of {peak_kind}",
                         "traffic": None if traffic_ratio is None else round(traffic_ratio * step_bytes / launches_per_step),
                         "traffic_source": None if traffic_ratio is None else NCU_TRAFFIC_SOURCE,
                         "per_gpu": True},
            "other_launch_form": {"what": "one launch per step (gn_multi_kernel)" if args.chain else
                                          "four launches per step, one per tensor (cluster ring / register kernels)",
                                  "value": round(to_gbs(statistics.median(other_ms)), 2), "unit": UNIT,
                                  "ms_per_step": round(statistics.median(other_ms) / K, 5)},
            "per_shape_single_launch": per_shape,
        }
        if parity is not None:
            line["parity_check"] = parity
        if world == 1 and not args.no_cpu_baseline:
            r = time_cpu_reference(steps=1000, warmup=1, budget_s=12.0, exact_steps=False)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
            line["cpu_baseline"]["opencl_cpu_runtime"] = r["opencl_cpu_runtime"]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# per-kernel table (--ops) and single cases for profiling (--case NAME)
# ---------------------------------------------------------------------------------------------
def op_cases(torch, ops, dev):
    """Every kernel of the path at the shapes of the five named workload configurations.
    Each case: name, algorithmic bytes, a factory and a spec for the CPU leg.  The factory
    allocates one set of buffers and returns a closure that enqueues one launch on them, so
    the caller can build a ring of buffer sets larger than L2."""
    gen = torch.Generator(device=dev).manual_seed(1234)

    def rnd(shape, dtype, scale=1.0):
        return (torch.randn(shape, device=dev, generator=gen) * scale).to(dtype)

    f16, f32 = torch.float16, torch.float32
    cases = []

    def gn(name, B, C, H, dtype, eps):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((B, C, H, H), dtype)
            y = torch.empty_like(x)
            g, b = 1 + 0.1 * rnd((C,), f32), 0.1 * rnd((C,), f32)
            return lambda: ops.groupnorm(x, g, b, 32, eps, True, out=y)
        cases.append((name, 2 * B * C * H * H * esz + 2 * C * 4, make, ("gn", B, C, H, eps)))

    gn("cfg1 GN+SiLU f32 [1,320,64,64]", 1, 320, 64, f32, 1e-5)
    for C, H in [(320, 64), (640, 32), (1280, 16), (1280, 8), (640, 64), (960, 64), (960, 32),
                 (1280, 32), (1920, 32), (1920, 16), (2560, 16), (2560, 8)]:
        gn(f"cfg3 GN+SiLU f16 [2,{C},{H},{H}]", 2, C, H, f16, 1e-5)
    for C, H in SHAPES:
        gn(f"cfg5 GN+SiLU f16 [8,{C},{H},{H}]", 8, C, H, f16, 1e-6)
    for C, H in SHAPES:
        gn(f"cfg5 GN+SiLU f16 [1,{C},{H},{H}] (8-GPU shard)", 1, C, H, f16, 1e-6)
    gn("profiling size GN+SiLU f16 [4,128,512,512]", 4, 128, 512, f16, 1e-6)
    gn("GN+SiLU f32 [8,256,256,256]", 8, 256, 256, f32, 1e-6)

    def gn_step(name, B):
        """The benchmark's step (the four VAE tensors) as ONE launch, at the shard size of 8 / B GPUs."""
        def make():
            xs = [rnd((B, C, H, H), f16) for C, H in SHAPES]
            ys = [torch.empty_like(x) for x in xs]
            gs = [1 + 0.1 * rnd((C,), f32) for C, H in SHAPES]
            bs = [0.1 * rnd((C,), f32) for C, H in SHAPES]
            return lambda: ops.groupnorm_multi(xs, gs, bs, 32, 1e-6, True, outs=ys)
        cases.append((name, sum(algorithmic_bytes(B, C, H) for C, H in SHAPES), make, ("gnstep", B)))

    for B in (8, 4, 2, 1):
        gn_step(f"cfg5 step GN+SiLU f16 batch {B}, four shapes in one launch", B)

    def gn_split(name, B, C, H, dtype, eps):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((B, C, H, H), dtype)
            y = torch.empty_like(x)
            g, b = 1 + 0.1 * rnd((C,), f32), 0.1 * rnd((C,), f32)
            return lambda: ops.groupnorm(x, g, b, 32, eps, True, out=y, path=ops.GN_SPLIT)
        cases.append((name, 2 * B * C * H * H * esz + 2 * C * 4, make, ("gn", B, C, H, eps)))

    gn_split("GN+SiLU f16 [4,128,512,512], split path (two kernels, three passes; any alignment)", 4, 128, 512, f16, 1e-6)

    def gn_by_name(name, B, C, H, dtype, eps):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((B, C, H, H), dtype)
            y = torch.empty_like(x)
            g, b = 1 + 0.1 * rnd((C,), f32), 0.1 * rnd((C,), f32)

            def run():
                mean = ops.local_reduction_mean(x, B * 32)
                var = ops.local_reduction_variance(x, mean, B * 32)
                ops.group_norm_apply(x, mean, var, g, b, (C // 32) * H * H, H * H, eps, C, out=y)
                ops.silu(y, out=y)
            return run
        cases.append((name, 2 * B * C * H * H * esz + 2 * C * 4, make, ("gn", B, C, H, eps)))

    gn_by_name("kernel by kernel (4 launches, 6 passes): mean, variance, group_norm, silu f32 [1,320,64,64]", 1, 320, 64, f32, 1e-5)
    gn_by_name("kernel by kernel (4 launches, 6 passes): mean, variance, group_norm, silu f16 [8,256,256,256]", 8, 256, 256, f16, 1e-6)

    def gn_bias(name, B, C, H, dtype, eps):
        esz = 2 if dtype == f16 else 4

        def make():
            x, e = rnd((B, C, H, H), dtype), rnd((B, C), dtype)
            y = torch.empty_like(x)
            g, b = 1 + 0.1 * rnd((C,), f32), 0.1 * rnd((C,), f32)
            return lambda: ops.groupnorm_bias(x, e, g, b, 32, eps, True, out=y)
        cases.append((name, 2 * B * C * H * H * esz + 2 * C * 4 + B * C * esz, make, ("gnbias", B, C, H, eps)))

    gn_bias("next: chunkwise_add+GN+SiLU f16 [2,320,64,64]", 2, 320, 64, f16, 1e-5)
    gn_bias("next: chunkwise_add+GN+SiLU f16 [2,1280,16,16]", 2, 1280, 16, f16, 1e-5)
    gn_bias("next: chunkwise_add+GN+SiLU f16 [8,256,256,256] (large)", 8, 256, 256, f16, 1e-5)

    def chadd(name, B, C, H, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((B, C, H, H), dtype)
            e = rnd((B, C), dtype)
            y = torch.empty_like(x)
            return lambda: ops.chunkwise_add(x, e, H * H, out=y)
        cases.append((name, 2 * B * C * H * H * esz + B * C * esz, make, ("chadd", B, C, H)))

    chadd("next: chunkwise_add f16 [2,320,64,64]", 2, 320, 64, f16)
    chadd("next: chunkwise_add f16 [8,256,256,256] (large)", 8, 256, 256, f16)

    def gn_nhwc(name, B, C, H, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((B, C, H, H), dtype)
            y = torch.empty((B, H * H, C), device=dev, dtype=dtype)
            g, b = 1 + 0.1 * rnd((C,), f32), 0.1 * rnd((C,), f32)
            return lambda: ops.groupnorm_nhwc(x, g, b, 32, 1e-6, False, out=y)
        cases.append((name, 2 * B * C * H * H * esz + 2 * C * 4, make, ("gnnhwc", B, C, H)))

    gn_nhwc("next: GN + channels-last store f16 [2,320,64,64]", 2, 320, 64, f16)
    gn_nhwc("next: GN + channels-last store f16 [2,1280,16,16]", 2, 1280, 16, f16)
    gn_nhwc("next: GN + channels-last store f32 [1,320,64,64]", 1, 320, 64, f32)
    gn_nhwc("next: GN + channels-last store f16 [8,512,128,128] (large)", 8, 512, 128, f16)
    gn_nhwc("next: GN + channels-last store f32 [4,512,128,128] (large)", 4, 512, 128, f32)

    def perm(name, I, J, K, dtype, add):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((I, J, K), dtype)
            r = rnd((I, K, J), dtype) if add else None
            y = torch.empty((I, K, J), device=dev, dtype=dtype)
            return (lambda: ops.permute_add(x, r, out=y)) if add else (lambda: ops.permute_021(x, out=y))
        cases.append((name, (3 if add else 2) * I * J * K * esz, make, ("perm", I, J, K, add)))

    perm("next: permute3D__0_2_1 f16 [2,320,4096]->[2,4096,320]", 2, 320, 4096, f16, False)
    perm("next: permute + residual add f16 [2,4096,320]->[2,320,4096]", 2, 4096, 320, f16, True)
    perm("next: permute3D__0_2_1 f16 [64,320,4096] (large)", 64, 320, 4096, f16, False)
    perm("next: permute + residual add f16 [64,4096,320] (large)", 64, 4096, 320, f16, True)
    perm("next: permute3D__0_2_1 f32 [64,1280,1024] (large)", 64, 1280, 1024, f32, False)

    def gn_cat(name, B, C1, C2, H, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            a, c = rnd((B, C1, H, H), dtype), rnd((B, C2, H, H), dtype)
            y = torch.empty((B, C1 + C2, H, H), device=dev, dtype=dtype)
            g, b = 1 + 0.1 * rnd((C1 + C2,), f32), 0.1 * rnd((C1 + C2,), f32)
            return lambda: ops.groupnorm_concat(a, c, g, b, 32, 1e-5, True, out=y)
        cases.append((name, 2 * B * (C1 + C2) * H * H * esz + 2 * (C1 + C2) * 4, make, ("gncat", B, C1, C2, H)))

    gn_cat("next: concat+GN+SiLU f16 [2,640+320,32,32]", 2, 640, 320, 32, f16)
    gn_cat("next: concat+GN+SiLU f16 [2,320+320,64,64]", 2, 320, 320, 64, f16)
    gn_cat("next: concat+GN+SiLU f16 [8,128+128,256,256] (large)", 8, 128, 128, 256, f16)

    def cat(name, B, C1, C2, H, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            a, c = rnd((B, C1, H, H), dtype), rnd((B, C2, H, H), dtype)
            y = torch.empty((B, C1 + C2, H, H), device=dev, dtype=dtype)
            return lambda: ops.concat_channels(a, c, out=y)
        cases.append((name, 2 * B * (C1 + C2) * H * H * esz, make, ("cat", B, C1, C2, H)))

    cat("next: concat_buffer f16 [2,640+320,32,32]", 2, 640, 320, 32, f16)
    cat("next: concat_buffer f16 [8,128+128,256,256] (large)", 8, 128, 128, 256, f16)

    def ups(name, B, C, H, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((B, C, H, H), dtype)
            y = torch.empty((B, C, 2 * H, 2 * H), device=dev, dtype=dtype)
            return lambda: ops.up_sample_nearest(x, 2, out=y)
        cases.append((name, 5 * B * C * H * H * esz, make, ("ups", B, C, H)))

    ups("next: up_sample_nearest x2 f16 [2,1280,16,16]", 2, 1280, 16, f16)
    ups("next: up_sample_nearest x2 f16 [8,512,128,128] (large)", 8, 512, 128, f16)

    def smax(name, rows, keys, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((rows, keys), dtype, 2.0)
            y = torch.empty_like(x)
            return lambda: ops.softmax(x, out=y)
        cases.append((name, 2 * rows * keys * esz, make, ("softmax", rows, keys)))

    smax("next: softmax f16 cross-attention [2*8*4096, 77]", 2 * 8 * 4096, 77, f16)
    smax("next: softmax f32 cross-attention [8*4096, 77] (reference dtype)", 8 * 4096, 77, f32)
    smax("next: softmax f16 self-attention [2*8*1024, 1024]", 2 * 8 * 1024, 1024, f16)
    smax("next: softmax f16 self-attention [8*4096, 4096] (large)", 8 * 4096, 4096, f16)
    smax("next: softmax f32 self-attention [8*4096, 4096] (large)", 8 * 4096, 4096, f32)

    def ln(name, rows, D, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((rows, D), dtype)
            y = torch.empty_like(x)
            g, b = 1 + 0.1 * rnd((D,), f32), 0.1 * rnd((D,), f32)
            return lambda: ops.layernorm(x, g, b, 1e-5, out=y)
        cases.append((name, 2 * rows * D * esz + 2 * D * 4, make, ("ln", rows, D)))

    ln("cfg2 LN f32 [2,77,768]", 154, 768, f32)
    ln("cfg2 LN f32 [1,77,1024] (reference width)", 77, 1024, f32)
    ln("cfg4 LN f16 [2,4096,320]", 8192, 320, f16)
    ln("LN f16 [16,4096,1280] (large)", 65536, 1280, f16)
    ln("LN f32 [16,4096,320] (large)", 65536, 320, f32)

    def add_ln(name, rows, D, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            x, r = rnd((rows, D), dtype), rnd((rows, D), dtype)
            ssum, y = torch.empty_like(x), torch.empty_like(x)
            g, b = 1 + 0.1 * rnd((D,), f32), 0.1 * rnd((D,), f32)
            return lambda: ops.add_layernorm(x, r, g, b, 1e-5, sum_out=ssum, out=y)
        cases.append((name, 4 * rows * D * esz + 2 * D * 4, make, ("addln", rows, D)))

    add_ln("next: add+LN f16 [2,4096,320]", 8192, 320, f16)
    add_ln("next: add+LN f16 [16,4096,1280] (large)", 65536, 1280, f16)

    def geglu(name, rows, D, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            ab = rnd((rows, 2 * D), dtype)
            y = torch.empty((rows, D), device=dev, dtype=dtype)
            return lambda: ops.gelu_multiply(ab, out=y)
        cases.append((name, 3 * rows * D * esz, make, ("geglu", rows, D)))

    geglu("cfg4 GEGLU f16 [2,4096,2560]->[2,4096,1280]", 8192, 1280, f16)
    geglu("GEGLU f16 [16,4096,2560] (large)", 65536, 1280, f16)
    geglu("GEGLU f32 [8,4096,2560] (large)", 32768, 1280, f32)

    def act(name, fn, n, dtype):
        esz = 2 if dtype == f16 else 4

        def make():
            x = rnd((n,), dtype)
            y = torch.empty_like(x)
            return lambda: fn(x, out=y)
        cases.append((name, 2 * n * esz, make, ("act", fn.__name__, n)))

    act("cfg2 quick_gelu f32 [2,77,3072]", ops.quick_gelu, 2 * 77 * 3072, f32)
    act("cfg2 gelu(erf) f32 [2,77,3072]", ops.gelu, 2 * 77 * 3072, f32)
    act("cfg4 SiLU f16 [2,1280]", ops.silu, 2 * 1280, f16)
    act("SiLU f16 256M elements (large)", ops.silu, 1 << 28, f16)
    act("gelu(erf) f32 128M elements (large)", ops.gelu, 1 << 27, f32)
    act("quick_gelu f16 256M elements (large)", ops.quick_gelu, 1 << 28, f16)

    tables = {}

    def emb(D):
        def make():
            if D not in tables:            # the 152-202 MB table is shared by the ring's sets
                tables[D] = (rnd((49408, D), f32, 0.02), rnd((77, D), f32, 0.02))
            table, pos = tables[D]
            ids = torch.randint(0, 49408, (2, 77), device=dev, generator=gen, dtype=torch.int64)
            out = torch.empty((2, 77, D), device=dev, dtype=f32)
            return lambda: ops.token_embedding(ids, table, pos, out=out)
        nbytes = 2 * 77 * 8 + 2 * (2 * 77 * D * 4) + 77 * D * 4
        cases.append((f"cfg2 token+pos embedding f32 [2,77]->[2,77,{D}]", nbytes, make, ("emb", D)))

    emb(768)
    emb(1024)

    def ts_make():
        t = torch.randint(0, 1000, (2,), device=dev, generator=gen, dtype=torch.int64)
        out = torch.empty((2, 320), device=dev, dtype=f16)
        return lambda: ops.timestep_embedding(t, 320, out=out)
    cases.append(("cfg4 timestep embedding f16 [2]->[2,320]", 2 * 8 + 2 * 320 * 2, ts_make, ("ts",)))

    def add_make():
        a_, b_ = rnd((1 << 27,), f32), rnd((1 << 27,), f32)
        c_ = torch.empty_like(a_)
        return lambda: ops.elemwise_add(a_, b_, out=c_)
    cases.append(("elemwise_add f32 128M elements (large)", 3 * (1 << 27) * 4, add_make, ("add", 1 << 27)))
    return cases


def cpu_reference_case(spec) -> dict:
    """The reference's CPU implementation of one case on this machine's host cores
    (oracle/_ref when built, else the plain-C port), on a bounded sample scaled linearly to the
    case's size.  fp32 arithmetic whatever the GPU case's storage type."""
    import numpy as np
    import oracle
    backend = "ref" if oracle.have_ref() else "port"
    rng = np.random.Generator(np.random.PCG64(99))
    kind = spec[0]

    def timed(fn, reps=3):
        fn()
        best = 1e30
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
        return best

    scale, note = 1.0, "full size"
    if kind == "gn":
        _, B, C, H, eps = spec
        x = rng.standard_normal((1, C, H, H), dtype=np.float32)
        g, b = np.ones(C, np.float32), np.zeros(C, np.float32)
        t = timed(lambda: oracle.group_norm(x, g, b, 32, eps, True, backend=backend), reps=2)
        scale, note = float(B), f"one image x {B}"
    elif kind == "gnstep":
        B = spec[1]
        t = 0.0
        for C, H in SHAPES:
            x = rng.standard_normal((1, C, H, H), dtype=np.float32)
            g, b = np.ones(C, np.float32), np.zeros(C, np.float32)
            t += timed(lambda: oracle.group_norm(x, g, b, 32, 1e-6, True, backend=backend), reps=1)
        scale, note = float(B), f"one image of each shape x {B}"
    elif kind == "gnbias":
        _, B, C, H, eps = spec
        x = rng.standard_normal((C, H, H), dtype=np.float32)
        e = rng.standard_normal(C, dtype=np.float32)
        g, b = np.ones(C, np.float32), np.zeros(C, np.float32)
        t = timed(lambda: oracle.group_norm(oracle.chunkwise_add(x, e, H * H, backend=backend)[None],
                                            g, b, 32, eps, True, backend=backend), reps=2)
        scale, note = float(B), f"one image x {B}"
    elif kind == "gnnhwc":
        _, B, C, H = spec
        x = rng.standard_normal((1, C, H, H), dtype=np.float32)
        g, b = np.ones(C, np.float32), np.zeros(C, np.float32)
        t = timed(lambda: oracle.permute_021(oracle.group_norm(x, g, b, 32, 1e-6, False, backend=backend)
                                             .reshape(1, C, H * H), backend=backend), reps=2)
        scale, note = float(B), f"one image x {B}"
    elif kind == "perm":
        _, I, J, K, add = spec
        i = min(I, 4)
        x = rng.standard_normal((i, J, K), dtype=np.float32)
        r = rng.standard_normal((i, K, J), dtype=np.float32)
        if add:
            t = timed(lambda: oracle.elemwise_add(oracle.permute_021(x, backend=backend), r, backend=backend))
        else:
            t = timed(lambda: oracle.permute_021(x, backend=backend))
        scale, note = I / i, f"{i} of {I} slices scaled"
    elif kind == "gncat":
        _, B, C1, C2, H = spec
        a = rng.standard_normal((1, C1, H, H), dtype=np.float32)
        c = rng.standard_normal((1, C2, H, H), dtype=np.float32)
        g, b = np.ones(C1 + C2, np.float32), np.zeros(C1 + C2, np.float32)
        t = timed(lambda: oracle.group_norm(oracle.concat_buffer(a, c), g, b, 32, 1e-5, True, backend=backend), reps=2)
        scale, note = float(B), f"one image x {B}"
    elif kind == "chadd":
        _, B, C, H = spec
        x = rng.standard_normal((C, H, H), dtype=np.float32)
        e = rng.standard_normal(C, dtype=np.float32)
        t = timed(lambda: oracle.chunkwise_add(x, e, H * H, backend=backend))
        scale, note = float(B), f"one image x {B}"
    elif kind == "cat":
        _, B, C1, C2, H = spec
        a = rng.standard_normal((1, C1, H, H), dtype=np.float32)
        c = rng.standard_normal((1, C2, H, H), dtype=np.float32)
        t = timed(lambda: oracle.concat_buffer(a, c))
        scale, note = float(B), f"one image x {B}"
    elif kind == "ups":
        _, B, C, H = spec
        x = rng.standard_normal((1, C, H, H), dtype=np.float32)
        t = timed(lambda: oracle.up_sample_nearest(x, 2, backend=backend))
        scale, note = float(B), f"one image x {B}"
    elif kind == "softmax":
        _, rows, keys = spec
        r = min(rows, 4096)
        x = (rng.standard_normal((r, keys), dtype=np.float32) * 2.0).astype(np.float32)
        t = timed(lambda: oracle.softmax(x, backend=backend))
        scale, note = rows / r, f"{r} rows scaled"
    elif kind == "ln":
        _, rows, D = spec
        r = min(rows, 8192)
        x = rng.standard_normal((r, D), dtype=np.float32)
        g, b = np.ones(D, np.float32), np.zeros(D, np.float32)
        t = timed(lambda: oracle.layer_norm(x, g, b, 1e-5, backend=backend if D % 64 == 0 else "port"))
        scale, note = rows / r, f"{r} rows scaled"
    elif kind == "addln":
        _, rows, D = spec
        r = min(rows, 8192)
        x = rng.standard_normal((r, D), dtype=np.float32)
        y = rng.standard_normal((r, D), dtype=np.float32)
        g, b = np.ones(D, np.float32), np.zeros(D, np.float32)
        t = timed(lambda: oracle.layer_norm(oracle.elemwise_add(x, y, backend=backend), g, b, 1e-5,
                                            backend=backend if D % 64 == 0 else "port"))
        scale, note = rows / r, f"{r} rows scaled"
    elif kind == "geglu":
        _, rows, D = spec
        r = min(rows, 8192)
        ab = rng.standard_normal((r, 2 * D), dtype=np.float32)
        t = timed(lambda: oracle.gelu_multiply(ab, backend=backend))
        scale, note = rows / r, f"{r} rows scaled"
    elif kind == "act":
        _, fname, n = spec
        m = min(n, 1 << 24)
        x = rng.standard_normal(m, dtype=np.float32)
        be = "port" if fname == "quick_gelu" else backend
        t = timed(lambda: getattr(oracle, fname)(x, backend=be))
        scale, note = n / m, f"{m} elements scaled"
    elif kind == "add":
        n = spec[1]
        m = min(n, 1 << 24)
        x, y = rng.standard_normal(m, dtype=np.float32), rng.standard_normal(m, dtype=np.float32)
        t = timed(lambda: oracle.elemwise_add(x, y, backend=backend))
        scale, note = n / m, f"{m} elements scaled"
    elif kind == "emb":
        D = spec[1]
        table = rng.standard_normal((49408, D), dtype=np.float32)
        pos = rng.standard_normal((77, D), dtype=np.float32)
        ids = rng.integers(0, 49408, (2, 77), dtype=np.int64)
        t = timed(lambda: oracle.token_embedding(ids, table, pos))
    else:
        tt = np.array([981, 17], np.int64)
        t = timed(lambda: oracle.timestep_embedding(tt, 320))
    return {"cpu_ms": round(t * scale * 1e3, 4), "cpu_cores": oracle.num_threads(backend),
            "cpu_kind": "reference kernels compiled as C++" if backend == "ref" else "plain-C port",
            "cpu_sample": note}


def run_ops(args) -> None:
    """--ops: one JSON line per kernel/shape (device time per launch with L2 flushed, GB/s of
    algorithmic bytes, fraction of the measured HBM peak).  --case SUBSTRING: run only the
    matching cases, `--steps` launches each (the form used under ncu)."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pkg = importlib.import_module("mobile-stable-diffusion_b200")
    ops = pkg.ops
    peak, peak_kind = measured_peak()
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
    reps = max(args.steps, 1) if args.case else 9
    stream = torch.cuda.Stream(device=dev)
    for name, nbytes, make, spec in op_cases(torch, ops, dev):
        if args.case and args.case not in name:
            continue
        ring_timing = not args.case or args.ring
        nring = min(64, max(2, -(-4 * L2_BYTES // nbytes))) if ring_timing else 1
        fns = [make() for _ in range(nring)]
        fn = fns[0]
        for _ in range(max(args.warmup, 1)):
            fn()
        times = []
        for _ in range(reps):
            flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize(dev)
            times.append(a.elapsed_time(b))
        t = statistics.median(times)
        gbs = nbytes / (t * 1e-3) / 1e9
        line = {"case": name, "bytes": nbytes, "single_launch_us": round(t * 1e3, 2),
                "single_launch_gbs": round(gbs, 1),
                "single_launch_timing": "CUDA events around one launch, L2 flushed before it, median "
                                        "(an empty launch costs about 6 us this way)",
                "peak": peak, "peak_source": f"of {peak_kind}"}
        if ring_timing:
            # K launches back to back as one CUDA graph, cycling through the ring of buffer sets
            # (a set comes back after >= 4 x L2 of other traffic unless the case is tiny)
            K = max(nring, 32)
            with torch.cuda.stream(stream):
                for f in fns:
                    f()
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for i in range(K):
                        fns[i % nring]()
                g.replay()
                stream.synchronize()
                rt = []
                for _ in range(21):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    g.replay()
                    b.record(stream)
                    stream.synchronize()
                    rt.append(a.elapsed_time(b) / K)
                del g
            tr = statistics.median(rt)
            line.update({"us": round(tr * 1e3, 2), "gbs": round(nbytes / (tr * 1e-3) / 1e9, 1),
                         "frac_of_peak": round(nbytes / (tr * 1e-3) / 1e9 / peak, 4),
                         "timing": f"CUDA graph of {K} back-to-back launches over a ring of {nring} buffer "
                                   f"sets ({nring * nbytes / 1e6:.0f} MB), median of 21 replays, per launch"})
        else:
            line.update({"us": line["single_launch_us"], "gbs": line["single_launch_gbs"],
                         "frac_of_peak": round(gbs / peak, 4), "timing": line["single_launch_timing"]})
        if args.cpu:
            line.update(cpu_reference_case(spec))
        print(json.dumps(line), flush=True)
        del fns, fn
        torch.cuda.empty_cache()
    assert ops.device_status() == 0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--blocks", type=int, default=25, help="timed blocks of --steps steps each (the median block is reported)")
    ap.add_argument("--chain", action="store_true", help="launch the step as four kernels, one per tensor, instead of one")
    ap.add_argument("--no-parity-check", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ops", action="store_true", help="per-kernel table over all named shapes")
    ap.add_argument("--case", default="", help="with --ops: only cases whose name contains this")
    ap.add_argument("--cpu", action="store_true", help="with --ops: also time the reference on the host cores")
    ap.add_argument("--ring", action="store_true", help="with --case: also run the back-to-back graph timing")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.ops or args.case:
        run_ops(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
