"""Generate tests/golden/reference_kernels.npz from the reference's own kernel source.

Runs ONLY where a reference checkout is present: it drives oracle/_ref/libsdfl_ref.so (the
reference's .cl files compiled as C++ by `make -C oracle ref`) on small seeded inputs and
stores inputs and outputs, so that machines without the reference can still check the plain-C
oracle and the CUDA kernels against what the reference's kernels produce.

    python tests/golden/make_golden.py

The two embedding host functions and quick_gelu are not in the file: the reference has no
stand-alone, compilable code for them (they are host code entangled with OpenCL buffer calls,
or do not exist), so there is nothing to run.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernels.npz")

# (name, C, H, W, groups, eps, silu, batch)
GN_CASES = [
    ("gn_c64_h8_g32_silu", 64, 8, 8, 32, 1e-5, True, 1),
    ("gn_c32_h16_g4_plain", 32, 16, 16, 4, 1e-6, False, 1),
    ("gn_c128_h8_g32_silu_b2", 128, 8, 8, 32, 1e-5, True, 2),
    ("gn_c16_h32x8_g2_silu", 16, 32, 8, 2, 1e-6, True, 1),
]
# (name, rows, D)
LN_CASES = [("ln_r6_d128", 6, 128), ("ln_r3_d320", 3, 320), ("ln_r5_d768", 5, 768)]


def main() -> None:
    if not oracle.have_ref():
        oracle.build()
    if not oracle.have_ref():
        raise SystemExit("no compiled reference (oracle/_ref): a reference checkout is required")
    data = {}
    for i, (name, C, H, W, G, eps, silu, B) in enumerate(GN_CASES):
        rng = np.random.Generator(np.random.PCG64(7000 + i))
        x = (rng.standard_normal((B, C, H, W)) * 1.5 + 0.25).astype(np.float32)
        gamma = (1.0 + 0.1 * rng.standard_normal(C)).astype(np.float32)
        beta = (0.1 * rng.standard_normal(C)).astype(np.float32)
        y, mean, var = oracle.group_norm(x, gamma, beta, G, eps, silu, backend="ref",
                                         return_stats=True)
        data.update({f"{name}.x": x, f"{name}.gamma": gamma, f"{name}.beta": beta,
                     f"{name}.y": y, f"{name}.mean": mean, f"{name}.var": var,
                     f"{name}.meta": np.array([G, int(silu)], np.int64),
                     f"{name}.eps": np.array([eps], np.float64)})
    for i, (name, rows, D) in enumerate(LN_CASES):
        rng = np.random.Generator(np.random.PCG64(7100 + i))
        x = (rng.standard_normal((rows, D)) * 2.0 - 0.5).astype(np.float32)
        gamma = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
        beta = (0.1 * rng.standard_normal(D)).astype(np.float32)
        y, mean, var = oracle.layer_norm(x, gamma, beta, 1e-5, backend="ref", return_stats=True)
        data.update({f"{name}.x": x, f"{name}.gamma": gamma, f"{name}.beta": beta,
                     f"{name}.y": y, f"{name}.mean": mean, f"{name}.var": var})
    rng = np.random.Generator(np.random.PCG64(7200))
    ab = (rng.standard_normal((5, 2 * 64)) * 2.0).astype(np.float32)
    data["geglu_r5_d64.ab"] = ab
    data["geglu_r5_d64.y"] = oracle.gelu_multiply(ab, backend="ref")
    x = (rng.standard_normal(1000) * 3.0).astype(np.float32)
    x[:8] = [0.0, -0.0, 1e-8, -1e-8, 20.0, -20.0, 88.0, -88.0]
    other = rng.standard_normal(1000).astype(np.float32)
    data["act.x"] = x
    data["act.other"] = other
    data["act.silu"] = oracle.silu(x, backend="ref")
    data["act.gelu"] = oracle.gelu(x, backend="ref")
    data["act.add"] = oracle.elemwise_add(x, other, backend="ref")
    a = rng.standard_normal((6, 40)).astype(np.float32)
    chunk = rng.standard_normal(6).astype(np.float32)
    data["chunk.a"], data["chunk.chunk"] = a, chunk
    data["chunk.y"] = oracle.chunkwise_add(a, chunk, 40, backend="ref")
    t3 = rng.standard_normal((2, 5, 7)).astype(np.float32)
    data["permute.x"] = t3
    data["permute.y"] = oracle.permute_021(t3, backend="ref")
    up = rng.standard_normal((3, 6, 6)).astype(np.float32)
    data["upsample.x"] = up
    data["upsample.y"] = oracle.up_sample_nearest(up, 2, backend="ref")
    for name, shape in (("softmax_r6_c77", (6, 77)), ("softmax_r3_c256", (3, 256))):
        x = (rng.standard_normal(shape) * 2.0).astype(np.float32)
        data[f"{name}.x"] = x
        data[f"{name}.y"] = oracle.softmax(x, backend="ref")
    # the text encoder's attention softmax: 3 heads of 77 x 77 scores plus the causal mask (-inf above
    # the diagonal), as local_softmax sees them (MultiHeadAttention.cpp:213-225), and an even row length
    for name, shape in (("local_softmax_h3_77", (3, 77, 77)), ("local_softmax_r5_64", (5, 64))):
        x = (rng.standard_normal(shape) * 2.0).astype(np.float32)
        if x.ndim == 3:
            x = x + np.triu(np.full(shape[1:], -np.inf, np.float32), 1)
        data[f"{name}.x"] = x
        data[f"{name}.y"] = oracle.local_softmax(x, backend="ref")
    np.savez_compressed(OUT, **data)
    print(f"wrote {OUT}: {len(data)} arrays, {os.path.getsize(OUT)} bytes")


if __name__ == "__main__":
    main()
