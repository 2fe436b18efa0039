"""Generates tests/golden/*.npz from the UNMODIFIED reference quant module (oracle/_ref, built by
oracle/Makefile from the reference sources where they lie).  Run in a container that has the
reference:

    python tests/golden/gen_golden.py

Inputs are re-derived from the seeds in tests/cases.py, so the fixtures hold only the parameters
and the reference's outputs.  The per-channel-scale and fused-ReLU fixtures are assembled from
reference runs only: channel k of the per-channel output is channel k of a reference run with the
scalar walpha[k]; the ReLU output is the reference conv followed by the reference relu op with
equal input and output scale / zero point.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from cases import EDGE_SHAPES, conv_inputs  # noqa: E402


def main():
    oracle.build(ref=True)
    R = oracle.ref()
    out = {}

    # ---- scale decomposition and rounding shift -------------------------------------------
    scales = np.array([0.02 * 0.005 / 0.05, 1.0, 3.7, 0.5, 0.25, 1e-3, 123.4, 7e-6, 0.9999999],
                      dtype=np.float32)
    rows = []
    for x in scales:
        for bits in (32, -16, 23, 24, 16):
            m, s = R.get_quant_scale(float(x), bits)
            rows.append((float(x), bits, m, s))
    out["scale_rows"] = np.array(rows, dtype=np.float64)
    rng = np.random.default_rng(1234)
    xs = rng.integers(-2**62, 2**62, 4000, dtype=np.int64)
    bs = rng.integers(1, 59, 4000).astype(np.int64)
    out["rshift_x"], out["rshift_b"] = xs, bs
    out["rshift_y"] = np.array([R.rshift_rn(int(a), int(b)) for a, b in zip(xs, bs)], dtype=np.int64)

    # ---- conv: 64 -> 64 channels, 3x3 on 56x56, per-tensor / per-channel / fused relu ------------------------
    n, c, h, w, k, r, s, st, pd, g = EDGE_SHAPES[0]
    x, wt, bias, walpha = conv_inputs(0, n, c, h, w, k, r, s, g)
    q = dict(ialpha=0.02, izp=128, wzp=128, oalpha=0.05, ozp=0)
    out["c0_scalar"] = R.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, walpha=float(walpha[0]), **q)
    per = np.empty_like(out["c0_scalar"])
    for kk in range(k):
        per[:, kk] = R.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, walpha=float(walpha[kk]), **q)[:, kk]
    out["c0_per_channel"] = per
    # a second quantization with a non-zero output zero point so that the relu clamp is visible
    q2 = dict(ialpha=0.02, izp=117, wzp=128, oalpha=0.4, ozp=77)
    y2 = R.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, walpha=float(walpha[0]), **q2)
    out["c0_zp_scalar"] = y2
    out["c0_zp_relu"] = R.relu_u8(y2, q2["oalpha"], q2["ozp"], q2["oalpha"], q2["ozp"])

    # ---- conv: the edge shapes, scalar walpha, odd zero points ---------------------------------
    for i, (n, c, h, w, k, r, s, st, pd, g) in enumerate(EDGE_SHAPES[1:], start=1):
        x, wt, bias, walpha = conv_inputs(100 + i, n, c, h, w, k, r, s, g)
        out["edge%d" % i] = R.conv2d_u8(
            x, wt, bias, (st, st), (pd, pd), g, ialpha=0.037, izp=(37 * i) % 256,
            walpha=float(walpha[0]), wzp=128, oalpha=0.05 * np.sqrt(c // g * r * s) / 4,
            ozp=(11 * i) % 200)

    # ---- the ops around the conv -----------------------------------------------------------------
    rng = np.random.default_rng(7)
    a = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    b = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    ia, iz = [0.037, 0.081], [117, 9]
    out["eltwise"] = R.eltwise_sum_u8([a, b], ia, iz, 0.093, 31)
    out["add"] = R.eltwise_sum_u8([a, b], ia, iz, 0.093, 31, use_add=True)
    out["relu_same"] = R.relu_u8(a, 0.037, 117, 0.037, 117)
    out["relu_rescale"] = R.relu_u8(a, 0.037, 117, 0.05, 20)
    out["pool_max"] = R.pool_u8(a, 0, (3, 3), (1, 1), (2, 2), 0, 0.037, 117, 0.093, 31)
    out["pool_max_ceil"] = R.pool_u8(a, 0, (3, 3), (1, 1), (2, 2), 1, 0.037, 117, 0.093, 31)
    out["pool_ave"] = R.pool_u8(a, 1, (3, 3), (1, 1), (2, 2), 0, 0.037, 117, 0.093, 31)
    out["pool_ave_ceil"] = R.pool_u8(a, 1, (3, 3), (1, 1), (2, 2), 1, 0.037, 117, 0.093, 31)
    out["pool_gap"] = R.pool_u8(a, 1, (14, 14), (0, 0), (1, 1), 0, 0.037, 117, 0.093, 31)
    f = (rng.standard_normal((2, 3, 20, 20)) * 3).astype(np.float32)
    out["quantize"] = R.quantize_u8(f, 0.037, 117)
    out["dequantize"] = R.dequantize_u8(a, 0.037, 117)
    xi = rng.integers(0, 256, (4, 512), dtype=np.uint8)
    wi = (rng.integers(-127, 128, (100, 512)) + 128).astype(np.uint8)
    bi = rng.integers(-4096, 4097, 100).astype(np.int32)
    out["ip"] = R.ip_u8(xi, wi, bi, 0.02, 100, 0.005, 128, 0.1, 50)

    path = os.path.join(HERE, "quant_ref.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
