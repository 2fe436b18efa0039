"""Generates tests/golden/quant_ref_s8.npz: outputs of the UNMODIFIED reference quant module (oracle/_ref)
on its int8 path -- conv_2d and ip on dtINT8 tensors, quantize with qtype SYMMETRIC, dequantize of int8.
Run where the reference sources are present:

    python tests/golden/gen_golden_s8.py

Inputs are re-derived from the seeds in tests/cases.py; the file holds the reference's outputs only.
The reference reads one weight scale per layer, so the per-channel fixture is assembled channel by
channel from reference runs with the scalar walpha[k].
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from cases import S8_SHAPES, conv_inputs_s8, s8_oalpha  # noqa: E402


def main():
    oracle.build(ref=True)
    R = oracle.ref()
    out = {}
    for i, (n, c, h, w, k, r, s, st, pd, g, ob) in enumerate(S8_SHAPES):
        x, wt, bias, walpha = conv_inputs_s8(300 + i, n, c, h, w, k, r, s, g)
        oa = s8_oalpha(c, g, r, s)
        out["conv%d_scalar" % i] = R.conv2d_i8(x, wt, bias, (st, st), (pd, pd), g, 0.02, float(walpha[0]), oa, ob)
        if i < 3:
            per = np.empty_like(out["conv%d_scalar" % i])
            for kk in range(k):
                per[:, kk] = R.conv2d_i8(x, wt, bias, (st, st), (pd, pd), g, 0.02, float(walpha[kk]), oa, ob)[:, kk]
            out["conv%d_per_channel" % i] = per
    rng = np.random.default_rng(77)
    xi = rng.integers(-127, 128, (4, 512)).astype(np.int8)
    wi = rng.integers(-127, 128, (100, 512)).astype(np.int8)
    bi = rng.integers(-4096, 4097, 100).astype(np.int32)
    out["ip"] = R.ip_i8(xi, wi, bi, 0.02, 0.005, 0.4, 7)
    f = (rng.standard_normal((2, 24, 9, 11)) * 3).astype(np.float32)
    f.reshape(-1)[:2001] = (np.arange(2001) - 1000) * np.float32(0.05) * np.float32(0.5)     # every half-step tie
    for ob in (8, 7, 4):
        out["quantize_%d" % ob] = R.quantize_i8(f, 0.05, ob)
    q = rng.integers(-128, 128, (2, 24, 9, 11)).astype(np.int8)
    out["dequantize"] = R.dequantize_i8(q, 0.037)
    path = os.path.join(HERE, "quant_ref_s8.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
