"""Times single quantized convolutions through the C-ABI: one shape, or the shape sweep of the
benchmark's config 1 ((C_in, C_out, H) in {(64,64,56), (128,128,28), (256,256,14), (512,512,7)},
1x1 and 3x3, stride 1 and 2, batch 1 / 32 / 256).

    python -m nart_b200.conv_bench --c 128 --k 128 --hw 28 --ks 3 --stride 1 --batch 256
    python -m nart_b200.conv_bench --sweep

Per shape it prints one JSON line: milliseconds per launch (CUDA events on the launching stream,
warm-up first), TOP/s on the true dims, and the algorithmic GB/s (each tensor once).  Inputs and
outputs rotate through enough buffers to exceed the L2 cache between launches of the same data.
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np
import torch

from . import ops

L2_BYTES = 126 << 20
SWEEP_SHAPES = [(64, 64, 56), (128, 128, 28), (256, 256, 14), (512, 512, 7)]


def time_conv(c, k, hw, ks, stride, batch, group=1, algo=ops.ALGO_AUTO, iters=20, warmup=5, seed=0, graph=False):
    rng = np.random.default_rng(seed)
    w = (rng.integers(-127, 128, (k, c // group, ks, ks)) + 128).astype(np.uint8)
    b = rng.integers(-4096, 4097, k).astype(np.int32)
    wa = rng.uniform(0.001, 0.01, k).astype(np.float32)
    conv = ops.Conv2d(w, b, in_hw=(hw, hw), stride=(stride, stride), pad=(ks // 2, ks // 2), group=group,
                      ialpha=0.02, izp=128, walpha=wa, oalpha=0.05, ozp=0, relu=True, algo=algo)
    oh, ow = conv.out_hw
    in_bytes, out_bytes = batch * hw * hw * c, batch * oh * ow * k
    # rotate buffers so that a launch never finds its operands in L2 from the previous one
    nbuf = max(2, min(8, -(-2 * L2_BYTES // max(1, in_bytes + out_bytes)) + 1))
    xs = [torch.randint(0, 256, (batch, hw, hw, c), dtype=torch.uint8, device="cuda") for _ in range(nbuf)]
    for i in range(max(warmup, nbuf)):
        y = conv(xs[i % nbuf])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        # the same launches replayed from a CUDA graph: the device time per launch without the
        # host's per-call cost (Python, output allocation, tensor-map encoding)
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for i in range(iters):
                    y = conv(xs[i % nbuf])
            g.replay()
            side.synchronize()
            e0.record(side)
            g.replay()
            e1.record(side)
        torch.cuda.synchronize()
    else:
        e0.record()
        for i in range(iters):
            y = conv(xs[i % nbuf])
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    assert ops.device_status() == 0
    ops_count = 2.0 * batch * oh * ow * k * (c // group) * ks * ks
    byts = in_bytes + out_bytes + w.size + 4 * k
    return dict(c=c, k=k, hw=hw, ks=ks, stride=stride, batch=batch, group=group, plan=conv.describe(),
                algo={1: "cuda_core", 2: "tcgen05_igemm"}[conv.algo], ms=ms, tops=ops_count / ms / 1e9,
                gbs=byts / ms / 1e6, intensity_op_per_byte=ops_count / byts, buffers=nbuf,
                timing="cuda graph replay" if graph else "eager launches")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--c", type=int, default=64)
    ap.add_argument("--k", type=int, default=64)
    ap.add_argument("--hw", type=int, default=56)
    ap.add_argument("--ks", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--group", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--direct", action="store_true", help="force the CUDA-core kernel")
    ap.add_argument("--graph", action="store_true", help="time the launches replayed from one CUDA graph")
    a = ap.parse_args(argv)
    algo = ops.ALGO_DIRECT if a.direct else ops.ALGO_AUTO
    if a.sweep:
        for c, k, hw in SWEEP_SHAPES:
            for ks in (1, 3):
                for stride in (1, 2):
                    for batch in (1, 32, 256):
                        print(json.dumps(time_conv(c, k, hw, ks, stride, batch, algo=algo, iters=a.iters, warmup=a.warmup,
                                                   graph=a.graph)))
    else:
        print(json.dumps(time_conv(a.c, a.k, a.hw, a.ks, a.stride, a.batch, a.group, algo, a.iters, a.warmup,
                                   graph=a.graph)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
