"""Times the bandwidth-bound ops around the convolution through the C-ABI, one op per call:

    python -m nart_b200.op_bench --op eltwise --c 256 --hw 56 --batch 256
    python -m nart_b200.op_bench --op maxpool --c 64 --hw 112 --batch 256
    python -m nart_b200.op_bench --op avgpool --c 2048 --hw 7 --batch 256
    python -m nart_b200.op_bench --op input_layout --c 3 --hw 224 --batch 256
    python -m nart_b200.op_bench --op quantize | dequantize | relu | depthwise | stem --...

Per op it prints one JSON line: milliseconds per launch (CUDA events on the launching stream after a
warm-up), the algorithmic bytes (every input and output tensor once) and the GB/s they give.  Inputs rotate
through enough buffers to exceed the L2 cache between launches of the same data.
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np
import torch

from . import ops

L2_BYTES = 126 << 20


def _time(fn, sets, iters, warmup):
    for i in range(max(warmup, len(sets))):
        fn(*sets[i % len(sets)])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(*sets[i % len(sets)])
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _nbuf(bytes_per_set):
    return max(2, min(8, -(-2 * L2_BYTES // max(1, bytes_per_set)) + 1))


def _u8(*shape):
    return torch.randint(0, 256, shape, dtype=torch.uint8, device="cuda")


def run(op, c, hw, batch, stride=1, iters=20, warmup=5):
    rng = np.random.default_rng(0)
    if op == "eltwise":
        byts = 3 * batch * hw * hw * c
        sets = [(_u8(batch, hw, hw, c), _u8(batch, hw, hw, c)) for _ in range(_nbuf(byts))]
        ms = _time(lambda a, b: ops.eltwise_sum([a, b], [0.037, 0.081], [117, 9], 0.093, 31, relu=True), sets, iters, warmup)
    elif op in ("maxpool", "avgpool"):
        method = ops.POOL_MAX if op == "maxpool" else ops.POOL_AVE
        k, p, s = ((3, 3), (1, 1), (2, 2)) if op == "maxpool" else ((hw, hw), (0, 0), (1, 1))
        oh, ow = ops.pool_out_dims(hw, hw, k, p, s, False)
        byts = batch * c * (hw * hw + oh * ow)
        sets = [(_u8(batch, hw, hw, c),) for _ in range(_nbuf(byts))]
        oa = 0.037 if op == "maxpool" else 0.02
        ms = _time(lambda a: ops.pool(a, method, k, p, s, False, 0.037, 117, oa, 117), sets, iters, warmup)
    elif op == "input_layout":
        cp = (c + 3) // 4 * 4
        byts = batch * hw * hw * (c + cp)
        sets = [(_u8(batch, c, hw, hw),) for _ in range(_nbuf(byts))]
        ms = _time(lambda a: ops.nchw_to_nhwc(a, c_pad=cp), sets, iters, warmup)
    elif op == "quantize":
        byts = batch * hw * hw * c * 5
        sets = [(torch.randn((batch, c, hw, hw), device="cuda"),) for _ in range(_nbuf(byts))]
        ms = _time(lambda a: ops.quantize(a, 0.037, 117), sets, iters, warmup)
    elif op == "dequantize":
        byts = batch * hw * hw * c * 5
        sets = [(_u8(batch, hw, hw, c),) for _ in range(_nbuf(byts))]
        ms = _time(lambda a: ops.dequantize(a, 0.037, 117), sets, iters, warmup)
    elif op == "relu":
        byts = 2 * batch * hw * hw * c
        sets = [(_u8(batch, hw, hw, c),) for _ in range(_nbuf(byts))]
        ms = _time(lambda a: ops.relu(a, 0.037, 117, 0.05, 20), sets, iters, warmup)
    elif op in ("depthwise", "stem"):
        if op == "depthwise":
            cin, k, ks, group, pad = c, c, 3, c, 1
        else:
            cin, k, ks, group, pad, stride = 4, c, 7, 1, 3, 2
        w = (rng.integers(-127, 128, (k, cin // group, ks, ks)) + 128).astype(np.uint8)
        b = rng.integers(-4096, 4097, k).astype(np.int32)
        wa = rng.uniform(0.001, 0.01, k).astype(np.float32)
        conv = ops.Conv2d(w, b, in_hw=(hw, hw), stride=(stride, stride), pad=(pad, pad), group=group, ialpha=0.02, izp=128,
                          walpha=wa, oalpha=0.05, ozp=3, relu=True)
        oh, ow = conv.out_hw
        byts = batch * (hw * hw * cin + oh * ow * k) + w.size
        sets = [(_u8(batch, hw, hw, cin),) for _ in range(_nbuf(byts))]
        ms = _time(conv, sets, iters, warmup)
    else:
        raise ValueError("unknown op " + op)
    assert ops.device_status() == 0
    return dict(op=op, c=c, hw=hw, batch=batch, stride=stride, ms=ms, bytes=byts, gbs=byts / ms / 1e6, buffers=len(sets))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["eltwise", "maxpool", "avgpool", "input_layout", "quantize", "dequantize",
                                                    "relu", "depthwise", "stem"])
    ap.add_argument("--c", type=int, default=64)
    ap.add_argument("--hw", type=int, default=56)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args(argv)
    print(json.dumps(run(a.op, a.c, a.hw, a.batch, a.stride, a.iters, a.warmup)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
