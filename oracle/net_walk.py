"""TEST INFRASTRUCTURE ONLY -- walks a network spec (nart_b200.nets) op by op over a CPU checker.

``backend`` is any object offering conv2d_u8 / ip_u8 / pool_u8 / eltwise_sum_u8 / relu_u8 /
dequantize_u8 on NCHW numpy arrays: ``oracle.port()`` or ``oracle.ref()``.
"""
from __future__ import annotations

import numpy as np


def run_net(spec, x, backend, per_channel: bool = True, keep=()):
    """Walks the spec with ``backend`` (an object offering conv2d_u8 / ip_u8 / pool_u8 /
    eltwise_sum_u8 / relu_u8 / dequantize_u8 on NCHW numpy arrays).  ``per_channel`` False passes
    only walpha[0], which is all the reference module reads.  Returns (float32 logits, uint8 output,
    {name: tensor} for the names in ``keep``)."""
    T = spec["tensors"]
    vals = {"input": np.ascontiguousarray(x, dtype=np.uint8)}
    kept = {}
    last_use = {}
    for i, op in enumerate(spec["ops"]):
        for n in op["ins"]:
            last_use[n] = i
    for i, op in enumerate(spec["ops"]):
        ti, to = T[op["ins"][0]], T[op["out"]]
        xin = vals[op["ins"][0]]
        if op["op"] in ("conv", "ip"):
            wa = op["walpha"] if per_channel else op["walpha"][:1]
            if op["op"] == "conv":
                kw = dict(relu=op["relu"]) if per_channel else {}
                y = backend.conv2d_u8(xin, op["w"], op["bias"], (op["stride"],) * 2, (op["pad"],) * 2, op["group"],
                                      ialpha=ti["alpha"], izp=ti["zp"], walpha=wa if per_channel else float(wa[0]),
                                      wzp=128, oalpha=to["alpha"], ozp=to["zp"], **kw)
                if not per_channel and op["relu"]:
                    y = backend.relu_u8(y, to["alpha"], to["zp"], to["alpha"], to["zp"])
            else:
                y = backend.ip_u8(xin.reshape(xin.shape[0], -1), op["w"], op["bias"], ti["alpha"], ti["zp"],
                                  wa if per_channel else float(wa[0]), 128, to["alpha"], to["zp"])
                y = y.reshape(y.shape[0], -1, 1, 1)
        elif op["op"] == "pool":
            y = backend.pool_u8(xin, op["method"], (op["ksize"],) * 2, (op["pad"],) * 2, (op["stride"],) * 2,
                                op["ceil_mode"], ti["alpha"], ti["zp"], to["alpha"], to["zp"])
        elif op["op"] == "eltwise":
            ins = [T[n] for n in op["ins"]]
            y = backend.eltwise_sum_u8([vals[n] for n in op["ins"]], [t["alpha"] for t in ins],
                                       [t["zp"] for t in ins], to["alpha"], to["zp"])
            if op["relu"]:
                y = backend.relu_u8(y, to["alpha"], to["zp"], to["alpha"], to["zp"])
        else:
            raise ValueError(op["op"])
        vals[op["out"]] = y
        if op["out"] in keep:
            kept[op["out"]] = y
        for n in op["ins"]:
            if last_use.get(n) == i and n != spec["output"] and n in vals:
                del vals[n]
    out = T[spec["output"]]
    q = vals[spec["output"]]
    return backend.dequantize_u8(q, out["alpha"], out["zp"]), q, kept
