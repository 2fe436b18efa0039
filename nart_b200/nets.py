"""Synthetic quantized networks for the path's benchmark configs: ResNet-18 / ResNet-50 (v1.5,
stride on the 3x3) and MobileNetV2-1.0, as flat op lists ("specs") with seeded random int8
weights and per-tensor activation scales / zero points.

A spec is backend-neutral and building one loads no native library: ``to_case`` turns it into a
GPU case through the C-ABI (and loads ``libnart_b200.so`` when called); the tests walk the same spec
op by op over their CPU checkers.  BatchNorm is assumed folded into the convs, the way the reference's exporter emits
quantized cases (python/nart/modules/quant.py of ModelTC/NART); ReLU after a conv or a residual
add is the fused clamp at the output zero point.
"""
from __future__ import annotations

import math

import numpy as np

# SETTING_POOL_MAX / SETTING_POOL_AVE (art/include/art/op_settings.h:62-63) and B200_CONV_ALGO_AUTO; the
# same values as in ._lib, repeated here so that importing this module loads no shared library
POOL_MAX, POOL_AVE = 0, 1
ALGO_AUTO = 0


class SpecBuilder:
    """Collects ops; every tensor carries (c, h, w, alpha, zp)."""

    def __init__(self, seed: int, in_chw, spread: bool):
        self.rng = np.random.default_rng(seed)
        self.spread = spread
        self.ops = []
        self.tensors = {}
        self.in_chw = tuple(in_chw)
        c, h, w = in_chw
        # the image: uint8 U[0,255]; as a quantized tensor it needs a scale and a zero point
        # `std` is a rough standard deviation of the tensor in quantized units, used only to pick
        # scales that keep the next tensor spread over the uint8 range
        self.tensors["input"] = dict(c=c, h=h, w=w, alpha=float(np.float32(self.rng.uniform(0.01, 0.1))),
                                     zp=int(self.rng.integers(0, 256)), std=74.0)
        self._n = 0

    def _name(self, kind):
        self._n += 1
        return "%s%d" % (kind, self._n)

    def _out_quant(self, real_std, relu):
        """Output scale / zero point / spread estimate.  Benchmark form: alpha ~ U(0.01, 0.1),
        zp ~ U{0..255}.  With random weights that saturates most outputs, so the parity nets use
        ``spread``: a scale matched to the estimated spread of the real values, which keeps the
        quantized values distributed over the range layer after layer."""
        zp = int(self.rng.integers(0, 256))
        alpha = float(np.float32(self.rng.uniform(0.01, 0.1)))
        std = 60.0
        if self.spread:
            std = float(self.rng.uniform(30.0, 60.0))
            alpha = float(np.float32(real_std / std))
            zp = int(self.rng.integers(60, 180))
        if relu:
            std *= 0.6
        return alpha, zp, std

    def conv(self, tin, k, ksize, stride, pad, group=1, relu=True):
        ti = self.tensors[tin]
        c = ti["c"]
        cg = c // group
        w = (self.rng.integers(-127, 128, (k, cg, ksize, ksize)) + 128).astype(np.uint8)
        bias = self.rng.integers(-4096, 4097, k).astype(np.int32)
        walpha = self.rng.uniform(0.001, 0.01, k).astype(np.float32)
        real_std = ti["alpha"] * ti["std"] * float(walpha.mean()) * 73.0 * math.sqrt(cg * ksize * ksize)
        oalpha, ozp, ostd = self._out_quant(real_std, relu)
        oh = (ti["h"] + 2 * pad - ksize) // stride + 1
        ow = (ti["w"] + 2 * pad - ksize) // stride + 1
        out = self._name("conv")
        self.tensors[out] = dict(c=k, h=oh, w=ow, alpha=oalpha, zp=ozp, std=ostd)
        self.ops.append(dict(op="conv", ins=[tin], out=out, w=w, bias=bias, walpha=walpha, stride=stride,
                             pad=pad, group=group, relu=relu))
        return out

    def pool(self, tin, method, ksize, stride, pad, ceil_mode=False):
        ti = self.tensors[tin]
        out = self._name("pool")
        v = (ti["h"] + 2 * pad - ksize) / stride + 1
        o = int(math.ceil(v) if ceil_mode else math.floor(v))
        if pad and (o - 1) * stride >= ti["h"] + pad:
            o -= 1
        # max-pool keeps the quantization of its input; the average gets a fresh output scale
        if method == POOL_MAX:
            alpha, zp, std = ti["alpha"], ti["zp"], ti["std"]
        else:
            # the mean of ksize^2 values is narrower: rescale so that it spreads again
            std = ti["std"]
            alpha = float(np.float32(ti["alpha"] * self.rng.uniform(0.5, 1.0) / (ksize if self.spread else 1)))
            zp = ti["zp"]
        self.tensors[out] = dict(c=ti["c"], h=o, w=o, alpha=alpha, zp=zp, std=std)
        self.ops.append(dict(op="pool", ins=[tin], out=out, method=method, ksize=ksize, stride=stride,
                             pad=pad, ceil_mode=ceil_mode))
        return out

    def add(self, ta, tb, relu=True):
        a, b = self.tensors[ta], self.tensors[tb]
        zp = int(self.rng.integers(0, 256))
        alpha = float(np.float32(self.rng.uniform(0.01, 0.1)))
        std = 60.0
        if self.spread:
            std = float(self.rng.uniform(30.0, 60.0))
            alpha = float(np.float32(math.hypot(a["alpha"] * a["std"], b["alpha"] * b["std"]) / std))
            zp = int(self.rng.integers(60, 180))
        if relu:
            std *= 0.6
        out = self._name("add")
        self.tensors[out] = dict(c=a["c"], h=a["h"], w=a["w"], alpha=alpha, zp=zp, std=std)
        self.ops.append(dict(op="eltwise", ins=[ta, tb], out=out, relu=relu))
        return out

    def ip(self, tin, k):
        ti = self.tensors[tin]
        chw = ti["c"] * ti["h"] * ti["w"]
        w = (self.rng.integers(-127, 128, (k, chw)) + 128).astype(np.uint8)
        bias = self.rng.integers(-4096, 4097, k).astype(np.int32)
        walpha = self.rng.uniform(0.001, 0.01, k).astype(np.float32)
        real_std = ti["alpha"] * ti["std"] * float(walpha.mean()) * 73.0 * math.sqrt(chw)
        oalpha, ozp, ostd = self._out_quant(real_std, False)
        out = self._name("ip")
        self.tensors[out] = dict(c=k, h=1, w=1, alpha=oalpha, zp=ozp, std=ostd)
        self.ops.append(dict(op="ip", ins=[tin], out=out, w=w, bias=bias, walpha=walpha))
        return out

    def finish(self, name, out, conv_macs_note=""):
        return dict(name=name, in_chw=self.in_chw, ops=self.ops, tensors=self.tensors, output=out)


def resnet(depth: int, seed: int = 2, hw: int = 224, spread: bool = False, width_div: int = 1,
           num_classes: int = 1000):
    """ResNet-18 / ResNet-50 v1.5.  ``width_div`` shrinks every width (test-sized nets)."""
    b = SpecBuilder(seed, (3, hw, hw), spread)
    wd = lambda c: max(16, c // width_div)
    t = b.conv("input", wd(64), 7, 2, 3)
    t = b.pool(t, POOL_MAX, 3, 2, 1, ceil_mode=False)
    if depth == 18:
        blocks, bottleneck = [2, 2, 2, 2], False
    elif depth == 50:
        blocks, bottleneck = [3, 4, 6, 3], True
    else:
        raise ValueError("depth must be 18 or 50")
    for stage, (nblk, width) in enumerate(zip(blocks, [64, 128, 256, 512])):
        width = wd(width)
        for i in range(nblk):
            stride = 2 if (stage > 0 and i == 0) else 1
            cin = b.tensors[t]["c"]
            if bottleneck:
                cout = width * 4
                u = b.conv(t, width, 1, 1, 0)
                u = b.conv(u, width, 3, stride, 1)
                u = b.conv(u, cout, 1, 1, 0, relu=False)
            else:
                cout = width
                u = b.conv(t, width, 3, stride, 1)
                u = b.conv(u, width, 3, 1, 1, relu=False)
            sc = t
            if stride != 1 or cin != cout:
                sc = b.conv(t, cout, 1, stride, 0, relu=False)
            t = b.add(u, sc, relu=True)
    t = b.pool(t, POOL_AVE, b.tensors[t]["h"], 1, 0)
    t = b.ip(t, num_classes)
    return b.finish("resnet%d" % depth, t)


def mobilenet_v2(seed: int = 4, hw: int = 224, spread: bool = False, num_classes: int = 1000):
    """MobileNetV2-1.0: inverted residuals with expansion 6.  The quant module has no ReLU6 op
    (art/modules/quant/src/quant_module.c:49-66), so the activations are the ReLU clamp."""
    b = SpecBuilder(seed, (3, hw, hw), spread)
    t = b.conv("input", 32, 3, 2, 1)
    cfg = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
    for expand, cout, reps, stride0 in cfg:
        for i in range(reps):
            stride = stride0 if i == 0 else 1
            cin = b.tensors[t]["c"]
            u = t
            if expand != 1:
                u = b.conv(u, cin * expand, 1, 1, 0)
            u = b.conv(u, cin * expand, 3, stride, 1, group=cin * expand)
            u = b.conv(u, cout, 1, 1, 0, relu=False)
            t = b.add(u, t, relu=False) if (stride == 1 and cin == cout) else u
    t = b.conv(t, 1280, 1, 1, 0)
    t = b.pool(t, POOL_AVE, b.tensors[t]["h"], 1, 0)
    t = b.ip(t, num_classes)
    return b.finish("mobilenet_v2", t)


def conv_ops_per_image(spec) -> float:
    """2 * MACs of the conv ops (true, unpadded dims); the FC (ip) is not counted."""
    total = 0.0
    for op in spec["ops"]:
        if op["op"] == "conv":
            to = spec["tensors"][op["out"]]
            k, cg, r, s = op["w"].shape
            total += 2.0 * to["h"] * to["w"] * k * cg * r * s
    return total


def to_case(spec, max_batch: int, algo: int = ALGO_AUTO, output_f32: bool = True, extra_outputs=(),
            fuse: bool = False):
    """Builds and prepares the GPU case.  Returns (case, tensor-id map).  ``fuse`` True folds the
    residual adds into the convs that feed them (see b200_case_set_fusion)."""
    from .case import Case
    cs = Case()
    cs.set_fusion(fuse)
    T = spec["tensors"]
    c, h, w = spec["in_chw"]
    ids = {"input": cs.input_u8(c, h, w)}
    for op in spec["ops"]:
        ti = T[op["ins"][0]]
        to = T[op["out"]]
        if op["op"] == "conv":
            ids[op["out"]] = cs.conv2d(
                ids[op["ins"][0]], op["w"], op["bias"], stride=(op["stride"],) * 2, pad=(op["pad"],) * 2,
                group=op["group"], ialpha=ti["alpha"], izp=ti["zp"], walpha=op["walpha"], oalpha=to["alpha"],
                ozp=to["zp"], relu=op["relu"], algo=algo)
        elif op["op"] == "ip":
            ids[op["out"]] = cs.ip(ids[op["ins"][0]], op["w"], op["bias"], ialpha=ti["alpha"], izp=ti["zp"],
                                   walpha=op["walpha"], oalpha=to["alpha"], ozp=to["zp"])
        elif op["op"] == "pool":
            ids[op["out"]] = cs.pool(ids[op["ins"][0]], op["method"], (op["ksize"],) * 2, (op["pad"],) * 2,
                                     (op["stride"],) * 2, op["ceil_mode"], ti["alpha"], ti["zp"], to["alpha"], to["zp"])
        elif op["op"] == "eltwise":
            ins = [T[n] for n in op["ins"]]
            ids[op["out"]] = cs.eltwise_sum([ids[n] for n in op["ins"]], [t["alpha"] for t in ins],
                                            [t["zp"] for t in ins], to["alpha"], to["zp"], relu=op["relu"])
        else:
            raise ValueError(op["op"])
    out = T[spec["output"]]
    if output_f32:
        cs.output_f32(ids[spec["output"]], out["alpha"], out["zp"])
    else:
        cs.output_u8(ids[spec["output"]])
    for name in extra_outputs:
        cs.output_u8(ids[name])
    cs.prepare(max_batch)
    return cs, ids
