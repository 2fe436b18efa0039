"""Serialized cases of NART's art runtime ("engine.bin", format version 2) for the quantized path:
a writer that turns one of this package's network specs into a file the reference's own loader
accepts, a reader, and a builder that runs a read file on the GPU case runner.

Layout (art/src/serialize_v2.c:26-103 and the writer src/serialize.cpp:181-306 of ModelTC/NART;
integers are raw little-endian host ints, a string is int32 length + bytes, art/src/serialize.c:162-184):

    head      int32 version (2), string name
    tensors   int32 tensor count (inputs + weights + every op output)
              inputs : int32 n, then per input  uint32 dtype, string name, shape, int32 has_transform (0)
              weights: int32 n, then per weight uint32 dtype, string name, shape, raw data
              shape  : int32 dim_size, int32 dims[dim_size], int32 channel_axis, int32 batch_axis
                       (src/serialize.cpp:54-58, reader art/src/serialize.c:230-240)
    ops       int32 n, then per op: int32 inputs (data inputs, then weight / bias tensors), int32 outputs,
              uint64 op code, int32 input tensor indices, int32 setting count, settings
              setting: int32 repeated, int32 item, int32 dtype, then the value, or int32 count + values
    outputs   int32 n, then per output int32 tensor index, string name
    shares    int32 n (0)

Tensor indices count the inputs first, then the weights, then the outputs of the ops in op order.
"""
from __future__ import annotations

import struct

import numpy as np

# ---- numeric codes of the reference's headers ------------------------------------------------------
# art/include/art/data_type.h
DT_INT8, DT_INT16, DT_INT32, DT_UINT8, DT_UINT16, DT_UINT32 = 1, 2, 3, 5, 6, 7
DT_FLOAT16, DT_FLOAT32, DT_FLOAT64, DT_STR, DT_BOOL = 9, 10, 11, 12, 15
_DT_NUMPY = {DT_INT8: np.int8, DT_INT16: np.int16, DT_INT32: np.int32, DT_UINT8: np.uint8, DT_UINT16: np.uint16,
             DT_UINT32: np.uint32, DT_FLOAT16: np.float16, DT_FLOAT32: np.float32, DT_FLOAT64: np.float64,
             DT_BOOL: np.uint8}
# art/include/art/op_tp.h; quantize / dequantize: art/modules/quant/include/art/quant/quant_op_tp.h:23-24
OP_GROUP_QUANT = 6
OP_ADD, OP_CONV_2D, OP_RELU, OP_POOL, OP_IP, OP_ELTWISE = 0x11, 0x100, 0x101, 0x102, 0x104, 0x10C
OP_QUANT_QUANTIZE = (OP_GROUP_QUANT << 32) | 0x80000000
OP_QUANT_DEQUANTIZE = (OP_GROUP_QUANT << 32) | 0x80000001
# art/include/art/op_settings.h
CONV_NUM_OUTPUT, CONV_PAD_H, CONV_PAD_W, CONV_KERNEL_H, CONV_KERNEL_W = 1, 2, 3, 4, 5
CONV_STRIDE_H, CONV_STRIDE_W, CONV_GROUP, CONV_RELU_FLAG = 6, 7, 8, 9
IP_NUM_OUTPUT = 1
ELTWISE_OPERATION, ELTWISE_COEFF, ELTWISE_OP_SUM = 1, 2, 1
POOL_METHOD, POOL_PAD_H, POOL_PAD_W, POOL_KERNEL_H, POOL_KERNEL_W = 1, 2, 3, 4, 5
POOL_STRIDE_H, POOL_STRIDE_W, POOL_CEIL_MODE = 6, 7, 8
POOL_MAX, POOL_AVE = 0, 1
# art/modules/quant/include/art/quant/quant_op_settings.h:26-40
Q_IALPHA, Q_IZERO_POINT, Q_IBITS = 0x00060101, 0x00060102, 0x00060103
Q_WALPHA, Q_WZERO_POINT, Q_WBITS = 0x00060104, 0x00060105, 0x00060106
Q_OALPHA, Q_OZERO_POINT, Q_OBITS = 0x00060107, 0x00060108, 0x00060109
Q_QTYPE, Q_BIASED = 0x0006010A, 1

# name -> value, for the test that pins this table to the compiled reference headers
CONSTANTS = {
    "OP_CONV_2D": OP_CONV_2D, "OP_IP": OP_IP, "OP_ELTWISE": OP_ELTWISE, "OP_ADD": OP_ADD, "OP_RELU": OP_RELU,
    "OP_POOL": OP_POOL, "OP_QUANT_QUANTIZE": OP_QUANT_QUANTIZE, "OP_QUANT_DEQUANTIZE": OP_QUANT_DEQUANTIZE,
    "SETTING_CONV_2D_RELU_FLAG": CONV_RELU_FLAG, "SETTING_CONV_2D_NUM_OUTPUT": CONV_NUM_OUTPUT,
    "SETTING_CONV_2D_KERNEL_H": CONV_KERNEL_H, "SETTING_CONV_2D_KERNEL_W": CONV_KERNEL_W,
    "SETTING_CONV_2D_PAD_H": CONV_PAD_H, "SETTING_CONV_2D_PAD_W": CONV_PAD_W,
    "SETTING_CONV_2D_STRIDE_H": CONV_STRIDE_H, "SETTING_CONV_2D_STRIDE_W": CONV_STRIDE_W,
    "SETTING_CONV_2D_GROUP": CONV_GROUP, "SETTING_IP_NUM_OUTPUT": IP_NUM_OUTPUT,
    "SETTING_ELTWISE_OPERATION": ELTWISE_OPERATION, "SETTING_ELTWISE_OP_SUM": ELTWISE_OP_SUM,
    "SETTING_ELTWISE_COEFF": ELTWISE_COEFF, "SETTING_POOL_METHOD": POOL_METHOD,
    "SETTING_POOL_KERNEL_H": POOL_KERNEL_H, "SETTING_POOL_KERNEL_W": POOL_KERNEL_W,
    "SETTING_POOL_PAD_H": POOL_PAD_H, "SETTING_POOL_PAD_W": POOL_PAD_W, "SETTING_POOL_STRIDE_H": POOL_STRIDE_H,
    "SETTING_POOL_STRIDE_W": POOL_STRIDE_W, "SETTING_POOL_CEIL_MODE": POOL_CEIL_MODE,
    "SETTING_POOL_MAX": POOL_MAX, "SETTING_POOL_AVE": POOL_AVE,
    "SETTING_QUANT_IALPHA": Q_IALPHA, "SETTING_QUANT_IZERO_POINT": Q_IZERO_POINT, "SETTING_QUANT_IBITS": Q_IBITS,
    "SETTING_QUANT_OALPHA": Q_OALPHA, "SETTING_QUANT_OZERO_POINT": Q_OZERO_POINT, "SETTING_QUANT_OBITS": Q_OBITS,
    "SETTING_QUANT_WALPHA": Q_WALPHA, "SETTING_QUANT_WZERO_POINT": Q_WZERO_POINT, "SETTING_QUANT_WBITS": Q_WBITS,
    "SETTING_QUANT_QTYPE": Q_QTYPE, "SETTING_QUANT_BIASED": Q_BIASED,
    "dtUINT8": DT_UINT8, "dtINT8": DT_INT8, "dtUINT32": DT_UINT32, "dtINT32": DT_INT32, "dtFLOAT32": DT_FLOAT32,
    "dtBOOL": DT_BOOL, "dtSTR": DT_STR,
}


# ---- writer --------------------------------------------------------------------------------------
class _Out:
    def __init__(self):
        self.parts = []

    def i32(self, v):
        self.parts.append(struct.pack("<i", int(v)))

    def u64(self, v):
        self.parts.append(struct.pack("<Q", int(v)))

    def string(self, s):
        b = (s or "").encode()
        self.i32(len(b))
        self.parts.append(b)

    def shape(self, dims):
        self.i32(len(dims))
        for d in dims:
            self.i32(d)
        self.i32(1 if len(dims) > 1 else 0)   # channel_axis
        self.i32(0)                           # batch_axis

    def raw(self, arr):
        self.parts.append(np.ascontiguousarray(arr).tobytes())

    def single(self, item, dtype, value):
        self.i32(0)
        self.i32(item)
        self.i32(dtype)
        self.raw(np.asarray([value], dtype=_DT_NUMPY[dtype]))

    def array(self, item, dtype, values):
        a = np.asarray(values, dtype=_DT_NUMPY[dtype]).ravel()
        self.i32(1)
        self.i32(item)
        self.i32(dtype)
        self.i32(a.size)
        self.raw(a)

    def bytes(self):
        return b"".join(self.parts)


def write_engine(spec, path, batch=1, per_channel=True, conv_relu_flag=True):
    """Writes ``spec`` (nart_b200.nets) as an engine.bin for a module of op group QUANT: uint8 NCHW
    input, the ops in order, the logits dequantized to float32.

    ``per_channel`` False stores one weight scale per layer (walpha[0]) -- all the reference's CPU
    module reads.  ``conv_relu_flag`` False writes the activation of a conv as a relu op of its own
    with equal input and output scale, which the CPU module executes (it ignores
    SETTING_CONV_2D_RELU_FLAG); True sets the flag, as exports for the reference's GPU module do.
    """
    T = spec["tensors"]
    c, h, w = spec["in_chw"]
    weights = []          # (dtype, name, array)
    ops = []              # (code, data input names, weight indices, n settings, settings writer, out name)
    for op in spec["ops"]:
        ti, to = T[op["ins"][0]], T[op["out"]]
        kind = op["op"]
        if kind in ("conv", "ip"):
            wt = np.ascontiguousarray(op["w"], dtype=np.uint8)
            k = wt.shape[0]
            if kind == "ip":
                wt = wt.reshape(k, -1, 1, 1)
            bias = np.zeros(k, np.int32) if op["bias"] is None else np.asarray(op["bias"], np.int32)
            wi = len(weights)
            weights.append((DT_UINT8, op["out"] + "_w", wt))
            weights.append((DT_INT32, op["out"] + "_b", bias))
            wa = np.asarray(op["walpha"], np.float32).ravel()
            wa = wa if per_channel else wa[:1]
            relu_as_op = kind == "conv" and op["relu"] and not conv_relu_flag

            def settings(o, op=op, kind=kind, ti=ti, to=to, wt=wt, wa=wa, k=k):
                n = 0
                if kind == "conv":
                    for item, v in ((CONV_NUM_OUTPUT, k), (CONV_KERNEL_H, wt.shape[2]), (CONV_KERNEL_W, wt.shape[3]),
                                    (CONV_PAD_H, op["pad"]), (CONV_PAD_W, op["pad"]), (CONV_STRIDE_H, op["stride"]),
                                    (CONV_STRIDE_W, op["stride"]), (CONV_GROUP, op["group"])):
                        o.single(item, DT_UINT32, v)
                        n += 1
                    if op["relu"] and conv_relu_flag:
                        o.single(CONV_RELU_FLAG, DT_BOOL, 1)
                        n += 1
                else:
                    o.single(IP_NUM_OUTPUT, DT_UINT32, k)
                    n += 1
                # one entry per op input, the weight and bias slots included (python/nart/modules/quant.py:175-215)
                o.array(Q_IALPHA, DT_FLOAT32, [ti["alpha"], wa[0], 1.0])
                o.array(Q_IZERO_POINT, DT_UINT8, [ti["zp"], 128, 0])
                o.array(Q_IBITS, DT_UINT8, [8, 8, 32])
                o.array(Q_WALPHA, DT_FLOAT32, wa)
                o.array(Q_WZERO_POINT, DT_UINT8, [128])
                o.array(Q_WBITS, DT_UINT8, [8])
                o.array(Q_OALPHA, DT_FLOAT32, [to["alpha"]])
                o.array(Q_OZERO_POINT, DT_UINT8, [to["zp"]])
                o.array(Q_OBITS, DT_UINT8, [8])
                return n + 9

            code = OP_CONV_2D if kind == "conv" else OP_IP
            if relu_as_op:
                ops.append((code, [op["ins"][0]], [wi, wi + 1], settings, op["out"] + "_pre"))
                ops.append((OP_RELU, [op["out"] + "_pre"], [], _act_settings([to], to), op["out"]))
            else:
                ops.append((code, [op["ins"][0]], [wi, wi + 1], settings, op["out"]))
        elif kind == "pool":
            def settings(o, op=op, ti=ti, to=to):
                for item, v in ((POOL_METHOD, op["method"]), (POOL_KERNEL_H, op["ksize"]), (POOL_KERNEL_W, op["ksize"]),
                                (POOL_PAD_H, op["pad"]), (POOL_PAD_W, op["pad"]), (POOL_STRIDE_H, op["stride"]),
                                (POOL_STRIDE_W, op["stride"])):
                    o.single(item, DT_UINT32, v)
                o.single(POOL_CEIL_MODE, DT_BOOL, int(bool(op["ceil_mode"])))
                return 8 + _act_settings([ti], to)(o)
            ops.append((OP_POOL, [op["ins"][0]], [], settings, op["out"]))
        elif kind == "eltwise":
            tis = [T[n] for n in op["ins"]]

            def settings(o, op=op, tis=tis, to=to):
                o.single(ELTWISE_OPERATION, DT_UINT32, ELTWISE_OP_SUM)
                n = 1 + _act_settings(tis, to)(o)
                return n
            if op["relu"]:
                # the add's ReLU as an op of its own, with equal scales: what both modules execute
                ops.append((OP_ELTWISE, list(op["ins"]), [], settings, op["out"] + "_pre"))
                ops.append((OP_RELU, [op["out"] + "_pre"], [], _act_settings([to], to), op["out"]))
            else:
                ops.append((OP_ELTWISE, list(op["ins"]), [], settings, op["out"]))
        else:
            raise ValueError("engine writer: op %r" % kind)
    out_t = T[spec["output"]]
    ops.append((OP_QUANT_DEQUANTIZE, [spec["output"]], [], _dequant_settings(out_t), "logits"))

    o = _Out()
    o.i32(2)
    o.string("")
    n_out = len(ops)
    o.i32(1 + len(weights) + n_out)
    o.i32(1)
    o.i32(DT_UINT8)
    o.string("input")
    o.shape([batch, c, h, w])
    o.i32(0)
    o.i32(len(weights))
    for dtype, name, arr in weights:
        o.i32(dtype)
        o.string(name)
        o.shape(list(arr.shape))
        o.raw(arr)
    index = {"input": 0}
    next_index = 1 + len(weights)
    o.i32(len(ops))
    for code, ins, widx, settings, out_name in ops:
        o.i32(len(ins) + len(widx))
        o.i32(1)
        o.u64(code if code >> 32 else (OP_GROUP_QUANT << 32) | code)
        for n in ins:
            o.i32(index[n])
        for wi in widx:
            o.i32(1 + wi)
        body = _Out()
        count = settings(body)
        o.i32(count)
        o.parts.extend(body.parts)
        index[out_name] = next_index
        next_index += 1
    o.i32(1)
    o.i32(index["logits"])
    o.string("logits")
    o.i32(0)
    with open(path, "wb") as f:
        f.write(o.bytes())


def _act_settings(tis, to):
    def settings(o):
        o.array(Q_IALPHA, DT_FLOAT32, [t["alpha"] for t in tis])
        o.array(Q_IZERO_POINT, DT_UINT8, [t["zp"] for t in tis])
        o.array(Q_IBITS, DT_UINT8, [8] * len(tis))
        o.array(Q_OALPHA, DT_FLOAT32, [to["alpha"]])
        o.array(Q_OZERO_POINT, DT_UINT8, [to["zp"]])
        o.array(Q_OBITS, DT_UINT8, [8])
        return 6
    return settings


def _dequant_settings(ti):
    def settings(o):
        o.array(Q_IALPHA, DT_FLOAT32, [ti["alpha"]])
        o.array(Q_IZERO_POINT, DT_UINT8, [ti["zp"]])
        o.array(Q_IBITS, DT_UINT8, [8])
        o.single(Q_QTYPE, DT_INT32, Q_BIASED)
        return 4
    return settings


# ---- reader --------------------------------------------------------------------------------------
class _In:
    def __init__(self, data):
        self.d = data
        self.p = 0

    def i32(self):
        v = struct.unpack_from("<i", self.d, self.p)[0]
        self.p += 4
        return v

    def u64(self):
        v = struct.unpack_from("<Q", self.d, self.p)[0]
        self.p += 8
        return v

    def string(self):
        n = self.i32()
        s = self.d[self.p:self.p + n].decode()
        self.p += n
        return s

    def shape(self):
        n = self.i32()
        dims = [self.i32() for _ in range(n)]
        self.i32()
        self.i32()
        return dims

    def raw(self, dtype, count):
        a = np.frombuffer(self.d, dtype=_DT_NUMPY[dtype], count=count, offset=self.p).copy()
        self.p += a.nbytes
        return a


def read_engine(path):
    """Parses a version-2 engine.bin into ``dict(inputs, weights, ops, outputs)``; tensors are
    referred to by their index in the file's numbering."""
    with open(path, "rb") as f:
        r = _In(f.read())
    version = r.i32()
    name = r.string()
    if version != 2:
        raise ValueError("engine.bin version %d is not supported (only 2)" % version)
    n_tensors = r.i32()
    inputs, weights = [], {}
    for _ in range(r.i32()):
        dtype, tname, dims = r.i32(), r.string(), r.shape()
        if r.i32():
            raise ValueError("input %r carries a preprocessing transform, which this reader does not support" % tname)
        inputs.append(dict(index=len(inputs), dtype=dtype, name=tname, dims=dims))
    base = len(inputs)
    for i in range(r.i32()):
        dtype, tname, dims = r.i32(), r.string(), r.shape()
        weights[base + i] = dict(dtype=dtype, name=tname, data=r.raw(dtype, int(np.prod(dims))).reshape(dims))
    next_index = base + len(weights)
    ops = []
    for _ in range(r.i32()):
        n_in, n_out, code = r.i32(), r.i32(), r.u64()
        ins = [r.i32() for _ in range(n_in)]
        settings = {}
        for _ in range(r.i32()):
            repeated, item, dtype = r.i32(), r.i32() & 0xFFFFFFFF, r.i32()
            if dtype == DT_STR:
                settings[item] = [r.string() for _ in range(r.i32())] if repeated else r.string()
            elif repeated:
                settings[item] = r.raw(dtype, r.i32())
            else:
                settings[item] = r.raw(dtype, 1)[0]
        ops.append(dict(code=code, ins=ins, outs=list(range(next_index, next_index + n_out)), settings=settings))
        next_index += n_out
    outputs = [dict(index=r.i32(), name=r.string()) for _ in range(r.i32())]
    shares = [(r.i32(), r.i32()) for _ in range(r.i32())]
    if next_index != n_tensors:
        raise ValueError("engine.bin: %d tensors announced, %d found" % (n_tensors, next_index))
    return dict(name=name, inputs=inputs, weights=weights, ops=ops, outputs=outputs, shares=shares)


# ---- builder: a read file on the GPU case runner ---------------------------------------------------
def engine_to_case(model, max_batch, algo=0, fuse=False, input_chw=None):
    """Builds and prepares a ``Case`` from ``read_engine`` output.  Supported: one uint8 (or float32 +
    quantize) NCHW input; conv_2d, ip, pool, eltwise SUM, add, relu; outputs uint8 or dequantized
    float32.  ``input_chw`` replaces the input's recorded (C, H, W) -- the reshape the reference applies
    with parade_apply_reshape (art/src/parade.c:199-215); every later shape follows from the ops.
    Returns (case, list of (is_float32, per-image shape) per output)."""
    from .case import Case
    if len(model["inputs"]) != 1:
        raise ValueError("engine_to_case: exactly one input is supported")
    cs = Case()
    cs.set_fusion(fuse)
    inp = model["inputs"][0]
    _, c, h, w = inp["dims"]
    if input_chw is not None:
        c, h, w = (int(v) for v in input_chw)
    ids, quant = {}, {}            # file tensor index -> case tensor id / (alpha, zp) where known
    pending_f32 = inp["dtype"] == DT_FLOAT32
    if not pending_f32:
        if inp["dtype"] != DT_UINT8:
            raise ValueError("engine_to_case: input dtype %d" % inp["dtype"])
        ids[0] = cs.input_u8(c, h, w)
    W = model["weights"]
    f32_outputs = {}
    for op in model["ops"]:
        code, s, ins, out = op["code"], op["settings"], op["ins"], op["outs"][0]
        low = code & 0xFFFFFFFF if not (code & 0x80000000) else code
        ia, iz = s.get(Q_IALPHA), s.get(Q_IZERO_POINT)
        oa = float(s[Q_OALPHA][0]) if Q_OALPHA in s else None
        oz = int(s[Q_OZERO_POINT][0]) if Q_OZERO_POINT in s else None
        ob = int(s[Q_OBITS][0]) if Q_OBITS in s else 8
        if low == OP_QUANT_QUANTIZE:
            if not (pending_f32 and ins == [0]):
                raise ValueError("engine_to_case: quantize is supported on the float32 input only")
            ids[out] = cs.input_f32(c, h, w, oa, oz, ob)
            pending_f32 = False
        elif low == OP_QUANT_DEQUANTIZE:
            f32_outputs[out] = (ins[0], float(ia[0]), int(iz[0]))
        elif low in (OP_CONV_2D, OP_IP):
            wt = W[ins[1]]["data"]
            bias = W[ins[2]]["data"] if len(ins) > 2 else None
            kw = dict(ialpha=float(ia[0]), izp=int(iz[0]), walpha=np.asarray(s[Q_WALPHA], np.float32),
                      wzp=int(s[Q_WZERO_POINT][0]), oalpha=oa, ozp=oz, obits=ob)
            if low == OP_CONV_2D:
                ids[out] = cs.conv2d(ids[ins[0]], wt, bias, stride=(int(s[CONV_STRIDE_H]), int(s[CONV_STRIDE_W])),
                                     pad=(int(s.get(CONV_PAD_H, 0)), int(s.get(CONV_PAD_W, 0))),
                                     group=int(s.get(CONV_GROUP, 1)), relu=bool(s.get(CONV_RELU_FLAG, 0)), algo=algo, **kw)
            else:
                ids[out] = cs.ip(ids[ins[0]], wt.reshape(wt.shape[0], -1), bias, **kw)
        elif low == OP_POOL:
            ids[out] = cs.pool(ids[ins[0]], int(s[POOL_METHOD]), (int(s[POOL_KERNEL_H]), int(s[POOL_KERNEL_W])),
                               (int(s.get(POOL_PAD_H, 0)), int(s.get(POOL_PAD_W, 0))),
                               (int(s[POOL_STRIDE_H]), int(s[POOL_STRIDE_W])), bool(s.get(POOL_CEIL_MODE, 1)),
                               float(ia[0]), int(iz[0]), oa, oz, ob)
        elif low in (OP_ELTWISE, OP_ADD):
            if low == OP_ELTWISE and int(s.get(ELTWISE_OPERATION, ELTWISE_OP_SUM)) != ELTWISE_OP_SUM:
                raise ValueError("engine_to_case: only eltwise SUM is supported")
            coeff = [float(v) for v in s[ELTWISE_COEFF]] if ELTWISE_COEFF in s else None
            ids[out] = cs.eltwise_sum([ids[i] for i in ins], [float(a) for a in ia], [int(z) for z in iz], oa, oz, ob,
                                      coeff=coeff)
        elif low == OP_RELU:
            ids[out] = cs.relu(ids[ins[0]], float(ia[0]), int(iz[0]), oa, oz, ob)
        else:
            raise ValueError("engine_to_case: op code 0x%x is not on the quantized path" % code)
    outs = []
    for o in model["outputs"]:
        if o["index"] in f32_outputs:
            src, alpha, zp = f32_outputs[o["index"]]
            cs.output_f32(ids[src], alpha, zp)
            outs.append((True, cs.dims(ids[src])))
        else:
            cs.output_u8(ids[o["index"]])
            outs.append((False, cs.dims(ids[o["index"]])))
    cs.prepare(max_batch)
    return cs, outs
