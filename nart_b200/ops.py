"""Host-side mirror of the reference's quant operator interface on top of the C-ABI.

Names and argument meaning follow the art ``quant`` module's ops (conv_2d, ip, quantize,
dequantize, eltwise, add, relu, pool -- art/modules/quant/src/quant_module.c:49-66 of
ModelTC/NART) and their ``SETTING_QUANT_*`` settings (ialpha/izp, walpha/wzp, oalpha/ozp/obits).
torch is used only to own device memory and to name the current stream; all compute goes through
``libnart_b200.so``.  Device activations are uint8 NHWC ``[N, H, W, C]`` tensors.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import ACT_S8, ACT_U8, ALGO_AUTO, ALGO_DIRECT, ALGO_IGEMM, POOL_AVE, POOL_MAX, ConvParams, check, lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev_u8(t: torch.Tensor) -> torch.Tensor:
    if not (t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous()):
        raise ValueError("expected a contiguous uint8 CUDA tensor")
    return t


def _dev_s8(t: torch.Tensor) -> torch.Tensor:
    if not (t.is_cuda and t.dtype == torch.int8 and t.is_contiguous()):
        raise ValueError("expected a contiguous int8 CUDA tensor")
    return t


def get_quant_scale(x: float, bits: int):
    m, s = C.c_uint32(0), C.c_int8(0)
    lib.b200_get_quant_scale(x, bits, C.byref(m), C.byref(s))
    return m.value, s.value


def _walpha_array(walpha, k):
    wa = np.atleast_1d(np.asarray(walpha, dtype=np.float32)).copy()
    if wa.size not in (1, k):
        raise ValueError("walpha must have 1 or k entries")
    return wa


class Conv2d:
    """conv_2d of the quant module (op_quant_conv_2d_tp_* + op_conv_2d_u8xu8_run).

    ``weight``: uint8 ``[K, C/group, R, S]`` (int8 value + 128, ``wzp`` = 128); ``bias``: int32
    ``[K]`` or None; ``in_hw``: input height and width the plan is prepared for.
    """

    def __init__(self, weight, bias, *, in_hw, stride=(1, 1), pad=(0, 0), group=1, ialpha, izp=0,
                 walpha, wzp=128, oalpha, ozp=0, obits=8, relu=False, algo=ALGO_AUTO, signed=False,
                 s8_wrap=False):
        """``signed`` True selects the reference's int8 (dtINT8) path: int8 weights, int8 NHWC activations in
        and out, no zero points; ``s8_wrap`` accepts obits == 8 with the reference's wrapping cast."""
        self.signed = bool(signed)
        w = np.ascontiguousarray(weight, dtype=np.int8 if signed else np.uint8)
        k, cg, r, s = w.shape
        self.k, self.c = k, cg * group
        wa = _walpha_array(walpha, k)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        p = ConvParams()
        p.c, p.h, p.w, p.k, p.r, p.s = self.c, in_hw[0], in_hw[1], k, r, s
        p.pad_h, p.pad_w, p.stride_h, p.stride_w, p.group = pad[0], pad[1], stride[0], stride[1], group
        p.ialpha, p.izp, p.wzp, p.ozp, p.obits, p.oalpha = ialpha, izp, wzp, ozp, obits, oalpha
        p.walpha = wa.ctypes.data_as(C.POINTER(C.c_float))
        p.n_walpha, p.relu, p.algo = wa.size, int(relu), algo
        p.act_type, p.s8_wrap = (ACT_S8 if signed else ACT_U8), int(s8_wrap)
        self._h = C.c_void_p()
        check(lib.b200_conv2d_create(
            C.byref(p), w.ctypes.data, None if b is None else b.ctypes.data, C.byref(self._h)))
        oh, ow = C.c_int32(), C.c_int32()
        check(lib.b200_conv2d_out_dims(self._h, C.byref(oh), C.byref(ow)))
        self.in_hw, self.out_hw = tuple(in_hw), (oh.value, ow.value)
        self.algo = lib.b200_conv2d_algo(self._h)

    def __call__(self, x: torch.Tensor, return_acc: bool = False):
        _dev_s8(x) if self.signed else _dev_u8(x)
        n, h, w, c = x.shape
        if (h, w) != self.in_hw or c != self.c:
            raise ValueError("input %s does not match the prepared plan" % (tuple(x.shape),))
        y = torch.empty((n, self.out_hw[0], self.out_hw[1], self.k), dtype=x.dtype, device=x.device)
        if return_acc:
            acc = torch.empty(y.shape, dtype=torch.int32, device=x.device)
            check(lib.b200_conv2d_run_acc(self._h, x.data_ptr(), n, y.data_ptr(), acc.data_ptr(), _stream()))
            return y, acc
        check(lib.b200_conv2d_run(self._h, x.data_ptr(), n, y.data_ptr(), _stream()))
        return y

    def describe(self) -> str:
        buf = C.create_string_buffer(256)
        check(lib.b200_conv2d_describe(self._h, buf, 256))
        return buf.value.decode()

    def fuse_residual_add(self, conv_input, ialpha, izp, oalpha, ozp, obits=8, coeff=None, relu=False):
        """Folds ``eltwise_sum((conv(x), res)[order], ...)`` into this plan (b200_conv2d_fuse_residual_add);
        raises B200Error (status ERR_UNSUPPORTED) when the plan cannot take it."""
        ia = (C.c_float * 2)(*[float(a) for a in ialpha])
        iz = (C.c_uint8 * 2)(*[int(z) for z in izp])
        cf = None if coeff is None else (C.c_float * 2)(*[float(v) for v in coeff])
        check(lib.b200_conv2d_fuse_residual_add(self._h, int(conv_input), ia, iz, cf, float(oalpha), int(ozp),
                                                int(obits), int(relu)))

    def run_residual(self, x: torch.Tensor, res: torch.Tensor):
        """y = eltwise_sum(conv(x), res) of a fused plan; res is NHWC with the output's shape."""
        _dev_u8(x)
        _dev_u8(res)
        n = x.shape[0]
        y = torch.empty((n, self.out_hw[0], self.out_hw[1], self.k), dtype=torch.uint8, device=x.device)
        if tuple(res.shape) != tuple(y.shape):
            raise ValueError("residual %s does not match the output %s" % (tuple(res.shape), tuple(y.shape)))
        check(lib.b200_conv2d_run_residual(self._h, x.data_ptr(), n, res.data_ptr(), y.data_ptr(), _stream()))
        return y

    def close(self):
        if self._h:
            lib.b200_conv2d_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class InnerProduct(Conv2d):
    """ip of the quant module (op_quant_ip_u8xu8_run): ``weight`` uint8 ``[K, C*H*W]`` in the
    reference's flattened NCHW column order; input NHWC ``[N, H, W, C]``, output ``[N, 1, 1, K]``."""

    def __init__(self, weight, bias, *, in_chw, ialpha, izp, walpha, wzp=128, oalpha, ozp, obits=8):
        c, h, w = in_chw
        wt = np.ascontiguousarray(weight, dtype=np.uint8)
        k = wt.shape[0]
        self.k, self.c, self.signed = k, c, False
        wa = _walpha_array(walpha, k)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        self._h = C.c_void_p()
        check(lib.b200_ip_create(
            c, h, w, k, ialpha, izp, wa.ctypes.data_as(C.POINTER(C.c_float)), wa.size, wzp, oalpha,
            ozp, obits, wt.ctypes.data, None if b is None else b.ctypes.data, C.byref(self._h)))
        self.in_hw, self.out_hw = (h, w), (1, 1)
        self.algo = lib.b200_conv2d_algo(self._h)


class InnerProductS8(Conv2d):
    """ip of the quant module on int8 activations (op_quant_ip_i8xi8_run): ``weight`` int8 ``[K, C*H*W]``."""

    def __init__(self, weight, bias, *, in_chw, ialpha, walpha, oalpha, obits=7, s8_wrap=False):
        c, h, w = in_chw
        wt = np.ascontiguousarray(weight, dtype=np.int8)
        k = wt.shape[0]
        self.k, self.c, self.signed = k, c, True
        wa = _walpha_array(walpha, k)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        self._h = C.c_void_p()
        check(lib.b200_ip_create_s8(
            c, h, w, k, ialpha, wa.ctypes.data_as(C.POINTER(C.c_float)), wa.size, oalpha, obits, int(s8_wrap),
            wt.ctypes.data, None if b is None else b.ctypes.data, C.byref(self._h)))
        self.in_hw, self.out_hw = (h, w), (1, 1)
        self.algo = lib.b200_conv2d_algo(self._h)


def quantize_s8(x: torch.Tensor, oalpha: float, obits: int = 8, nhwc: bool = True):
    """quantize with qtype SYMMETRIC: float32 NCHW -> int8 (NHWC by default)."""
    if not (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 4):
        raise ValueError("expected a contiguous float32 NCHW CUDA tensor")
    n, c, h, w = x.shape
    y = torch.empty((n, h, w, c) if nhwc else (n, c, h, w), dtype=torch.int8, device=x.device)
    check(lib.b200_quantize_s8(x.data_ptr(), y.data_ptr(), n, c, h, w, oalpha, obits, int(nhwc), _stream()))
    return y


def dequantize_s8(x: torch.Tensor, ialpha: float, nhwc: bool = True):
    """dequantize of an int8 tensor (NHWC by default) -> float32 NCHW."""
    _dev_s8(x)
    if nhwc:
        n, h, w, c = x.shape
    else:
        n, c, h, w = x.shape
    y = torch.empty((n, c, h, w), dtype=torch.float32, device=x.device)
    check(lib.b200_dequantize_s8(x.data_ptr(), y.data_ptr(), n, c, h, w, ialpha, int(nhwc), _stream()))
    return y


def quantize(x: torch.Tensor, oalpha: float, ozp: int, obits: int = 8, nhwc: bool = True):
    """quantize: float32 NCHW -> uint8 (NHWC by default, the device layout)."""
    if not (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 4):
        raise ValueError("expected a contiguous float32 NCHW CUDA tensor")
    n, c, h, w = x.shape
    y = torch.empty((n, h, w, c) if nhwc else (n, c, h, w), dtype=torch.uint8, device=x.device)
    check(lib.b200_quantize_u8(x.data_ptr(), y.data_ptr(), n, c, h, w, oalpha, ozp, obits, int(nhwc), _stream()))
    return y


def dequantize(x: torch.Tensor, ialpha: float, izp: int, nhwc: bool = True):
    """dequantize: uint8 (NHWC by default) -> float32 NCHW."""
    _dev_u8(x)
    if nhwc:
        n, h, w, c = x.shape
    else:
        n, c, h, w = x.shape
    y = torch.empty((n, c, h, w), dtype=torch.float32, device=x.device)
    check(lib.b200_dequantize_u8(x.data_ptr(), y.data_ptr(), n, c, h, w, ialpha, izp, int(nhwc), _stream()))
    return y


def nchw_to_nhwc(x: torch.Tensor, c_pad: int | None = None, fill: int = 0):
    _dev_u8(x)
    n, c, h, w = x.shape
    c_pad = c if c_pad is None else c_pad
    y = torch.empty((n, h, w, c_pad), dtype=torch.uint8, device=x.device)
    check(lib.b200_nchw_to_nhwc_u8(x.data_ptr(), y.data_ptr(), n, c, h, w, c_pad, fill, _stream()))
    return y


def nhwc_to_nchw(x: torch.Tensor, c: int | None = None):
    _dev_u8(x)
    n, h, w, c_pad = x.shape
    c = c_pad if c is None else c
    y = torch.empty((n, c, h, w), dtype=torch.uint8, device=x.device)
    check(lib.b200_nhwc_to_nchw_u8(x.data_ptr(), y.data_ptr(), n, c, h, w, c_pad, _stream()))
    return y


def eltwise_sum(xs, ialpha, izp, oalpha, ozp, obits: int = 8, coeff=None, relu: bool = False):
    """eltwise SUM / add of the quant module on same-shaped uint8 tensors."""
    xs = [_dev_u8(t) for t in xs]
    n = len(xs)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in xs])
    ia = (C.c_float * n)(*[float(a) for a in ialpha])
    iz = (C.c_uint8 * n)(*[int(z) for z in izp])
    cf = None if coeff is None else (C.c_float * n)(*[float(v) for v in coeff])
    y = torch.empty_like(xs[0])
    check(lib.b200_eltwise_sum_u8(ptrs, n, xs[0].numel(), ia, iz, cf, oalpha, ozp, obits, int(relu),
                                  y.data_ptr(), _stream()))
    return y


def add(x0, x1, ialpha, izp, oalpha, ozp, obits: int = 8):
    """add of the quant module: the two-input eltwise SUM."""
    return eltwise_sum([x0, x1], ialpha, izp, oalpha, ozp, obits)


def relu(x: torch.Tensor, ialpha, izp, oalpha, ozp, obits: int = 8):
    _dev_u8(x)
    y = torch.empty_like(x)
    check(lib.b200_relu_u8(x.data_ptr(), x.numel(), ialpha, izp, oalpha, ozp, obits, y.data_ptr(), _stream()))
    return y


def pool_out_dims(h, w, kernel, pad, stride, ceil_mode):
    oh, ow = C.c_int32(), C.c_int32()
    check(lib.b200_pool_out_dims(h, w, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1],
                                 int(ceil_mode), C.byref(oh), C.byref(ow)))
    return oh.value, ow.value


def pool(x: torch.Tensor, method: int, kernel, pad, stride, ceil_mode, ialpha, izp, oalpha, ozp,
         obits: int = 8):
    """pool of the quant module (method POOL_MAX / POOL_AVE) on a uint8 NHWC tensor."""
    _dev_u8(x)
    n, h, w, c = x.shape
    oh, ow = pool_out_dims(h, w, kernel, pad, stride, ceil_mode)
    y = torch.empty((n, oh, ow, c), dtype=torch.uint8, device=x.device)
    check(lib.b200_pool_u8(x.data_ptr(), n, c, h, w, method, kernel[0], kernel[1], pad[0], pad[1],
                           stride[0], stride[1], int(ceil_mode), ialpha, izp, oalpha, ozp, obits,
                           y.data_ptr(), _stream()))
    return y


def device_status() -> int:
    """Reads and clears the status word of the kernels' bounded waits (0 = none ran out)."""
    w = C.c_int(0)
    check(lib.b200_device_status(_stream(), C.byref(w)))
    return w.value
