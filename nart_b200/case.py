"""Python face of the C-ABI case runner (``b200_case_*``): a prepared op list bound to one GPU,
the counterpart of the reference's parade (art/src/parade.c:169-197 of ModelTC/NART).  Inputs
and outputs cross in the reference's NCHW layout as numpy arrays or pinned torch tensors."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import ConvParams, check, lib


class Case:
    def __init__(self):
        self._h = C.c_void_p()
        check(lib.b200_case_create(C.byref(self._h)))
        self._keep = []          # host arrays referenced while building
        self.n_inputs = 0
        self.n_outputs = 0
        self.max_batch = 0

    # ---- building ---------------------------------------------------------------------------
    def input_u8(self, c, h, w) -> int:
        t = C.c_int32()
        check(lib.b200_case_input_u8(self._h, c, h, w, C.byref(t)))
        self.n_inputs += 1
        return t.value

    def input_f32(self, c, h, w, oalpha, ozp, obits=8) -> int:
        t = C.c_int32()
        check(lib.b200_case_input_f32(self._h, c, h, w, oalpha, ozp, obits, C.byref(t)))
        self.n_inputs += 1
        return t.value

    def dims(self, tensor):
        c, h, w = C.c_int32(), C.c_int32(), C.c_int32()
        check(lib.b200_case_tensor_dims(self._h, tensor, C.byref(c), C.byref(h), C.byref(w)))
        return c.value, h.value, w.value

    def conv2d(self, tin, weight, bias, *, stride=(1, 1), pad=(0, 0), group=1, ialpha, izp, walpha,
               wzp=128, oalpha, ozp, obits=8, relu=False, algo=0) -> int:
        w = np.ascontiguousarray(weight, dtype=np.uint8)
        k, cg, r, s = w.shape
        c, h, wd = self.dims(tin)
        wa = np.atleast_1d(np.asarray(walpha, dtype=np.float32)).copy()
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        p = ConvParams()
        p.c, p.h, p.w, p.k, p.r, p.s = c, h, wd, k, r, s
        p.pad_h, p.pad_w, p.stride_h, p.stride_w, p.group = pad[0], pad[1], stride[0], stride[1], group
        p.ialpha, p.izp, p.wzp, p.ozp, p.obits, p.oalpha = ialpha, izp, wzp, ozp, obits, oalpha
        p.walpha = wa.ctypes.data_as(C.POINTER(C.c_float))
        p.n_walpha, p.relu, p.algo = wa.size, int(relu), algo
        t = C.c_int32()
        check(lib.b200_case_conv2d(self._h, tin, C.byref(p), w.ctypes.data,
                                   None if b is None else b.ctypes.data, C.byref(t)))
        return t.value

    def ip(self, tin, weight, bias, *, ialpha, izp, walpha, wzp=128, oalpha, ozp, obits=8) -> int:
        w = np.ascontiguousarray(weight, dtype=np.uint8)
        k = w.shape[0]
        wa = np.atleast_1d(np.asarray(walpha, dtype=np.float32)).copy()
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        t = C.c_int32()
        check(lib.b200_case_ip(self._h, tin, k, ialpha, izp, wa.ctypes.data_as(C.POINTER(C.c_float)),
                               wa.size, wzp, oalpha, ozp, obits, w.ctypes.data,
                               None if b is None else b.ctypes.data, C.byref(t)))
        return t.value

    def eltwise_sum(self, tins, ialpha, izp, oalpha, ozp, obits=8, coeff=None, relu=False) -> int:
        n = len(tins)
        ids = (C.c_int32 * n)(*tins)
        ia = (C.c_float * n)(*[float(a) for a in ialpha])
        iz = (C.c_uint8 * n)(*[int(z) for z in izp])
        cf = None if coeff is None else (C.c_float * n)(*[float(v) for v in coeff])
        t = C.c_int32()
        check(lib.b200_case_eltwise_sum(self._h, ids, n, ia, iz, cf, oalpha, ozp, obits, int(relu), C.byref(t)))
        return t.value

    def relu(self, tin, ialpha, izp, oalpha, ozp, obits=8) -> int:
        t = C.c_int32()
        check(lib.b200_case_relu(self._h, tin, ialpha, izp, oalpha, ozp, obits, C.byref(t)))
        return t.value

    def pool(self, tin, method, kernel, pad, stride, ceil_mode, ialpha, izp, oalpha, ozp, obits=8) -> int:
        t = C.c_int32()
        check(lib.b200_case_pool(self._h, tin, method, kernel[0], kernel[1], pad[0], pad[1], stride[0],
                                 stride[1], int(ceil_mode), ialpha, izp, oalpha, ozp, obits, C.byref(t)))
        return t.value

    def output_u8(self, tensor):
        check(lib.b200_case_output_u8(self._h, tensor))
        self.n_outputs += 1

    def output_f32(self, tensor, ialpha, izp):
        check(lib.b200_case_output_f32(self._h, tensor, ialpha, izp))
        self.n_outputs += 1

    def prepare(self, max_batch: int):
        check(lib.b200_case_prepare(self._h, max_batch))
        self.max_batch = max_batch

    # ---- running ----------------------------------------------------------------------------
    def io_bytes(self, is_output: bool, index: int) -> int:
        v = C.c_size_t()
        check(lib.b200_case_io_bytes(self._h, int(is_output), index, C.byref(v)))
        return v.value

    def io_device_ptr(self, is_output: bool, index: int) -> int:
        p = C.c_void_p()
        check(lib.b200_case_io_device_ptr(self._h, int(is_output), index, C.byref(p)))
        return p.value

    def tensor_device_ptr(self, tensor: int) -> int:
        p = C.c_void_p()
        check(lib.b200_case_tensor_device_ptr(self._h, tensor, C.byref(p)))
        return p.value

    def launch_count(self) -> int:
        v = C.c_int32()
        check(lib.b200_case_launch_count(self._h, C.byref(v)))
        return v.value

    def use_graph(self, enable: bool = True):
        """Replay run_device as one CUDA graph per batch size (see b200_case_use_graph)."""
        check(lib.b200_case_use_graph(self._h, int(enable)))

    def set_fusion(self, enable: bool):
        """Residual adds inside the feeding conv's epilogue (default off); call before prepare."""
        check(lib.b200_case_set_fusion(self._h, int(enable)))

    def set_profiling(self, enable: bool):
        check(lib.b200_case_set_profiling(self._h, int(enable)))

    def profile(self):
        """(ms, kind) per launch of the last profiled run, in launch order."""
        cap = self.launch_count()
        ms = (C.c_float * cap)()
        kinds = (C.c_int32 * cap)()
        n = C.c_int32()
        check(lib.b200_case_profile(self._h, ms, kinds, cap, C.byref(n)))
        return [(ms[i], kinds[i]) for i in range(n.value)]

    def run_device(self, batch: int, stream: int = 0):
        check(lib.b200_case_run_device(self._h, batch, stream))

    def run_host_ptrs(self, batch: int, in_ptrs, out_ptrs, stream: int = 0):
        """Host pointers (pinned for full copy speed); synchronizes before returning."""
        ins = (C.c_void_p * len(in_ptrs))(*in_ptrs)
        outs = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        check(lib.b200_case_run_host(self._h, batch, ins, outs, stream))

    def submit_host_ptrs(self, batch: int, in_ptrs, out_ptrs):
        """Queues one batch (pinned host pointers) and returns; see b200_case_submit_host."""
        ins = (C.c_void_p * len(in_ptrs))(*in_ptrs)
        outs = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        check(lib.b200_case_submit_host(self._h, batch, ins, outs))

    def wait(self):
        check(lib.b200_case_wait(self._h))

    def run_host(self, inputs, out_dtypes_shapes, stream: int = 0):
        """numpy in, numpy out.  ``out_dtypes_shapes``: list of (dtype, per-image shape)."""
        batch = inputs[0].shape[0]
        ins = [np.ascontiguousarray(a) for a in inputs]
        outs = [np.empty((batch,) + tuple(shape), dtype=dt) for dt, shape in out_dtypes_shapes]
        self.run_host_ptrs(batch, [a.ctypes.data for a in ins], [o.ctypes.data for o in outs], stream)
        return outs

    def close(self):
        if self._h:
            lib.b200_case_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
