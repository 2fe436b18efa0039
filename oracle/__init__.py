"""TEST INFRASTRUCTURE ONLY -- numpy-facing bindings of the two CPU checkers.

``port``  the restatement in ``oracle/port.c`` (``libnart_port.so``).  Always available once
          ``make -C oracle port`` has run.  Handles batch > 1, per-channel weight scales and a
          fused ReLU clamp.
``ref``   the unmodified reference ``quant`` module compiled into ``oracle/_ref/libnart_ref.so``
          and driven through its op API by ``oracle/ref_shim.c``.  Present only where the
          reference sources were available at build time (or the prebuilt file travelled).

Both take and return arrays in the reference's layout: activations ``[N][C][H][W]`` uint8,
weights ``[K][C/group][R][S]`` uint8 (an int8 weight ``v`` is stored as ``v + 128`` with
``wzp = 128``, python/nart/modules/quant.py:53-58 of the reference), bias int32 ``[K]``.

Only ``tests/``, the smoke check and the CPU-baseline / reference legs of ``bench.py`` may import
this package; the shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(_HERE, "libnart_port.so")
REF_SO = os.path.join(_HERE, "_ref", "libnart_ref.so")

_u8p = C.POINTER(C.c_uint8)
_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)


def reference_root() -> str | None:
    """Folder of the reference project's checkout when it is present on this machine: ``$NART_REF_ROOT``,
    else a folder called ``reference`` beside this repository.  None elsewhere (the GPU boxes)."""
    cand = os.environ.get("NART_REF_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.exists(os.path.join(cand, "art", "src", "op.c")) else None


def build(ref: bool | None = None) -> None:
    """Compile the restatement, and the reference when its sources are present."""
    target = "all" if ref is None else ("all" if ref else "port")
    cmd = ["make", "-s", "-C", _HERE, target]
    root = reference_root()
    if root is not None:
        cmd.append("REF=" + root)
    subprocess.check_call(cmd)


def _p(a, tp):
    return a.ctypes.data_as(tp) if a is not None else None


def _u8(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8, a.dtype
    return a


def conv_out_dim(i, k, pad, stride):
    return (i + 2 * pad - k) // stride + 1


class _Common:
    """Shared numpy plumbing; subclasses bind one shared library."""

    prefix = ""
    per_channel = False

    def __init__(self, path):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        f = getattr(self.lib, self.prefix + "_rshift_rn")
        f.restype = C.c_int64
        f.argtypes = [C.c_int64, C.c_uint8]
        g = getattr(self.lib, self.prefix + "_get_quant_scale")
        g.restype = None

    def rshift_rn(self, x, bits):
        return int(getattr(self.lib, self.prefix + "_rshift_rn")(int(x), int(bits)))

    def get_quant_scale(self, x, bits):
        """bits: 32 -> get_quant_scale_int32, -16 -> get_quant_scale_int16, else generic."""
        m, s = C.c_uint32(0), C.c_int8(0)
        fn = getattr(self.lib, self.prefix + "_get_quant_scale")
        if self.prefix == "ref":
            fn(C.c_float(x), C.c_int(bits), C.byref(m), C.byref(s))
        else:
            fn(C.c_float(x), C.c_int(bits), C.byref(m), C.byref(s))
        return m.value, s.value

    # -- ops that have identical C signatures in both libraries ---------------------------
    def relu_u8(self, x, ialpha, izp, oalpha, ozp, obits=8):
        x = _u8(x)
        y = np.empty_like(x)
        rc = getattr(self.lib, self.prefix + "_relu_u8")(
            _p(x, _u8p), C.c_size_t(x.size), C.c_float(ialpha), C.c_uint8(izp), C.c_float(oalpha),
            C.c_uint8(ozp), C.c_uint8(obits), _p(y, _u8p))
        assert rc == 0
        return y

    def pool_u8(self, x, method, kernel, pad, stride, ceil_mode, ialpha, izp, oalpha, ozp,
                obits=8):
        x = _u8(x)
        n, c, h, w = x.shape
        kh, kw = kernel
        ph, pw = pad
        sh, sw = stride
        hw = (C.c_int * 2)()
        fn = getattr(self.lib, self.prefix + "_pool_u8")
        args = [C.c_int(n), C.c_int(c), C.c_int(h), C.c_int(w), C.c_int(method), C.c_int(kh),
                C.c_int(kw), C.c_int(ph), C.c_int(pw), C.c_int(sh), C.c_int(sw),
                C.c_int(int(ceil_mode)), C.c_float(ialpha), C.c_uint8(izp), C.c_float(oalpha),
                C.c_uint8(ozp), C.c_uint8(obits)]
        rc = fn(_p(x, _u8p), *args, None, hw)
        assert rc == 0
        y = np.empty((n, c, hw[0], hw[1]), np.uint8)
        rc = fn(_p(x, _u8p), *args, _p(y, _u8p), hw)
        assert rc == 0
        return y

    def quantize_u8(self, x, oalpha, ozp, obits=8):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(x.shape, np.uint8)
        rc = getattr(self.lib, self.prefix + "_quantize_u8")(
            _p(x, _f32p), C.c_size_t(x.size), C.c_float(oalpha), C.c_uint8(ozp), C.c_uint8(obits),
            _p(y, _u8p))
        assert rc == 0
        return y

    def dequantize_u8(self, x, ialpha, izp):
        x = _u8(x)
        y = np.empty(x.shape, np.float32)
        rc = getattr(self.lib, self.prefix + "_dequantize_u8")(
            _p(x, _u8p), C.c_size_t(x.size), C.c_float(ialpha), C.c_uint8(izp), _p(y, _f32p))
        assert rc == 0
        return y


_i8p = C.POINTER(C.c_int8)


def _i8(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.int8, a.dtype
    return a


class _CommonI8:
    """The int8 (symmetric, no zero points) ops; the C signatures of the two libraries differ only in
    walpha (one float for the reference, an array for the restatement)."""

    def _wa(self, walpha):
        wa = np.atleast_1d(np.asarray(walpha, dtype=np.float32)).copy()
        if self.prefix == "ref":
            return [C.c_float(float(wa[0]))]
        return [_p(wa, _f32p), C.c_int(wa.size)]

    def conv2d_i8(self, x, w, bias, stride, pad, group, ialpha, walpha, oalpha, obits=7):
        x, w = _i8(x), _i8(w)
        n, c, h, wd = x.shape
        k, cg, r, s = w.shape
        assert cg * group == c
        sh, sw = stride
        ph, pw = pad
        oh, ow = conv_out_dim(h, r, ph, sh), conv_out_dim(wd, s, pw, sw)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        y = np.empty((n, k, oh, ow), np.int8)
        rc = getattr(self.lib, self.prefix + "_conv2d_i8")(
            _p(x, _i8p), C.c_int(n), C.c_int(c), C.c_int(h), C.c_int(wd), _p(w, _i8p), _p(b, _i32p),
            C.c_int(k), C.c_int(r), C.c_int(s), C.c_int(ph), C.c_int(pw), C.c_int(sh), C.c_int(sw),
            C.c_int(group), C.c_float(ialpha), *self._wa(walpha), C.c_float(oalpha), C.c_uint8(obits), _p(y, _i8p))
        assert rc == 0
        return y

    def ip_i8(self, x, w, bias, ialpha, walpha, oalpha, obits=7):
        x, w = _i8(x), _i8(w)
        n = x.shape[0]
        chw = x.size // n
        k = w.shape[0]
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        y = np.empty((n, k), np.int8)
        rc = getattr(self.lib, self.prefix + "_ip_i8")(
            _p(x, _i8p), C.c_int(n), C.c_int(chw), _p(w, _i8p), _p(b, _i32p), C.c_int(k), C.c_float(ialpha),
            *self._wa(walpha), C.c_float(oalpha), C.c_uint8(obits), _p(y, _i8p))
        assert rc == 0
        return y

    def quantize_i8(self, x, oalpha, obits=8):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(x.shape, np.int8)
        rc = getattr(self.lib, self.prefix + "_quantize_i8")(
            _p(x, _f32p), C.c_size_t(x.size), C.c_float(oalpha), C.c_uint8(obits), _p(y, _i8p))
        assert rc == 0
        return y

    def dequantize_i8(self, x, ialpha, ibits=8):
        x = _i8(x)
        y = np.empty(x.shape, np.float32)
        extra = [C.c_uint8(ibits)] if self.prefix == "ref" else []
        rc = getattr(self.lib, self.prefix + "_dequantize_i8")(
            _p(x, _i8p), C.c_size_t(x.size), C.c_float(ialpha), *extra, _p(y, _f32p))
        assert rc == 0
        return y


class Port(_Common, _CommonI8):
    prefix = "port"
    per_channel = True

    def __init__(self):
        super().__init__(PORT_SO)

    def conv2d_u8(self, x, w, bias, stride, pad, group, ialpha, izp, walpha, wzp, oalpha, ozp,
                  obits=8, relu=False, return_acc=False):
        x, w = _u8(x), _u8(w)
        n, c, h, wd = x.shape
        k, cg, r, s = w.shape
        assert cg * group == c
        sh, sw = stride
        ph, pw = pad
        oh, ow = conv_out_dim(h, r, ph, sh), conv_out_dim(wd, s, pw, sw)
        wa = np.atleast_1d(np.asarray(walpha, dtype=np.float32)).copy()
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        y = np.empty((n, k, oh, ow), np.uint8)
        acc = np.empty((n, k, oh, ow), np.int32) if return_acc else None
        rc = self.lib.port_conv2d_u8(
            _p(x, _u8p), C.c_int(n), C.c_int(c), C.c_int(h), C.c_int(wd), _p(w, _u8p),
            _p(b, _i32p), C.c_int(k), C.c_int(r), C.c_int(s), C.c_int(ph), C.c_int(pw),
            C.c_int(sh), C.c_int(sw), C.c_int(group), C.c_float(ialpha), C.c_uint8(izp),
            _p(wa, _f32p), C.c_int(wa.size), C.c_uint8(wzp), C.c_float(oalpha), C.c_uint8(ozp),
            C.c_uint8(obits), C.c_int(int(relu)), _p(y, _u8p), _p(acc, _i32p))
        assert rc == 0
        return (y, acc) if return_acc else y

    def ip_u8(self, x, w, bias, ialpha, izp, walpha, wzp, oalpha, ozp, obits=8):
        x, w = _u8(x), _u8(w)
        n = x.shape[0]
        chw = x.size // n
        k = w.shape[0]
        wa = np.atleast_1d(np.asarray(walpha, dtype=np.float32)).copy()
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        y = np.empty((n, k), np.uint8)
        rc = self.lib.port_ip_u8(
            _p(x, _u8p), C.c_int(n), C.c_int(chw), _p(w, _u8p), _p(b, _i32p), C.c_int(k),
            C.c_float(ialpha), C.c_uint8(izp), _p(wa, _f32p), C.c_int(wa.size), C.c_uint8(wzp),
            C.c_float(oalpha), C.c_uint8(ozp), C.c_uint8(obits), _p(y, _u8p))
        assert rc == 0
        return y

    def eltwise_sum_u8(self, xs, ialpha, izp, oalpha, ozp, obits=8, coeff=None, relu=False):
        xs = [_u8(a) for a in xs]
        n = len(xs)
        ptrs = (_u8p * n)(*[_p(a, _u8p) for a in xs])
        ia = np.asarray(ialpha, dtype=np.float32).copy()
        iz = np.asarray(izp, dtype=np.uint8).copy()
        cf = None if coeff is None else np.asarray(coeff, dtype=np.float32).copy()
        y = np.empty_like(xs[0])
        rc = self.lib.port_eltwise_sum_u8(
            ptrs, C.c_int(n), C.c_size_t(xs[0].size), _p(ia, _f32p), _p(iz, _u8p), _p(cf, _f32p),
            C.c_float(oalpha), C.c_uint8(ozp), C.c_uint8(obits), C.c_int(int(relu)), _p(y, _u8p))
        assert rc == 0
        return y


class Ref(_Common, _CommonI8):
    prefix = "ref"
    per_channel = False

    def __init__(self):
        # RTLD_GLOBAL: an art plugin loaded afterwards resolves the runtime's symbols against it,
        # the way a plugin dlopen'ed by the reference's drivers resolves them against libart
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        C.CDLL(REF_SO, mode=C.RTLD_GLOBAL)
        super().__init__(REF_SO)
        self._plugins = {}

    def use_module(self, plugin_path=None, symbol=None, whole_batch=False, conv_relu=False):
        """Routes every op of this object through another art module (``plugin_path`` exporting
        the ``module_t`` named ``symbol``), or back to the reference quant module when called
        without arguments."""
        ptr = None
        if plugin_path is not None:
            if plugin_path not in self._plugins:
                self._plugins[plugin_path] = C.CDLL(plugin_path, mode=C.RTLD_GLOBAL)
            ptr = C.c_void_p.in_dll(self._plugins[plugin_path], symbol)
            ptr = C.addressof(ptr)
        self.lib.ref_use_module.argtypes = [C.c_void_p, C.c_int, C.c_int]
        self.lib.ref_use_module.restype = None
        self.lib.ref_use_module(ptr, int(whole_batch), int(conv_relu))

    def constant(self, name: str):
        """Value of a named constant of the reference's headers (None if the shim does not list it)."""
        found = C.c_int(0)
        self.lib.ref_constant.restype = C.c_uint64
        self.lib.ref_constant.argtypes = [C.c_char_p, C.POINTER(C.c_int)]
        v = self.lib.ref_constant(name.encode(), C.byref(found))
        return int(v) if found.value else None

    def open_engine(self, path):
        """Loads a serialized case with the reference's deserializer and prepares its parade on the module
        selected by use_module.  Returns a handle for engine_input / engine_run / engine_output / close_engine:
        the reference's own calling sequence (host view of the inputs, parade_run, host view of the outputs)."""
        L = self.lib
        L.ref_parade_open.restype = C.c_void_p
        L.ref_parade_open.argtypes = [C.c_char_p]
        L.ref_parade_io_bytes.restype = C.c_size_t
        L.ref_parade_io_bytes.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.ref_parade_input_ptr.restype = C.c_void_p
        L.ref_parade_input_ptr.argtypes = [C.c_void_p, C.c_int]
        L.ref_parade_output_ptr.restype = C.c_void_p
        L.ref_parade_output_ptr.argtypes = [C.c_void_p, C.c_int]
        L.ref_parade_run_only.restype = None
        L.ref_parade_run_only.argtypes = [C.c_void_p]
        L.ref_parade_close.argtypes = [C.c_void_p]
        h = L.ref_parade_open(os.fsencode(path))
        if not h:
            raise RuntimeError("the reference could not load %s" % path)
        return h

    def engine_input(self, h, index, dtype=np.uint8):
        """The host view of input `index` as a numpy array (no copy); asking for it marks it as written."""
        n = self.lib.ref_parade_io_bytes(h, 0, index)
        p = self.lib.ref_parade_input_ptr(h, index)
        return np.ctypeslib.as_array((C.c_uint8 * n).from_address(p)).view(dtype)

    def engine_run(self, h):
        self.lib.ref_parade_run_only(h)

    def engine_output(self, h, index, dtype=np.float32):
        """The host view of output `index` (downloads it from the module's memory if that is newer)."""
        n = self.lib.ref_parade_io_bytes(h, 1, index)
        p = self.lib.ref_parade_output_ptr(h, index)
        return np.ctypeslib.as_array((C.c_uint8 * n).from_address(p)).view(dtype)

    def close_engine(self, h):
        self.lib.ref_parade_close(h)

    def run_engine(self, path, inputs, output_dtypes):
        """Loads a serialized case with the reference's own deserializer and parade, bound to the
        module selected by use_module, and runs it once.  inputs: numpy arrays in the file's input
        order and shapes; returns one flat numpy array per output."""
        L = self.lib
        L.ref_parade_open.restype = C.c_void_p
        L.ref_parade_open.argtypes = [C.c_char_p]
        L.ref_parade_io_bytes.restype = C.c_size_t
        L.ref_parade_io_bytes.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.ref_parade_run.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
        L.ref_parade_close.argtypes = [C.c_void_p]
        h = L.ref_parade_open(os.fsencode(path))
        if not h:
            raise RuntimeError("the reference could not load %s" % path)
        try:
            ins = [np.ascontiguousarray(a) for a in inputs]
            for i, a in enumerate(ins):
                want = L.ref_parade_io_bytes(h, 0, i)
                if a.nbytes != want:
                    raise ValueError("input %d has %d bytes, the case expects %d" % (i, a.nbytes, want))
            outs = [np.empty(L.ref_parade_io_bytes(h, 1, i) // np.dtype(dt).itemsize, dtype=dt)
                    for i, dt in enumerate(output_dtypes)]
            ip = (C.c_void_p * len(ins))(*[a.ctypes.data for a in ins])
            op = (C.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
            assert L.ref_parade_run(h, ip, op) == 0
            return outs
        finally:
            L.ref_parade_close(h)

    def conv2d_u8(self, x, w, bias, stride, pad, group, ialpha, izp, walpha, wzp, oalpha, ozp,
                  obits=8):
        x, w = _u8(x), _u8(w)
        n, c, h, wd = x.shape
        k, cg, r, s = w.shape
        sh, sw = stride
        ph, pw = pad
        oh, ow = conv_out_dim(h, r, ph, sh), conv_out_dim(wd, s, pw, sw)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        y = np.empty((n, k, oh, ow), np.uint8)
        rc = self.lib.ref_conv2d_u8(
            _p(x, _u8p), C.c_int(n), C.c_int(c), C.c_int(h), C.c_int(wd), _p(w, _u8p),
            _p(b, _i32p), C.c_int(k), C.c_int(r), C.c_int(s), C.c_int(ph), C.c_int(pw),
            C.c_int(sh), C.c_int(sw), C.c_int(group), C.c_float(ialpha),
            C.c_uint8(izp), C.c_float(float(walpha)), C.c_uint8(wzp), C.c_float(oalpha),
            C.c_uint8(ozp), C.c_uint8(obits), _p(y, _u8p))
        assert rc == 0
        return y

    def ip_u8(self, x, w, bias, ialpha, izp, walpha, wzp, oalpha, ozp, obits=8):
        x, w = _u8(x), _u8(w)
        n = x.shape[0]
        chw = x.size // n
        k = w.shape[0]
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
        y = np.empty((n, k), np.uint8)
        rc = self.lib.ref_ip_u8(
            _p(x, _u8p), C.c_int(n), C.c_int(chw), _p(w, _u8p), _p(b, _i32p), C.c_int(k),
            C.c_float(ialpha), C.c_uint8(izp), C.c_float(float(walpha)), C.c_uint8(wzp),
            C.c_float(oalpha), C.c_uint8(ozp), C.c_uint8(obits), _p(y, _u8p))
        assert rc == 0
        return y

    def eltwise_sum_u8(self, xs, ialpha, izp, oalpha, ozp, obits=8, coeff=None, use_add=False):
        xs = [_u8(a) for a in xs]
        n = len(xs)
        ptrs = (_u8p * n)(*[_p(a, _u8p) for a in xs])
        ia = np.asarray(ialpha, dtype=np.float32).copy()
        iz = np.asarray(izp, dtype=np.uint8).copy()
        cf = None if coeff is None else np.asarray(coeff, dtype=np.float32).copy()
        y = np.empty_like(xs[0])
        rc = self.lib.ref_eltwise_sum_u8(
            ptrs, C.c_int(n), C.c_size_t(xs[0].size), _p(ia, _f32p), _p(iz, _u8p), _p(cf, _f32p),
            C.c_float(oalpha), C.c_uint8(ozp), C.c_uint8(obits), C.c_int(int(use_add)),
            _p(y, _u8p))
        assert rc == 0
        return y


_port = None
_ref = None


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref() -> Ref:
    global _ref
    if _ref is None:
        _ref = Ref()
    return _ref


def have_ref() -> bool:
    return os.path.exists(REF_SO)
