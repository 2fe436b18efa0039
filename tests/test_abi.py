"""CPU: the C-ABI library loads, exports every symbol the header declares, and its host-only
entry points (scale decomposition, argument validation that precedes any CUDA call) behave."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_ref.npz"))


@pytest.fixture(scope="module")
def L():
    lib_path = os.path.join(ROOT, "nart_b200", "libnart_b200.so")
    if not os.path.exists(lib_path):
        from nart_b200 import build
        build.build_library()
    from nart_b200 import _lib
    return _lib


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nart_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"B200_API\s+[^;(]*?\b(b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(L):
    names = declared_symbols()
    assert len(names) > 40
    for n in names:
        assert hasattr(L.lib, n), n
        assert n in L.SIGNATURES, "python binding misses " + n
    assert sorted(L.SIGNATURES) == names


def test_scale_decomposition_matches_reference_fixture(L):
    for x, bits, m, s in GOLD["scale_rows"]:
        mm, ss = C.c_uint32(0), C.c_int8(0)
        L.lib.b200_get_quant_scale(float(np.float32(x)), int(bits), C.byref(mm), C.byref(ss))
        assert (mm.value, ss.value) == (int(m), int(s))


def _params(L, **kw):
    p = L.ConvParams()
    d = dict(c=16, h=8, w=8, k=16, r=3, s=3, pad_h=1, pad_w=1, stride_h=1, stride_w=1, group=1,
             ialpha=0.02, izp=128, wzp=128, ozp=0, obits=8, oalpha=0.05, n_walpha=1, relu=0, algo=0)
    d.update(kw)
    for k, v in d.items():
        setattr(p, k, v)
    return p


def test_conv_create_refuses_cleanly(L):
    wa = (C.c_float * 1)(0.005)
    w = np.full((16, 16, 3, 3), 128, np.uint8)
    h = C.c_void_p()
    for kw, status in ((dict(ialpha=1e-12), L.ERR_UNSUPPORTED), (dict(group=3), L.ERR_INVALID),
                       (dict(obits=9), L.ERR_INVALID), (dict(n_walpha=5), L.ERR_INVALID),
                       (dict(oalpha=0.0), L.ERR_INVALID), (dict(stride_h=0), L.ERR_INVALID),
                       (dict(algo=7), L.ERR_INVALID)):
        p = _params(L, **kw)
        p.walpha = wa
        rc = L.lib.b200_conv2d_create(C.byref(p), w.ctypes.data, None, C.byref(h))
        assert rc == status, (kw, rc, L.lib.b200_last_error())
        assert L.lib.b200_last_error() != b""
    assert L.lib.b200_strerror(L.ERR_UNSUPPORTED) == b"unsupported configuration"


def test_pool_out_dims_follow_reference_shape_rule(L):
    # art/src/op.c:934-956: 112 -> 57 with ceil_mode (the default), 56 without
    oh, ow = C.c_int32(), C.c_int32()
    assert L.lib.b200_pool_out_dims(112, 112, 3, 3, 1, 1, 2, 2, 1, C.byref(oh), C.byref(ow)) == 0
    assert (oh.value, ow.value) == (57, 57)
    assert L.lib.b200_pool_out_dims(112, 112, 3, 3, 1, 1, 2, 2, 0, C.byref(oh), C.byref(ow)) == 0
    assert (oh.value, ow.value) == (56, 56)
    assert L.lib.b200_pool_out_dims(14, 14, 3, 3, 1, 1, 2, 2, 1, C.byref(oh), C.byref(ow)) == 0
    assert (oh.value, ow.value) == tuple(GOLD["pool_max_ceil"].shape[2:])


def test_eltwise_refuses_terms_that_would_not_fit_32_bits(L):
    """Argument checks that precede any CUDA call (count == 0: nothing is launched).  The kernels form
    x * m + add in int32; a scale ratio of 2^27 between the inputs would need more (the reference's
    rshift_rn works on int64), so such an op is declined instead of computed differently."""
    x = (C.c_void_p * 2)(256, 512)          # aligned dummies; never dereferenced with count == 0
    izp = (C.c_uint8 * 2)(0, 0)
    ok = (C.c_float * 2)(0.02, 0.02 * 1024)
    assert L.lib.b200_eltwise_sum_u8(x, 2, 0, ok, izp, None, 0.05, 3, 8, 0, 1024, None) == L.OK
    extreme = (C.c_float * 2)(0.02, 0.02 * 2.0 ** 27)
    rc = L.lib.b200_eltwise_sum_u8(x, 2, 0, extreme, izp, None, 0.05, 3, 8, 0, 1024, None)
    assert rc == L.ERR_UNSUPPORTED, L.lib.b200_last_error()


def test_selftest_argument_check(L):
    assert L.lib.b200_selftest_wait_expiry(0, None) == L.ERR_INVALID
    assert L.lib.b200_selftest_wait_expiry(3_000_000_000, None) == L.ERR_INVALID
