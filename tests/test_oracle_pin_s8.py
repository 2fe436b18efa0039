"""CPU: the restatement's int8 (dtINT8, symmetric) functions against the fixtures the unmodified
reference produced (tests/golden/quant_ref_s8.npz) and, where oracle/_ref is available, live."""
import os

import numpy as np
import pytest

from cases import S8_SHAPES, conv_inputs_s8, s8_oalpha

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_ref_s8.npz"))


def s8_float_inputs():
    rng = np.random.default_rng(77)
    xi = rng.integers(-127, 128, (4, 512)).astype(np.int8)
    wi = rng.integers(-127, 128, (100, 512)).astype(np.int8)
    bi = rng.integers(-4096, 4097, 100).astype(np.int32)
    f = (rng.standard_normal((2, 24, 9, 11)) * 3).astype(np.float32)
    f.reshape(-1)[:2001] = (np.arange(2001) - 1000) * np.float32(0.05) * np.float32(0.5)
    q = rng.integers(-128, 128, (2, 24, 9, 11)).astype(np.int8)
    return xi, wi, bi, f, q


@pytest.mark.parametrize("i", range(len(S8_SHAPES)))
def test_conv_i8_golden(port, i):
    n, c, h, w, k, r, s, st, pd, g, ob = S8_SHAPES[i]
    x, wt, bias, walpha = conv_inputs_s8(300 + i, n, c, h, w, k, r, s, g)
    oa = s8_oalpha(c, g, r, s)
    y = port.conv2d_i8(x, wt, bias, (st, st), (pd, pd), g, 0.02, walpha[:1], oa, ob)
    assert np.array_equal(y, GOLD["conv%d_scalar" % i])
    if i < 3:
        y = port.conv2d_i8(x, wt, bias, (st, st), (pd, pd), g, 0.02, walpha, oa, ob)
        assert np.array_equal(y, GOLD["conv%d_per_channel" % i])
    if ob == 8:       # the reference's quirk is in the fixture: values beyond +-127 have wrapped
        wide = port.conv2d_i8(x, wt, bias, (st, st), (pd, pd), g, 0.02, walpha[:1], oa / 4, ob)
        clipped = port.conv2d_i8(x, wt, bias, (st, st), (pd, pd), g, 0.02, walpha[:1], oa / 4, 7)
        assert (wide != clipped).any()


def test_ip_quantize_dequantize_i8_golden(port):
    xi, wi, bi, f, q = s8_float_inputs()
    assert np.array_equal(port.ip_i8(xi, wi, bi, 0.02, 0.005, 0.4, 7), GOLD["ip"])
    for ob in (8, 7, 4):
        got = port.quantize_i8(f, 0.05, ob)
        assert np.array_equal(got, GOLD["quantize_%d" % ob])
        assert got.max() == 2 ** (ob - 1) - 1 and got.min() == -(2 ** (ob - 1) - 1)
    assert np.array_equal(port.dequantize_i8(q, 0.037).view(np.uint32), GOLD["dequantize"].view(np.uint32))


def test_live_reference_i8(port, ref):
    rng = np.random.default_rng(9)
    for trial in range(6):
        c = int(rng.choice([8, 16, 24]))
        k = int(rng.choice([8, 16, 40]))
        h, w = int(rng.integers(3, 10)), int(rng.integers(3, 10))
        ks = int(rng.choice([1, 3]))
        st = int(rng.choice([1, 2]))
        ob = int(rng.choice([4, 7, 8]))
        x, wt, bias, walpha = conv_inputs_s8(1000 + trial, 2, c, h, w, k, ks, ks)
        oa = s8_oalpha(c, 1, ks, ks) / 2
        a = port.conv2d_i8(x, wt, bias, (st, st), (ks // 2, ks // 2), 1, 0.03, walpha[:1], oa, ob)
        b = ref.conv2d_i8(x, wt, bias, (st, st), (ks // 2, ks // 2), 1, 0.03, walpha[:1], oa, ob)
        assert np.array_equal(a, b), (c, k, h, w, ks, st, ob)
    f = (rng.standard_normal(50000) * 40).astype(np.float32)
    for ob in (2, 3, 6, 8):
        assert np.array_equal(port.quantize_i8(f, 0.31, ob), ref.quantize_i8(f, 0.31, ob))
