"""CPU: the restatement (oracle/port.c) against the committed fixtures that the unmodified
reference produced (tests/golden/quant_ref.npz), and against the compiled reference itself where
oracle/_ref is available."""
import os

import numpy as np
import pytest

from cases import EDGE_SHAPES, conv_inputs

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_ref.npz"))


def test_scale_decomposition_golden(port):
    for x, bits, m, s in GOLD["scale_rows"]:
        assert port.get_quant_scale(float(np.float32(x)), int(bits)) == (int(m), int(s))


def test_rshift_rn_golden(port):
    for x, b, y in zip(GOLD["rshift_x"], GOLD["rshift_b"], GOLD["rshift_y"]):
        assert port.rshift_rn(int(x), int(b)) == int(y)


def test_rshift_rn_is_round_half_up(port):
    # rshift_rn(x, b) == floor((x + 2^(b-1)) / 2^b): the identity the device code relies on
    rng = np.random.default_rng(5)
    for _ in range(20000):
        x = int(rng.integers(-2**62, 2**62))
        b = int(rng.integers(1, 63))
        assert port.rshift_rn(x, b) == (x + (1 << (b - 1))) >> b
    assert port.rshift_rn(-3, 1) == -1 and port.rshift_rn(5, 1) == 3


def _c0():
    n, c, h, w, k, r, s, st, pd, g = EDGE_SHAPES[0]
    return conv_inputs(0, n, c, h, w, k, r, s, g), (st, st), (pd, pd), g


def test_conv_config0_golden(port):
    (x, wt, bias, walpha), st, pd, g = _c0()
    q = dict(ialpha=0.02, izp=128, wzp=128, oalpha=0.05, ozp=0)
    y = port.conv2d_u8(x, wt, bias, st, pd, g, walpha=walpha[:1], **q)
    assert np.array_equal(y, GOLD["c0_scalar"])
    y = port.conv2d_u8(x, wt, bias, st, pd, g, walpha=walpha, **q)
    assert np.array_equal(y, GOLD["c0_per_channel"])


def test_conv_fused_relu_golden(port):
    (x, wt, bias, walpha), st, pd, g = _c0()
    q2 = dict(ialpha=0.02, izp=117, wzp=128, oalpha=0.4, ozp=77)
    y = port.conv2d_u8(x, wt, bias, st, pd, g, walpha=walpha[:1], **q2)
    assert np.array_equal(y, GOLD["c0_zp_scalar"])
    yr = port.conv2d_u8(x, wt, bias, st, pd, g, walpha=walpha[:1], relu=True, **q2)
    assert np.array_equal(yr, GOLD["c0_zp_relu"])
    assert (yr >= 77).all() and (y < 77).any()


@pytest.mark.parametrize("i", range(1, len(EDGE_SHAPES)))
def test_conv_edge_shapes_golden(port, i):
    n, c, h, w, k, r, s, st, pd, g = EDGE_SHAPES[i]
    x, wt, bias, walpha = conv_inputs(100 + i, n, c, h, w, k, r, s, g)
    y = port.conv2d_u8(
        x, wt, bias, (st, st), (pd, pd), g, ialpha=0.037, izp=(37 * i) % 256, walpha=walpha[:1],
        wzp=128, oalpha=0.05 * np.sqrt(c // g * r * s) / 4, ozp=(11 * i) % 200)
    assert np.array_equal(y, GOLD["edge%d" % i])


def test_conv_batch_equals_per_image(port):
    x, wt, bias, walpha = conv_inputs(9, 4, 32, 9, 9, 32, 3, 3)
    q = dict(ialpha=0.02, izp=99, wzp=128, oalpha=0.3, ozp=3)
    y = port.conv2d_u8(x, wt, bias, (1, 1), (1, 1), 1, walpha=walpha, **q)
    for i in range(4):
        yi = port.conv2d_u8(x[i:i + 1], wt, bias, (1, 1), (1, 1), 1, walpha=walpha, **q)
        assert np.array_equal(y[i:i + 1], yi)


def _other_inputs():
    rng = np.random.default_rng(7)
    a = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    b = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    f = (rng.standard_normal((2, 3, 20, 20)) * 3).astype(np.float32)
    xi = rng.integers(0, 256, (4, 512), dtype=np.uint8)
    wi = (rng.integers(-127, 128, (100, 512)) + 128).astype(np.uint8)
    bi = rng.integers(-4096, 4097, 100).astype(np.int32)
    return a, b, f, xi, wi, bi


def test_other_ops_golden(port):
    a, b, f, xi, wi, bi = _other_inputs()
    ia, iz = [0.037, 0.081], [117, 9]
    y = port.eltwise_sum_u8([a, b], ia, iz, 0.093, 31)
    assert np.array_equal(y, GOLD["eltwise"]) and np.array_equal(y, GOLD["add"])
    assert np.array_equal(port.relu_u8(a, 0.037, 117, 0.037, 117), GOLD["relu_same"])
    assert np.array_equal(GOLD["relu_same"], np.maximum(a, 117))
    assert np.array_equal(port.relu_u8(a, 0.037, 117, 0.05, 20), GOLD["relu_rescale"])
    for name, m, cm in (("pool_max", 0, 0), ("pool_max_ceil", 0, 1), ("pool_ave", 1, 0), ("pool_ave_ceil", 1, 1)):
        assert np.array_equal(port.pool_u8(a, m, (3, 3), (1, 1), (2, 2), cm, 0.037, 117, 0.093, 31), GOLD[name])
    assert np.array_equal(port.pool_u8(a, 1, (14, 14), (0, 0), (1, 1), 0, 0.037, 117, 0.093, 31), GOLD["pool_gap"])
    assert np.array_equal(port.quantize_u8(f, 0.037, 117), GOLD["quantize"])
    assert np.array_equal(port.dequantize_u8(a, 0.037, 117).view(np.uint32), GOLD["dequantize"].view(np.uint32))
    assert np.array_equal(port.ip_u8(xi, wi, bi, 0.02, 100, 0.005, 128, 0.1, 50), GOLD["ip"])


# ---- live against the compiled reference (skipped where oracle/_ref did not travel) ---------------
def test_live_reference_random_convs(port, ref):
    rng = np.random.default_rng(42)
    for t in range(12):
        g = int(rng.choice([1, 1, 1, 2, 4]))
        c = g * int(rng.integers(1, 9)) * 2
        k = g * int(rng.integers(1, 9))
        h, w = int(rng.integers(3, 15)), int(rng.integers(3, 15))
        r, s = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        st, pd = int(rng.integers(1, 3)), int(rng.integers(0, 2))
        x, wt, bias, walpha = conv_inputs(1000 + t, 2, c, h, w, k, r, s, g)
        q = dict(ialpha=float(rng.uniform(0.01, 0.1)), izp=int(rng.integers(0, 256)), wzp=128,
                 oalpha=float(rng.uniform(0.05, 2.0)), ozp=int(rng.integers(0, 256)))
        yr = ref.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, walpha=float(walpha[0]), **q)
        yp = port.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, walpha=walpha[:1], **q)
        assert np.array_equal(yr, yp), (t, c, k, h, w, r, s, st, pd, g)


def test_live_reference_weight_zero_points(port, ref):
    """Weight zero points other than 128 (asymmetric weights, any stored byte): port == reference."""
    rng = np.random.default_rng(43)
    for t, wzp in enumerate((0, 3, 77, 127, 131, 200, 255)):
        g = (1, 1, 2, 1, 4, 1, 1)[t]
        c, k = g * 6, g * 5
        h, w = int(rng.integers(4, 12)), int(rng.integers(4, 12))
        r, s = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        st, pd = int(rng.integers(1, 3)), int(rng.integers(0, 2))
        x = rng.integers(0, 256, (2, c, h, w), dtype=np.uint8)
        wt = rng.integers(0, 256, (k, c // g, r, s), dtype=np.uint8)
        bias = rng.integers(-4096, 4097, k).astype(np.int32)
        q = dict(ialpha=float(rng.uniform(0.01, 0.1)), izp=int(rng.integers(0, 256)), wzp=wzp,
                 oalpha=float(rng.uniform(0.05, 2.0)), ozp=int(rng.integers(0, 256)))
        yr = ref.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, walpha=0.004, **q)
        yp = port.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, walpha=np.float32([0.004]), **q)
        assert np.array_equal(yr, yp), (t, wzp, c, k, h, w, r, s, st, pd, g)
        assert len(np.unique(yp)) > 8


def test_live_reference_eltwise_all_byte_pairs(port, ref):
    # every (a, b) byte pair once: 65536 elements
    a = np.repeat(np.arange(256, dtype=np.uint8), 256).reshape(1, 256, 16, 16)
    b = np.tile(np.arange(256, dtype=np.uint8), 256).reshape(1, 256, 16, 16)
    for ia, iz, oa, oz in (([0.037, 0.081], [117, 9], 0.093, 31), ([0.1, 0.01], [0, 255], 0.05, 128)):
        assert np.array_equal(ref.eltwise_sum_u8([a, b], ia, iz, oa, oz), port.eltwise_sum_u8([a, b], ia, iz, oa, oz))
        assert np.array_equal(ref.eltwise_sum_u8([a, b], ia, iz, oa, oz, use_add=True), port.eltwise_sum_u8([a, b], ia, iz, oa, oz))


def test_live_reference_relu_equals_clamp(port, ref):
    x = np.arange(256, dtype=np.uint8).reshape(1, 256, 1, 1)
    for zp in (0, 1, 77, 128, 255):
        assert np.array_equal(ref.relu_u8(x, 0.4, zp, 0.4, zp), np.maximum(x, zp))
