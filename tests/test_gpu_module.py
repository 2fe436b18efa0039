"""GPU: the art plugin (libart_module_b200.so) driven through the reference's own op API --
workspace_new_op / op_setting_*_set / op_config / op_prepare / op_run on `b200_module_tp`, by the
same shim that drives the reference quant module -- gives the reference module's bytes.  The art
core it runs under is the reference's, compiled unmodified into oracle/_ref."""
import os

import numpy as np
import pytest

from cases import EDGE_SHAPES, conv_inputs
from gpu_util import assert_same

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN = os.path.join(ROOT, "nart_b200", "libart_module_b200.so")
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_ref.npz"))


@pytest.fixture()
def plugin(ref):
    if not os.path.exists(PLUGIN):
        pytest.skip("libart_module_b200.so was not built (the art headers were not available)")
    ref.use_module(PLUGIN, "b200_module_tp", whole_batch=True)
    yield ref
    ref.use_module()


def test_plugin_conv_config0(plugin):
    n, c, h, w, k, r, s, st, pd, g = EDGE_SHAPES[0]
    x, wt, bias, walpha = conv_inputs(0, n, c, h, w, k, r, s, g)
    y = plugin.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, 0.02, 128, float(walpha[0]), 128, 0.05, 0)
    assert_same(y, GOLD["c0_scalar"], "plugin conv config 0")


@pytest.mark.parametrize("i", range(1, len(EDGE_SHAPES)))
def test_plugin_conv_edge_shapes(plugin, i):
    n, c, h, w, k, r, s, st, pd, g = EDGE_SHAPES[i]
    x, wt, bias, walpha = conv_inputs(100 + i, n, c, h, w, k, r, s, g)
    y = plugin.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, 0.037, (37 * i) % 256, float(walpha[0]), 128,
                         0.05 * np.sqrt(c // g * r * s) / 4, (11 * i) % 200)
    assert_same(y, GOLD["edge%d" % i], "plugin edge%d" % i)


def test_plugin_fused_relu_flag(ref):
    if not os.path.exists(PLUGIN):
        pytest.skip("plugin not built")
    n, c, h, w, k, r, s, st, pd, g = EDGE_SHAPES[0]
    x, wt, bias, walpha = conv_inputs(0, n, c, h, w, k, r, s, g)
    ref.use_module(PLUGIN, "b200_module_tp", whole_batch=True, conv_relu=True)
    try:
        y = ref.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, 0.02, 117, float(walpha[0]), 128, 0.4, 77)
    finally:
        ref.use_module()
    assert_same(y, GOLD["c0_zp_relu"], "plugin conv + relu flag")


def test_plugin_conv_asymmetric_weights(ref):
    """Weight zero points other than 128, as the reference's calibrator writes them by default: the
    plugin gives the bytes of the reference's own CPU module, run live on the same inputs."""
    if not os.path.exists(PLUGIN):
        pytest.skip("plugin not built")
    rng = np.random.default_rng(21)
    for wzp, (c, k, ks, st, pd, g, h, w) in ((77, (64, 32, 3, 1, 1, 1, 9, 10)), (201, (32, 64, 1, 2, 0, 1, 8, 8)),
                                             (5, (12, 8, 3, 1, 1, 2, 7, 7)), (140, (4, 32, 7, 2, 3, 1, 20, 20))):
        x = rng.integers(0, 256, (2, c, h, w), dtype=np.uint8)
        wt = rng.integers(0, 256, (k, c // g, ks, ks), dtype=np.uint8)
        bias = rng.integers(-4096, 4097, k).astype(np.int32)
        q = (0.03, 128, 0.004, wzp, 0.03 * 0.004 * 74 * 74 * np.sqrt(c // g * ks * ks) / 40, 120)
        want = ref.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, *q)
        assert len(np.unique(want)) > 16
        ref.use_module(PLUGIN, "b200_module_tp", whole_batch=True)
        try:
            got = ref.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, *q)
        finally:
            ref.use_module()
        assert_same(got, want, "plugin wzp=%d" % wzp)


def test_plugin_other_ops(plugin):
    rng = np.random.default_rng(7)
    a = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    b = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    f = (rng.standard_normal((2, 3, 20, 20)) * 3).astype(np.float32)
    xi = rng.integers(0, 256, (4, 512), dtype=np.uint8)
    wi = (rng.integers(-127, 128, (100, 512)) + 128).astype(np.uint8)
    bi = rng.integers(-4096, 4097, 100).astype(np.int32)
    ia, iz = [0.037, 0.081], [117, 9]
    assert_same(plugin.eltwise_sum_u8([a, b], ia, iz, 0.093, 31), GOLD["eltwise"], "eltwise")
    assert_same(plugin.eltwise_sum_u8([a, b], ia, iz, 0.093, 31, use_add=True), GOLD["add"], "add")
    assert_same(plugin.relu_u8(a, 0.037, 117, 0.037, 117), GOLD["relu_same"], "relu")
    assert_same(plugin.relu_u8(a, 0.037, 117, 0.05, 20), GOLD["relu_rescale"], "relu rescale")
    for name, m, cm in (("pool_max", 0, 0), ("pool_max_ceil", 0, 1), ("pool_ave", 1, 0), ("pool_ave_ceil", 1, 1)):
        assert_same(plugin.pool_u8(a, m, (3, 3), (1, 1), (2, 2), cm, 0.037, 117, 0.093, 31), GOLD[name], name)
    assert_same(plugin.pool_u8(a, 1, (14, 14), (0, 0), (1, 1), 0, 0.037, 117, 0.093, 31), GOLD["pool_gap"], "gap")
    assert_same(plugin.quantize_u8(f, 0.037, 117), GOLD["quantize"], "quantize")
    assert_same(plugin.dequantize_u8(a, 0.037, 117).view(np.uint32), GOLD["dequantize"].view(np.uint32), "dequantize")
    assert_same(plugin.ip_u8(xi, wi, bi, 0.02, 100, 0.005, 128, 0.1, 50), GOLD["ip"], "ip")


def test_plugin_int8_path(ref, monkeypatch):
    """dtINT8 tensors through the plugin: conv_2d and ip dispatch on the dtype of input 0, quantize /
    dequantize on qtype SYMMETRIC, exactly as the reference module does; the bytes are the reference's
    (fixtures produced by the compiled reference)."""
    if not os.path.exists(PLUGIN):
        pytest.skip("plugin not built")
    from cases import S8_SHAPES, conv_inputs_s8, s8_oalpha
    from test_oracle_pin_s8 import s8_float_inputs
    S8 = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_ref_s8.npz"))
    monkeypatch.setenv("NART_B200_S8_WRAP", "1")          # the obits = 8 case of the list wraps, as in the reference
    ref.use_module(PLUGIN, "b200_module_tp", whole_batch=True)
    try:
        for i, (n, c, h, w, k, r, s, st, pd, g, ob) in enumerate(S8_SHAPES):
            x, wt, bias, walpha = conv_inputs_s8(300 + i, n, c, h, w, k, r, s, g)
            y = ref.conv2d_i8(x, wt, bias, (st, st), (pd, pd), g, 0.02, float(walpha[0]), s8_oalpha(c, g, r, s), ob)
            assert_same(y, S8["conv%d_scalar" % i], "plugin int8 conv %d" % i)
        xi, wi, bi, f, q = s8_float_inputs()
        assert_same(ref.ip_i8(xi, wi, bi, 0.02, 0.005, 0.4, 7), S8["ip"], "plugin int8 ip")
        for ob in (8, 7, 4):
            assert_same(ref.quantize_i8(f, 0.05, ob), S8["quantize_%d" % ob], "plugin int8 quantize %d" % ob)
        assert_same(ref.dequantize_i8(q, 0.037).view(np.uint32), S8["dequantize"].view(np.uint32), "plugin int8 dequantize")
    finally:
        ref.use_module()
