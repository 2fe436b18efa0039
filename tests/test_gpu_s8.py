"""GPU: the int8 (dtINT8) path through the C-ABI -- conv on both kernels, ip, quantize, dequantize --
bit for bit against the fixtures the compiled reference produced and against the CPU restatement."""
import os

import numpy as np
import pytest

from cases import S8_SHAPES, conv_inputs_s8, s8_oalpha
from gpu_util import assert_same
from test_oracle_pin_s8 import s8_float_inputs

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_ref_s8.npz"))


@pytest.fixture(scope="module")
def ops():
    import torch
    assert torch.cuda.is_available()
    from nart_b200 import ops as o
    return o


def dev(x_nchw):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x_nchw.transpose(0, 2, 3, 1))).cuda()


def host(y_nhwc):
    return np.ascontiguousarray(y_nhwc.cpu().numpy().transpose(0, 3, 1, 2))


def algos(ops, c, k, g, ob):
    a = [ops.ALGO_DIRECT]
    if g == 1 and c % 16 == 0 and k % 16 == 0 and ob < 8:
        a.append(ops.ALGO_IGEMM)
    return a


@pytest.mark.parametrize("i", range(len(S8_SHAPES)))
def test_conv_s8(ops, port, i):
    from nart_b200._lib import B200Error, ERR_UNSUPPORTED
    n, c, h, w, k, r, s, st, pd, g, ob = S8_SHAPES[i]
    x, wt, bias, walpha = conv_inputs_s8(300 + i, n, c, h, w, k, r, s, g)
    oa = s8_oalpha(c, g, r, s)
    common = dict(in_hw=(h, w), stride=(st, st), pad=(pd, pd), group=g, ialpha=0.02, oalpha=oa, obits=ob, signed=True,
                  s8_wrap=(ob == 8))
    for algo in algos(ops, c, k, g, ob):
        conv = ops.Conv2d(wt, bias, walpha=walpha[:1], algo=algo, **common)
        assert conv.algo == algo
        assert_same(host(conv(dev(x))), GOLD["conv%d_scalar" % i], "s8 conv %d algo %d" % (i, algo))
        # one scale per output channel, and a fused ReLU, against the restatement
        want = port.conv2d_i8(x, wt, bias, (st, st), (pd, pd), g, 0.02, walpha, oa, ob)
        convp = ops.Conv2d(wt, bias, walpha=walpha, algo=algo, **common)
        assert_same(host(convp(dev(x))), want, "s8 conv %d algo %d per channel" % (i, algo))
        if i < 3:
            assert_same(want, GOLD["conv%d_per_channel" % i], "fixture")
        convr = ops.Conv2d(wt, bias, walpha=walpha, algo=algo, relu=True, **common)
        if ob < 8:
            assert_same(host(convr(dev(x))), np.maximum(want, 0), "s8 conv %d algo %d relu" % (i, algo))
        assert ops.device_status() == 0
    if ob == 8:      # without the flag the wrapping case is refused, with a reason
        with pytest.raises(B200Error) as ei:
            ops.Conv2d(wt, bias, walpha=walpha[:1], **dict(common, s8_wrap=False))
        assert ei.value.status == ERR_UNSUPPORTED and "wrap" in ei.value.detail


def test_conv_s8_larger_batch_tensor_cores(ops, port):
    """A ResNet-sized layer on the tensor-core path: many tiles per CTA, images from both ends compared."""
    n, c, h, k = 64, 64, 28, 128
    x, wt, bias, walpha = conv_inputs_s8(41, n, c, h, h, k, 3, 3)
    oa = s8_oalpha(c, 1, 3, 3)
    conv = ops.Conv2d(wt, bias, in_hw=(h, h), stride=(1, 1), pad=(1, 1), ialpha=0.02, walpha=walpha, oalpha=oa, obits=7,
                      signed=True, algo=ops.ALGO_IGEMM)
    y = conv(dev(x))
    pick = [0, 31, 63]
    want = port.conv2d_i8(x[pick], wt, bias, (1, 1), (1, 1), 1, 0.02, walpha, oa, 7)
    assert_same(host(y[pick]), want, "s8 batch 64")
    assert len(np.unique(want)) > 100


def test_ip_quantize_dequantize_s8(ops):
    import torch
    xi, wi, bi, f, q = s8_float_inputs()
    ip = ops.InnerProductS8(wi, bi, in_chw=(512, 1, 1), ialpha=0.02, walpha=0.005, oalpha=0.4, obits=7)
    y = ip(torch.from_numpy(xi.reshape(4, 1, 1, 512)).cuda())
    assert_same(y.cpu().numpy().reshape(4, 100), GOLD["ip"], "s8 ip")
    fd = torch.from_numpy(f).cuda()
    for ob in (8, 7, 4):
        for nhwc in (True, False):
            got = ops.quantize_s8(fd, 0.05, ob, nhwc=nhwc).cpu().numpy()
            if nhwc:
                got = np.ascontiguousarray(got.transpose(0, 3, 1, 2))
            assert_same(got, GOLD["quantize_%d" % ob], "s8 quantize obits %d nhwc %s" % (ob, nhwc))
    qd = torch.from_numpy(np.ascontiguousarray(q.transpose(0, 2, 3, 1))).cuda()
    got = ops.dequantize_s8(qd, 0.037).cpu().numpy()
    assert_same(got.view(np.uint32), GOLD["dequantize"].view(np.uint32), "s8 dequantize")
