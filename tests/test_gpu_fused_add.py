"""GPU parity of the residual add fused into the tensor-core conv's epilogue: the fused plan must give
the bytes of the two separate ops, conv_2d followed by eltwise SUM, as the CPU restatement computes
them (art/modules/quant/src/op/conv_2d_uint8_impl.c:39-165 then eltwise.c:137-174 of ModelTC/NART)."""
import numpy as np
import pytest

from cases import conv_inputs
from gpu_util import assert_same, to_dev_nhwc, to_host_nchw
from oracle.net_walk import run_net

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from nart_b200 import ops as o
    return o


# (n, c, h, w, k, kernel, stride, pad): 1x1 expand, padded 3x3 (several border classes), stride 2,
# ragged maps (partial tiles), a wide layer with several channel tiles
SHAPES = [
    (3, 64, 14, 14, 256, 1, 1, 0),
    (2, 64, 9, 11, 64, 3, 1, 1),
    (2, 128, 13, 13, 512, 1, 2, 0),
    (5, 32, 7, 7, 96, 3, 1, 1),
    (2, 256, 6, 6, 1024, 1, 1, 0),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("conv_input", [0, 1])
@pytest.mark.parametrize("relu", [False, True])
def test_fused_residual_add_matches_separate_ops(ops, port, shape, conv_input, relu):
    n, c, h, w, k, ks, st, pd = shape
    x, wt, bias, walpha = conv_inputs(7 + k + conv_input, n, c, h, w, k, ks, ks, 1)
    rng = np.random.default_rng(11 * k + ks)
    cq = dict(ialpha=0.031, izp=121, wzp=128, oalpha=0.05 * np.sqrt(c * ks * ks) / 4, ozp=113, walpha=walpha)
    conv_out = port.conv2d_u8(x, wt, bias, (st, st), (pd, pd), 1, cq["ialpha"], cq["izp"], walpha, 128,
                              cq["oalpha"], cq["ozp"])
    res = rng.integers(0, 256, conv_out.shape, dtype=np.uint8)
    res_alpha, res_zp = 0.043, 97
    ins = [conv_out, res] if conv_input == 0 else [res, conv_out]
    ia = [np.float32(cq["oalpha"]), res_alpha] if conv_input == 0 else [res_alpha, np.float32(cq["oalpha"])]
    iz = [cq["ozp"], res_zp] if conv_input == 0 else [res_zp, cq["ozp"]]
    eq = dict(oalpha=0.06, ozp=9 if relu else 140, obits=8, relu=relu)
    want = port.eltwise_sum_u8(ins, ia, iz, eq["oalpha"], eq["ozp"], relu=relu)

    conv = ops.Conv2d(wt, bias, in_hw=(h, w), stride=(st, st), pad=(pd, pd), algo=ops.ALGO_IGEMM, **cq)
    conv.fuse_residual_add(conv_input, ia, iz, **eq)
    got = to_host_nchw(conv.run_residual(to_dev_nhwc(x), to_dev_nhwc(res)))
    assert ops.device_status() == 0
    assert_same(got, want, "fused add %s conv_input=%d relu=%s" % (shape, conv_input, relu))
    # the separate kernels give the same bytes
    plain = ops.Conv2d(wt, bias, in_hw=(h, w), stride=(st, st), pad=(pd, pd), algo=ops.ALGO_IGEMM, **cq)
    y = plain(to_dev_nhwc(x))
    r = to_dev_nhwc(res)
    sep = ops.eltwise_sum([y, r] if conv_input == 0 else [r, y], ia, iz, eq["oalpha"], eq["ozp"], relu=relu)
    assert_same(to_host_nchw(sep), want, "separate kernels")


def test_fused_plan_refuses_the_plain_entry_and_odd_plans(ops):
    from nart_b200._lib import ERR_INVALID, ERR_UNSUPPORTED, B200Error
    x, wt, bias, walpha = conv_inputs(3, 1, 64, 8, 8, 64, 1, 1, 1)
    q = dict(ialpha=0.02, izp=128, wzp=128, oalpha=0.05, ozp=3, walpha=walpha)
    conv = ops.Conv2d(wt, bias, in_hw=(8, 8), algo=ops.ALGO_IGEMM, **q)
    conv.fuse_residual_add(0, [np.float32(0.05), 0.04], [3, 7], 0.06, 0)
    with pytest.raises(B200Error) as e:
        conv(to_dev_nhwc(x))
    assert e.value.status == ERR_INVALID
    with pytest.raises(B200Error) as e:            # a second fusion on the same plan
        conv.fuse_residual_add(0, [np.float32(0.05), 0.04], [3, 7], 0.06, 0)
    assert e.value.status == ERR_INVALID
    direct = ops.Conv2d(wt, bias, in_hw=(8, 8), algo=ops.ALGO_DIRECT, **q)
    with pytest.raises(B200Error) as e:            # the CUDA-core plan keeps the separate eltwise kernel
        direct.fuse_residual_add(0, [np.float32(0.05), 0.04], [3, 7], 0.06, 0)
    assert e.value.status == ERR_UNSUPPORTED
    other = ops.Conv2d(wt, bias, in_hw=(8, 8), algo=ops.ALGO_IGEMM, **q)
    with pytest.raises(B200Error) as e:            # the eltwise input is not this conv's output tensor
        other.fuse_residual_add(0, [0.07, 0.04], [3, 7], 0.06, 0)
    assert e.value.status == ERR_UNSUPPORTED


def test_case_fusion_on_and_off_agree(port):
    """A ResNet through the case runner with the fusion pass on and off (the default): same bytes,
    fewer launches with it on, both equal to the CPU restatement."""
    from nart_b200 import nets
    spec = nets.resnet(50, seed=12, hw=64, width_div=2, spread=True, num_classes=64)
    x = np.random.default_rng(9).integers(0, 256, (3, 3, 64, 64), dtype=np.uint8)
    want_logits, _, _ = run_net(spec, x, port)
    outs, launches = [], []
    for fuse in (True, False):
        cs, ids = nets.to_case(spec, 4, fuse=fuse)
        (got,) = cs.run_host([x], [(np.float32, (64, 1, 1))])
        outs.append(got.reshape(want_logits.shape))
        launches.append(cs.launch_count())
        cs.close()
    assert_same(outs[0].view(np.uint32), want_logits.view(np.uint32), "fused case vs restatement")
    assert_same(outs[1].view(np.uint32), want_logits.view(np.uint32), "unfused case vs restatement")
    assert launches[0] == launches[1] - 16      # the 16 residual adds of ResNet-50 ride in conv epilogues
