"""GPU parity, through the C-ABI: every op of the path against the CPU restatement (oracle/port.c)
and the reference-produced fixtures, bit for bit."""
import os

import numpy as np
import pytest

from cases import EDGE_SHAPES, SWEEP, conv_inputs
from gpu_util import assert_same, to_dev_nhwc, to_host_nchw

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_ref.npz"))


@pytest.fixture(scope="module")
def ops():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from nart_b200 import ops as o   # raises if libnart_b200.so is missing: there is no fallback
    return o


def algos_for(ops, c, k, group):
    a = [ops.ALGO_DIRECT]
    if group == 1 and c % 16 == 0 and k % 16 == 0:
        a.append(ops.ALGO_IGEMM)
    return a


def run_conv(ops, x, wt, bias, st, pd, g, algo, return_acc=False, **q):
    conv = ops.Conv2d(wt, bias, in_hw=x.shape[2:], stride=(st, st), pad=(pd, pd), group=g, algo=algo, **q)
    assert conv.algo == algo
    out = conv(to_dev_nhwc(x), return_acc=return_acc)
    assert ops.device_status() == 0
    if return_acc:
        return to_host_nchw(out[0]), to_host_nchw(out[1])
    return to_host_nchw(out)


@pytest.mark.parametrize("algo_i", [0, 1])
def test_conv_config0_golden(ops, algo_i):
    n, c, h, w, k, r, s, st, pd, g = EDGE_SHAPES[0]
    algo = algos_for(ops, c, k, g)[algo_i]
    x, wt, bias, walpha = conv_inputs(0, n, c, h, w, k, r, s, g)
    q = dict(ialpha=0.02, izp=128, wzp=128, oalpha=0.05, ozp=0)
    assert_same(run_conv(ops, x, wt, bias, st, pd, g, algo, walpha=walpha[:1], **q), GOLD["c0_scalar"], "scalar")
    assert_same(run_conv(ops, x, wt, bias, st, pd, g, algo, walpha=walpha, relu=True, **q), GOLD["c0_per_channel"], "per-channel")
    q2 = dict(ialpha=0.02, izp=117, wzp=128, oalpha=0.4, ozp=77)
    assert_same(run_conv(ops, x, wt, bias, st, pd, g, algo, walpha=walpha[:1], **q2), GOLD["c0_zp_scalar"], "zp")
    assert_same(run_conv(ops, x, wt, bias, st, pd, g, algo, walpha=walpha[:1], relu=True, **q2), GOLD["c0_zp_relu"], "zp relu")


@pytest.mark.parametrize("i", range(1, len(EDGE_SHAPES)))
def test_conv_edge_shapes(ops, port, i):
    n, c, h, w, k, r, s, st, pd, g = EDGE_SHAPES[i]
    x, wt, bias, walpha = conv_inputs(100 + i, n, c, h, w, k, r, s, g)
    q = dict(ialpha=0.037, izp=(37 * i) % 256, wzp=128, oalpha=0.05 * np.sqrt(c // g * r * s) / 4, ozp=(11 * i) % 200)
    for algo in algos_for(ops, c, k, g):
        y = run_conv(ops, x, wt, bias, st, pd, g, algo, walpha=walpha[:1], **q)
        assert_same(y, GOLD["edge%d" % i], "edge%d algo%d" % (i, algo))
        # per-channel scales + fused relu against the restatement
        want = port.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, walpha=walpha, relu=True, **q)
        y = run_conv(ops, x, wt, bias, st, pd, g, algo, walpha=walpha, relu=True, **q)
        assert_same(y, want, "edge%d algo%d per-channel relu" % (i, algo))


def test_conv_accumulators(ops, port):
    x, wt, bias, walpha = conv_inputs(77, 2, 32, 9, 11, 48, 3, 3)
    q = dict(ialpha=0.02, izp=131, wzp=128, oalpha=0.3, ozp=5)
    want_y, want_acc = port.conv2d_u8(x, wt, bias, (1, 1), (1, 1), 1, walpha=walpha, return_acc=True, **q)
    y, acc = run_conv(ops, x, wt, bias, 1, 1, 1, ops.ALGO_DIRECT, return_acc=True, walpha=walpha, **q)
    assert_same(acc, want_acc, "acc")
    assert_same(y, want_y, "y")


@pytest.mark.parametrize("c,k,h,ks,st", SWEEP)
@pytest.mark.parametrize("batch", [1, 3])
def test_conv_sweep_shapes(ops, port, c, k, h, ks, st, batch):
    """The single-conv sweep shapes at small batch (the restatement finishes in seconds)."""
    x, wt, bias, walpha = conv_inputs(c + h + ks + st, batch, c, h, h, k, ks, ks)
    q = dict(ialpha=0.02, izp=128, wzp=128, oalpha=0.05 * np.sqrt(c * ks * ks) / 8, ozp=0)
    want = port.conv2d_u8(x, wt, bias, (st, st), (ks // 2, ks // 2), 1, walpha=walpha, relu=True, **q)
    for algo in algos_for(ops, c, k, 1):
        y = run_conv(ops, x, wt, bias, st, ks // 2, 1, algo, walpha=walpha, relu=True, **q)
        assert_same(y, want, "sweep algo%d" % algo)


@pytest.mark.parametrize("c,k,h,ks,st", SWEEP)
@pytest.mark.parametrize("batch", [32, 256])
def test_conv_sweep_shapes_at_bench_batches(ops, port, c, k, h, ks, st, batch):
    """The same 16 shapes at the batches the throughput figures are quoted on.  Batch changes the
    M-tile box, the grid and the number of tiles a CTA walks, so these are kernel configurations of
    their own.  The whole output goes through the tensor-core path; images from both ends, the middle
    and either side of a tile boundary are compared with the restatement (every image of a conv is
    independent of the others), and the full tensor must equal a second run."""
    x, wt, bias, walpha = conv_inputs(1000 + c + h + ks + st + batch, batch, c, h, h, k, ks, ks)
    q = dict(ialpha=0.02, izp=128, wzp=128, oalpha=0.05 * np.sqrt(c * ks * ks) / 8, ozp=0)
    conv = ops.Conv2d(wt, bias, in_hw=(h, h), stride=(st, st), pad=(ks // 2, ks // 2), group=1, algo=ops.ALGO_IGEMM,
                      walpha=walpha, relu=True, **q)
    xd = to_dev_nhwc(x)
    y1 = conv(xd)
    y2 = conv(xd)
    assert ops.device_status() == 0
    assert bool((y1 == y2).all())
    pick = sorted({0, 1, batch // 2 - 1, batch // 2, batch - 2, batch - 1})
    want = port.conv2d_u8(x[pick], wt, bias, (st, st), (ks // 2, ks // 2), 1, walpha=walpha, relu=True, **q)
    got = to_host_nchw(y1[pick])
    assert_same(got, want, "sweep c%d h%d k%dx%d s%d batch %d" % (c, h, ks, ks, st, batch))
    assert len(np.unique(want)) > 16


def test_conv_large_scale_generic_requant_path(ops, port):
    """Scales >= 0.25 give shift <= 32: the 64-bit requantize branch."""
    x, wt, bias, walpha = conv_inputs(5, 2, 16, 6, 6, 16, 3, 3)
    for oalpha in (1e-4, 3e-6):
        q = dict(ialpha=0.02, izp=128, wzp=128, oalpha=oalpha, ozp=100)
        want = port.conv2d_u8(x, wt, bias, (1, 1), (1, 1), 1, walpha=walpha, **q)
        for algo in algos_for(ops, 16, 16, 1):
            assert_same(run_conv(ops, x, wt, bias, 1, 1, 1, algo, walpha=walpha, **q), want, "oalpha %g" % oalpha)


def test_conv_empty_batch_and_errors(ops):
    import torch
    x, wt, bias, walpha = conv_inputs(1, 1, 16, 5, 5, 16, 3, 3)
    conv = ops.Conv2d(wt, bias, in_hw=(5, 5), pad=(1, 1), ialpha=0.02, izp=1, walpha=walpha, oalpha=0.1, ozp=0)
    y = conv(torch.empty((0, 5, 5, 16), dtype=torch.uint8, device="cuda"))
    assert y.shape == (0, 5, 5, 16)
    with pytest.raises(ValueError):
        conv(torch.zeros((1, 6, 5, 16), dtype=torch.uint8, device="cuda"))


def test_ip(ops, port):
    rng = np.random.default_rng(7)
    rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8); rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    rng.standard_normal((2, 3, 20, 20))
    xi = rng.integers(0, 256, (4, 512), dtype=np.uint8)
    wi = (rng.integers(-127, 128, (100, 512)) + 128).astype(np.uint8)
    bi = rng.integers(-4096, 4097, 100).astype(np.int32)
    ip = ops.InnerProduct(wi, bi, in_chw=(512, 1, 1), ialpha=0.02, izp=100, walpha=0.005, oalpha=0.1, ozp=50)
    y = ip(to_dev_nhwc(xi.reshape(4, 512, 1, 1)))
    assert_same(y.cpu().numpy().reshape(4, 100), GOLD["ip"], "ip 1x1")
    # spatial input: the reference flattens NCHW
    x = rng.integers(0, 256, (3, 16, 3, 3), dtype=np.uint8)
    w2 = (rng.integers(-127, 128, (24, 144)) + 128).astype(np.uint8)
    want = port.ip_u8(x, w2, None, 0.05, 7, [0.004], 128, 0.5, 9)
    ip2 = ops.InnerProduct(w2, None, in_chw=(16, 3, 3), ialpha=0.05, izp=7, walpha=0.004, oalpha=0.5, ozp=9)
    assert_same(ip2(to_dev_nhwc(x)).cpu().numpy().reshape(3, 24), want, "ip 3x3")
    # asymmetric weights (any byte, zero point other than 128): 1x1 and spatial inputs
    for wzp, shape in ((90, (5, 64, 1, 1)), (201, (3, 16, 3, 3))):
        x = rng.integers(0, 256, shape, dtype=np.uint8)
        w3 = rng.integers(0, 256, (40, int(np.prod(shape[1:]))), dtype=np.uint8)
        b3 = rng.integers(-4096, 4097, 40).astype(np.int32)
        want = port.ip_u8(x, w3, b3, 0.05, 131, [0.004], wzp, 0.3, 120)
        assert len(np.unique(want)) > 16
        ip3 = ops.InnerProduct(w3, b3, in_chw=shape[1:], ialpha=0.05, izp=131, walpha=0.004, wzp=wzp, oalpha=0.3, ozp=120)
        assert_same(ip3(to_dev_nhwc(x)).cpu().numpy().reshape(shape[0], 40), want, "ip wzp=%d" % wzp)


def test_layout_roundtrip(ops):
    import torch
    rng = np.random.default_rng(3)
    for shape in ((2, 3, 17, 19), (1, 64, 7, 7), (3, 40, 5, 6), (2, 16, 1, 1)):
        x = rng.integers(0, 256, shape, dtype=np.uint8)
        d = ops.nchw_to_nhwc(torch.from_numpy(x).cuda())
        assert_same(d.cpu().numpy(), x.transpose(0, 2, 3, 1), "nchw->nhwc %s" % (shape,))
        assert_same(ops.nhwc_to_nchw(d).cpu().numpy(), x, "nhwc->nchw %s" % (shape,))
    x = rng.integers(0, 256, (2, 3, 9, 9), dtype=np.uint8)
    d = ops.nchw_to_nhwc(torch.from_numpy(x).cuda(), c_pad=4, fill=9)
    assert (d[..., 3] == 9).all() and np.array_equal(d[..., :3].cpu().numpy(), x.transpose(0, 2, 3, 1))
    assert_same(ops.nhwc_to_nchw(d, c=3).cpu().numpy(), x, "strip pad")


def test_quantize_dequantize(ops, port):
    import torch
    rng = np.random.default_rng(7)
    a = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    f = (rng.standard_normal((2, 3, 20, 20)) * 3).astype(np.float32)
    q = ops.quantize(torch.from_numpy(f).cuda(), 0.037, 117)
    assert_same(to_host_nchw(q), GOLD["quantize"], "quantize nhwc")
    q = ops.quantize(torch.from_numpy(f).cuda(), 0.037, 117, nhwc=False)
    assert_same(q.cpu().numpy(), GOLD["quantize"], "quantize nchw")
    d = ops.dequantize(to_dev_nhwc(a), 0.037, 117)
    assert_same(d.cpu().numpy().view(np.uint32), GOLD["dequantize"].view(np.uint32), "dequantize")
    # values on and around the rounding boundaries, saturation at both ends
    alpha, zp = np.float32(0.1), 10
    grid = ((np.arange(-40, 600, dtype=np.float32) * np.float32(0.5)) - zp) * alpha
    vals = np.concatenate([grid, np.nextafter(grid, np.float32(1e9)), np.nextafter(grid, np.float32(-1e9))]).astype(np.float32)
    vals = vals[: vals.size // 4 * 4].reshape(1, 4, -1, 1)
    got = ops.quantize(torch.from_numpy(vals).cuda(), float(alpha), zp)
    assert_same(to_host_nchw(got), port.quantize_u8(vals, float(alpha), zp), "quantize boundaries")
    big = (rng.standard_normal((2, 64, 30, 31)) * 4).astype(np.float32)
    assert_same(to_host_nchw(ops.quantize(torch.from_numpy(big).cuda(), 0.05, 128)), port.quantize_u8(big, 0.05, 128), "quantize big")


def test_eltwise_all_byte_pairs(ops, port):
    a = np.repeat(np.arange(256, dtype=np.uint8), 256).reshape(1, 256, 16, 16)
    b = np.tile(np.arange(256, dtype=np.uint8), 256).reshape(1, 256, 16, 16)
    import torch
    for ia, iz, oa, oz in (([0.037, 0.081], [117, 9], 0.093, 31), ([0.1, 0.01], [0, 255], 0.05, 128), ([0.02, 0.02], [3, 250], 0.3, 0)):
        for relu in (False, True):
            want = port.eltwise_sum_u8([a, b], ia, iz, oa, oz, relu=relu)
            got = ops.eltwise_sum([torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()], ia, iz, oa, oz, relu=relu)
            assert_same(got.cpu().numpy(), want, "eltwise %s relu=%s" % (ia, relu))
    rng = np.random.default_rng(7)
    a = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    b = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    got = ops.add(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), [0.037, 0.081], [117, 9], 0.093, 31)
    assert_same(got.cpu().numpy(), GOLD["add"], "add golden")
    # ragged length (tail path) and three inputs
    xs = [rng.integers(0, 256, 1000 + 7, dtype=np.uint8) for _ in range(3)]
    want = port.eltwise_sum_u8(xs, [0.03, 0.05, 0.02], [1, 2, 3], 0.08, 17, coeff=[1.0, 0.5, 2.0])
    got = ops.eltwise_sum([torch.from_numpy(v).cuda() for v in xs], [0.03, 0.05, 0.02], [1, 2, 3], 0.08, 17, coeff=[1.0, 0.5, 2.0])
    assert_same(got.cpu().numpy(), want, "eltwise 3 inputs")


def test_relu(ops, port):
    import torch
    x = np.arange(256, dtype=np.uint8).repeat(3).reshape(1, 1, 3, 256)
    for ia, iz, oa, oz in ((0.037, 117, 0.037, 117), (0.037, 117, 0.05, 20), (0.4, 0, 0.1, 255)):
        got = ops.relu(torch.from_numpy(x).cuda(), ia, iz, oa, oz)
        assert_same(got.cpu().numpy(), port.relu_u8(x, ia, iz, oa, oz), "relu")


def test_pool(ops, port):
    rng = np.random.default_rng(7)
    a = rng.integers(0, 256, (2, 32, 14, 14), dtype=np.uint8)
    for name, m, cm in (("pool_max", 0, 0), ("pool_max_ceil", 0, 1), ("pool_ave", 1, 0), ("pool_ave_ceil", 1, 1)):
        got = ops.pool(to_dev_nhwc(a), m, (3, 3), (1, 1), (2, 2), cm, 0.037, 117, 0.093, 31)
        assert_same(to_host_nchw(got), GOLD[name], name)
    got = ops.pool(to_dev_nhwc(a), 1, (14, 14), (0, 0), (1, 1), 0, 0.037, 117, 0.093, 31)
    assert_same(to_host_nchw(got), GOLD["pool_gap"], "gap")
    # ragged channel counts (4- and 1-byte vector paths), odd sizes
    for c in (20, 7, 64):
        x = rng.integers(0, 256, (3, c, 13, 9), dtype=np.uint8)
        for m in (0, 1):
            want = port.pool_u8(x, m, (3, 2), (1, 0), (2, 1), 1, 0.05, 33, 0.07, 12)
            got = ops.pool(to_dev_nhwc(x), m, (3, 2), (1, 0), (2, 1), 1, 0.05, 33, 0.07, 12)
            assert_same(to_host_nchw(got), want, "pool c=%d m=%d" % (c, m))
    # even output widths and the common windows (3x3 stride 1 or 2, 2x2 stride 2) take the
    # two-outputs-per-thread max kernel, with and without the identity table; 3x5 stays generic
    x = rng.integers(0, 256, (2, 48, 11, 16), dtype=np.uint8)
    for kern, pad, stride, cm in (((3, 3), (1, 1), (1, 1), 0), ((2, 2), (0, 0), (2, 2), 1), ((3, 3), (1, 1), (2, 2), 0),
                                  ((3, 3), (0, 0), (2, 2), 1), ((3, 5), (1, 2), (2, 2), 0)):
        for oa, oz in ((0.05, 33), (0.07, 12)):
            want = port.pool_u8(x, 0, kern, pad, stride, cm, 0.05, 33, oa, oz)
            got = ops.pool(to_dev_nhwc(x), 0, kern, pad, stride, cm, 0.05, 33, oa, oz)
            assert_same(to_host_nchw(got), want, "pool pair %s %s %s" % (kern, stride, oa))
    # the ResNet shapes: 3x3 s2 p1 max on 112x112 (ceil_mode false) and 7x7 global average
    x = rng.integers(0, 256, (2, 64, 112, 112), dtype=np.uint8)
    want = port.pool_u8(x, 0, (3, 3), (1, 1), (2, 2), 0, 0.05, 3, 0.05, 3)
    assert want.shape[2:] == (56, 56)
    assert_same(to_host_nchw(ops.pool(to_dev_nhwc(x), 0, (3, 3), (1, 1), (2, 2), 0, 0.05, 3, 0.05, 3)), want, "resnet maxpool")
    x = rng.integers(0, 256, (4, 2048, 7, 7), dtype=np.uint8)
    want = port.pool_u8(x, 1, (7, 7), (0, 0), (1, 1), 0, 0.05, 3, 0.02, 0)
    assert_same(to_host_nchw(ops.pool(to_dev_nhwc(x), 1, (7, 7), (0, 0), (1, 1), 0, 0.05, 3, 0.02, 0)), want, "resnet gap")


@pytest.mark.parametrize("k,ks,st,pd,h,w", [(64, 7, 2, 3, 33, 35), (32, 3, 2, 1, 20, 22), (16, 3, 1, 1, 9, 8),
                                             (48, 5, 1, 0, 12, 17), (64, 7, 2, 3, 224, 224)])
def test_conv_four_channel_image_row_lowering(ops, port, k, ks, st, pd, h, w):
    """4-channel (padded RGB) inputs take the tensor-core path through the row-lowering kernel."""
    x, wt, bias, walpha = conv_inputs(k + ks + h, 2, 4, h, w, k, ks, ks)
    wt[:, 3] = 128            # the padding channel carries zero weights
    q = dict(ialpha=0.02, izp=97, wzp=128, oalpha=0.05 * np.sqrt(3 * ks * ks) / 2, ozp=13)
    want = port.conv2d_u8(x, wt, bias, (st, st), (pd, pd), 1, walpha=walpha, relu=True, **q)
    conv = ops.Conv2d(wt, bias, in_hw=(h, w), stride=(st, st), pad=(pd, pd), walpha=walpha, relu=True, **q)
    assert conv.algo == ops.ALGO_IGEMM
    got = to_host_nchw(conv(to_dev_nhwc(x)))
    assert ops.device_status() == 0
    assert_same(got, want, "row lowering k=%d ks=%d" % (k, ks))
    # a second call at a smaller batch reuses the scratch tensor
    got1 = to_host_nchw(conv(to_dev_nhwc(x[:1])))
    assert_same(got1, want[:1], "row lowering, smaller batch")


@pytest.mark.parametrize("k", [32, 48, 16])
def test_conv_requantize_variants_on_both_paths(ops, port, k):
    """Epilogue variants of the tensor-core path: shifts below 32 (large scales), output widths
    below 8 bits, channel tiles of 16 and of 48 (a 32-column chunk plus a 16-column tail)."""
    x, wt, bias, walpha = conv_inputs(40 + k, 3, 32, 9, 10, k, 3, 3)
    for oalpha, obits, ozp in ((0.3, 8, 11), (1e-4, 8, 100), (3e-6, 8, 7), (0.3, 7, 40), (0.5, 4, 5), (2e-5, 6, 20)):
        q = dict(ialpha=0.02, izp=101, wzp=128, oalpha=oalpha, ozp=ozp, obits=obits)
        for relu in (False, True):
            want = port.conv2d_u8(x, wt, bias, (1, 1), (1, 1), 1, walpha=walpha, relu=relu, **q)
            for algo in (ops.ALGO_DIRECT, ops.ALGO_IGEMM):
                got = run_conv(ops, x, wt, bias, 1, 1, 1, algo, walpha=walpha, relu=relu, **q)
                assert_same(got, want, "k=%d oalpha=%g obits=%d relu=%s algo=%d" % (k, oalpha, obits, relu, algo))


@pytest.mark.parametrize("c,h,w,sh,sw,pd", [(32, 9, 9, 1, 1, 1), (64, 7, 12, 1, 1, 0), (16, 5, 3, 1, 1, 1), (48, 11, 10, 2, 1, 1),
                                            (16, 3, 4, 1, 1, 0), (32, 12, 12, 2, 2, 1), (48, 9, 11, 2, 2, 1), (16, 7, 7, 2, 2, 0),
                                            (16, 8, 9, 1, 2, 1), (32, 5, 5, 2, 2, 1), (16, 3, 3, 2, 2, 1)])
def test_depthwise3x3_two_pixels_per_thread(ops, port, c, h, w, sh, sw, pd):
    """Depthwise 3x3 with two output pixels (and, where the strides agree, two output rows) per thread:
    strides 1 and 2, odd and even output sizes, with and without padding, maps smaller than the
    thread's reach."""
    rng = np.random.default_rng(c * 100 + h * 10 + w)
    n = 3
    x = rng.integers(0, 256, (n, c, h, w), dtype=np.uint8)
    wt = (rng.integers(-127, 128, (c, 1, 3, 3)) + 128).astype(np.uint8)
    bias = rng.integers(-4096, 4097, c).astype(np.int32)
    walpha = rng.uniform(0.001, 0.01, c).astype(np.float32)
    q = dict(ialpha=0.04, izp=int(rng.integers(0, 256)), wzp=128, oalpha=0.12, ozp=int(rng.integers(0, 200)), walpha=walpha)
    for relu in (False, True):
        want = port.conv2d_u8(x, wt, bias, (sh, sw), (pd, pd), c, q["ialpha"], q["izp"], walpha, 128, q["oalpha"], q["ozp"],
                              relu=relu)
        conv = ops.Conv2d(wt, bias, in_hw=(h, w), stride=(sh, sw), pad=(pd, pd), group=c, algo=ops.ALGO_DIRECT, relu=relu, **q)
        got = to_host_nchw(conv(to_dev_nhwc(x)))
        assert ops.device_status() == 0
        assert_same(got, want, "dw pair c=%d %dx%d stride %dx%d pad=%d relu=%d" % (c, h, w, sh, sw, pd, relu))
    assert len(np.unique(want)) > 16


# (c, k, kernel, stride, pad, group, h, w, algo name): every kernel that forms products
WZP_SHAPES = [(64, 64, 3, 1, 1, 1, 13, 11, "igemm"), (32, 48, 1, 1, 0, 1, 9, 9, "igemm"), (128, 32, 3, 2, 1, 1, 12, 12, "igemm"),
              (256, 272, 1, 1, 0, 1, 7, 7, "igemm"), (4, 64, 7, 2, 3, 1, 30, 34, "igemm"), (64, 64, 3, 1, 1, 1, 13, 11, "direct"),
              (12, 10, 3, 1, 1, 2, 8, 9, "direct"), (7, 5, 2, 1, 0, 1, 6, 6, "direct"), (32, 32, 3, 1, 1, 32, 10, 10, "direct"),
              (16, 16, 5, 2, 2, 16, 11, 9, "direct")]


@pytest.mark.parametrize("shape", WZP_SHAPES)
@pytest.mark.parametrize("wzp", [0, 77, 131, 255])
def test_conv_weight_zero_point(ops, port, shape, wzp):
    """Asymmetric weights: any stored byte, any zero point.  The kernels multiply by (stored - 128) and
    take (wzp - 128) times the window sum of the activations off the accumulator."""
    c, k, ks, st, pd, g, h, w, algo_name = shape
    rng = np.random.default_rng(1000 + c + k + wzp)
    n = 3
    x = rng.integers(0, 256, (n, c, h, w), dtype=np.uint8)
    wt = rng.integers(0, 256, (k, c // g, ks, ks), dtype=np.uint8)
    walpha = rng.uniform(0.001, 0.01, k).astype(np.float32)
    izp = int(rng.integers(0, 256))
    # weights with a non-zero mean push the accumulators far from 0: the bias centres every channel,
    # and the output scale comes from the accumulators' spread, so that the bytes use the range
    zero = np.zeros(k, np.int32)
    _, acc = port.conv2d_u8(x, wt, zero, (st, st), (pd, pd), g, 0.03, izp, walpha, wzp, 1.0, 0, return_acc=True)
    bias = (-acc.astype(np.float64).mean(axis=(0, 2, 3))).round().astype(np.int32) + rng.integers(-4096, 4097, k).astype(np.int32)
    real = (acc + bias[None, :, None, None]).astype(np.float64) * 0.03 * walpha.astype(np.float64)[None, :, None, None]
    oalpha = float(np.float32(real.std() / 45.0))
    ozp = int(rng.integers(100, 156))
    q = dict(ialpha=0.03, izp=izp, wzp=wzp, oalpha=oalpha, ozp=ozp, walpha=walpha)
    want = port.conv2d_u8(x, wt, bias, (st, st), (pd, pd), g, q["ialpha"], q["izp"], walpha, wzp, q["oalpha"], q["ozp"],
                          relu=bool(wzp & 1))
    algo = ops.ALGO_IGEMM if algo_name == "igemm" else ops.ALGO_DIRECT
    got = run_conv(ops, x, wt, bias, st, pd, g, algo, relu=bool(wzp & 1), **q)
    assert_same(got, want, "wzp=%d %s" % (wzp, shape))
    assert len(np.unique(want)) > 16


@pytest.mark.parametrize("c,k,ks,st,hw", [(16, 96, 1, 1, 14), (48, 32, 3, 1, 9), (80, 48, 3, 2, 12), (144, 24, 1, 1, 7),
                                          (16, 16, 3, 1, 8), (208, 64, 1, 2, 10), (96, 576, 1, 1, 6)])
def test_conv_channels_not_multiple_of_32_on_tensor_cores(ops, port, c, k, ks, st, hw):
    """Input channel counts that are multiples of 16 but not of 32 (MobileNetV2's 16, 96, 144, 576 ...):
    the tensor-core path pads the repacked weights to 32 and lets TMA zero-fill the activations."""
    n, pd = 3, ks // 2
    x, wt, bias, walpha = conv_inputs(900 + c + k, n, c, hw, hw, k, ks, ks, 1)
    q = dict(ialpha=0.029, izp=101, wzp=128, oalpha=0.05 * np.sqrt(c * ks * ks) / 4, ozp=33, walpha=walpha)
    want = port.conv2d_u8(x, wt, bias, (st, st), (pd, pd), 1, q["ialpha"], q["izp"], walpha, 128, q["oalpha"], q["ozp"],
                          relu=True)
    got = run_conv(ops, x, wt, bias, st, pd, 1, ops.ALGO_IGEMM, relu=True, **q)
    assert_same(got, want, "c=%d k=%d %dx%d s%d" % (c, k, ks, ks, st))


def test_bounded_wait_expiry_is_reported_and_the_context_survives(ops, port):
    """The give-up path of the kernels' bounded waits, exercised the harmless way: a one-warp kernel
    waits on a barrier nothing arrives at, with a limit of about a millisecond; it gives up, writes its
    code to the device status word and ends normally.  The status call reports the code once, a case run
    that follows such a kernel returns B200_ERR_DEVICE_WAIT, and ordinary work is correct afterwards."""
    import ctypes as C
    import time
    import torch
    from nart_b200 import nets
    from nart_b200._lib import B200Error, ERR_DEVICE_WAIT, ERR_INVALID, check, lib
    from oracle.net_walk import run_net
    side = torch.cuda.Stream()
    stream = side.cuda_stream
    assert ops.device_status() == 0
    assert lib.b200_selftest_wait_expiry(0, stream) == ERR_INVALID
    t = time.perf_counter()
    check(lib.b200_selftest_wait_expiry(2_000_000, stream))
    word = C.c_int(0)
    check(lib.b200_device_status(stream, C.byref(word)))
    assert time.perf_counter() - t < 5.0           # about a millisecond of waiting, not the kernels' two seconds
    assert word.value == 0x1FF
    check(lib.b200_device_status(stream, C.byref(word)))
    assert word.value == 0                          # reading clears it

    # the host-buffer entry point of a case maps the word to the error status
    spec = nets.resnet(18, seed=31, hw=32, width_div=4, spread=True, num_classes=10)
    x = np.random.default_rng(12).integers(0, 256, (2, 3, 32, 32), dtype=np.uint8)
    want, _, _ = run_net(spec, x, port)
    cs, _ = nets.to_case(spec, 2)
    check(lib.b200_selftest_wait_expiry(1_000_000, stream))
    with pytest.raises(B200Error) as ei:
        cs.run_host([x], [(np.float32, (10, 1, 1))], stream)
    assert ei.value.status == ERR_DEVICE_WAIT
    # ... and the same case, same context, right after: correct results, clean status
    (got,) = cs.run_host([x], [(np.float32, (10, 1, 1))], stream)
    assert_same(got.reshape(want.shape).view(np.uint32), want.view(np.uint32), "after an expired wait")
    assert ops.device_status() == 0
    cs.close()


@pytest.mark.parametrize("shape", [(256, 256, 14, 3, 1, 5), (512, 256, 7, 3, 2, 3), (1024, 512, 7, 1, 1, 9), (128, 320, 9, 3, 1, 2)])
def test_conv_on_cta_pairs(ops, port, monkeypatch, shape):
    """The kernel variant in which two CTAs of a cluster run every MMA together (tcgen05 cta_group::2, M = 256),
    forced onto small shapes: odd numbers of M tiles (the second CTA of the last pair has no tile), several
    channel tiles, stride 2, a channel tile narrower than 256."""
    c, k, h, ks, st, batch = shape
    monkeypatch.setenv("B200_IGEMM_CTA_PAIR", "1")
    x, wt, bias, walpha = conv_inputs(700 + c + k + h, batch, c, h, h, k, ks, ks)
    q = dict(ialpha=0.02, izp=119, wzp=128, oalpha=0.05 * np.sqrt(c * ks * ks) / 8, ozp=3)
    conv = ops.Conv2d(wt, bias, in_hw=(h, h), stride=(st, st), pad=(ks // 2, ks // 2), algo=ops.ALGO_IGEMM, walpha=walpha,
                      relu=True, **q)
    y = conv(to_dev_nhwc(x))
    assert "cta-pair" in conv.describe(), conv.describe()
    assert ops.device_status() == 0
    want = port.conv2d_u8(x, wt, bias, (st, st), (ks // 2, ks // 2), 1, walpha=walpha, relu=True, **q)
    assert_same(to_host_nchw(y), want, "cta pair %s" % (shape,))


def test_conv_picks_cta_pairs_on_long_launches(ops, port):
    """Without any switch a 256-wide, reduction-heavy layer runs on CTA pairs once the launch is long enough
    (six pair tiles per cluster), and on single CTAs below that; both give the restatement's bytes."""
    c = k = 256
    h, ks = 14, 3
    x, wt, bias, walpha = conv_inputs(4321, 640, c, h, h, k, ks, ks)
    q = dict(ialpha=0.02, izp=128, wzp=128, oalpha=0.05 * np.sqrt(c * ks * ks) / 8, ozp=0)
    conv = ops.Conv2d(wt, bias, in_hw=(h, h), stride=(1, 1), pad=(1, 1), algo=ops.ALGO_IGEMM, walpha=walpha, relu=True, **q)
    xd = to_dev_nhwc(x)
    y_small = conv(xd[:8].contiguous())
    assert "cta-pair (" not in conv.describe(), conv.describe()
    y = conv(xd)
    assert "cta-pair (" in conv.describe(), conv.describe()
    assert ops.device_status() == 0
    pick = [0, 7, 320, 639]
    want = port.conv2d_u8(x[pick], wt, bias, (1, 1), (1, 1), 1, walpha=walpha, relu=True, **q)
    assert_same(to_host_nchw(y[pick]), want, "long launch on cta pairs")
    assert_same(to_host_nchw(y_small[[0, 7]]), want[:2], "short launch on single CTAs")
