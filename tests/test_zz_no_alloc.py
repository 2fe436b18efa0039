"""GPU: the allocation-free convolution entry point, b200_conv2d_run_static_scratch, against the
regular one and against the CPU restatement.

Some hosts of the library cannot let it allocate while it runs: a serving loop where the
device-wide synchronization of cudaMalloc / cudaFree would stall every stream, or an application
that has handed all device memory to its own pool, so that an allocation from inside a plugin
fails.  For them the row-lowered stem convolution keeps its scratch tensor in a fixed 32 MiB device
array that is part of the library.  This file is collected last on purpose (its name sorts after
the others), and it also passes on its own in a fresh process, where the new entry point is the
very first kernel launch.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _stem(seed, n, h, w, k, ks, stride, pad):
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 256, (n, h, w, 4), dtype=np.uint8)          # NHWC, 4 channels
    wt = (rng.integers(-127, 128, (k, 4, ks, ks)) + 128).astype(np.uint8)
    bias = rng.integers(-4096, 4097, k).astype(np.int32)
    walpha = rng.uniform(0.001, 0.01, k).astype(np.float32)
    return x, wt, bias, walpha


def _static_status(lib, stream):
    word = C.c_int(-1)
    rc = lib.b200_static_scratch_status(stream, C.byref(word))
    return rc, word.value


def test_static_scratch_matches_regular_entry_point_twice(port):
    import torch
    from nart_b200 import ops
    from nart_b200._lib import ERR_INVALID, ERR_UNSUPPORTED, check, lib
    n, h, w, k = 3, 64, 72, 64
    x, wt, bias, walpha = _stem(1, n, h, w, k, 7, 2, 3)
    q = dict(ialpha=0.02, izp=113, walpha=walpha, oalpha=0.3, ozp=9, relu=True)
    conv = ops.Conv2d(wt, bias, in_hw=(h, w), stride=(2, 2), pad=(3, 3), **q)
    assert conv.algo == ops.ALGO_IGEMM
    stream = torch.cuda.current_stream().cuda_stream
    oh, ow = conv.out_hw
    for call in range(2):            # two calls in a row, different data: nothing stale may survive
        xh = np.roll(x, call * 5, axis=1).copy()
        xd = torch.from_numpy(xh).cuda()
        y_static = torch.zeros((n, oh, ow, k), dtype=torch.uint8, device="cuda")
        check(lib.b200_conv2d_run_static_scratch(conv._h, xd.data_ptr(), n, y_static.data_ptr(), stream))
        y_regular = conv(xd)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        assert _static_status(lib, stream) == (0, 0)
        assert torch.equal(y_static, y_regular), "call %d: outputs differ" % call
        assert int(y_regular.max()) > 9 and len(torch.unique(y_regular)) > 8
        # and against the CPU restatement (NCHW, the 4 stored channels)
        want = port.conv2d_u8(np.ascontiguousarray(xh.transpose(0, 3, 1, 2)), wt, bias, (2, 2), (3, 3), 1, wzp=128, **q)
        got = np.ascontiguousarray(y_static.cpu().numpy().transpose(0, 3, 1, 2))
        assert np.array_equal(got, want), "call %d: differs from the restatement" % call

    # A second plan of another shape straight after, on the same stream, with a batch that fills most of
    # the 32 MiB: whatever the first plan left in the array lies inside this tensor's extent and beyond
    # it, and must not show.  The steady-state call (the second with the same buffers) must leave the
    # amount of free device memory exactly as it found it.
    n2, h2, w2, k2 = 128, 96, 160, 32
    x2, wt2, bias2, walpha2 = _stem(7, n2, h2, w2, k2, 5, 2, 2)
    q2 = dict(ialpha=0.05, izp=31, walpha=walpha2, oalpha=0.2, ozp=77, relu=False)
    conv_b = ops.Conv2d(wt2, bias2, in_hw=(h2, w2), stride=(2, 2), pad=(2, 2), **q2)
    assert conv_b.algo == ops.ALGO_IGEMM
    oh2, ow2 = conv_b.out_hw
    assert 28 * 2**20 < n2 * h2 * ow2 * 32 <= 32 * 2**20
    x2d = torch.from_numpy(x2).cuda()
    y2d = torch.zeros((n2, oh2, ow2, k2), dtype=torch.uint8, device="cuda")
    check(lib.b200_conv2d_run_static_scratch(conv_b._h, x2d.data_ptr(), n2, y2d.data_ptr(), stream))
    torch.cuda.synchronize()
    first = y2d.clone()
    y2d.zero_()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    check(lib.b200_conv2d_run_static_scratch(conv_b._h, x2d.data_ptr(), n2, y2d.data_ptr(), stream))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the steady-state call changed free device memory by %d bytes" % (free_before - free_after)
    assert _static_status(lib, stream) == (0, 0)
    assert torch.equal(y2d, first)
    pick = [0, 29, n2 - 1]
    want = port.conv2d_u8(np.ascontiguousarray(x2[pick].transpose(0, 3, 1, 2)), wt2, bias2, (2, 2), (2, 2), 1, wzp=128, **q2)
    got = np.ascontiguousarray(y2d[pick].cpu().numpy().transpose(0, 3, 1, 2))
    assert np.array_equal(got, want), "second plan differs from the restatement"
    assert len(np.unique(want)) > 16

    # a smaller batch through the same array
    y1 = torch.zeros((1, oh, ow, k), dtype=torch.uint8, device="cuda")
    xd = torch.from_numpy(x[:1].copy()).cuda()
    check(lib.b200_conv2d_run_static_scratch(conv._h, xd.data_ptr(), 1, y1.data_ptr(), stream))
    assert torch.equal(y1, conv(xd))

    # beyond the fixed array: a clear refusal, nothing launched
    big = 32 * 1024 * 1024 // (h * ow * 32) + 1
    rc = lib.b200_conv2d_run_static_scratch(conv._h, xd.data_ptr(), big, y1.data_ptr(), stream)
    assert rc == ERR_UNSUPPORTED and b"static array holds" in lib.b200_last_error()

    # a plan without a scratch tensor is not this entry point's business
    wt2 = (np.random.default_rng(2).integers(-127, 128, (32, 32, 3, 3)) + 128).astype(np.uint8)
    conv2 = ops.Conv2d(wt2, None, in_hw=(8, 8), pad=(1, 1), ialpha=0.02, izp=1, walpha=0.005, oalpha=0.1, ozp=0)
    x2 = torch.zeros((1, 8, 8, 32), dtype=torch.uint8, device="cuda")
    y2 = torch.zeros((1, 8, 8, 32), dtype=torch.uint8, device="cuda")
    rc = lib.b200_conv2d_run_static_scratch(conv2._h, x2.data_ptr(), 1, y2.data_ptr(), stream)
    assert rc == ERR_INVALID
