"""GPU: the allocation-free convolution entry point, b200_conv2d_run_static_scratch, against the
regular one.

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


def test_static_scratch_matches_regular_entry_point_twice():
    import torch
    from nart_b200 import ops
    from nart_b200._lib import ERR_INVALID, ERR_UNSUPPORTED, check, lib
    n, h, w, k = 3, 64, 72, 64
    x, wt, bias, walpha = _stem(1, n, h, w, k, 7, 2, 3)
    conv = ops.Conv2d(wt, bias, in_hw=(h, w), stride=(2, 2), pad=(3, 3), ialpha=0.02, izp=113, walpha=walpha,
                      oalpha=0.3, ozp=9, relu=True)
    assert conv.algo == ops.ALGO_IGEMM
    stream = torch.cuda.current_stream().cuda_stream
    oh, ow = conv.out_hw
    for call in range(2):            # two calls in a row, different data: nothing stale may survive
        xd = torch.from_numpy(np.roll(x, call * 5, axis=1).copy()).cuda()
        y_static = torch.zeros((n, oh, ow, k), dtype=torch.uint8, device="cuda")
        check(lib.b200_conv2d_run_static_scratch(conv._h, xd.data_ptr(), n, y_static.data_ptr(), stream))
        y_regular = conv(xd)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        assert torch.equal(y_static, y_regular), "call %d: outputs differ" % call
        assert int(y_regular.max()) > 9 and len(torch.unique(y_regular)) > 8

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
