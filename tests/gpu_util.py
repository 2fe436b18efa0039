"""Helpers for the GPU parity tests: numpy NCHW <-> device NHWC through the library's own layout
kernels or torch permutes (both are exercised)."""
import numpy as np
import torch


def to_dev_nhwc(x_nchw: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x_nchw.transpose(0, 2, 3, 1))).cuda()


def to_host_nchw(y_nhwc: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(y_nhwc.cpu().numpy().transpose(0, 3, 1, 2))


def assert_same(a: np.ndarray, b: np.ndarray, what=""):
    if not np.array_equal(a, b):
        bad = np.argwhere(a != b)
        raise AssertionError("%s: %d of %d differ; first at %s: got %s want %s" % (
            what, len(bad), a.size, tuple(bad[0]), a[tuple(bad[0])], b[tuple(bad[0])]))
