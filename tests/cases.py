"""Seeded synthetic inputs shared by the CPU and GPU tests (the single 3x3 conv on 56x56, the conv shape sweep and the small
edge-case shapes).  Everything is drawn from numpy's default_rng(seed)."""
import numpy as np


def conv_inputs(seed, n, c, h, w, k, r, s, group=1, per_channel=True):
    """uint8 activations U[0,255]; int8 weights U[-127,127] stored +128; int32 bias U[-4096,4096];
    per-channel weight scales U(0.001, 0.01)."""
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 256, (n, c, h, w), dtype=np.uint8)
    wt = (rng.integers(-127, 128, (k, c // group, r, s)) + 128).astype(np.uint8)
    bias = rng.integers(-4096, 4097, k).astype(np.int32)
    walpha = rng.uniform(0.001, 0.01, k).astype(np.float32)
    if not per_channel:
        walpha = walpha[:1]
    return x, wt, bias, walpha


# (n, c, h, w, k, r, s, stride, pad, group) -- edge shapes: odd sizes, ragged channel counts,
# grouped, depthwise, stem, tiny maps, asymmetric kernels
EDGE_SHAPES = [
    (1, 64, 56, 56, 64, 3, 3, 1, 1, 1),      # the single-conv benchmark case
    (2, 32, 9, 9, 32, 3, 3, 1, 1, 1),
    (3, 16, 7, 5, 48, 1, 1, 1, 0, 1),
    (2, 32, 11, 13, 16, 3, 3, 2, 1, 1),
    (1, 3, 33, 35, 8, 7, 7, 2, 3, 1),        # stem-like, C=3
    (2, 32, 10, 10, 32, 3, 3, 1, 1, 32),     # depthwise
    (2, 48, 9, 9, 48, 3, 3, 2, 1, 48),       # depthwise stride 2
    (2, 16, 8, 8, 24, 5, 5, 2, 2, 2),        # grouped
    (1, 20, 6, 6, 10, 3, 2, 1, 0, 1),        # asymmetric kernel, c % 16 != 0
    (2, 64, 1, 1, 40, 1, 1, 1, 0, 1),        # 1x1 map
    (1, 128, 4, 4, 128, 3, 3, 1, 1, 1),
    (5, 64, 7, 7, 64, 3, 3, 2, 1, 1),
]

# conv shape sweep: (c, k, h) x kernel {1,3} x stride {1,2}
SWEEP = [(c, k, h, ks, st) for (c, k, h) in [(64, 64, 56), (128, 128, 28), (256, 256, 14), (512, 512, 7)]
         for ks in (1, 3) for st in (1, 2)]


def conv_inputs_s8(seed, n, c, h, w, k, r, s, group=1):
    """The int8 (symmetric) path: int8 activations and weights in [-127, 127], int32 bias, one weight scale
    per output channel."""
    rng = np.random.default_rng(seed)
    x = rng.integers(-127, 128, (n, c, h, w)).astype(np.int8)
    wt = rng.integers(-127, 128, (k, c // group, r, s)).astype(np.int8)
    bias = rng.integers(-4096, 4097, k).astype(np.int32)
    walpha = rng.uniform(0.001, 0.01, k).astype(np.float32)
    return x, wt, bias, walpha


# (n, c, h, w, k, r, s, stride, pad, group, obits) for the int8 path; obits 8 is the reference's wrapping case
S8_SHAPES = [
    (2, 64, 14, 14, 64, 3, 3, 1, 1, 1, 7),
    (3, 32, 9, 11, 48, 1, 1, 1, 0, 1, 7),
    (2, 128, 8, 8, 256, 1, 1, 2, 0, 1, 7),
    (1, 16, 7, 9, 32, 3, 3, 2, 1, 1, 8),
    (2, 32, 6, 6, 32, 3, 3, 1, 1, 32, 7),     # depthwise
    (1, 16, 5, 5, 16, 5, 5, 1, 2, 2, 4),      # grouped, 4-bit outputs
    (2, 20, 6, 6, 10, 3, 2, 1, 0, 1, 6),      # c % 16 != 0
    (2, 64, 10, 10, 96, 3, 3, 1, 1, 1, 5),
]


def s8_oalpha(c, group, r, s):
    return float(np.float32(0.05 * np.sqrt(c // group * r * s) / 4))
