"""Asymmetric weights inside the case runner: a chain of convs with weight zero points other than 128
through tensors whose channel count is padded in the device buffers (24 -> 32), a depthwise conv among
them, against the CPU restatement op by op."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_case_with_weight_zero_points(port):
    from nart_b200.case import Case
    rng = np.random.default_rng(31)
    n, c, h, w = 3, 16, 10, 12

    def layer(k, cg, ks, wzp, fan):
        wt = rng.integers(0, 256, (k, cg, ks, ks), dtype=np.uint8)
        bias = rng.integers(-4096, 4097, k).astype(np.int32)
        walpha = rng.uniform(0.002, 0.006, k).astype(np.float32)
        return dict(wt=wt, bias=bias, walpha=walpha, wzp=wzp, oalpha=float(0.03 * 0.004 * 74 * 74 * np.sqrt(fan) / 40))

    l1 = layer(24, 16, 3, 100, 16 * 9)      # 24 output channels: padded to 32 on the device
    l2 = layer(24, 1, 3, 201, 9)            # depthwise on the padded tensor
    l3 = layer(32, 24, 1, 77, 24)           # reads the padded tensor
    x = rng.integers(0, 256, (n, c, h, w), dtype=np.uint8)
    zps = [128, 120, 131, 125]
    alphas = [0.03, l1["oalpha"], l2["oalpha"], l3["oalpha"]]
    # the zero points of asymmetric weights shift the accumulators: centre them with the bias, per channel
    acts = [x]
    for i, (l, group, pad) in enumerate(((l1, 1, 1), (l2, 24, 1), (l3, 1, 0))):
        zero = np.zeros_like(l["bias"])
        _, acc = port.conv2d_u8(acts[-1], l["wt"], zero, (1, 1), (pad, pad), group, alphas[i], zps[i], l["walpha"], l["wzp"],
                                1.0, 0, return_acc=True)
        l["bias"] = l["bias"] - acc.astype(np.float64).mean(axis=(0, 2, 3)).round().astype(np.int32)
        real = (acc + l["bias"][None, :, None, None]).astype(np.float64) * alphas[i] * l["walpha"].astype(np.float64)[None, :, None, None]
        alphas[i + 1] = float(np.float32(real.std() / 40.0))
        acts.append(port.conv2d_u8(acts[-1], l["wt"], l["bias"], (1, 1), (pad, pad), group, alphas[i], zps[i], l["walpha"],
                                   l["wzp"], alphas[i + 1], zps[i + 1], relu=(i == 0)))
        assert len(np.unique(acts[-1])) > 16

    cs = Case()
    t = cs.input_u8(c, h, w)
    outs = []
    for i, (l, group, pad) in enumerate(((l1, 1, 1), (l2, 24, 1), (l3, 1, 0))):
        t = cs.conv2d(t, l["wt"], l["bias"], pad=(pad, pad), group=group, ialpha=alphas[i], izp=zps[i], walpha=l["walpha"],
                      wzp=l["wzp"], oalpha=alphas[i + 1], ozp=zps[i + 1], relu=(i == 0))
        outs.append(t)
    cs.output_u8(outs[-1])
    cs.prepare(n)
    (got,) = cs.run_host([x], [(np.uint8, acts[-1].shape[1:])])
    cs.close()
    assert np.array_equal(got.reshape(acts[-1].shape), acts[-1])
