"""CPU: the network walker over the restatement agrees with the same walk over the compiled
reference (per-tensor weight scale, the only form the reference executes), and the spec
generators are deterministic."""
import numpy as np

from nart_b200 import nets
from oracle.net_walk import run_net


def test_spec_is_seeded():
    a = nets.resnet(18, seed=2, hw=32, width_div=4)
    b = nets.resnet(18, seed=2, hw=32, width_div=4)
    assert all(np.array_equal(x["w"], y["w"]) for x, y in zip(a["ops"], b["ops"]) if "w" in x)
    assert a["tensors"] == b["tensors"]


def test_resnet50_conv_work_matches_the_known_figure():
    # 4.0871 GMAC of convolution per 224x224 image
    spec = nets.resnet(50)
    assert abs(nets.conv_ops_per_image(spec) / 2 / 1e9 - 4.0871) < 0.01
    spec = nets.resnet(18)
    assert abs(nets.conv_ops_per_image(spec) / 2 / 1e9 - 1.8136) < 0.01


def test_small_resnet_port_equals_reference(port, ref):
    rng = np.random.default_rng(0)
    for depth in (18, 50):
        spec = nets.resnet(depth, seed=11, hw=96, width_div=4, spread=True, num_classes=10)
        x = rng.integers(0, 256, (2, 3, 96, 96), dtype=np.uint8)  # maps stay >= 3x3: the reference mis-handles maps smaller than the kernel
        lp, qp, _ = run_net(spec, x, port, per_channel=False)
        lr, qr, _ = run_net(spec, x, ref, per_channel=False)
        assert np.array_equal(qp, qr)
        assert np.array_equal(lp.view(np.uint32), lr.view(np.uint32))
        assert len(np.unique(qp)) > 4   # the outputs are spread, not saturated
