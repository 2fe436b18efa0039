"""The calibrator hand-off end to end: an fp32 two-conv net, per-batch extremes -> max_min entries ->
scales, zero points and integer weights (nart_b200/quant_param.py) -> a GPU case.  The quantized
net must track the fp32 one to within a few quantization steps."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from nart_b200 import quant_param as qp

pytestmark = pytest.mark.gpu


def test_float_net_through_max_min_to_gpu_case():
    from nart_b200.case import Case
    rng = np.random.default_rng(5)
    w1 = (rng.normal(0, 0.08, (32, 16, 3, 3)) + 0.05).astype(np.float32)     # off-centre: asymmetric ranges
    b1 = rng.normal(0, 0.1, 32).astype(np.float32)
    w2 = (rng.normal(0, 0.12, (16, 32, 1, 1)) - 0.04).astype(np.float32)
    b2 = rng.normal(0, 0.1, 16).astype(np.float32)

    def forward(x):
        t = torch.from_numpy(x)
        h1 = F.relu(F.conv2d(t, torch.from_numpy(w1), torch.from_numpy(b1), padding=1))
        h2 = F.conv2d(h1, torch.from_numpy(w2), torch.from_numpy(b2))
        return {"data": x, "conv1": h1.numpy(), "conv2": h2.numpy()}

    # calibration: extremes of every tensor over a few batches
    ext = {k: {"max": [], "min": []} for k in ("data", "conv1", "conv2")}
    for _ in range(4):
        acts = forward(rng.uniform(-1.0, 1.5, (8, 16, 12, 12)).astype(np.float32))
        for k, a in acts.items():
            ext[k]["max"].append(float(a.max()))
            ext[k]["min"].append(float(a.min()))
    # the calibrator's defaults: biased (asymmetric) weights and activations, each with its own zero point
    param = qp.weight_entries({"conv1": w1, "conv2": w2})
    param.update(qp.activation_entries(ext))
    param.update(qp.bias_entries([("conv1", "data"), ("conv2", "conv1")], param))
    q = qp.convert_quant_param(param, zero_point_quotient=True)
    for k in ("data", "conv1", "conv2", "conv1_weight_0", "conv2_weight_0"):
        assert q[k].qtype == qp.BIASED and 0 <= q[k].zero_point <= 255 and q[k].alpha > 0
    assert q["conv1_weight_0"].zero_point != 128 and q["conv2_weight_0"].zero_point != 128
    # the bias step of the hand-off is the product of the two step sizes it is added between
    assert q["conv1_weight_1"].alpha == pytest.approx(q["conv1_weight_0"].alpha * q["data"].alpha, rel=1e-6)

    cs = Case()
    t0 = cs.input_f32(16, 12, 12, q["data"].alpha, q["data"].zero_point)
    qw1, qw2 = q["conv1_weight_0"], q["conv2_weight_0"]
    t1 = cs.conv2d(t0, qp.quantize_weight(w1, qw1), qp.quantize_weight(b1, q["conv1_weight_1"]),
                   pad=(1, 1), ialpha=q["data"].alpha, izp=q["data"].zero_point, walpha=qw1.alpha,
                   wzp=qw1.zero_point, oalpha=q["conv1"].alpha, ozp=q["conv1"].zero_point, relu=True)
    t2 = cs.conv2d(t1, qp.quantize_weight(w2, qw2), qp.quantize_weight(b2, q["conv2_weight_1"]),
                   ialpha=q["conv1"].alpha, izp=q["conv1"].zero_point, walpha=qw2.alpha,
                   wzp=qw2.zero_point, oalpha=q["conv2"].alpha, ozp=q["conv2"].zero_point)
    cs.output_f32(t2, q["conv2"].alpha, q["conv2"].zero_point)
    cs.prepare(8)

    x = rng.uniform(-1.0, 1.5, (8, 16, 12, 12)).astype(np.float32)
    want = forward(x)["conv2"]
    got = cs.run_host([x], [(np.float32, (16, 12, 12))])[0]
    cs.close()
    step = q["conv2"].alpha
    err = np.abs(got - want)
    inside = (want > ext["conv2"]["min"][0]) & (want < ext["conv2"]["max"][0])    # values the 8-bit range can hold
    assert inside.mean() > 0.99
    assert err[inside].max() < 6 * step, (err[inside].max(), step)
    assert err[inside].mean() < 1.5 * step, (err[inside].mean(), step)
