"""The calibrator hand-off (nart_b200/quant_param.py) against outputs of the reference's own Python
functions (tests/golden/quant_param_ref.json, written by gen_quant_param_golden.py)."""
import json
import os

import numpy as np
import pytest

from nart_b200 import quant_param as qp

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "quant_param_ref.json")))


def test_convert_quant_param_matches_reference():
    got = qp.convert_quant_param(GOLD["entries"])
    assert set(got) == set(GOLD["converted"])
    n_biased_minmax = 0
    for k, want in GOLD["converted"].items():
        q = got[k]
        assert q.alpha == want["alpha"], k                 # same float operations: equal to the last bit
        assert q.zero_point == want["zero_point"], k
        assert (q.bits, q.qtype) == (want["bits"], want["qtype"]), k
        b = q.to_biased()
        assert [b.alpha, b.zero_point, b.bits, b.qtype] == want["to_biased"], k
        n_biased_minmax += "max" in GOLD["entries"][k] and GOLD["entries"][k]["type"] == "biased"
    assert n_biased_minmax > 20


def test_zero_point_forms():
    e = {"x": {"max": 6.0, "min": -2.0, "bit": 8, "type": "biased"}}
    ref = qp.convert_quant_param(e)["x"]
    assert ref.alpha == 8.0 / 255 and ref.zero_point == round(8.0 / 255 * 2.0)      # the reference's product form
    quo = qp.convert_quant_param(e, zero_point_quotient=True)["x"]
    assert quo.zero_point == round(2.0 / (8.0 / 255)) == 64                         # min -> 0, max -> 255
    # ranges that do not straddle 0 are widened to include it
    pos = qp.convert_quant_param({"x": {"max": 4.0, "min": 1.0, "bit": 8, "type": "biased"}})["x"]
    assert pos.alpha == 4.0 / 255 and pos.zero_point == 0
    sym = qp.convert_quant_param({"x": {"max": 1.0, "min": -3.0, "bit": 8, "type": "symmetric"}})["x"]
    assert sym.alpha == 3.0 / 127 and sym.zero_point == 0
    assert sym.to_biased().zero_point == 128 and sym.to_biased().qtype == qp.SYMMETRIC


def test_errors_follow_the_reference():
    with pytest.raises(RuntimeError, match="`type` is required"):
        qp.convert_quant_param({"x": {"max": 1.0, "min": 0.0, "bit": 8}})
    with pytest.raises(RuntimeError, match="`type` can be"):
        qp.convert_quant_param({"x": {"max": 1.0, "min": 0.0, "bit": 8, "type": "affine"}})
    with pytest.raises(RuntimeError, match="`bit` is required"):
        qp.convert_quant_param({"x": {"max": 1.0, "min": 0.0, "type": "biased"}})
    with pytest.raises(RuntimeError, match="is required for quantization"):
        qp.convert_quant_param({"x": {"max": 1.0, "bit": 8, "type": "biased"}})
    assert qp.convert_quant_param(None) is None


def test_calibrator_entries_match_reference():
    weights = {k: np.array(v, dtype=np.float32).reshape(8, 4, 3, 3) for k, v in GOLD["weights"].items()}
    layers = [("conv%d" % i, "blob%d" % i) for i in range(6)]
    for mode in ("biased", "symmetric"):
        want = GOLD["calibrator"][mode]
        sym = mode == "symmetric"
        param = qp.weight_entries(weights, 8, sym)
        for k, w in param.items():
            assert w["type"] == want[k]["type"] and w["bit"] == want[k]["bit"], k
            assert float(w["max"]) == want[k]["max"] and float(w["min"]) == want[k]["min"], k
        for i in range(6):
            param["blob%d" % i] = want["blob%d" % i]
        bias = qp.bias_entries(layers, param, 8, sym)
        for k, b in bias.items():
            assert b == want[k], k
        assert len(bias) == 6


def test_activation_entries():
    ext = {"a": {"max": [1.0, 3.0], "min": [-1.0, -0.5]}, "b": {"max": [2.0, 4.0], "min": [0.5, 1.5]}}
    got = qp.activation_entries(ext)
    assert got["a"] == {"max": 2.0, "min": -0.75, "bit": 8, "type": "biased"}
    assert got["b"]["min"] == 1.0                                   # clamped to 0 later, in convert_quant_param
    sym = qp.activation_entries(ext, symmetric=True)
    assert sym["a"] == {"max": 2.0, "min": -2.0, "bit": 8, "type": "symmetric"}
    assert sym["b"] == {"max": 3.0, "min": -3.0, "bit": 8, "type": "symmetric"}


def test_quantize_weight():
    w = np.array([-1.0, -0.26, 0.0, 0.26, 0.5, 9.0], dtype=np.float32)
    q = qp.quantize_weight(w, qp.QuantParam(0.01, 128, 8, qp.BIASED))
    assert q.dtype == np.uint8 and q.tolist() == [28, 102, 128, 154, 178, 255]
    q = qp.quantize_weight(w, qp.QuantParam(0.01, 0, 8, qp.SYMMETRIC))
    assert q.dtype == np.int8 and q.tolist() == [-100, -26, 0, 26, 50, 127]
    q = qp.quantize_weight(w * 1000, qp.QuantParam(0.01, 0, 32, qp.SYMMETRIC))
    assert q.dtype == np.int32 and q[-1] == 900000
    q = qp.quantize_weight(w, qp.QuantParam(0.001, 0, 16, qp.DEFAULT))
    assert q.dtype == np.int16 and q[0] == -1000


def test_load_max_min(tmp_path):
    p = tmp_path / "max_min.json"
    p.write_text(json.dumps({"data": {"max": 2.0, "min": -2.0, "bit": 8, "type": "biased"}}))
    got = qp.load_max_min(str(p))
    assert got["data"].alpha == 4.0 / 255
