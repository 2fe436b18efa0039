"""Regenerates quant_param_ref.json from the reference's own Python source.

The reference package cannot be imported here (it needs its compiled runtime and caffe), so the
functions this path mirrors are cut out of their source files with ``ast`` and executed on their own:
``QuantParam`` and ``convert_quant_param`` from python/nart/modules/quant.py, ``quant_weights`` and
``quant_bias`` from python/nart/calibrator.py.  Usage:

    python tests/golden/gen_quant_param_golden.py <path to the reference checkout>
"""
import ast
import json
import os
import sys
from types import SimpleNamespace

import numpy as np


def cut(path, class_name, names):
    tree = ast.parse(open(path).read())
    body = tree.body
    if class_name:
        body = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == class_name).body
    picked = [n for n in body if isinstance(n, (ast.ClassDef, ast.FunctionDef)) and n.name in names]
    assert len(picked) == len(names), (path, names)
    return picked


def main():
    ref = sys.argv[1]
    rng = np.random.default_rng(11)

    # ---- quant.py: QuantParam + convert_quant_param, as members of a stand-in class -----------------
    nodes = cut(os.path.join(ref, "python/nart/modules/quant.py"), "CaffeQuantParser", ["QuantParam", "convert_quant_param"])
    holder = ast.ClassDef(name="Holder", bases=[], keywords=[], body=nodes, decorator_list=[])
    mod = ast.Module(body=[holder], type_ignores=[])
    ast.fix_missing_locations(mod)
    ns = {}
    exec(compile(mod, "quant.py", "exec"), ns)
    Holder = ns["Holder"]
    ns["QuantParam"] = Holder.QuantParam          # to_biased names the class without a qualifier
    obj = Holder()

    entries = {}
    for i in range(60):
        bit = int(rng.choice([4, 8, 8, 8, 16]))
        tp = "symmetric" if rng.random() < 0.4 else "biased"
        lo, hi = sorted(rng.normal(0, 3, 2).tolist())
        if rng.random() < 0.15:
            lo, hi = abs(lo) + 0.1, abs(lo) + abs(hi) + 0.2      # all-positive range: min is clamped to 0
        if rng.random() < 0.1:
            lo, hi = -abs(lo) - abs(hi) - 0.2, -abs(hi) - 0.1    # all-negative range
        entries["t%d" % i] = {"max": hi, "min": lo, "bit": bit, "type": tp}
    for i in range(12):
        entries["a%d" % i] = {"alpha": float(rng.uniform(0.001, 0.1)), "zero_point": int(rng.integers(0, 256)),
                              "bit": 8, "type": "symmetric" if i % 3 == 0 else "biased"}
    conv = obj.convert_quant_param(entries)
    converted = {}
    for k, q in conv.items():
        b = q.to_biased()
        converted[k] = {"alpha": q.alpha, "zero_point": q.zero_point, "bits": q.bits, "qtype": q.qtype,
                        "to_biased": [b.alpha, b.zero_point, b.bits, b.qtype]}

    # ---- calibrator.py: quant_weights (min/max form) and quant_bias ---------------------------------
    nodes = cut(os.path.join(ref, "python/nart/calibrator.py"), None, ["quant_weights", "quant_bias"])
    mod = ast.Module(body=nodes, type_ignores=[])
    ast.fix_missing_locations(mod)
    cns = {"np": np}
    exec(compile(mod, "calibrator.py", "exec"), cns)
    weights = {}
    layers = []
    for i in range(6):
        w = (rng.normal(0, 0.05, (8, 4, 3, 3)) + (0.08 if i == 4 else 0.0) - (0.3 if i == 5 else 0.0)).astype(np.float32)
        weights["conv%d" % i] = w
        layers.append(SimpleNamespace(
            type="Convolution" if i % 2 == 0 else "InnerProduct", name="conv%d" % i, bottom=["blob%d" % i],
            blobs=[SimpleNamespace(data=w.ravel().tolist())],
            convolution_param=SimpleNamespace(bias_term=True), inner_product_param=SimpleNamespace(bias_term=True)))
    model = SimpleNamespace(layer=layers)
    calib = {}
    for symmetric in (False, True):
        args = SimpleNamespace(symmetric=symmetric, kl_divergence=False, bit_width=8)
        param = cns["quant_weights"](args, model)
        for i in range(6):
            lo, hi = sorted(rng.normal(0, 4, 2).tolist())
            if symmetric:
                hi = max(abs(lo), abs(hi)); lo = -hi
            param["blob%d" % i] = {"max": hi, "min": lo, "bit": 8, "type": "symmetric" if symmetric else "biased"}
        cns["quant_bias"](args, model, param)
        calib["symmetric" if symmetric else "biased"] = {
            k: {kk: (float(vv) if isinstance(vv, (float, np.floating)) else vv) for kk, vv in v.items()}
            for k, v in param.items()}

    out = {"entries": entries, "converted": converted,
           "weights": {k: v.ravel().tolist() for k, v in weights.items()}, "calibrator": calib}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_param_ref.json")
    with open(path, "wt") as f:
        json.dump(out, f)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
