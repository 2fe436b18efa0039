"""The calibrator hand-off: from the ``max_min.json`` a calibration run writes to the scales, zero
points and quantized weights a quantized case is built from.

Mirrors, for this path, the reference's
  * ``CaffeQuantParser.convert_quant_param`` / ``QuantParam`` (python/nart/modules/quant.py:42-124 of
    ModelTC/NART): one entry per tensor, ``{"max", "min"}`` or ``{"alpha", "zero_point"}``, plus the
    required ``"bit"`` and ``"type"`` ("symmetric" | "biased");
  * the weight rounding of ``param_to_tensor`` (quant.py:133-163);
  * the entries the calibrator derives without running a network: ``quant_weights``
    (python/nart/calibrator.py:59-100, min/max form) and ``quant_bias`` (calibrator.py:344-368);
  * the default (min/max, no KL) reduction of per-batch activation extremes in ``quant_activation``
    (calibrator.py:216-231, 281-290, 310-316).

Running the fp32 network over calibration data (the reference uses caffe for that) is the caller's
business: this module starts from the per-batch extremes.  Names follow the reference:
``<layer>_weight_0`` for a layer's weights, ``<layer>_weight_1`` for its bias.

The reference's behaviour is kept where it is surprising:
  * a biased ``max``/``min`` entry gets ``zero_point = round(-alpha * min)`` (quant.py:114) -- the
    product, not the quotient ``-min / alpha``;
  * an ``alpha`` entry always takes ``zero_point`` from the entry, symmetric or not (quant.py:102-106).
``zero_point_quotient=True`` in ``convert_quant_param`` selects ``round(-min / alpha)`` instead, the
value under which ``min`` maps to 0 and ``max`` to ``2^bit - 1``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

import numpy as np

DEFAULT, BIASED, SYMMETRIC = 0, 1, 2


@dataclass
class QuantParam:
    """quant.py:42-58."""
    alpha: float = 1.0
    zero_point: int = 0
    bits: int = 8
    qtype: int = DEFAULT

    def to_biased(self) -> "QuantParam":
        if self.qtype == BIASED or self.zero_point != 0:
            return self
        return QuantParam(self.alpha, 2 ** (self.bits - 1), self.bits, SYMMETRIC)


def convert_quant_param(quant_param, zero_point_quotient: bool = False):
    """dict name -> entry  ==>  dict name -> QuantParam (quant.py:70-124).  Raises RuntimeError with
    the reference's messages for a missing ``type`` / ``bit`` or an entry with neither form."""
    if quant_param is None:
        return None
    res = {}
    for k, v in quant_param.items():
        if "type" not in v:
            raise RuntimeError(f"`type` is required for quantization [{k}]")
        if v["type"] not in ["symmetric", "biased"]:
            raise RuntimeError(f"`type` can be `symmetric` or `biased`, but got {v['type']} for [{k}]")
        qtp = SYMMETRIC if v["type"] == "symmetric" else BIASED
        if "bit" not in v:
            raise RuntimeError(f"`bit` is required for quantization [{k}]")
        bit = v["bit"]
        if "alpha" in v:
            alpha = v["alpha"]
            zp = v["zero_point"]
        elif "max" in v and "min" in v:
            dmax = max(v["max"], 0.0)
            dmin = min(v["min"], 0.0)
            if qtp == SYMMETRIC:
                dmax = max(dmax, -dmin)
                alpha = dmax / (2 ** (bit - 1) - 1)
                zp = 0
            else:
                alpha = (dmax - dmin) / (2 ** bit - 1)
                zp = round(-dmin / alpha) if (zero_point_quotient and alpha > 0) else round(-alpha * dmin)
        else:
            raise RuntimeError(f"`max, min` or `alpha, zero_point` is required for quantization [{k}]")
        res[k] = QuantParam(alpha, zp, bit, qtp)
    return res


def load_max_min(path, zero_point_quotient: bool = False):
    """Reads a ``max_min.json`` and converts it."""
    with open(path, "rt") as f:
        return convert_quant_param(json.load(f), zero_point_quotient)


def quantize_weight(data, qparam: QuantParam) -> np.ndarray:
    """fp32 weights -> stored integers (quant.py:141-163): biased entries round ``w / alpha + zp`` and
    clip to ``0 .. 2^bits - 1`` (unsigned storage), the others round ``w / alpha`` and clip to
    ``+-(2^(bits-1) - 1)``; 8 / 16 / 32-bit storage by ``bits``."""
    w = np.array(data, dtype="float32")
    if qparam.qtype == BIASED:
        q = np.round(w / qparam.alpha + qparam.zero_point).clip(0, 2 ** qparam.bits - 1)
        prefix = "u"
    else:
        lim = 2 ** (qparam.bits - 1) - 1
        q = np.round(w / qparam.alpha).clip(-lim, lim)
        prefix = ""
    if qparam.bits <= 8:
        return q.astype(prefix + "int8")
    if qparam.bits <= 16:
        return q.astype(prefix + "int16")
    return q.astype(prefix + "int32")


def weight_entries(weights, bit_width: int = 8, symmetric: bool = False):
    """``{layer: fp32 weight array}`` -> ``{"<layer>_weight_0": entry}`` (calibrator.py:59-100 without
    the KL search): extremes widened to include 0; ``symmetric`` mirrors the larger magnitude."""
    ret = {}
    for name, w in weights.items():
        w = np.array(w, dtype=np.float64)   # the reference reads the blob as Python floats: double arithmetic from here on
        wmax = max(float(w.max()), 0.0)
        wmin = min(float(w.min()), 0.0)
        ret[f"{name}_weight_0"] = {"max": wmax, "min": wmin, "bit": bit_width, "type": "biased"}
    if symmetric:
        for k in ret:
            imax, imin = float(ret[k]["max"]), float(ret[k]["min"])
            ret[k]["max"] = max(abs(imax), abs(imin))
            ret[k]["min"] = -ret[k]["max"]
            ret[k]["type"] = "symmetric"
    return ret


def activation_entries(batch_extremes, bit_width: int = 8, symmetric: bool = False):
    """``{tensor: {"max": [per batch], "min": [per batch]}}`` -> entries, the calibrator's default
    reduction: the mean of the per-batch extremes (calibrator.py:310-316); ``symmetric`` clamps the
    means at 0 and mirrors the larger magnitude (calibrator.py:281-290)."""
    ret = {}
    for k, v in batch_extremes.items():
        if symmetric:
            amax = max(np.average(v["max"]), 0)
            amin = min(np.average(v["min"]), 0)
            m = max(abs(amax), abs(amin))
            ret[k] = {"max": m, "min": -m, "bit": bit_width, "type": "symmetric"}
        else:
            ret[k] = {"max": float(np.array(v["max"]).mean()), "min": float(np.array(v["min"]).mean()),
                      "bit": bit_width, "type": "biased"}
    return ret


def bias_entries(layers, param, bit_width: int = 8, symmetric: bool = False):
    """``layers``: iterable of (layer name, name of its input tensor) for the layers that have a bias;
    ``param``: the entries so far (weights and activations).  Returns ``{"<layer>_weight_1": entry}``
    with ``alpha = walpha * ialpha``, 32 bits, symmetric (calibrator.py:344-368; the step sizes there
    use ``2^bit - 1`` levels, or ``2^bit - 2`` when symmetric)."""
    ret = {}
    levels = 2 ** bit_width - (2 if symmetric else 1)
    for name, bottom in layers:
        w, i = param[f"{name}_weight_0"], param[bottom]
        walpha = (w["max"] - w["min"]) / levels
        ialpha = (i["max"] - i["min"]) / levels
        ret[f"{name}_weight_1"] = {"alpha": walpha * ialpha, "zero_point": 0, "type": "symmetric", "bit": 32}
    return ret
