"""The engine.bin writer and reader (nart_b200/engine.py) against the reference's own loader:
a written case must load with deserialize_parade (art/src/serialize_v2.c) and, run by the reference's
parade on its CPU `quant` module, give what the op-by-op walk of the same network gives."""
import os

import numpy as np
import pytest

from nart_b200 import engine, nets
from oracle.net_walk import run_net


def test_constants_match_the_reference_headers(ref):
    for name, value in engine.CONSTANTS.items():
        assert ref.constant(name) == value, name


def test_write_read_round_trip(tmp_path):
    spec = nets.resnet(18, seed=21, hw=32, width_div=8, spread=True, num_classes=10)
    path = os.path.join(tmp_path, "engine.bin")
    engine.write_engine(spec, path, batch=3, per_channel=True)
    m = engine.read_engine(path)
    assert [i["dims"] for i in m["inputs"]] == [[3, 3, 32, 32]]
    convs = [op for op in spec["ops"] if op["op"] in ("conv", "ip")]
    assert len(m["weights"]) == 2 * len(convs)
    n_relu_ops = sum(1 for op in spec["ops"] if op["op"] == "eltwise" and op["relu"])
    assert len(m["ops"]) == len(spec["ops"]) + n_relu_ops + 1        # + the final dequantize
    first = m["ops"][0]
    assert first["code"] == (6 << 32) | engine.OP_CONV_2D and first["ins"][0] == 0
    w0 = m["weights"][first["ins"][1]]["data"]
    np.testing.assert_array_equal(w0, convs[0]["w"])
    np.testing.assert_array_equal(first["settings"][engine.Q_WALPHA], convs[0]["walpha"].astype(np.float32))
    assert m["outputs"][0]["name"] == "logits"


def test_written_case_runs_on_the_reference_parade(ref, tmp_path):
    """Batch 1 (the reference conv cannot take more), one weight scale per layer, activations as
    relu ops of their own: the file's result equals the op-by-op walk through the same module."""
    spec = nets.resnet(18, seed=22, hw=96, width_div=4, spread=True, num_classes=12)
    path = os.path.join(tmp_path, "engine.bin")
    engine.write_engine(spec, path, batch=1, per_channel=False, conv_relu_flag=False)
    x = np.random.default_rng(3).integers(0, 256, (1, 3, 96, 96), dtype=np.uint8)
    ref.use_module()
    (got,) = ref.run_engine(path, [x], [np.float32])
    want, _, _ = run_net(spec, x, ref, per_channel=False)
    np.testing.assert_array_equal(got.view(np.uint32), want.reshape(-1).view(np.uint32))


def test_promark_runtime_config(tmp_path):
    """The reference driver's runtime JSON (tools/promark.cpp:136-187, 314-321) as this driver reads it: the
    workspace "b200" and no other, an optional device."""
    import json

    import pytest
    from nart_b200 import promark

    def write(obj, name="cfg.json"):
        path = os.path.join(tmp_path, name)
        with open(path, "w") as f:
            f.write(obj if isinstance(obj, str) else json.dumps(obj))
        return path

    assert promark.parse_runtime_config(write({"workspaces": {"b200": {}}, "input_workspace": "b200"})) is None
    assert promark.parse_runtime_config(write({"workspaces": {"b200": {"device": 3}}})) == 3
    for bad, text in (({"workspaces": {"quant": {}}, "input_workspace": "quant"}, "module [quant] not found"),
                      ({"workspaces": {"b200": {}, "default": {}}}, "module [default] not found"),
                      ({"workspaces": {"b200": {}}, "input_workspace": "cuda"}, "input_workspace"),
                      ({"workspaces": {}}, "workspaces"),
                      ({"workspaces": {"b200": {"device": -1}}}, "device"),
                      ("{not json", "not JSON")):
        with pytest.raises(ValueError, match=__import__("re").escape(text)):
            promark.parse_runtime_config(write(bad))


def test_art_runtime_context(tmp_path):
    """nart_b200.art mirrors the reference's nart.art (python/nart/art/__init__.py:31-55): a context from the
    runtime JSON; one backend, so only the workspace "b200" loads."""
    import json

    from nart_b200 import art
    path = os.path.join(tmp_path, "engine.bin.json")
    with open(path, "w") as f:
        json.dump({"workspaces": {"b200": {}}, "input_workspace": "b200"}, f)
    ctx = art.create_context_from_json(path)
    assert ctx.loaded_workspaces == ["b200"] and ctx.input_module == "b200"
    assert art.create_context_for_target("b200").loaded_workspaces == ["b200"]
    with pytest.raises(RuntimeError, match="module \\[quant\\] not found"):
        art.RuntimeContext(["quant"], "quant")
    with pytest.raises(RuntimeError, match="input workspace"):
        art.RuntimeContext(["b200"], "default")
    with pytest.raises(KeyError):
        art.create_context_for_target("cuda")
