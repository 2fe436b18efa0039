"""GPU: serialized cases (engine.bin).  (1) A file read by nart_b200.engine runs on the GPU case
runner.  (2) The same file, untouched, loaded by the reference's own deserializer and parade with
the b200 plugin as the only workspace -- the drop-in: what `promark -m engine.bin` does when the
runtime JSON lists "b200" (tools/promark.cpp:58-72,122-187).  Both give the CPU restatement's bits."""
import os

import numpy as np
import pytest

from gpu_util import assert_same
from oracle.net_walk import run_net

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN = os.path.join(ROOT, "nart_b200", "libart_module_b200.so")


@pytest.mark.parametrize("depth,relu_flag", [(18, True), (50, True), (18, False)])
def test_engine_file_on_the_case_runner(port, tmp_path, depth, relu_flag):
    from nart_b200 import engine, nets
    spec = nets.resnet(depth, seed=30 + depth, hw=64, width_div=2, spread=True, num_classes=40)
    path = os.path.join(tmp_path, "engine.bin")
    engine.write_engine(spec, path, batch=3, per_channel=True, conv_relu_flag=relu_flag)
    x = np.random.default_rng(depth).integers(0, 256, (3, 3, 64, 64), dtype=np.uint8)
    want, _, _ = run_net(spec, x, port)
    cs, outs = engine.engine_to_case(engine.read_engine(path), 4)
    assert outs == [(True, (40, 1, 1))]
    (got,) = cs.run_host([x], [(np.float32, (40, 1, 1))])
    cs.close()
    assert_same(got.reshape(want.shape).view(np.uint32), want.view(np.uint32), "engine.bin on the case runner")


def test_engine_file_through_the_reference_parade_on_the_plugin(ref, port, tmp_path):
    if not os.path.exists(PLUGIN):
        pytest.skip("libart_module_b200.so was not built (the art headers were not available)")
    from nart_b200 import engine, nets
    spec = nets.resnet(50, seed=41, hw=64, width_div=2, spread=True, num_classes=24)
    path = os.path.join(tmp_path, "engine.bin")
    engine.write_engine(spec, path, batch=2, per_channel=True, conv_relu_flag=True)
    x = np.random.default_rng(8).integers(0, 256, (2, 3, 64, 64), dtype=np.uint8)
    want, _, _ = run_net(spec, x, port)
    ref.use_module(PLUGIN, "b200_module_tp", whole_batch=True)
    try:
        (got,) = ref.run_engine(path, [x], [np.float32])
    finally:
        ref.use_module()
    assert_same(got.reshape(want.shape).view(np.uint32), want.view(np.uint32), "engine.bin through parade + plugin")


def test_promark_cli(port, tmp_path, monkeypatch, capsys):
    """python -m nart_b200.promark: the reference benchmark driver's options on the case runner;
    -i / -s read and write raw NCHW files."""
    from nart_b200 import engine, nets, promark
    spec = nets.resnet(18, seed=51, hw=64, width_div=4, spread=True, num_classes=10)
    path = os.path.join(tmp_path, "engine.bin")
    engine.write_engine(spec, path, batch=2)
    x = np.random.default_rng(4).integers(0, 256, (2, 3, 64, 64), dtype=np.uint8)
    x.tofile(os.path.join(tmp_path, "in.bin"))
    monkeypatch.chdir(tmp_path)
    assert promark.main(["-m", path, "-n", "2", "-y", "-s", "-i", "in.bin"]) == 0
    text = capsys.readouterr().out
    assert "input tensors:" in text and "Process 1 : cost" in text and "average cost" in text
    got = np.fromfile(os.path.join(tmp_path, "nart-out-logits.bin"), dtype=np.float32)
    want, _, _ = run_net(spec, x, port)
    assert_same(got.view(np.uint32), want.reshape(-1).view(np.uint32), "promark -s")
    assert promark.main(["-m", path, "-n", "2", "-b", "4", "-d"]) == 0      # device-resident timing, other batch

    # -c: the reference driver's runtime JSON; one backend here, so "b200" is the only workspace it may list
    import json
    with open(os.path.join(tmp_path, "b200.json"), "w") as f:
        json.dump({"workspaces": {"b200": {"device": 0}}, "input_workspace": "b200"}, f)
    with open(os.path.join(tmp_path, "quant.json"), "w") as f:
        json.dump({"workspaces": {"quant": {}}, "input_workspace": "quant"}, f)
    capsys.readouterr()
    assert promark.main(["-m", path, "-c", "b200.json", "-n", "1"]) == 0
    assert promark.main(["-m", path, "-c", "quant.json", "-n", "1"]) == 1
    assert "module [quant] not found" in capsys.readouterr().err
    # --gpus: replicas as child processes (one here: the test asks for no more GPUs than it is sure to have)
    import torch
    rc = promark.main(["-m", path, "-n", "2", "-b", "2", "--gpus", "2"])
    cap = capsys.readouterr()
    if torch.cuda.device_count() >= 2:
        assert rc == 0 and "2 replicas:" in cap.out
    else:       # the second replica finds no device: reported, the first one still counted
        assert rc == 1 and "replica 1 failed" in cap.err and "replica 0 on device 0:" in cap.out and "1 replicas:" in cap.out


def test_promark_reshape(port, tmp_path, monkeypatch, capsys):
    """-r name:n,c,h,w: the recorded input shape is replaced before the case is prepared and every later
    shape follows (what parade_apply_reshape does in the reference's driver)."""
    from nart_b200 import engine, nets, promark

    def build(h, w):
        b = nets.SpecBuilder(77, (3, h, w), True)
        t = b.conv("input", 32, 3, 2, 1)
        t = b.conv(t, 48, 3, 1, 1)
        t = b.pool(t, nets.POOL_MAX, 2, 2, 0)
        return b.finish("reshape-net", t)

    small, large = build(16, 16), build(24, 20)
    path = os.path.join(tmp_path, "engine.bin")
    engine.write_engine(small, path, batch=2)
    name = engine.read_engine(path)["inputs"][0]["name"]
    x = np.random.default_rng(9).integers(0, 256, (3, 3, 24, 20), dtype=np.uint8)
    x.tofile(os.path.join(tmp_path, "in.bin"))
    monkeypatch.chdir(tmp_path)
    assert promark.main(["-m", path, "-n", "1", "-r", "%s:3,3,24,20" % name, "-s", "-i", "in.bin"]) == 0
    assert "%s: 3, 3, 24, 20" % name in capsys.readouterr().out
    want, _, _ = run_net(large, x, port)          # the file's output is the dequantized last tensor
    out_name = engine.read_engine(path)["outputs"][0]["name"].replace("/", "_")
    got = np.fromfile(os.path.join(tmp_path, "nart-out-%s.bin" % out_name), dtype=np.float32)
    assert got.size == want.size == 3 * 48 * 6 * 5
    assert_same(got.view(np.uint32), want.reshape(-1).view(np.uint32), "promark -r")


def test_art_python_interface(port, tmp_path):
    """nart_b200.art: the reference's Python runtime interface (python/nart/art/__init__.py, the pybind Parade of
    python/src/art/module.cpp:285-509) on the case runner -- load, shapes and dtypes, run with dicts of arrays,
    its argument checks, reshape."""
    import json

    from nart_b200 import art, engine, nets
    spec = nets.resnet(18, seed=23, hw=64, width_div=4, spread=True, num_classes=10)
    path = os.path.join(tmp_path, "engine.bin")
    engine.write_engine(spec, path, batch=2)
    with open(path + ".json", "w") as f:
        json.dump({"workspaces": {"b200": {}}, "input_workspace": "b200"}, f)
    ctx = art.create_context_from_json(path + ".json")
    parade = art.load_parade(path, ctx)
    (iname,), (oname,) = parade.get_input_names(), parade.get_output_names()
    assert parade.input_shapes() == {iname: [2, 3, 64, 64]} and parade.output_shapes() == {oname: [2, 10, 1, 1]}
    assert parade.get_tensor_dtype(iname) == "uint8" and parade.get_tensor_dtype(oname) == "float32"
    assert parade.get_tensor_shape(oname) == [2, 10, 1, 1]
    inputs, outputs = art.get_empty_io(parade)
    x = np.random.default_rng(5).integers(0, 256, (2, 3, 64, 64), dtype=np.uint8)
    inputs[iname][:] = x
    assert parade.run(inputs, outputs) is True
    want, _, _ = run_net(spec, x, port)
    assert_same(outputs[oname].reshape(want.shape).view(np.uint32), want.view(np.uint32), "art.Parade.run")
    parade.forward()                                       # the device-resident run of the same data
    # the reference's argument checks
    with pytest.raises(ValueError, match="input shape not match"):
        parade.run({iname: x[:1]}, outputs)
    with pytest.raises(ValueError, match="input dtype not match"):
        parade.run({iname: x.astype(np.float32)}, outputs)
    with pytest.raises(ValueError, match="output dtype not match"):
        parade.run(inputs, {oname: outputs[oname].astype(np.float64)})
    with pytest.raises(ValueError, match="some output not given"):
        parade.run(inputs, {})
    parade.close()

    # reshape: another batch and image size; every later shape follows
    def build(h, w):
        b = nets.SpecBuilder(77, (3, h, w), True)
        t = b.conv("input", 32, 3, 2, 1)
        t = b.conv(t, 48, 3, 1, 1)
        t = b.pool(t, nets.POOL_MAX, 2, 2, 0)
        return b.finish("reshape-net", t)

    small, large = build(16, 16), build(24, 20)
    engine.write_engine(small, path, batch=2)
    parade = art.load_parade(path, ctx)
    (iname,), (oname,) = parade.get_input_names(), parade.get_output_names()
    assert parade.reshape({"no such input": [1, 3, 8, 8]}) is False
    assert parade.reshape({iname: [3, 3, 24, 20]}) is True
    assert parade.input_shapes() == {iname: [3, 3, 24, 20]} and parade.output_shapes() == {oname: [3, 48, 6, 5]}
    inputs, outputs = art.get_empty_io(parade)
    x = np.random.default_rng(6).integers(0, 256, (3, 3, 24, 20), dtype=np.uint8)
    inputs[iname][:] = x
    parade.run(inputs, outputs)
    want, _, _ = run_net(large, x, port)
    assert_same(outputs[oname].reshape(want.shape).view(np.uint32), want.view(np.uint32), "art.Parade.run after reshape")
    parade.close()
