"""GPU parity of whole networks through the C-ABI case runner: every intermediate tensor and the
final logits against the CPU restatement, bit for bit."""
import numpy as np
import pytest

from gpu_util import assert_same
from oracle.net_walk import run_net

pytestmark = pytest.mark.gpu


def _check(spec, x, port, algo=0, max_batch=None):
    from nart_b200 import nets
    names = [op["out"] for op in spec["ops"]]
    want_logits, want_q, kept = run_net(spec, x, port, keep=set(names))
    cs, ids = nets.to_case(spec, max_batch or x.shape[0], algo=algo, extra_outputs=names)
    T = spec["tensors"]
    shapes = [(np.float32, (T[spec["output"]]["c"], 1, 1))] + [
        (np.uint8, (T[n]["c"], T[n]["h"], T[n]["w"])) for n in names]
    outs = cs.run_host([x], shapes)
    for n, got in zip(names, outs[1:]):
        assert_same(got, kept[n], "%s tensor %s" % (spec["name"], n))
    assert_same(outs[0].reshape(want_logits.shape).view(np.uint32), want_logits.view(np.uint32), "logits")
    assert cs.launch_count() >= len(spec["ops"]) + 1 + 1 + len(names)
    cs.close()


@pytest.mark.parametrize("spread", [True, False])
def test_resnet18_small(port, spread):
    from nart_b200 import nets
    spec = nets.resnet(18, seed=5, hw=64, width_div=2, spread=spread, num_classes=40)
    x = np.random.default_rng(1).integers(0, 256, (3, 3, 64, 64), dtype=np.uint8)
    _check(spec, x, port)


def test_resnet50_small(port):
    from nart_b200 import nets
    spec = nets.resnet(50, seed=6, hw=64, width_div=2, spread=True, num_classes=1000)
    x = np.random.default_rng(2).integers(0, 256, (2, 3, 64, 64), dtype=np.uint8)
    _check(spec, x, port, max_batch=4)


def test_resnet18_direct_only(port):
    from nart_b200 import nets, ops
    spec = nets.resnet(18, seed=7, hw=32, width_div=4, spread=True, num_classes=16)
    x = np.random.default_rng(3).integers(0, 256, (2, 3, 32, 32), dtype=np.uint8)
    _check(spec, x, port, algo=ops.ALGO_DIRECT)


def test_mobilenet_v2_small(port):
    from nart_b200 import nets
    spec = nets.mobilenet_v2(seed=8, hw=64, spread=True, num_classes=24)
    x = np.random.default_rng(4).integers(0, 256, (2, 3, 64, 64), dtype=np.uint8)
    _check(spec, x, port)


def test_resnet50_full_size_one_image(port):
    """The 224x224 network of the benchmark, batch 2, final logits only."""
    from nart_b200 import nets
    spec = nets.resnet(50, seed=2, spread=True)
    x = np.random.default_rng(5).integers(0, 256, (2, 3, 224, 224), dtype=np.uint8)
    want_logits, want_q, _ = run_net(spec, x, port)
    cs, ids = nets.to_case(spec, 2)
    (got,) = cs.run_host([x], [(np.float32, (1000, 1, 1))])
    assert_same(got.reshape(want_logits.shape).view(np.uint32), want_logits.view(np.uint32), "resnet50 logits")
    assert len(np.unique(want_q)) > 16
    cs.close()


def test_graph_replay_matches_eager(port):
    """b200_case_use_graph: eager first run, captured second run, replays -- all identical."""
    import torch
    from nart_b200 import nets
    from nart_b200._lib import check, lib
    spec = nets.resnet(50, seed=9, hw=64, width_div=2, spread=True, num_classes=64)
    rng = np.random.default_rng(6)
    cs, ids = nets.to_case(spec, 4)
    cs.use_graph(True)
    side = torch.cuda.Stream()          # the default stream cannot be captured
    stream = side.cuda_stream
    for it in range(5):
        x = rng.integers(0, 256, (4, 3, 64, 64), dtype=np.uint8)
        ref_logits, _, _ = run_net(spec, x, port)
        (got,) = cs.run_host([x], [(np.float32, (64, 1, 1))], stream)
        assert_same(got.reshape(ref_logits.shape).view(np.uint32), ref_logits.view(np.uint32), "graph run %d" % it)
    # a different batch size gets its own graph
    x = rng.integers(0, 256, (2, 3, 64, 64), dtype=np.uint8)
    ref_logits, _, _ = run_net(spec, x, port)
    for it in range(3):
        (got,) = cs.run_host([x], [(np.float32, (64, 1, 1))], stream)
        assert_same(got.reshape(ref_logits.shape).view(np.uint32), ref_logits.view(np.uint32), "graph batch 2 run %d" % it)
    cs.close()


def test_graphs_of_several_batch_sizes_keep_their_scratch(port):
    """Graphs captured at a small batch are replayed after a larger batch has run: the convs' scratch
    tensors (the row-lowered stem) are sized once at prepare (b200_conv2d_reserve), so the addresses
    a captured graph holds stay valid."""
    import torch
    from nart_b200 import nets
    spec = nets.resnet(18, seed=14, hw=64, width_div=2, spread=True, num_classes=32)
    rng = np.random.default_rng(10)
    cs, ids = nets.to_case(spec, 6)
    cs.use_graph(True)
    side = torch.cuda.Stream()
    xs = {b: rng.integers(0, 256, (b, 3, 64, 64), dtype=np.uint8) for b in (2, 6, 3)}
    want = {b: run_net(spec, x, port)[0] for b, x in xs.items()}
    for b in (2, 2, 2, 6, 6, 6, 2, 3, 3, 3, 6, 2):     # eager, capture, replay per size; then replays interleaved
        (got,) = cs.run_host([xs[b]], [(np.float32, (32, 1, 1))], side.cuda_stream)
        assert_same(got.reshape(want[b].shape).view(np.uint32), want[b].view(np.uint32), "batch %d" % b)
    cs.close()


def test_pipelined_submit_matches_reference(port):
    """b200_case_submit_host / b200_case_wait: three batches in flight back to back."""
    import torch
    from nart_b200 import nets
    spec = nets.resnet(18, seed=12, hw=64, width_div=2, spread=True, num_classes=32)
    rng = np.random.default_rng(8)
    cs, ids = nets.to_case(spec, 4)
    cs.use_graph(True)
    for rnd in range(2):
        xs = [torch.from_numpy(rng.integers(0, 256, (4, 3, 64, 64), dtype=np.uint8)).pin_memory() for _ in range(3)]
        ys = [torch.zeros((4, 32), dtype=torch.float32).pin_memory() for _ in range(3)]
        for x, y in zip(xs, ys):
            cs.submit_host_ptrs(4, [x.data_ptr()], [y.data_ptr()])
        cs.wait()
        for i, (x, y) in enumerate(zip(xs, ys)):
            want, _, _ = run_net(spec, x.numpy(), port)
            assert_same(y.numpy().reshape(want.shape).view(np.uint32), want.view(np.uint32), "round %d batch %d" % (rnd, i))
    cs.close()


def test_resnet50_bench_size_paths_agree(port):
    """The benchmark's own size (ResNet-50, batch 256): the eager run, the CUDA-graph replay, the
    pipelined submit and the case with fused residual adds give the same 256 x 1000 logits bit for
    bit, and images taken from both ends and the middle of the batch equal the CPU restatement."""
    import torch
    from nart_b200 import nets
    spec = nets.resnet(50, seed=3)
    batch = 256
    x = torch.from_numpy(np.random.default_rng(11).integers(0, 256, (batch, 3, 224, 224), dtype=np.uint8)).pin_memory()
    side = torch.cuda.Stream()
    results = {}
    for name, fuse in (("plain", False), ("fused", True)):
        cs, _ = nets.to_case(spec, batch, fuse=fuse)
        y = torch.zeros((batch, 1000), dtype=torch.float32).pin_memory()
        cs.run_host_ptrs(batch, [x.data_ptr()], [y.data_ptr()], side.cuda_stream)
        results[name + " eager"] = y.numpy().copy()
        if not fuse:
            cs.use_graph(True)
            for _ in range(3):      # eager, capture, replay
                y.zero_()
                cs.run_host_ptrs(batch, [x.data_ptr()], [y.data_ptr()], side.cuda_stream)
            results["graph replay"] = y.numpy().copy()
            y.zero_()
            cs.submit_host_ptrs(batch, [x.data_ptr()], [y.data_ptr()])
            cs.wait()
            results["submit"] = y.numpy().copy()
        cs.close()
    base = results["plain eager"]
    for name, got in results.items():
        assert_same(got.view(np.uint32), base.view(np.uint32), name + " vs plain eager")
    pick = [0, 131, 255]
    want, _, _ = run_net(spec, x.numpy()[pick], port)
    assert_same(base[pick].view(np.uint32), want.reshape(len(pick), -1).view(np.uint32), "batch-256 images vs restatement")
    assert len(np.unique(base)) > 16          # not a collapsed network: the uint8 logits take many values


def _bench_size_check(spec, batch, port, seed, n_classes=1000):
    """A network at the batch and image size its throughput is quoted on: the eager run and the CUDA-graph
    replay give the same logits bit for bit, and images from both ends and the middle of the batch equal
    the CPU restatement."""
    import torch
    from nart_b200 import nets
    c, h, w = spec["in_chw"]
    x = torch.from_numpy(np.random.default_rng(seed).integers(0, 256, (batch, c, h, w), dtype=np.uint8)).pin_memory()
    side = torch.cuda.Stream()
    cs, _ = nets.to_case(spec, batch)
    y = torch.zeros((batch, n_classes), dtype=torch.float32).pin_memory()
    cs.run_host_ptrs(batch, [x.data_ptr()], [y.data_ptr()], side.cuda_stream)
    eager = y.numpy().copy()
    cs.use_graph(True)
    for _ in range(3):      # eager, capture, replay
        y.zero_()
        cs.run_host_ptrs(batch, [x.data_ptr()], [y.data_ptr()], side.cuda_stream)
    assert_same(y.numpy().view(np.uint32), eager.view(np.uint32), "graph replay vs eager")
    cs.close()
    pick = [0, batch // 2 + 3, batch - 1]
    want, want_q, _ = run_net(spec, x.numpy()[pick], port)
    assert_same(eager[pick].view(np.uint32), want.reshape(len(pick), -1).view(np.uint32), "%s batch %d vs restatement" % (spec["name"], batch))
    assert len(np.unique(want_q)) > 16


def test_resnet18_bench_size(port):
    """ResNet-18, batch 64, 3 x 224 x 224 (the synthetic quantization of the ResNet-50 benchmark)."""
    from nart_b200 import nets
    _bench_size_check(nets.resnet(18, seed=4), 64, port, seed=21)


def test_mobilenet_v2_bench_size(port):
    """MobileNetV2-1.0, batch 256, 3 x 224 x 224: 1x1 convs on the tensor-core path, depthwise 3x3 on dp4a."""
    from nart_b200 import nets
    _bench_size_check(nets.mobilenet_v2(seed=5), 256, port, seed=22)
