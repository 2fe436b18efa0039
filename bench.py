#!/usr/bin/env python
"""Benchmark of the quantized-convolution path on B200: int8 ResNet-50 (batch 256 per GPU,
3x224x224 uint8 input, synthetic quantization), images per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One process per GPU (the driver launches torchrun for N > 1); the batch is sharded by replica, no
collective is on the data path.  A step is one pass of the whole network over one batch.

  value     whole-job images/s with the input batch already resident in HBM (CUDA events, max
            over ranks).
  e2e       the same through the host-buffer entry point b200_case_run_host: pinned host input
            copied host->device and the logits copied device->host inside every step.
  roofline  the tensor-core convolution kernel (all of its launches in a step): algorithmic bytes
            and ops over the kernel's own time, measured with CUDA events around every launch.
  cpu_baseline / --impl reference
            the reference's CPU quant module (oracle/_ref, compiled unmodified from the reference
            sources) on the host cores, one process per core, each running whole images.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH = 256
# DRAM bytes per launch of the conv kernel, averaged over the 54 launches of one batch-256 step:
# dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this script (3.850 GB per step)
IGEMM_DRAM_BYTES_PER_LAUNCH = 3.850e9 / 54
WORKLOAD = "ResNet-50 v1.5 int8, batch 256 per GPU, 3x224x224 uint8 input, synthetic per-layer quantization"
SEED = 3


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16=float(d["bf16_tflops_sustained"]), src="measured")
    return dict(hbm_gbs=6650.0, bf16=1400.0, src="fallback")


# ---------------------------------------------------------------------------------------------
# clocks: sampled by nvidia-smi while the timed region runs
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        busy = sorted(sm)[len(sm) // 2:]   # the upper half: samples taken under load
        return dict(sm_mhz=float(np.median(busy)), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference quant module on the host cores
# ---------------------------------------------------------------------------------------------
_CPU_STATE = {}


def _cpu_init(kind):
    """Per worker process, outside any timed step: the network spec and the CPU module."""
    os.environ["OMP_NUM_THREADS"] = "1"
    import oracle
    from nart_b200 import nets
    _CPU_STATE["spec"] = nets.resnet(50, seed=SEED)
    _CPU_STATE["be"] = oracle.ref() if kind == "reference" else oracle.port()
    _CPU_STATE["kind"] = kind


def _cpu_worker(args):
    seed, n_images = args
    from oracle.net_walk import run_net
    if n_images == 0:          # warm-up call: the worker exists and is initialised
        return 0.0
    x = np.random.default_rng(seed).integers(0, 256, (n_images, 3, 224, 224), dtype=np.uint8)
    t = time.perf_counter()
    run_net(_CPU_STATE["spec"], x, _CPU_STATE["be"], per_channel=(_CPU_STATE["kind"] != "reference"))
    return time.perf_counter() - t


def cpu_images_per_sec(images_per_core: int = 1, procs: int | None = None):
    """Runs `procs` processes, each pushing `images_per_core` images through the CPU module; returns
    (images/s, kind, procs, seconds)."""
    import multiprocessing as mp
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    procs = procs or max(1, (os.cpu_count() or 1))
    ctx = mp.get_context("spawn")
    with ctx.Pool(procs, initializer=_cpu_init, initargs=(kind,)) as pool:
        pool.map(_cpu_worker, [(1, 0)] * procs)          # every worker is up and initialised
        t = time.perf_counter()
        pool.map(_cpu_worker, [(100 + i, images_per_core) for i in range(procs)], chunksize=1)
        dt = time.perf_counter() - t
    return procs * images_per_core / dt, kind, procs, dt


def run_reference_arm(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    procs = max(1, min(os.cpu_count() or 1, 64))
    import multiprocessing as mp
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    ctx = mp.get_context("spawn")
    times = []
    with ctx.Pool(procs, initializer=_cpu_init, initargs=(kind,)) as pool:
        pool.map(_cpu_worker, [(1, 0)] * procs)
        for step in range(a.warmup + a.steps):
            t = time.perf_counter()
            pool.map(_cpu_worker, [(100 + i, 1) for i in range(procs)], chunksize=1)
            dt = time.perf_counter() - t
            if step >= a.warmup:
                times.append(dt)
    total = sum(times)
    value = procs * len(times) / total
    sample = "%d image(s) per step on each of %d host processes (one per core), whole ResNet-50 per image" % (1, procs)
    line = dict(
        impl="reference", metric="resnet50_int8_images_per_sec", value=value, unit="images/s", n_gpus=a.gpus,
        steps=a.steps, warmup=a.warmup, ms_per_step=1e3 * total / len(times), higher_is_better=True, scaling="weak",
        vs_baseline=None, dtype="u8", data="synthetic",
        config=dict(workload=WORKLOAD, note="CPU arm: a step is %s; the reference reads one weight scale per layer" % sample),
        cpu_baseline=dict(value=value, unit="images/s", cores=procs, kind=kind, sample=sample),
        e2e=dict(value=value, unit="images/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
        gpu_launches=0)
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def pin_to_gpu_numa_node(local: int):
    """Best effort: run this rank's host threads on the cores of the NUMA node its GPU hangs off, so
    that the pinned batch buffers (first touch) and the copy engine's reads stay on that node.
    Returns a short description for the JSON line."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(local).pci_bus_id, torch.cuda.get_device_properties(local).pci_device_id
        dom = torch.cuda.get_device_properties(local).pci_domain_id
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0" % (dom, bus[0], bus[1])
        node = int(open(path + "/numa_node").read().strip())
        if node < 0:
            return "gpu reports no NUMA node"
        cpus = []
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.extend(range(int(lo), int(hi or lo) + 1))
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if not allowed:
            return "node %d has no core this process may use" % node
        os.sched_setaffinity(0, allowed)
        return "node %d, %d cores" % (node, len(allowed))
    except Exception as e:          # containers without /sys, restricted affinity: leave the process where it is
        return "not pinned (%s)" % type(e).__name__


def verify_ranks(cs, batch, stream, rank, world, device):
    """Every rank pushes the SAME seeded batch through its replica once, outside any timed region;
    the logits' bytes are hashed per rank, gathered, and must agree with rank 0's; rank 0 compares
    three images of them with the CPU restatement.  Returns (ranks_identical, images_checked)."""
    import hashlib
    import torch
    x = torch.from_numpy(np.random.default_rng(4242).integers(0, 256, (batch, 3, 224, 224), dtype=np.uint8)).pin_memory()
    y = torch.zeros((batch, 1000), dtype=torch.float32).pin_memory()
    cs.run_host_ptrs(batch, [x.data_ptr()], [y.data_ptr()], stream)
    digest = hashlib.sha256(y.numpy().tobytes()).digest()[:8]
    from nart_b200 import replicas
    identical = replicas.all_ranks_hold(digest, device)
    checked = 0
    if rank == 0:
        import oracle
        from oracle.net_walk import run_net
        from nart_b200 import nets
        pick = [0, batch // 2, batch - 1] if batch >= 3 else list(range(batch))
        want, _, _ = run_net(nets.resnet(50, seed=SEED), x.numpy()[pick], oracle.port())
        if not np.array_equal(y.numpy()[pick].view(np.uint32), want.reshape(len(pick), -1).view(np.uint32)):
            raise SystemExit("bench: the logits of the verification batch differ from the CPU restatement")
        checked = len(pick)
    if not identical:
        raise SystemExit("bench: ranks disagree on the logits of the same batch")
    return identical, checked


def fused_residual_convs(spec):
    """Names of the conv outputs whose residual add the case runner folds into the conv: the later
    produced input of a two-input eltwise op, when a conv makes it and nothing else reads it."""
    ops = spec["ops"]
    producer = {op["out"]: i for i, op in enumerate(ops)}
    readers = {}
    for op in ops:
        for n in op["ins"]:
            readers[n] = readers.get(n, 0) + 1
    readers[spec["output"]] = readers.get(spec["output"], 0) + 1
    out = set()
    for op in ops:
        if op["op"] != "eltwise" or len(op["ins"]) != 2:
            continue
        p = max(producer.get(op["ins"][0], -1), producer.get(op["ins"][1], -1))
        if p >= 0 and ops[p]["op"] == "conv" and readers.get(ops[p]["out"], 0) == 1:
            out.add(ops[p]["out"])
    return out


def conv_bytes_ops(spec, batch):
    """Algorithmic bytes and ops of each conv op: every tensor once (1 B/element), weights and
    bias once, 2*MACs; true dims."""
    T = spec["tensors"]
    out = []
    for op in spec["ops"]:
        if op["op"] not in ("conv", "ip"):
            out.append(None)
            continue
        ti, to = T[op["ins"][0]], T[op["out"]]
        if op["op"] == "conv":
            k, cg, r, s = op["w"].shape
        else:
            k, cg, r, s = op["w"].shape[0], ti["c"], ti["h"], ti["w"]
        ops = 2.0 * batch * to["h"] * to["w"] * k * cg * r * s
        byts = batch * (ti["c"] * ti["h"] * ti["w"] + to["c"] * to["h"] * to["w"]) + k * cg * r * s + 4 * k
        out.append((byts, ops))
    return out


def measure_int8_peak(lib, check, stream, local):
    """The dense int8 rate of the tensor pipe on this GPU: a short burst (best of five launches of about
    half a millisecond) and a sustained run of about a second, with the clocks seen during the latter."""
    import ctypes as C
    ms, ops = C.c_float(0), C.c_double(0)

    def run(mmas):
        check(lib.b200_measure_mma_i8_peak(int(mmas), C.byref(ms), C.byref(ops), stream))
        return ops.value / (ms.value * 1e-3) / 1e12, ms.value

    run(4096)
    burst = max(run(4096)[0] for _ in range(5))
    tops, t = run(1 << 17)
    per_ms = (1 << 17) / t
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.15)
    sustained, t_long = run(min(int(per_ms * 1000), 30000000))
    clocks = sampler.stop()
    return dict(burst_tops=burst, sustained_tops=sustained, sustained_ms=t_long, clocks_sustained=clocks,
                shape="tcgen05.mma kind::i8 M128 N256 K32, operands resident in shared memory, all SMs")


def conv_sweep_rows(peaks, int8_peak_tops, batch=256):
    """The 16 single-conv shapes (C = K in 64/128/256/512 on 56/28/14/7 pixel maps, 1x1 and 3x3, stride 1 and 2)
    at `batch`: device time per launch from a CUDA-graph replay of 20 launches, TOP/s on the true dims,
    algorithmic GB/s, and the fraction of the roof that binds the shape (the larger of ops / measured int8
    rate and bytes / measured copy bandwidth, over the measured time)."""
    from nart_b200 import conv_bench
    rows = []
    for c, k, hw in conv_bench.SWEEP_SHAPES:
        for ks in (1, 3):
            for stride in (1, 2):
                r = conv_bench.time_conv(c, k, hw, ks, stride, batch, iters=20, warmup=3, graph=True)
                ops = r["tops"] * 1e12 * r["ms"] * 1e-3
                byts = r["gbs"] * 1e9 * r["ms"] * 1e-3
                t_tensor = ops / (int8_peak_tops * 1e12) * 1e3
                t_hbm = byts / (peaks["hbm_gbs"] * 1e9) * 1e3
                rows.append(dict(c=c, k=k, hw=hw, ks=ks, stride=stride, batch=batch, ms=round(r["ms"], 5),
                                 tops=round(r["tops"], 1), gbs=round(r["gbs"], 1),
                                 bound="tensor" if t_tensor > t_hbm else "hbm",
                                 roof_frac=round(max(t_tensor, t_hbm) / r["ms"], 3)))
    return rows


def time_network(spec, batch, hw, steps=10):
    """One of the other benchmark networks: images/s of the CUDA-graph replay with the batch resident."""
    import torch
    from nart_b200 import nets
    from nart_b200._lib import check, lib
    cs, _ = nets.to_case(spec, batch)
    side = torch.cuda.Stream()
    x = torch.from_numpy(np.random.default_rng(7).integers(0, 256, (batch, 3, hw, hw), dtype=np.uint8)).pin_memory()
    check(lib.b200_memcpy_h2d(cs.io_device_ptr(False, 0), x.data_ptr(), x.numel(), side.cuda_stream))
    cs.use_graph(True)
    for _ in range(4):
        cs.run_device(batch, side.cuda_stream)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(side)
    for _ in range(steps):
        cs.run_device(batch, side.cuda_stream)
    e1.record(side)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    cs.close()
    return dict(network=spec["name"], batch=batch, ms_per_step=round(ms, 4), images_per_sec=round(batch / ms * 1e3, 1),
                conv_tops=round(nets.conv_ops_per_image(spec) * batch / ms / 1e9, 1))


def plugin_e2e(spec, batch, steps, x_ref, logits_ref):
    """The drop-in route: the network written as an engine.bin and run by the reference's own loader and
    parade (deserialize_parade / parade_prepare / parade_run, art/src/parade.c:169-197) with
    libart_module_b200.so as the only workspace, op by op on the default stream, the way the reference's
    promark drives a case (tools/promark.cpp:457-492).  A step marks the input's host view as written
    (so parade_run uploads it: the host->device copy is inside the step), runs the parade and takes the
    output's host view (device->host).  Needs the art core (compiled unmodified into oracle/_ref); the
    logits must equal the case runner's bit for bit."""
    import tempfile
    plugin = os.path.join(ROOT, "nart_b200", "libart_module_b200.so")
    try:
        import oracle
        if not (oracle.have_ref() and os.path.exists(plugin)):
            return dict(unavailable="the art core (oracle/_ref) or libart_module_b200.so is not present")
        from nart_b200 import engine
        R = oracle.ref()
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "engine.bin")
            engine.write_engine(spec, path, batch=batch, per_channel=True, conv_relu_flag=True)
            R.use_module(plugin, "b200_module_tp", whole_batch=True)
            try:
                h = R.open_engine(path)
                try:
                    R.engine_input(h, 0)[:] = x_ref.reshape(-1)
                    R.engine_run(h)
                    got = R.engine_output(h, 0).copy()
                    same = bool(np.array_equal(got.view(np.uint32), logits_ref.reshape(-1).view(np.uint32)))
                    for _ in range(2):
                        R.engine_input(h, 0)
                        R.engine_run(h)
                        R.engine_output(h, 0)
                    t = time.perf_counter()
                    for _ in range(steps):
                        R.engine_input(h, 0)          # host view requested: the next run uploads the batch again
                        R.engine_run(h)
                        R.engine_output(h, 0)         # downloads the logits, synchronizes
                    dt = time.perf_counter() - t
                finally:
                    R.close_engine(h)
            finally:
                R.use_module()
        return dict(value=batch * steps / dt, unit="images/s", ms_per_step=dt / steps * 1e3, steps=steps,
                    logits_equal_case_runner=same, clock="host (perf_counter) around input view / parade_run / output view",
                    host_runtime="the reference's art core (loader, parade and op loop), compiled unmodified; every op "
                                 "dispatches to libart_module_b200.so")
    except Exception as e:       # the main line must not depend on this leg
        return dict(unavailable="%s: %s" % (type(e).__name__, e))


def run_gpu_arm(a):
    import torch
    import torch.distributed as dist
    from nart_b200 import nets, replicas

    rank, world, local = replicas.env_rank_world()
    torch.cuda.set_device(local)
    numa = pin_to_gpu_numa_node(local)
    replicas.init("nccl", torch.device("cuda", local))

    batch = a.batch
    spec = nets.resnet(50, seed=SEED)
    cs, ids = nets.to_case(spec, batch)
    side = torch.cuda.Stream()   # a stream of its own: the default stream cannot be captured into a graph
    torch.cuda.set_stream(side)
    stream = side.cuda_stream
    n_launch = cs.launch_count()

    # host batch (pinned) and its resident copy in the case's input staging buffer
    rng = np.random.default_rng(1000 + rank)
    in_bytes = cs.io_bytes(False, 0) * batch
    out_bytes = cs.io_bytes(True, 0) * batch
    x_host = torch.from_numpy(rng.integers(0, 256, (batch, 3, 224, 224), dtype=np.uint8)).pin_memory()
    y_host = torch.empty((batch, 1000), dtype=torch.float32).pin_memory()
    from nart_b200._lib import check, lib
    check(lib.b200_memcpy_h2d(cs.io_device_ptr(False, 0), x_host.data_ptr(), in_bytes, stream))
    torch.cuda.synchronize()

    def barrier():
        replicas.barrier()
        torch.cuda.synchronize()

    # ---- every replica computes the same thing ---------------------------------------------------
    ranks_identical, oracle_images = verify_ranks(cs, batch, stream, rank, world, torch.device("cuda", local))
    check(lib.b200_memcpy_h2d(cs.io_device_ptr(False, 0), x_host.data_ptr(), in_bytes, stream))
    torch.cuda.synchronize()

    # ---- device-resident throughput -----------------------------------------------------------
    # The case replays its launches as one CUDA graph (eager first run, captured second run).
    cs.use_graph(not a.no_graph)
    for _ in range(max(a.warmup, 3)):
        cs.run_device(batch, stream)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        cs.run_device(batch, stream)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    ms_max = replicas.max_over_ranks(ms_total, "cuda")
    value = replicas.images_per_sec(batch, a.steps, ms_total, "cuda")

    # ---- the same K steps again with a CUDA-event pair around every launch: kernel times ---------
    # (op-by-op launches on the same stream and data; the graph is bypassed while profiling is on)
    cs.set_profiling(True)
    per_kind = {}
    igemm_ms = 0.0
    igemm_launches = 0
    igemm_bytes = igemm_ops = 0.0
    # conv launches come in the order of the spec's conv / ip ops; a conv that carries a residual add
    # in its epilogue also reads the residual tensor (1 B per output element)
    cb = [c for c in conv_bytes_ops(spec, batch) if c is not None]
    fused = fused_residual_convs(spec)
    if cs.launch_count() != len(spec["ops"]) + 3 - len(fused):   # input layout, row lowering, output; one less per fusion
        fused = set()
    conv_names = [op["out"] for op in spec["ops"] if op["op"] in ("conv", "ip")]
    for _ in range(a.steps):
        cs.run_device(batch, stream)
        prof = cs.profile()
        ci = 0
        for ms, kind in prof:
            per_kind[kind] = per_kind.get(kind, 0.0) + ms
            if kind in (1, 2):
                byts, ops = cb[ci]
                if conv_names[ci] in fused:
                    t = spec["tensors"][conv_names[ci]]
                    byts += batch * t["c"] * t["h"] * t["w"]
                ci += 1
                if kind == 1:
                    igemm_ms += ms
                    igemm_launches += 1
                    igemm_bytes += byts
                    igemm_ops += ops
    cs.set_profiling(False)

    # ---- end to end through the host-buffer entry points ------------------------------------------
    # Every step copies its 256 images host->device and its logits device->host inside the timed
    # region.  b200_case_submit_host queues a step and returns, so the copy of step i+1 overlaps the
    # kernels of step i; two pinned input/output buffer pairs alternate.
    x_hosts = [x_host, x_host.clone().pin_memory()]
    y_hosts = [y_host, torch.empty_like(y_host).pin_memory()]
    for i in range(3):
        cs.submit_host_ptrs(batch, [x_hosts[i % 2].data_ptr()], [y_hosts[i % 2].data_ptr()])
    cs.wait()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    e2.record()                                        # device timestamps on the (idle) bench stream ...
    for i in range(a.steps):
        cs.submit_host_ptrs(batch, [x_hosts[i % 2].data_ptr()], [y_hosts[i % 2].data_ptr()])
    cs.wait()                                          # ... around submit...wait, which drains the case's streams
    e3.record()
    e3.synchronize()
    e2e_wall_ms = (time.perf_counter() - w0) * 1e3
    e2e_ms = e2.elapsed_time(e3)
    barrier()
    e2e_value = replicas.images_per_sec(batch, a.steps, e2e_ms, "cuda")
    # the blocking single-call form, for comparison
    w0 = time.perf_counter()
    for _ in range(a.steps):
        cs.run_host_ptrs(batch, [x_host.data_ptr()], [y_host.data_ptr()], stream)
    wall_ms = (time.perf_counter() - w0) * 1e3
    logits_checksum = float(y_host.double().abs().sum().item())
    # ---- single-GPU extras, inside the clock-sampled region ------------------------------------------
    extras = {}
    if rank == 0 and world == 1 and not a.no_extras:
        peaks0 = measured_peaks()
        torch.cuda.synchronize()
        extras["int8_peak"] = measure_int8_peak(lib, check, stream, local)
        extras["conv_sweep_batch256"] = conv_sweep_rows(peaks0, extras["int8_peak"]["burst_tops"])
        extras["other_networks"] = [time_network(nets.resnet(18, seed=SEED), 64, 224),
                                    time_network(nets.mobilenet_v2(seed=SEED), 256, 224)]
        xv = torch.from_numpy(np.random.default_rng(4242).integers(0, 256, (batch, 3, 224, 224), dtype=np.uint8)).pin_memory()
        yv = torch.zeros((batch, 1000), dtype=torch.float32).pin_memory()
        cs.run_host_ptrs(batch, [xv.data_ptr()], [yv.data_ptr()], stream)
        extras["e2e_plugin"] = plugin_e2e(spec, batch, max(3, a.steps // 2), xv.numpy(), yv.numpy())
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        peaks = measured_peaks()
        kind_names = {0: "input_layout", 1: "conv_igemm_tcgen05", 2: "conv_cuda_core", 3: "eltwise_add", 4: "relu",
                      5: "pool", 6: "output_dequantize"}
        tot = sum(per_kind.values())
        breakdown = {kind_names[k]: round(v / a.steps, 4) for k, v in sorted(per_kind.items())}
        sec = igemm_ms / 1e3
        hbm_ach = igemm_bytes / sec / 1e9
        tops_ach = igemm_ops / sec / 1e12
        int8_peak = 2.0 * peaks["bf16"]
        int8_src = "2 x bf16_tflops_sustained of %s (no int8 entry in MEASURED_PEAKS.json)" % peaks["src"]
        if "int8_peak" in extras:
            int8_peak = extras["int8_peak"]["sustained_tops"]
            int8_src = ("measured in this run: %.0f TOP/s sustained over %.0f ms (%.0f burst), resident-operand kind::i8 loop"
                        % (int8_peak, extras["int8_peak"]["sustained_ms"], extras["int8_peak"]["burst_tops"]))
        cpu_val, cpu_kind, cpu_procs, cpu_dt = (None, None, None, None)
        cpu = None
        if world == 1 and not a.no_cpu:
            per_core = 4   # about 2.5 s of wall clock, 40 core-seconds on a 16-core host
            cpu_val, cpu_kind, cpu_procs, cpu_dt = cpu_images_per_sec(per_core)
            cpu = dict(value=cpu_val, unit="images/s", cores=cpu_procs, kind=cpu_kind,
                       sample="%d images in total, %d whole ResNet-50 images per host process, %d processes, %.1f s"
                              % (cpu_procs * per_core, per_core, cpu_procs, cpu_dt))
        line = dict(
            metric="resnet50_int8_images_per_sec", value=value, unit="images/s", n_gpus=world, steps=a.steps,
            warmup=max(a.warmup, 3), ms_per_step=ms_max / a.steps, higher_is_better=True, scaling="weak",
            vs_baseline=None, dtype="u8", data="synthetic",
            config=dict(workload=WORKLOAD, batch_per_gpu=batch, parallelism="replicas x%d, batch-sharded, no collective" % world,
                        l2="working set per step (5.6 GB of activations) is far larger than L2; no flush needed",
                        launch="one CUDA graph per step" if not a.no_graph else "op by op",
                        kernel_times="CUDA events around every launch, a second pass of the same K steps",
                        fused_residual_adds=len(fused),
                        conv_tops=igemm_ops / sec / 1e12, ms_per_step_by_kernel=breakdown,
                        conv_gop_per_image=nets.conv_ops_per_image(spec) / 1e9, logits_checksum=logits_checksum,
                        ranks_identical=ranks_identical, images_checked_against_cpu_restatement=oracle_images,
                        host_numa="rank 0: " + numa),
            roofline=dict(bound="hbm", achieved=hbm_ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=hbm_ach / peaks["hbm_gbs"],
                          traffic=IGEMM_DRAM_BYTES_PER_LAUNCH if batch == BATCH else None,
                          traffic_source="ncu dram__bytes_read.sum + dram__bytes_write.sum over the 54 launches of one "
                                         "step at batch 256, average per launch (profiles/resnet50_b256_igemm_dram_traffic.md)",
                          algorithmic_bytes_per_launch=igemm_bytes / max(1, igemm_launches),
                          kernel="conv_igemm_i8_kernel", launches_per_step=igemm_launches // a.steps,
                          peak_source=peaks["src"]),
            roofline_tensor=dict(bound="tensor", achieved=tops_ach, peak=int8_peak / 1.0, unit="TOP/s",
                                 frac=tops_ach / int8_peak,
                                 peak_source=int8_src),
            cpu_baseline=cpu,
            e2e=dict(value=e2e_value, unit="images/s", h2d_bytes_per_step=in_bytes, d2h_bytes_per_step=out_bytes,
                     api="b200_case_submit_host + b200_case_wait (copy of step i+1 overlaps the kernels of step i)",
                     ms_per_step=e2e_ms / a.steps, host_clock_ms_per_step=e2e_wall_ms / a.steps,
                     blocking_run_host_ms_per_step=wall_ms / a.steps),
            gpu_launches=n_launch * a.steps,
            clocks=clocks)
        line.update(extras)
        print(json.dumps(line))
    cs.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="launch op by op instead of replaying a CUDA graph")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the single-GPU extras (int8 peak, conv sweep, other networks, plugin route)")
    a = ap.parse_args()
    if a.impl == "reference":
        return run_reference_arm(a)
    return run_gpu_arm(a)


if __name__ == "__main__":
    sys.exit(main())
