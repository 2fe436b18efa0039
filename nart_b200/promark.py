"""Times a serialized case on the GPU case runner, with the options and the report of the
reference's benchmark driver (tools/promark.cpp:208-522 of ModelTC/NART):

    python -m nart_b200.promark -m engine.bin [-c runtime.json] [-n runs] [-b batch] [-r name:n,c,h,w]
                                [-i input.bin ...] [-s] [-d] [-y] [--gpus N]

  -m  the case file (format version 2)
  -n  timed runs (default 10), after one warm-up run
  -b  batch size (default: the batch recorded in the file)
  -r  reshape the named input to n,c,h,w before the case is prepared (the reference's
      parade_apply_reshape path); n sets the batch unless -b is given
  -i  raw input file in the input's dtype and NCHW shape, one per model input
  -s  save the outputs as nart-out-<name>.bin (raw, NCHW)
  -d  fresh random input data before every run
  -y  include the host<->device copies in the timed region (otherwise the device-resident run)
  --fuse  fold residual adds into the convs that feed them

  -c  the runtime JSON of the reference's driver (promark.cpp:136-187, 314-321):
      {"workspaces": {"b200": {}}, "input_workspace": "b200"}.  This driver has one backend, so the
      file must list the workspace "b200" and nothing else (any other name is the error the
      reference reports for a module it cannot find); "b200": {"device": 2} picks the GPU, as the
      NART_B200_DEVICE variable does for the plugin.  Without -c: the b200 workspace on the current
      device.
  --gpus N  one replica of the case per GPU (child processes, each with the full batch on its own
      device, no communication between them); the report adds the sum of their rates
"""
from __future__ import annotations

import argparse
import sys
import time

import numpy as np


def parse_runtime_config(path):
    """Reads the reference driver's runtime JSON and returns the device the "b200" workspace asks for
    (None: the current one).  Raises ValueError with the reference's kind of message for a workspace
    this driver cannot serve or a malformed file."""
    import json
    with open(path) as f:
        try:
            cfg = json.load(f)
        except json.JSONDecodeError as e:
            raise ValueError("runtime config %s is not JSON: %s" % (path, e))
    ws = cfg.get("workspaces")
    if not isinstance(ws, dict) or not ws:
        raise ValueError('runtime config needs a "workspaces" object')
    for name in ws:
        if name != "b200":
            raise ValueError("module [%s] not found: this driver serves the workspace \"b200\" only" % name)
    if cfg.get("input_workspace", "b200") != "b200":
        raise ValueError('"input_workspace" must be "b200"')
    settings = ws["b200"] if isinstance(ws["b200"], dict) else {}
    dev = settings.get("device")
    if dev is not None and (not isinstance(dev, int) or dev < 0):
        raise ValueError('"device" must be a non-negative integer')
    return dev


def run_replicas(a, argv):
    """--gpus N: N child processes of this driver, child i on device i, same arguments otherwise."""
    import re
    import subprocess
    args = []
    skip = False
    for tok in argv:                      # drop --gpus / --device of the parent
        if skip:
            skip = False
            continue
        if tok in ("--gpus", "--device"):
            skip = True
            continue
        if tok.startswith("--gpus=") or tok.startswith("--device="):
            continue
        args.append(tok)
    import os
    env = dict(os.environ)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))      # the children import this package too
    env["PYTHONPATH"] = root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    procs = [subprocess.Popen([sys.executable, "-m", "nart_b200.promark"] + args + ["--device", str(i)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for i in range(a.gpus)]
    total, failed = 0.0, 0
    for i, pr in enumerate(procs):
        out, _ = pr.communicate()
        m = re.search(r"([0-9.]+) images/s at batch", out)
        if pr.returncode != 0 or not m:
            failed += 1
            print("replica %d failed (exit %d):\n%s" % (i, pr.returncode, out[-2000:]), file=sys.stderr)
            continue
        rate = float(m.group(1))
        total += rate
        print("replica %d on device %d: %.1f images/s" % (i, i, rate))
    print("%d replicas: %.1f images/s" % (a.gpus - failed, total))
    return 1 if failed else 0


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m nart_b200.promark", add_help=True)
    ap.add_argument("-m", dest="model", required=True)
    ap.add_argument("-n", dest="runs", type=int, default=10)
    ap.add_argument("-b", dest="batch", type=int, default=-1)
    ap.add_argument("-r", dest="reshape", action="append", default=[])
    ap.add_argument("-i", dest="inputs", action="append", default=[])
    ap.add_argument("-s", dest="save", action="store_true")
    ap.add_argument("-d", dest="random", action="store_true")
    ap.add_argument("-y", dest="copies", action="store_true")
    ap.add_argument("--fuse", action="store_true")
    ap.add_argument("-c", dest="config", default=None)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--device", type=int, default=None, help=argparse.SUPPRESS)   # set for the children of --gpus
    a = ap.parse_args(argv)

    device = a.device
    if a.config:
        try:
            device_from_cfg = parse_runtime_config(a.config)
        except ValueError as e:
            print("Error: %s" % e, file=sys.stderr)
            return 1
        if device is None:
            device = device_from_cfg
    if a.gpus > 1:
        return run_replicas(a, sys.argv[1:] if argv is None else list(argv))

    import torch
    from . import engine
    if device is not None:
        torch.cuda.set_device(device)
    print("parse args ...")
    model = engine.read_engine(a.model)
    inp = model["inputs"][0]
    batch = a.batch if a.batch > 0 else int(inp["dims"][0])
    chw = tuple(int(d) for d in inp["dims"][1:])
    for spec in a.reshape:
        name, _, dims = spec.partition(":")
        if name != inp["name"]:
            print("warning: -r %s names no input of the model" % name, file=sys.stderr)
            continue
        shape = [int(d) for d in dims.split(",")]
        if len(shape) != 4:
            ap.error("-r takes name:n,c,h,w")
        chw = tuple(shape[1:])
        if a.batch <= 0:
            batch = shape[0]
    cs, outs = engine.engine_to_case(model, batch, fuse=a.fuse, input_chw=chw)
    in_dtype = np.float32 if inp["dtype"] == engine.DT_FLOAT32 else np.uint8
    in_shape = (batch,) + chw
    print("input tensors:")
    print("\t%s: %s" % (inp["name"], ", ".join(str(d) for d in in_shape)))
    print("output tensors:")
    for o, (is_f32, chw) in zip(model["outputs"], outs):
        print("\t%s: %s" % (o["name"], ", ".join(str(d) for d in (batch,) + tuple(chw))))

    rng = np.random.default_rng(0)

    def random_input():
        if in_dtype == np.uint8:
            return rng.integers(0, 256, in_shape, dtype=np.uint8)
        return rng.standard_normal(in_shape).astype(np.float32)

    x = random_input()
    if a.inputs:
        x = np.fromfile(a.inputs[0], dtype=in_dtype).reshape(in_shape)
    out_spec = [(np.float32 if is_f32 else np.uint8, chw) for is_f32, chw in outs]
    stream = torch.cuda.Stream()
    result = cs.run_host([x], out_spec, stream.cuda_stream)          # warm-up; also fills the device input
    print("\nFinish warm up")
    total = 0.0
    for i in range(a.runs):
        if a.random:
            print("use randomized data.")
            x = random_input()
            if not a.copies:
                cs.run_host([x], out_spec, stream.cuda_stream)
        t0 = time.perf_counter()
        if a.copies:
            result = cs.run_host([x], out_spec, stream.cuda_stream)
        else:
            cs.run_device(batch, stream.cuda_stream)
            stream.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        total += ms
        print("Process %d : cost %gms" % (i, ms))
    print("\nTest finised, average cost: %gms\n" % (total / max(1, a.runs)))
    print("%.1f images/s at batch %d" % (batch * a.runs / (total / 1e3), batch))
    if a.save:
        result = cs.run_host([x], out_spec, stream.cuda_stream)
        print("Info: Saving output tensors ...", file=sys.stderr)
        for o, arr in zip(model["outputs"], result):
            arr.tofile("nart-out-%s.bin" % o["name"].replace("/", "_"))
    cs.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
