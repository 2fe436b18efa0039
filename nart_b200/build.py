"""In-tree build of ``libnart_b200.so`` (CUDA kernels + C-ABI) and, where the art runtime headers
are available, of the art plugin ``libart_module_b200.so``.

    python -m nart_b200.build            # build what is stale
    python -m nart_b200.build --force

Everything is compiled for sm_100a only; nvcc cross-compiles without a GPU.  The CUDA runtime is
linked statically so the library does not depend on which libcudart the host process carries.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
MODSRC = os.path.join(PKG, "module")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libnart_b200.so")
MODULE_LIB = os.path.join(PKG, "libart_module_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(ROOT, "include", "nart_b200.h"))
    return hs


def _compile_one(src: str, force: bool) -> str:
    obj = os.path.join(OBJ, os.path.basename(src) + ".o")
    if force or _stale(obj, [src] + _headers()):
        cmd = [_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        with open(obj + ".log", "w") as f:
            f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s%s" % (src, res.stdout, res.stderr))
    return obj


def build_library(force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, force), srcs))
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-cudart", "static", "-ldl", "-lpthread", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB


def art_include_dirs() -> list[str] | None:
    """Include directories of the art runtime (the plugin's ABI headers).  They belong to the
    reference project and are used where they lie; ``NART_ART_ROOT`` names its ``art`` folder (default:
    a checkout called ``reference`` beside this repository).  None when there is no such folder: the
    plugin is then not rebuilt."""
    root = os.environ.get("NART_ART_ROOT") or os.path.join(os.path.dirname(ROOT), "reference", "art")
    inc = os.path.join(root, "include")
    if not os.path.exists(os.path.join(inc, "art", "module.h")):
        return None
    return [inc, os.path.join(root, "modules", "quant", "include")]


def build_module(force: bool = False) -> str | None:
    """The art plugin (C).  Built only where the art headers exist; returns None otherwise."""
    if not os.path.isdir(MODSRC):
        return None
    incs = art_include_dirs()
    if incs is None:
        return MODULE_LIB if os.path.exists(MODULE_LIB) else None
    srcs = sorted(os.path.join(MODSRC, f) for f in os.listdir(MODSRC) if f.endswith(".c"))
    hdrs = [os.path.join(MODSRC, f) for f in os.listdir(MODSRC) if f.endswith(".h")]
    if not srcs:
        return None
    if force or _stale(MODULE_LIB, srcs + hdrs + [LIB]):
        cmd = ["gcc", "-std=gnu99", "-O2", "-fPIC", "-shared", "-fvisibility=hidden",
               "-DNART_LOG_LEVEL=1", "-Wall", "-Wno-unused-function"]
        cmd += ["-I" + d for d in incs] + ["-I" + os.path.join(ROOT, "include")]
        cmd += srcs + ["-o", MODULE_LIB, "-L" + PKG, "-lnart_b200", "-Wl,-rpath,$ORIGIN", "-lm"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("module build failed:\n" + res.stdout + res.stderr)
    return MODULE_LIB


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel from the last compile logs."""
    out = []
    if os.path.isdir(OBJ):
        for f in sorted(os.listdir(OBJ)):
            if f.endswith(".log"):
                out.append(open(os.path.join(OBJ, f)).read())
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas", action="store_true", help="print the ptxas -v report")
    a = ap.parse_args(argv)
    print(build_library(a.force))
    print(build_module(a.force))
    if a.ptxas:
        print(ptxas_report())
    return 0


if __name__ == "__main__":
    sys.exit(main())
