"""In-tree build of the native libraries (no CMake, no JIT cache).

    python -m infiniops_b200.build            # build what is out of date
    python -m infiniops_b200.build --force    # rebuild everything

Produces, next to this file:

* ``lib/libinfiniops_b200.so`` -- the CUDA kernels and their C ABI (``include/infiniops_b200.h``),
  compiled by nvcc for sm_100a only;
* ``../infini/ops*.so``         -- the pybind11 module ``infini.ops`` (the C++ ``infini::ops``
  operator layer of ``include/`` -- ``#include <infini/ops.h>`` -- on top of the C ABI), compiled by g++.
"""

from __future__ import annotations

import argparse
import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys
import sysconfig

PKG = pathlib.Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
BUILD = ROOT / "build"
LIB = PKG / "lib" / "libinfiniops_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
    "-I", str(ROOT / "include"), "-I", str(CSRC),
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")


def _newer(target: pathlib.Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(pathlib.Path(s).stat().st_mtime <= t for s in sources)


def _run(cmd, log: pathlib.Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("build step failed: " + " ".join(map(str, cmd)))


def build_kernels(force: bool = False) -> pathlib.Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted((ROOT / "include").glob("*.h"))
    BUILD.mkdir(exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    objects = []
    for src in sources:
        obj = BUILD / (src.stem + ".o")
        objects.append(obj)
        if force or not _newer(obj, [src, *headers]):
            jobs.append(([nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)], BUILD / (src.stem + ".ptxas.log")))
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        for fut in [pool.submit(_run, cmd, log) for cmd, log in jobs]:
            fut.result()
    if force or jobs or not _newer(LIB, objects):
        _run([nvcc, "-shared", "-o", str(LIB), *map(str, objects), "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC"])
    return LIB


def build_bindings(force: bool = False) -> pathlib.Path | None:
    src_dir = PKG / "cpp"
    binding = src_dir / "bindings.cc"
    if not binding.exists():
        return None
    import pybind11

    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    out = ROOT / "infini" / f"ops{suffix}"
    out.parent.mkdir(exist_ok=True)
    deps = [*src_dir.rglob("*.h"), *src_dir.rglob("*.cc"), *(ROOT / "include").rglob("*.h"), LIB]
    if not force and _newer(out, deps):
        return out
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall",
           "-I", str(ROOT / "include"), "-I", str(src_dir), "-I", pybind11.get_include(),
           "-I", sysconfig.get_paths()["include"], "-I", "/usr/local/cuda/include",
           *[str(p) for p in sorted(src_dir.glob("*.cc"))],
           "-L", str(LIB.parent), "-linfiniops_b200", f"-Wl,-rpath,{LIB.parent}", "-Wl,-rpath,$ORIGIN/../infiniops_b200/lib",
           "-o", str(out)]
    _run(cmd)
    return out


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_bindings(force)


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    build_all(parser.parse_args().force)
    print("built", LIB)
