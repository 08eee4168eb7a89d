"""Build libnano_omni_b200.so in-tree with nvcc for sm_100a.

Usage: ``python -m nano_omni_b200.build [--force] [--verbose] [--checked]``.
Each ``csrc/*.cu`` is compiled to an object (only when its sources are newer),
then linked into one shared library next to this file.

``--checked`` builds ``libnano_omni_b200_checked.so`` beside it with ``-DNOB200_CHECKED``: the kernels test every
hand-computed store index against its tensor's extent, skip a store that fails and report it in bit 5 of the
status word (nothing traps).  ``NOB200_LIBRARY=<path>`` makes the Python front end load that library, e.g. to run
the parity tests against it.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libnano_omni_b200.so")

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-std=c++17",
    "-O3",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build the kernels")
    return path


def _sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    found = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    found += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    return found


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    stamp = os.path.getmtime(target)
    return any(os.path.getmtime(d) > stamp for d in deps)


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    obj_dir = OBJ_DIR + ("_checked" if checked else "")
    lib = LIB.replace(".so", "_checked.so") if checked else LIB
    flags = NVCC_FLAGS + (["-DNOB200_CHECKED"] if checked else [])
    os.makedirs(obj_dir, exist_ok=True)
    headers = _headers()
    jobs = []
    for src in _sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc(), *flags, "-I", INCLUDE, "-c", src, "-o", obj]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        return src, proc

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, proc in pool.map(compile_one, jobs):
            if verbose or proc.returncode != 0:
                sys.stderr.write(f"== {os.path.basename(src)}\n{proc.stdout}{proc.stderr}\n")
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
    objects = [os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o") for s in _sources()]
    if force or jobs or _stale(lib, objects):
        cmd = [nvcc(), "-shared", "-o", lib, *objects, "-gencode", "arch=compute_100a,code=sm_100a"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError(f"linking {os.path.basename(lib)} failed")
    return lib


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--checked", action="store_true", help="the library with index checks on every store")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose, checked=args.checked))
