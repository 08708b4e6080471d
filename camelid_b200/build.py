"""Builds ``libcamelid_b200.so`` (the C-ABI library) with nvcc for sm_100a, in-tree.

    python -m camelid_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libcamelid_b200.so"
STATIC_LIB = PKG / "libcamelid_b200.a"  # the same objects as an archive, for callers that link the engine in

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]
# Per-file extras: formats.cu must not contract a*b+c (bit-exact dequantisation and generator).
EXTRA = {"formats.cu": ["-fmad=false"]}


def nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; the library can only be built with the CUDA toolkit")
    return cand


def _stamp(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for f in [src, CSRC / "common.cuh", PKG.parent / "include" / "camelid_b200.h", *sorted(CSRC.glob("*.cuh"))]:
        h.update(f.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    host_cc = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else None
    jobs = []
    for src in sources:
        flags = ARCH + COMMON + EXTRA.get(src.name, []) + (["-Xptxas", "-v"] if verbose else [])
        if host_cc:
            flags = ["-ccbin", host_cc] + flags
        obj = OBJ / (src.stem + ".o")
        stamp_file = OBJ / (src.stem + ".stamp")
        stamp = _stamp(src, flags)
        if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
            continue
        jobs.append((src, obj, flags, stamp_file, stamp))

    def compile_one(job):
        src, obj, flags, stamp_file, stamp = job
        cmd = [nvcc(), *flags, "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
        stamp_file.write_text(stamp)
        return src.name

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name in ex.map(compile_one, jobs):
                if verbose:
                    print("compiled", name)
    if jobs or not LIB.exists():
        objs = [str(OBJ / (s.stem + ".o")) for s in sources]
        cmd = [nvcc(), *ARCH, "-shared", "-cudart", "static", "-o", str(LIB), *objs]
        if host_cc:
            cmd[1:1] = ["-ccbin", host_cc]
        cmd += ["-ldl", "-lpthread", "-lrt", "-Xlinker", "--no-undefined"]  # NCCL is bound with dlopen when a sharded engine first needs it
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if jobs or not STATIC_LIB.exists():
        # Static form: link with the CUDA runtime, e.g.
        #   g++ app.cpp libcamelid_b200.a -L$CUDA/lib64 -lcudart_static -ldl -lpthread -lrt
        STATIC_LIB.unlink(missing_ok=True)
        res = subprocess.run(["ar", "rcs", str(STATIC_LIB), *[str(OBJ / (s.stem + ".o")) for s in sources]], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"ar failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
