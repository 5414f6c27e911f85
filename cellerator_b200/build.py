"""Builds the native libraries of this package in-tree with nvcc for sm_100a.

    python -m cellerator_b200.build            # build what is out of date
    python -m cellerator_b200.build --force    # rebuild everything

Outputs (git-ignored, kept beside the sources so they travel with the tree):
    cellerator_b200/lib/libcellerator_b200.so       kernels + C ABI (include/cellerator_b200.h)
    cellerator_b200/lib/libcb200_synth.so           seeded workload generator used by bench/tests
    cellerator_b200/lib/libcb200_candidates.so      host/b200_candidates.cc, the C++ operation-core candidates over the
                                                    C ABI; compiles against the Cellerator headers, so it is built only
                                                    where CELLERATOR_REFERENCE names a Cellerator source tree
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(HERE, "build")

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "-I", os.path.join(ROOT, "include")] + os.environ.get("CB200_NVCC_EXTRA", "").split()

KERNEL_SOURCES = ["capi.cu", "host_contract.cu", "fleet.cu", "host_stage.cu", "qcsr_forward.cu", "qcsr_forward_tiled.cu", "qcsr_forward_mma.cu", "qcsr_forward_blocked.cu", "qcsr_forward_dense.cu", "qcsr_forward_codes.cu", "qcsr_transpose.cu", "qcsr_transpose_blocked.cu", "bell_lowering.cu", "public_route.cu", "gene_major.cu", "qbell_forward.cu", "qbell_tcgen05.cu",
                  "codec.cu"]
SYNTH_SOURCES = ["synth.cu"]

TARGETS = {
    "libcellerator_b200.so": [os.path.join(CSRC, s) for s in KERNEL_SOURCES],
    "libcb200_synth.so": [os.path.join(CSRC, s) for s in SYNTH_SOURCES],
}


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _headers() -> list[str]:
    out = [os.path.join(ROOT, "include", "cellerator_b200.h")]
    for d in (CSRC, HOST):
        if os.path.isdir(d):
            out += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".cuh", ".hh", ".h"))]
    return out


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def _compile(src: str, force: bool, extra: list[str]) -> str:
    obj = os.path.join(OBJ, os.path.basename(src) + ".o")
    if force or _newer(obj, [src] + _headers()):
        _run([NVCC, *ARCH, *NVCC_FLAGS, *extra, "-c", src, "-o", obj])
    return obj


def reference_root() -> str | None:
    """The Cellerator source tree the C++ host layer compiles against: the directory CELLERATOR_REFERENCE
    names, else a checkout called `reference` beside this repository."""
    for root in (os.environ.get("CELLERATOR_REFERENCE", ""), os.path.join(os.path.dirname(ROOT), "reference")):
        if root and os.path.isdir(os.path.join(root, "include", "Cellerator")):
            return os.path.abspath(root)
    return None


def build(force: bool = False, verbose: bool = False) -> dict[str, str]:
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    targets = {k: [s for s in v if os.path.exists(s)] for k, v in TARGETS.items()}
    jobs = {}
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        for lib, srcs in targets.items():
            for s in srcs:
                jobs[s] = pool.submit(_compile, s, force, [])
        objs = {s: f.result() for s, f in jobs.items()}
    out = {}
    for lib, srcs in targets.items():
        if not srcs:
            continue
        path = os.path.join(LIB, lib)
        deps = [objs[s] for s in srcs]
        if force or _newer(path, deps):
            _run([NVCC, *ARCH, "-shared", "-o", path, *deps, "-ldl"])  # dl: NCCL is bound at run time (fleet.cu)
        out[lib] = path
        if verbose:
            print("built", path)
    ref = reference_root()
    candidates = os.path.join(HOST, "b200_candidates.cc")
    if ref is not None and os.path.exists(candidates):
        # the product's own C++ host layer: operation_candidate records over the C ABI
        path = os.path.join(LIB, "libcb200_candidates.so")
        deps = [candidates] + _headers()
        if force or _newer(path, deps + [out["libcellerator_b200.so"]]):
            cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
            cuda_inc = os.path.join(os.path.dirname(os.path.dirname(NVCC)), "include")
            _run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-I", os.path.join(ref, "include"), "-I", cuda_inc,
                  "-I", os.path.join(ROOT, "include"), "-I", HOST, "-o", path, candidates, "-L", LIB, "-lcellerator_b200",
                  "-Wl,-rpath,$ORIGIN"])
        out["libcb200_candidates.so"] = path
        if verbose:
            print("built", path)
    return out


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
