"""Builds libnatten_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python natten_b200/build.py [--force]

The library links the CUDA runtime statically and looks the driver entry point it needs
(cuTensorMapEncodeTiled) up at run time, so it loads on machines without a GPU driver too.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libnatten_b200.so")
# The same library with -DB200NA_TEST_HOOKS in the forward kernel: bounded waits of about a
# millisecond and a host switch that holds one producer arrive back. Used by one GPU test
# (tests/test_gpu_robustness.py) to make a wait expire; the package never loads it.
HOOK_LIB_PATH = os.path.join(LIB_DIR, "libnatten_b200_testhooks.so")
SOURCES = ["capi.cu", "tokperm.cu", "merge.cu", "na_simt.cu", "na_bwd_simt.cu", "fna_sm100.cu", "fna_bwd_sm100.cu", "na_fused.cu"]
HEADERS = ["common.cuh", "ptx.cuh", "fna_host.cuh", "fna_device.cuh", "fna_instrument.cuh", os.path.join("..", "..", "include", "natten_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; natten_b200 needs the CUDA toolkit to build")
    return cand


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    nvcc = _nvcc()
    procs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_dir, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    hook_src = os.path.join(CSRC, "fna_sm100.cu")
    hook_obj = os.path.join(obj_dir, "fna_sm100_testhooks.o")
    hook_proc = None
    if force or _stale(hook_obj, [hook_src] + hdrs):
        hook_proc = subprocess.Popen([nvcc] + NVCC_FLAGS + ["-DB200NA_TEST_HOOKS=1", "-c", hook_src,
                                                            "-o", hook_obj],
                                     stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(out.decode())
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    if hook_proc is not None:
        out, _ = hook_proc.communicate()
        if hook_proc.returncode != 0:
            sys.stderr.write(out.decode())
            raise RuntimeError("nvcc failed on fna_sm100.cu (test-hook build)")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"]
    if force or procs or _stale(LIB_PATH, objs):
        subprocess.run(link + ["-o", LIB_PATH] + objs + ["-cudart", "static"], check=True)
    hook_objs = [hook_obj if o.endswith(os.sep + "fna_sm100.o") else o for o in objs]
    if force or procs or hook_proc is not None or _stale(HOOK_LIB_PATH, hook_objs):
        subprocess.run(link + ["-o", HOOK_LIB_PATH] + hook_objs + ["-cudart", "static"], check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
