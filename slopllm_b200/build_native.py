"""Builds the native libraries in-tree with nvcc / g++ (no torch headers: plain C ABI).

* `_lib/libslopllm_kernels.so`  - every sm_100a CUDA kernel (`csrc/*.cu`)
* `_lib/libslopllm_runtime.so`  - host-side C++ runtime (`csrc/runtime/*.cpp`): heap and page
  allocators, prefix matching, checkpoint mappings with multi-threaded strided window copies

Run `python -m slopllm_b200.build_native` (or `__graft_entry__.build()`).
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIB = os.path.join(ROOT, "_lib")
KERNELS_SO = os.path.join(LIB, "libslopllm_kernels.so")
RUNTIME_SO = os.path.join(LIB, "libslopllm_runtime.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
              "-Xptxas", "-v"]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, log_path=None):
    p = subprocess.run(cmd, capture_output=True, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + p.stdout + p.stderr)
    if p.returncode != 0:
        sys.stderr.write(p.stdout + p.stderr)
        raise RuntimeError("build failed: " + " ".join(cmd[:4]) + " ...")
    return p.stdout + p.stderr


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    cus = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    objs = []
    jobs = []
    for cu in cus:
        obj = os.path.join(LIB, os.path.basename(cu)[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [cu] + hdrs):
            jobs.append((cu, obj))

    def compile_one(job):
        cu, obj = job
        out = _run(["nvcc", *NVCC_FLAGS, "-I", CSRC, "-c", cu, "-o", obj], obj + ".log")
        if verbose:
            print(out)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    if jobs or force or _newer(KERNELS_SO, objs):
        _run(["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", KERNELS_SO, *objs])
    return KERNELS_SO


def build_runtime(force: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    cpps = sorted(glob.glob(os.path.join(CSRC, "runtime", "*.cpp")))
    hdrs = glob.glob(os.path.join(CSRC, "runtime", "*.h"))
    if cpps and (force or _newer(RUNTIME_SO, cpps + hdrs)):
        _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-pthread", "-o", RUNTIME_SO, *cpps])
    return RUNTIME_SO


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_runtime(force)
    build_kernels(force, verbose)


def main() -> int:
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", KERNELS_SO, RUNTIME_SO)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
