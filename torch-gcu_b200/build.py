"""Builds the native pieces in-tree.

  python torch-gcu_b200/build.py kernels   -> torch-gcu_b200/lib/libb200ops.so
  python torch-gcu_b200/build.py host      -> torch-gcu_b200/torch_gcu/_C*.so   (needs kernels)
  python torch-gcu_b200/build.py all

Every .cu file is compiled for sm_100a only
(`-gencode arch=compute_100a,code=sm_100a -lineinfo`), one nvcc process per
file, and linked with the static CUDA runtime so the library carries no
dependency on the interpreter's CUDA wheels.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
KERNEL_DIR = os.path.join(HERE, "csrc", "kernels")
BUILD_DIR = os.path.join(HERE, "build")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libb200ops.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-I" + os.path.join(ROOT, "include"), "-I" + KERNEL_DIR,
]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return r.stdout + r.stderr


def build_kernels(verbose=False, force=False):
    os.makedirs(BUILD_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    headers = [os.path.join(KERNEL_DIR, f) for f in os.listdir(KERNEL_DIR) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "b200ops.h"))
    sources = sorted(f for f in os.listdir(KERNEL_DIR) if f.endswith(".cu"))
    jobs = []
    objects = []
    for f in sources:
        src = os.path.join(KERNEL_DIR, f)
        obj = os.path.join(BUILD_DIR, f[:-3] + ".o")
        objects.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for out in ex.map(_run, jobs):
            if verbose and out.strip():
                print(out)
    if jobs or not os.path.exists(LIB_PATH):
        _run([NVCC, "-shared", "-o", LIB_PATH] + objects + ["-cudart", "static", "-Xlinker", "--no-undefined",
             "-lpthread", "-ldl", "-lrt"])
    return LIB_PATH


def build_host(verbose=False, force=False):
    sys.path.insert(0, HERE)
    import build_host  # noqa: deferred: needs torch
    return build_host.build(verbose=verbose, force=force)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    verbose = "-v" in sys.argv
    force = "-f" in sys.argv
    if what in ("kernels", "all"):
        print(build_kernels(verbose, force))
    if what in ("host", "all") and os.path.exists(os.path.join(HERE, "build_host.py")):
        print(build_host(verbose, force))
