"""Builds the PrivateUse1 host extension in-tree: torch_gcu/_C*.so.

Runs the code generator (codegen/gen_backend_stubs.py -> csrc/host/aten/generated)
and compiles csrc/host/**/*.cpp with the host compiler through
torch.utils.cpp_extension (ninja). The extension holds no device code; it links
the kernel library (lib/libb200ops.so, found at run time through an $ORIGIN
rpath), the static CUDA runtime and the NCCL library that ships with PyTorch.
"""
import glob
import importlib.util
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
HOST = os.path.join(HERE, "csrc", "host")
PKG = os.path.join(HERE, "torch_gcu")


def _nccl_paths():
    import nvidia.nccl as n
    base = os.path.dirname(n.__file__) if getattr(n, "__file__", None) else list(n.__path__)[0]
    return os.path.join(base, "include"), os.path.join(base, "lib")


def build(verbose=False, force=False):
    spec = importlib.util.spec_from_file_location("gen_backend_stubs", os.path.join(HERE, "codegen", "gen_backend_stubs.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    gen.run(os.path.join(HERE, "codegen", "gcu_native_functions.yaml"), os.path.join(HOST, "aten", "generated"))

    # the system compiler: its libstdc++ is the shared one the interpreter loads (a
    # toolchain that links libstdc++ statically gives the extension a second,
    # uninitialised copy of the iostream state)
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils import cpp_extension
    sources = sorted(glob.glob(os.path.join(HOST, "**", "*.cpp"), recursive=True))
    build_selftest(verbose, force)
    nccl_inc, nccl_lib = _nccl_paths()
    build_dir = os.path.join(HERE, "build", "host")
    os.makedirs(build_dir, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    existing = glob.glob(os.path.join(PKG, "_C*.so"))
    if existing and not force:
        newest_src = max(os.path.getmtime(p) for p in sources + glob.glob(os.path.join(HOST, "**", "*.h*"), recursive=True) +
                         [os.path.join(ROOT, "include", "b200ops.h")])
        if os.path.getmtime(existing[0]) > newest_src:
            return existing[0]
    # compile + link only (ninja); the library is NOT loaded into this process, so
    # building and importing torch_gcu in one interpreter registers everything once
    cpp_extension._write_ninja_file_and_build_library(
        name="_C",
        sources=sources,
        extra_cflags=["-O2", "-std=c++17", "-fvisibility=hidden", "-Wno-deprecated-declarations"],
        extra_cuda_cflags=[],
        extra_sycl_cflags=[],
        extra_ldflags=["-L" + os.path.join(HERE, "lib"), "-lb200ops", "-Wl,-rpath,'$$ORIGIN/../lib'",
                       "-L" + os.path.join(cuda_home, "lib64"), "-lcudart_static", "-lrt", "-ldl", "-lpthread",
                       "-L" + nccl_lib, "-l:libnccl.so.2", "-Wl,-rpath," + nccl_lib],
        extra_include_paths=[HOST, os.path.join(ROOT, "include"), os.path.join(cuda_home, "include"), nccl_inc],
        build_directory=build_dir,
        verbose=verbose,
        with_cuda=False,
        with_sycl=False,
        is_standalone=False,
    )
    built = os.path.join(build_dir, "_C.so")
    target = os.path.join(PKG, "_C.so")
    shutil.copy2(built, target)
    return target


def build_selftest(verbose=False, force=False):
    """tests/native/_gcu_selftest.so: the host-side policies (caching allocator, collective
    watchdog) compiled together with fakes of the device and of the communicator, for the CPU
    test-suite. Test infrastructure: the product never loads it."""
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils import cpp_extension
    native = os.path.join(ROOT, "tests", "native")
    sources = sorted(glob.glob(os.path.join(native, "*.cpp"))) + [
        os.path.join(HOST, "runtime", "gcu_allocator.cpp"), os.path.join(HOST, "runtime", "gcu_runtime.cpp"),
        os.path.join(HOST, "distributed", "work_watchdog.cpp")]
    target = os.path.join(native, "_gcu_selftest.so")
    deps = sources + glob.glob(os.path.join(HOST, "runtime", "*.h")) + glob.glob(os.path.join(HOST, "distributed", "*.h"))
    if os.path.exists(target) and not force and os.path.getmtime(target) > max(os.path.getmtime(p) for p in deps):
        return target
    build_dir = os.path.join(HERE, "build", "selftest")
    os.makedirs(build_dir, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cpp_extension._write_ninja_file_and_build_library(
        name="_gcu_selftest",
        sources=sources,
        extra_cflags=["-O1", "-std=c++17", "-fvisibility=hidden", "-Wno-deprecated-declarations"],
        extra_cuda_cflags=[],
        extra_sycl_cflags=[],
        extra_ldflags=["-L" + os.path.join(cuda_home, "lib64"), "-lcudart_static", "-lrt", "-ldl", "-lpthread"],
        extra_include_paths=[HOST, os.path.join(ROOT, "include"), os.path.join(cuda_home, "include")],
        build_directory=build_dir,
        verbose=verbose,
        with_cuda=False,
        with_sycl=False,
        is_standalone=False,
    )
    shutil.copy2(os.path.join(build_dir, "_gcu_selftest.so"), target)
    return target


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
