"""Builds libloom_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libloom_b200.so")
SOURCES = ["errors.cpp", "contract.cpp", "driver.cpp", "command.cpp", "graph.cpp",
           "providers.cpp", "peer_group.cpp", "prefill_provider.cpp", "prefill_kernels.cu", "prefill_tiled_kernel.cu", "decode_kernels.cu", "decode_stream_kernel.cu", "append_kernels.cu", "static_scratch.cu"]
HEADERS = ["runtime.hpp", "kernels.hpp", "peer_group.hpp", "decode_device.cuh", "dependent_launch.cuh", "prefill_device.cuh", "tcgen05_device.cuh", os.path.join(ROOT, "include", "loom_b200.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
         "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-x", "cu",
         "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def is_stale(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    built = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, s) for s in sources()] + [
        h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


# Checked builds (libraries of their own beside the product; `python build.py --asan` ...):
#   asan          host code with AddressSanitizer + UndefinedBehaviorSanitizer, for the host-side
#                 tests under the fake driver (the stand-in for compute-sanitizer's host checks)
#   debug-bounds  every computed global index of the decode and append kernels checked against the
#                 length of the operand it indexes (LB_DEBUG_BOUNDS): a violation sets the status
#                 word and skips the access, it never traps
VARIANTS = {
    "asan": ["-g", "-Xcompiler", "-fsanitize=address,-fsanitize=undefined,-fno-omit-frame-pointer"],
    "debug-bounds": ["-DLB_DEBUG_BOUNDS=1"],
}


def variant_path(variant: str) -> str:
    return os.path.join(HERE, f"libloom_b200_{variant.replace('-', '_')}.so")


def build(force: bool = False, verbose: bool = False, variant: str = "") -> str:
    lib = variant_path(variant) if variant else LIB
    if not force and not is_stale(lib):
        return lib
    obj_dir = os.path.join(HERE, "build", variant) if variant else os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    extra = VARIANTS[variant] if variant else []
    objects = []
    procs = []
    for source in sources():
        obj = os.path.join(obj_dir, os.path.splitext(source)[0] + ".o")
        objects.append(obj)
        cmd = [NVCC, *FLAGS, *extra, "-c", os.path.join(CSRC, source), "-o", obj]
        if verbose and source.endswith(".cu"):
            cmd.insert(1, "-Xptxas=-v")
        procs.append((source, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                               stderr=subprocess.STDOUT, text=True)))
    failed = False
    for source, proc in procs:
        output, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            sys.stderr.write(f"--- {source}\n{output}\n")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link_extra = ["-Xcompiler", "-fsanitize=address,-fsanitize=undefined"] if variant == "asan" else []
    subprocess.run([NVCC, "-shared", "-o", lib, *objects, "-gencode",
                    "arch=compute_100a,code=sm_100a", "-ldl", *link_extra], check=True)
    return lib


NATIVE_BENCH = os.path.join(HERE, "loom_native_bench")


def build_native_bench(force: bool = False) -> str:
    """The C++ latency harness over the C ABI (csrc/native_bench.cpp), linked to the library."""
    source = os.path.join(CSRC, "native_bench.cpp")
    lib = build()
    if (not force and os.path.exists(NATIVE_BENCH)
            and os.path.getmtime(NATIVE_BENCH) > max(os.path.getmtime(source),
                                                     os.path.getmtime(lib))):
        return NATIVE_BENCH
    subprocess.run([NVCC, "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), source,
                    "-o", NATIVE_BENCH, "-L", HERE, "-lloom_b200",
                    "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"], check=True)
    return NATIVE_BENCH


if __name__ == "__main__":
    chosen = [v for v in VARIANTS if f"--{v}" in sys.argv]
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv,
                variant=chosen[0] if chosen else ""))
    if "--native-bench" in sys.argv:
        print(build_native_bench(force="--force" in sys.argv))
