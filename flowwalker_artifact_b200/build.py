"""Builds libflowwalker.so (C ABI + CUDA kernels, sm_100a only) in-tree with nvcc.

Run as `python -m flowwalker_artifact_b200.build` or call build().  nvcc
cross-compiles without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libflowwalker.so")
CLI = os.path.join(HERE, "flowwalker")
SOURCES = ["fw_graph.cpp", "fw_rmat.cu", "fw_walk.cu"]
HEADERS = ["fw_internal.h", "fw_spec.cuh", "fw_kernels.cuh", os.path.join("..", "..", "include", "flowwalker.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # no implicit a*b+c contraction: the walk must match the CPU golden walker bit for bit
    "-fmad=false",
    "-Xcompiler", "-fPIC,-Wall,-Wextra,-Wno-unused-parameter",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compiles every CUDA/C++ source of the package; returns the library path."""
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    if force or _stale(LIB, deps):
        objs = []
        for s in SOURCES:
            obj = os.path.join(CSRC, s.rsplit(".", 1)[0] + ".o")
            src = os.path.join(CSRC, s)
            if force or _stale(obj, deps):
                cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", src, "-o", obj]
                subprocess.run(cmd, check=True, env=env)
            objs.append(obj)
        subprocess.run([_nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"],
                       check=True, env=env)
    cli_src = os.path.join(CSRC, "fw_cli.cpp")
    if os.path.exists(cli_src) and (force or _stale(CLI, [cli_src, LIB, os.path.join(CSRC, "fw_flags.h")])):
        subprocess.run(["g++", "-std=c++17", "-O2", "-Wall", "-Wextra", "-pthread", cli_src, "-o", CLI,
                        "-L" + HERE, "-lflowwalker", "-Wl,-rpath,$ORIGIN"], check=True, env=env)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
