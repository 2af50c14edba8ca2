"""Builds libzrnn.so (the C-ABI library with every CUDA kernel) in-tree with nvcc for sm_100a."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libzrnn.so")
CLI = os.path.join(HERE, "bin", "zoph_rnn")
SOURCES = ["kernels.cu", "tc_gemm.cu", "tc_decoder.cu", "zrnn_api.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]


def _newest(names_ok):
    t = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(root):
            if names_ok(f):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


def _newest_source():
    """Newest file that goes into libzrnn.so (the front end's own sources do not)."""
    return _newest(lambda f: f.endswith((".cu", ".cuh", ".h", ".hpp")) and f != "text_data.hpp")


def _newest_cli_source():
    return _newest(lambda f: f in ("cli_main.cpp", "text_data.hpp", "model_file.hpp", "zrnn.h"))


def build_cli(force=False):
    """Compile the command-line front end (host C++ only) against libzrnn.so; returns the binary's path."""
    if not force and os.path.exists(CLI) and os.path.getmtime(CLI) >= max(_newest_cli_source(), os.path.getmtime(LIB)):
        return CLI
    os.makedirs(os.path.dirname(CLI), exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    subprocess.check_call([cxx, "-O2", "-std=c++17", "-Wall", "-pthread", os.path.join(CSRC, "cli_main.cpp"), "-o", CLI,
                           "-L" + HERE, "-lzrnn", "-Wl,-rpath,$ORIGIN/.."])
    return CLI


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ into libzrnn.so and the front end binary; returns the library path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source():
        build_cli()
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        subprocess.check_call(cmd)
        objs.append(obj)
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs + ["-lcudart"])
    build_cli(force=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
