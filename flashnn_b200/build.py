"""Builds the C-ABI shared library (libflashnn_b200.so) with nvcc for sm_100a.

    python -m flashnn_b200.build [--force] [--verbose]

The library is built in-tree, next to this file, and loaded with ctypes by
`flashnn_b200._lib`.  There is no other backend: if the library is missing the
operators raise.
"""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB_PATH = os.path.join(HERE, "libflashnn_b200.so")
SOURCES = ["capi.cu", "dynamic_quant.cu", "gemm_a8w8.cu", "gemv_weight_only.cu", "gemv_w4_imma.cu", "gemm_weight_only.cu", "norm_dquant.cu", "fused_moe_a16w4.cu", "gemv_w4_tok.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return deps


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(d) > t for d in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every kernel source into one shared library; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = nvcc_path()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    common = [nvcc, "-std=c++17", "-O3", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC,-Wall",
              "-I", INCLUDE, "--expt-relaxed-constexpr"]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = common + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {src} (exit {pr.returncode})\n{out}\n")
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    link = [nvcc, "-shared", *ARCH_FLAGS, "-o", LIB_PATH, *objs, "-lcudart"]
    subprocess.run(link, check=True)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/shared-memory usage")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
