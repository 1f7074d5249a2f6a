"""Build libnvfp4_b200.so from csrc/*.cu with nvcc, for sm_100a only, in-tree.

    python -m nvfp4_sm120_b200.build          # build if sources are newer than the library
    python -m nvfp4_sm120_b200.build --force
"""
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libnvfp4_b200.so")
CLI = os.path.join(PKG, "nvfp4_gemm_cli")          # stand-alone C driver of the ABI (csrc/tools)
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "--threads", "4"]


def sources():
    return sorted(glob.glob(os.path.join(PKG, "csrc", "*.cu")))


def _deps():
    return sources() + glob.glob(os.path.join(PKG, "csrc", "*.cuh")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h")) + glob.glob(os.path.join(PKG, "csrc", "tools", "*.cu"))


def up_to_date():
    if not os.path.exists(LIB) or not os.path.exists(CLI):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(p) <= t for p in _deps())


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libnvfp4_b200.so")
    cmd = [nvcc] + NVCC_FLAGS + ["-I", os.path.join(ROOT, "include"), "-I", os.path.join(PKG, "csrc")]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += sources() + ["-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    # the C driver links the library it sits beside (rpath $ORIGIN)
    cli_cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
               "-I", os.path.join(ROOT, "include"), os.path.join(PKG, "csrc", "tools", "nvfp4_gemm_cli.cu"),
               "-L", PKG, "-lnvfp4_b200", "-Xlinker", "-rpath=$ORIGIN", "-o", CLI]
    res = subprocess.run(cli_cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed on the C driver:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
