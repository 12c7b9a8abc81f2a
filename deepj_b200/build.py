"""Builds libdeepj_cuda_jni.so (sm_100a only) in-tree with nvcc, and the CPU oracle.

`python -m deepj_b200.build` compiles every .cu under deepj_b200/csrc for
`-gencode arch=compute_100a,code=sm_100a` and links them into
deepj_b200/libdeepj_cuda_jni.so.  No GPU is needed to build.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
BUILD = os.path.join(PKG_DIR, "csrc", "build")
LIB = os.path.join(PKG_DIR, "libdeepj_cuda_jni.so")
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "libdeepj_oracle.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # multiply and add are fused only where the source says fmaf()
    "-fmad=false",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libdeepj_cuda_jni.so cannot be built")
    return exe


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _jni_includes() -> list[str]:
    """Include paths of the JDK named by JAVA_HOME; with them csrc/jni_shim.cpp adds the JNI natives."""
    home = os.environ.get("JAVA_HOME", "")
    inc = os.path.join(home, "include")
    if not home or not os.path.exists(os.path.join(inc, "jni.h")):
        return []
    return ["-I", inc, "-I", os.path.join(inc, "linux")]


def _compile(src: str, obj: str, headers: list[str], verbose: bool) -> str:
    if _newer(obj, [src] + headers):
        return ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), *_jni_includes(), "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return res.stderr if verbose else ""


def build_cuda(verbose: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    sources = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(ROOT, "include", "deepj_cuda.h"))
    objs = [os.path.join(BUILD, os.path.basename(s) + ".o") for s in sources]
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        logs = list(ex.map(lambda so: _compile(so[0], so[1], headers, verbose), zip(sources, objs)))
    if verbose:
        for log in logs:
            if log:
                print(log)
    if not _newer(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


def build_oracle() -> str:
    src = os.path.join(ORACLE_DIR, "deepj_oracle.cpp")
    if not _newer(ORACLE_LIB, [src]):
        res = subprocess.run(["make", "-C", ORACLE_DIR], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"oracle build failed:\n{res.stdout}\n{res.stderr}")
    return ORACLE_LIB


if __name__ == "__main__":
    v = "-v" in sys.argv
    print(build_cuda(verbose=v))
    print(build_oracle())
