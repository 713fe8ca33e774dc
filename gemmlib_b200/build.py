"""In-tree build of the C-ABI library ``libms_blkq4gemm.so`` for sm_100a.

``python -m gemmlib_b200.build`` compiles every ``csrc/*.cu`` with nvcc
(``-gencode arch=compute_100a,code=sm_100a``; nvcc cross-compiles without a GPU)
and links them into ``gemmlib_b200/libms_blkq4gemm.so``.  Objects are rebuilt
only when a source or header is newer.  ``build_ext()`` builds the PyTorch C++
extension ``ms_blkq4linear_ext`` that links against it.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libms_blkq4gemm.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the library cannot be built")
    return nvcc


def _newest(paths) -> float:
    return max(os.path.getmtime(p) for p in paths)


def build_lib(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    hdr_time = _newest(headers + [os.path.abspath(__file__)])
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for log in ex.map(run, jobs):
                if verbose and log:
                    print(log, file=sys.stderr)
    if jobs or not os.path.exists(LIB) or os.path.getmtime(LIB) < _newest(objs):
        run([nvcc, "-shared", "-o", LIB, *objs, "-lcudart"])
    return LIB


EXT_NAME = "ms_blkq4linear_ext"


def ext_path():
    import sysconfig

    return os.path.join(PKG, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build_ext(force: bool = False) -> str:
    """Build the PyTorch extension ``ms_blkq4linear_ext`` next to the library it links."""
    build_lib()
    out = ext_path()
    src = os.path.join(CSRC, "ms_blkq4linear_ext.cpp")
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(src), os.path.getmtime(LIB)):
        return out
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    inc = cpp_extension.include_paths("cuda")
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=" + EXT_NAME,
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I" + os.path.join(ROOT, "include"), "-I" + sysconfig.get_paths()["include"]]
    cmd += ["-isystem" + p for p in inc]
    cmd += [src, "-o", out, "-L" + PKG, "-l:libms_blkq4gemm.so", "-Wl,-rpath,$ORIGIN",
            "-L" + tlib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Wl,-rpath," + tlib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building ms_blkq4linear_ext failed:\n" + r.stdout + r.stderr)
    return out


if __name__ == "__main__":
    print(build_lib(verbose="-v" in sys.argv, force="-f" in sys.argv))
    if "--ext" in sys.argv:
        print(build_ext(force="-f" in sys.argv))

