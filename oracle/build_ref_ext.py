"""Compile the reference's own PyTorch extension, UNCHANGED, against this library.

``python oracle/build_ref_ext.py [reference_dir]`` compiles
``<reference>/python/ms_blkq4linear_ext/ms_blkq4linear.cpp`` from where it lies with the include
directory and the shared library of this repository in the places the reference's
``python/setup.py:16-22`` gives to its own header and ``libms_blkq4gemm``.  The output,
``oracle/_ref/ms_blkq4linear_ext<suffix>.so`` (git-ignored), is what the drop-in test loads: the
reference's caller, this library's kernels.  Test infrastructure; nothing of it is shipped.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def default_reference_dir():
    return os.environ.get("BLKQ4_REFERENCE_DIR", os.path.join(ROOT, os.pardir, "reference"))


def output_path():
    return os.path.join(HERE, "_ref", "ms_blkq4linear_ext" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference_dir=None):
    import torch
    from torch.utils import cpp_extension

    ref = os.path.abspath(reference_dir or default_reference_dir())
    src = os.path.join(ref, "python", "ms_blkq4linear_ext", "ms_blkq4linear.cpp")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    lib_dir = os.path.join(ROOT, "gemmlib_b200")
    if not os.path.exists(os.path.join(lib_dir, "libms_blkq4gemm.so")):
        raise FileNotFoundError("build the library first: python -m gemmlib_b200.build")
    out = output_path()
    os.makedirs(os.path.dirname(out), exist_ok=True)
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=ms_blkq4linear_ext",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I" + os.path.join(ROOT, "include"), "-I" + sysconfig.get_paths()["include"]]
    cmd += ["-isystem" + p for p in cpp_extension.include_paths("cuda")]
    cmd += [src, "-o", out, "-L" + lib_dir, "-l:libms_blkq4gemm.so", "-Wl,-rpath,$ORIGIN/../../gemmlib_b200",
            "-L" + tlib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Wl,-rpath," + tlib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compiling the reference extension failed:\n" + r.stdout + r.stderr)
    return out


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
