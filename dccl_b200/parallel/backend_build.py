"""Builds the PyTorch backend extension (csrc/torch/pg_dccl.cpp) in-tree, next to libdccl.so.

The extension only uses the library's public C++ API and libtorch; it is compiled with the system
C++ compiler against the headers of the installed torch and linked to ``dccl_b200/lib/libdccl.so``
by relative rpath, so the built file can be moved with the package.
"""
import os
import shutil
import subprocess
import sys
import sysconfig

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
_ROOT = os.path.dirname(_PKG)
SRC = os.path.join(_ROOT, "csrc", "torch", "pg_dccl.cpp")
OUT = os.path.join(_PKG, "lib", "_dccl_torch.so")


def needs_build():
    if not os.path.exists(OUT):
        return True
    newest = max(os.path.getmtime(SRC), os.path.getmtime(os.path.join(_ROOT, "include", "dccl", "dccl.hpp")))
    return os.path.getmtime(OUT) < newest


def build(force=False, verbose=False):
    if not force and not needs_build():
        return OUT
    import torch
    from torch.utils import cpp_extension
    from .._lib import LIB_PATH, lib
    lib()   # makes sure libdccl.so exists
    # a compiler that links libstdc++ dynamically, like torch itself does
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "c++")
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    incs = cpp_extension.include_paths(device_type="cuda")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", SRC, "-o", OUT,
           "-DTORCH_EXTENSION_NAME=_dccl_torch", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + os.path.join(_ROOT, "include"), "-I" + os.path.join(cuda_home, "include"), "-I" + sysconfig.get_paths()["include"]]
    cmd += ["-I" + p for p in incs]
    cmd += ["-L" + tlib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-L" + os.path.dirname(LIB_PATH), "-ldccl", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib, "-Wno-attributes", "-Wno-interference-size"]
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building the torch backend failed:\n" + " ".join(cmd) + "\n" + res.stderr[-6000:])
    if verbose:
        print(res.stderr, file=sys.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose=True))
