"""Builds ampstein_b200/libampstein_b200.so (the torch-free C-ABI library with every CUDA kernel)
in-tree with nvcc for sm_100a. Run as `python -m ampstein_b200.build [-f]`."""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "..", "build", "obj")
LIB = os.path.join(HERE, "libampstein_b200.so")

NVCC = os.environ.get("NVCC", "nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# (source, object name, extra flags)
def units():
    out = []
    for name in sorted(os.listdir(CSRC)):
        if not name.endswith(".cu"):
            continue
        if name == "exl3_gemv_inst.cu":
            for k in range(1, 9):
                out.append((name, "exl3_gemv_inst_k%d.o" % k, ["-DAMP_GEMV_K=%d" % k]))
        else:
            out.append((name, name[:-3] + ".o", []))
    return out


def _newest_header():
    return max(os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC)
               if f.endswith((".cuh", ".h")))


def _compile(unit, force, verbose):
    src, obj, extra = unit
    srcp, objp = os.path.join(CSRC, src), os.path.join(OBJ, obj)
    if (not force and os.path.exists(objp)
            and os.path.getmtime(objp) >= max(os.path.getmtime(srcp), _newest_header())):
        return objp, False
    cmd = [NVCC] + FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", srcp, "-o", objp]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    if verbose:
        sys.stderr.write(r.stderr)
    return objp, True


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    us = units()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        res = list(ex.map(lambda u: _compile(u, force, verbose), us))
    objs = [r[0] for r in res]
    if any(r[1] for r in res) or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return LIB


GLUE_SRC = os.path.join(HERE, "csrc_torch", "torch_glue.cpp")
GLUE = os.path.join(HERE, "_torch_glue.so")


def build_torch_glue(force=False):
    """Builds ampstein_b200/_torch_glue.so: the libtorch C++ layer with the reference's at::Tensor
    signatures over the C ABI (plain g++, linked against the installed libtorch and the library
    above)."""
    build()
    if not force and os.path.exists(GLUE) and os.path.getmtime(GLUE) >= max(
            os.path.getmtime(GLUE_SRC), os.path.getmtime(os.path.join(HERE, "..", "include", "ampstein_b200.h"))):
        return GLUE
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    inc = ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    libdirs = ce.library_paths("cuda")
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=_torch_glue",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    cmd += ["-I" + p for p in inc] + [GLUE_SRC, "-o", GLUE]
    cmd += ["-L" + p for p in libdirs] + ["-L" + HERE, "-lampstein_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu",
                                          "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
                                          "-Wl,-rpath,$ORIGIN"] + ["-Wl,-rpath," + p for p in libdirs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("torch glue build failed:\n%s\n%s" % (r.stdout, r.stderr[-4000:]))
    return GLUE


if __name__ == "__main__":
    print(build(force="-f" in sys.argv, verbose="-v" in sys.argv))
    if "--glue" in sys.argv:
        print(build_torch_glue(force="-f" in sys.argv))
