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


if __name__ == "__main__":
    print(build(force="-f" in sys.argv, verbose="-v" in sys.argv))
