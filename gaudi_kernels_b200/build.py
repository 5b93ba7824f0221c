"""Build libbfp8.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m gaudi_kernels_b200.build [--force] [--timeline]

--timeline writes libbfp8_timeline.so instead: the same sources compiled with -DBFP8_TIMELINE, in which the GEMM
kernels log clock stamps of their pipeline events (read with `python -m gaudi_kernels_b200.timeline`).  A diagnostic
build; the package never loads it.

nvcc cross-compiles without a GPU.  The shared object is written next to this file; it links the
CUDA runtime statically and resolves the one driver entry point it needs at run time, so it loads
on a machine without a GPU driver.
"""

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libbfp8.so")
SOURCES = ["codec.cu", "gemm_tcgen05.cu", "gemm_smallm.cu", "gemm_pair.cu", "gemm_channel.cu", "gemm_api.cu",
           "rank_sum.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libbfp8.so cannot be built")
    return exe


def _deps():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "bfp8.h")]
    return max(os.path.getmtime(f) for f in files)


def up_to_date():
    return os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps()


TIMELINE_LIB = os.path.join(HERE, "libbfp8_timeline.so")


def build(force=False, verbose=False, timeline=False):
    """Compile every .cu under csrc/ and link libbfp8.so (or the diagnostic libbfp8_timeline.so).  Returns the path."""
    if timeline:
        return _build(TIMELINE_LIB, os.path.join(HERE, "build", "timeline"), ["-DBFP8_TIMELINE"], verbose)
    if not force and up_to_date():
        return LIB
    return _build(LIB, os.path.join(HERE, "build"), [], verbose)


def _build(lib, objdir, defines, verbose):
    nvcc = _nvcc()
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = ([nvcc] + ARCH_FLAGS + CFLAGS + defines + (["-Xptxas", "-v"] if verbose else [])
               + ["-c", os.path.join(CSRC, src), "-o", obj])
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, pr in procs:
        out, _ = pr.communicate()
        if verbose and out:
            print(out)
        if pr.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s" % (" ".join(cmd), out))
    link = [nvcc] + ARCH_FLAGS + ["-shared", "-cudart", "static", "-o", lib] + objs
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed: %s\n%s" % (" ".join(link), res.stdout))
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, timeline="--timeline" in sys.argv))
