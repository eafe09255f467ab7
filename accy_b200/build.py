"""Builds libaccy_b200.so (C++17 host library behind the C ABI) in-tree with g++ and nvcc.

Needs the CUDA toolkit (nvcc and libcudart_static.a under $CUDA_HOME, default /usr/local/cuda):
the fixed-function kernels of CU_SOURCES are compiled ahead of time for sm_100a and linked with
the static CUDA runtime.  No GPU is needed to build or to load the library: libcuda and libnvrtc
are dlopen'ed at run time, and the static runtime touches no device until one of its entry points
is called.  All other kernels are CUDA templates the library instantiates per program and compiles
for sm_100a through NVRTC; `check_kernels_with_nvcc` cross-compiles the same sources with nvcc to
prove they build and to record registers/spills/shared memory (-Xptxas -v).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libaccy_b200.so")
SOURCES = ["program.cpp", "wire.cpp", "planner.cpp", "emit_row.cpp", "emit_gemm.cpp", "emit_tc.cpp", "emit_attn.cpp", "shard.cpp", "transform.cpp",
           "driver.cpp", "session.cpp", "sharded.cpp"]


def needs_build():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    for name in os.listdir(CSRC):
        if os.path.getmtime(os.path.join(CSRC, name)) > built:
            return True
    return os.path.getmtime(os.path.join(HERE, "..", "include", "accy_b200.h")) > built


CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
CU_SOURCES = ["noalloc.cu", "probe.cu"]   # fixed-function kernels compiled ahead of time by nvcc for sm_100a


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    objects = []
    nvcc = os.path.join(CUDA_HOME, "bin", "nvcc")
    if not os.path.exists(nvcc):
        raise RuntimeError("building libaccy_b200.so needs the CUDA toolkit: %s not found (set CUDA_HOME)" % nvcc)
    for cu in CU_SOURCES:
        obj = os.path.join(HERE, cu.replace(".cu", ".o"))
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
               "-std=c++17", "-Xcompiler", "-fPIC", "-c", os.path.join(CSRC, cu), "-o", obj]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
        objects.append(obj)
    cmd = ["g++", "-std=c++17", "-O2", "-g", "-fPIC", "-shared", "-Wall", "-Wextra", "-Wno-unused-parameter",
           "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES] + objects + [
               "-L" + os.path.join(CUDA_HOME, "lib64"), "-lcudart_static", "-lrt", "-ldl", "-lpthread"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return LIB


def check_kernels_with_nvcc(sources, out_dir, verbose=False):
    """Cross-compiles generated kernel sources for sm_100a with nvcc; returns ptxas -v text per kernel.

    `sources` is a list of (name, cuda_source, options) as returned by CompiledProgram.kernels().
    """
    os.makedirs(out_dir, exist_ok=True)
    reports = {}
    for name, source, options in sources:
        cu = os.path.join(out_dir, name + ".cu")
        with open(cu, "w") as f:
            f.write(source)
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
               "-Xptxas", "-v", "-cubin", "-o", os.path.join(out_dir, name + ".cubin"), cu]
        cmd += [o for o in options.split() if o.startswith("--fmad")]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (name, proc.stderr))
        reports[name] = proc.stderr
        if verbose:
            print(proc.stderr)
    return reports


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
