"""Builds libfa_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m flash_attn_b200.build [--force] [--verbose]

The library is rebuilt only when a source is newer than the binary.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libfa_b200.so")
SOURCES = ["fa_api.cu", "fa_fwd_tiled.cu", "fa_decode.cu", "fa_aux.cu", "fa_static_scratch.cu", "fa_ring.cu"]
HEADERS = ["fa_internal.h", "sm100_ptx.cuh", "philox.cuh", os.path.join("..", "..", "include", "fa_b200.h")]


def nvcc_path():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    objs = []
    build_dir = os.path.join(PKG, "build")
    os.makedirs(build_dir, exist_ok=True)
    common = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v" if verbose else "-warn-spills"]
    procs = []
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", os.path.join(CSRC, src), "-o", obj],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(out)
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    subprocess.check_call([nvcc_path(), "-shared", "-o", LIB] + objs + ["-Xcompiler", "-fPIC", "-ldl"])
    return LIB


TEST_LIB = os.path.join(PKG, "libfa_b200_shortwait.so")


def build_test_variant(force=False):
    """Builds libfa_b200_shortwait.so, the library compiled with -DFA_TEST_SHORT_WAIT: bounded waits give
    up after about 2 ms and the producer of the tiled kernel can be told to leave one KV tile out
    (fa_test_skip_kv_tile).  Used only by the GPU test of the give-up path."""
    if not force and os.path.exists(TEST_LIB) and not any(
            os.path.getmtime(os.path.join(CSRC, f)) > os.path.getmtime(TEST_LIB) for f in SOURCES + HEADERS):
        return TEST_LIB
    build_dir = os.path.join(PKG, "build", "shortwait")
    os.makedirs(build_dir, exist_ok=True)
    common = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-DFA_TEST_SHORT_WAIT", "-Xcompiler", "-fPIC", "-Xptxas", "-warn-spills"]
    procs, objs = [], []
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", os.path.join(CSRC, src), "-o", obj],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {src} (test variant)")
    subprocess.check_call([nvcc_path(), "-shared", "-o", TEST_LIB] + objs + ["-Xcompiler", "-fPIC", "-ldl"])
    return TEST_LIB


BENCH = os.path.join(PKG, "fa_bench")


def build_driver(force=False):
    """Builds the C benchmark driver (csrc/fa_main.c) against the library with gcc."""
    src = os.path.join(CSRC, "fa_main.c")
    build()
    if not force and os.path.exists(BENCH) and os.path.getmtime(BENCH) > max(os.path.getmtime(src), os.path.getmtime(LIB)):
        return BENCH
    cuda = os.path.dirname(os.path.dirname(nvcc_path()))
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    subprocess.check_call([cc, "-std=c99", "-O2", "-Wall", "-I", os.path.join(PKG, "..", "include"),
                           "-I", os.path.join(cuda, "include"), src, "-o", BENCH,
                           "-L", PKG, "-lfa_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lm", "-lpthread",
                           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda, "lib64")])
    return BENCH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
    print(build_driver(force="--force" in sys.argv))
    print(build_test_variant(force="--force" in sys.argv))
