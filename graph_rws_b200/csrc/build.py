"""Compiles libgrws_b200.so in-tree with nvcc for sm_100a (no other architecture is built)."""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, os.environ.get("GRWS_LIB_NAME", "libgrws_b200.so"))
NVCC = os.environ.get("GRWS_NVCC", "/usr/local/cuda/bin/nvcc")
EXTRA = os.environ.get("GRWS_NVCC_EXTRA", "").split()
FLAGS = EXTRA + ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-ccbin", "/usr/bin/g++"]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    deps = sources() + glob.glob(os.path.join(HERE, "*.cuh")) + [os.path.join(HERE, "..", "..", "include", "grws_b200.h")]
    return any(os.path.getmtime(d) > os.path.getmtime(LIB) for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return LIB
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for src in sources():
        obj = os.path.join(HERE, "build", os.path.basename(src) + ".o")
        objs.append(obj)
        cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([NVCC, "-shared", "-o", LIB] + objs + ["-lcudart", "-ccbin", "/usr/bin/g++"])
    return LIB


SELFTEST_LIB = os.path.join(HERE, "libgrws_b200_selftest.so")


def build_selftest(force: bool = False) -> str:
    """The same library with the SpMM kernel's profiling build compiled in (-DGRWS_TC5_PROFILING):
    per-role wait counters, and the switch the time-out self-test uses to withhold one barrier
    arrive.  Only spmm_tcgen05.cu is compiled again; the other objects are the product's."""
    build()
    src = os.path.join(HERE, "spmm_tcgen05.cu")
    if not force and os.path.exists(SELFTEST_LIB) and os.path.getmtime(SELFTEST_LIB) >= os.path.getmtime(LIB):
        return SELFTEST_LIB
    obj = os.path.join(HERE, "build", "spmm_tcgen05.selftest.o")
    subprocess.check_call([NVCC] + FLAGS + ["-DGRWS_TC5_PROFILING", "-c", src, "-o", obj])
    objs = [os.path.join(HERE, "build", os.path.basename(s) + ".o") for s in sources() if s != src] + [obj]
    subprocess.check_call([NVCC, "-shared", "-o", SELFTEST_LIB] + objs + ["-lcudart", "-ccbin", "/usr/bin/g++"])
    return SELFTEST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    # the self-test build shares every object but one with the product: it is kept in step with it
    # (a variant build under another name, GRWS_LIB_NAME, has no self-test twin)
    if "--selftest" in sys.argv or (os.path.exists(SELFTEST_LIB) and "GRWS_LIB_NAME" not in os.environ):
        print(build_selftest(force="--force" in sys.argv))
