"""Builds libatlas_kernels (shared object and static archive) for sm_100a with nvcc.

The static archive keeps the name the reference's build script links
(crates/atlas-tensor/build.rs:56,104: `static=atlas_kernels`); the shared object is what the
Python binding loads.  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "lib")
SOURCES = ["ctx.cu", "gemv.cu", "attention.cu", "elementwise.cu", "legacy_abi.cu", "model.cu", "comm.cu", "gemv_mma.cu", "loader.cu", "sampling.cu", "attention_mma.cu", "gemv_umma.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
LIB_SO = os.path.join(OUT, "libatlas_kernels.so")
LIB_A = os.path.join(OUT, "libatlas_kernels.a")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(OUT, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".inl"))]
    headers.append(os.path.join(HERE, "..", "include", "atlas_kernels.h"))
    nvcc = os.environ.get("NVCC", "nvcc")
    extra = os.environ.get("AX_EXTRA_NVCC_FLAGS", "").split()
    objs, jobs = [], []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OUT, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            jobs.append((src, [nvcc] + NVCC_FLAGS + extra + ["-c", s, "-o", o]))

    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = os.path.join(OUT, name + ".ptxas.log")
        with open(log, "w") as f:
            f.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (name, (r.stdout + r.stderr)[-6000:]))
        if verbose:
            sys.stderr.write("built %s\n" % name)

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    if force or jobs or _stale(LIB_SO, objs):
        r = subprocess.run([nvcc, "-shared", "-o", LIB_SO] + objs + ["-lcudart_static", "-ldl", "-lpthread", "-lrt"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        if os.path.exists(LIB_A):
            os.remove(LIB_A)
        subprocess.run(["ar", "rcs", LIB_A] + objs, check=True)
    return LIB_SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
