"""Builds dist/libnextsycl-llm.so from nextsycl_b200/csrc/*.cu with nvcc for sm_100a.

The library keeps the reference's output name (kernels/build.sh:70-106 produces dist/libnextsycl-llm.so), so an engine
switches to it by pointing NEXTSYCL_LIB at this file. Objects go to build/ and the library to dist/; both are built
artefacts, kept out of version control, and the library file travels with a copy of the working tree to machines where no
compiler runs.
"""
import concurrent.futures
import glob
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "nextsycl_b200", "csrc")
OUT = os.path.join(ROOT, "dist", "libnextsycl-llm.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def _nvcc():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_library(force=False, verbose=False):
    """Compiles what changed and links the library; returns its path."""
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    os.makedirs(os.path.join(ROOT, "build"), exist_ok=True)
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    nvcc = _nvcc()
    env = dict(os.environ)
    env.pop("CXX", None)
    env.pop("CC", None)
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(ROOT, "build", os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            jobs.append([nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return cmd, r.returncode, r.stdout

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, rc, out in ex.map(run, jobs):
            if verbose or rc != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + out)
            if rc != 0:
                raise RuntimeError("nvcc failed on " + cmd[-3])
    if force or jobs or _newer(OUT, objs):
        cmd, rc, out = run([nvcc, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart_static", "-ldl", "-lpthread", "-lrt"])
        if rc != 0:
            sys.stderr.write(out)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
