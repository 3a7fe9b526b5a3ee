"""In-tree build of libdsuf_qmm.so (nvcc, sm_100a only).

``python deepseek-ultrafast_b200/build.py`` or ``build()`` from Python.  Objects are cached under
``csrc/build/`` and rebuilt when a source or header is newer.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libdsuf_qmm.so")
SOURCES = ["abi.cu", "quant.cu", "moe_aux.cu", "stream_launch.cu", "noalloc.cu", "ep_comm.cu", "peak_probe.cu", "lm_head.cu", "pack.cc", "loader.cc"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
         "-Xptxas", "-v", "--expt-relaxed-constexpr", "-ccbin", "/usr/bin/g++"] + os.environ.get("DSUF_EXTRA_NVCC_FLAGS", "").split()


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "include", "dsuf_qmm.h"))
    return hs


def _compile(src, obj, log):
    cmd = [NVCC, *FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    if src.endswith(".cc"):
        cmd = [NVCC, "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++", "-x", "cu", "-c",
               os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")


def build(verbose=False):
    bdir = os.path.join(CSRC, "build")
    os.makedirs(bdir, exist_ok=True)
    newest_h = max(os.path.getmtime(h) for h in _headers())
    jobs, objs = [], []
    for s in SOURCES:
        if not os.path.exists(os.path.join(CSRC, s)):
            continue
        obj = os.path.join(bdir, s + ".o")
        objs.append(obj)
        src_m = max(os.path.getmtime(os.path.join(CSRC, s)), newest_h)
        if not os.path.exists(obj) or os.path.getmtime(obj) < src_m:
            jobs.append((s, obj, os.path.join(bdir, s + ".log")))
    if jobs:
        with ThreadPoolExecutor(max_workers=8) as ex:
            list(ex.map(lambda j: _compile(*j), jobs))
    if jobs or not os.path.exists(OUT):
        # link beside the target and rename: a reader never sees a half-written library
        cmd = [NVCC, "-shared", "-o", OUT + ".tmp", *objs, "-ccbin", "/usr/bin/g++", "-lcudart", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        os.replace(OUT + ".tmp", OUT)
    if verbose:
        for s, _, log in jobs:
            print(open(log).read())
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
