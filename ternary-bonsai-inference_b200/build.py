"""Builds libbonsai_kv.so (the CUDA kernels + C ABI) in-tree for sm_100a with nvcc.

    python ternary-bonsai-inference_b200/build.py [--force] [--verbose]

No GPU is needed to build.  The library lands next to this file so that it is found by
the ctypes loader in this package and travels with the source tree.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libbonsai_kv.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++20", "-O3", "-lineinfo", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
          "-Xcompiler", "-fPIC,-ffp-contract=off,-fvisibility=hidden,-Wall"]
# Per-file extras.  The files that decide stored bits are compiled without FMA contraction on
# top of their explicit round-to-nearest intrinsics; division and sqrt stay IEEE (nvcc default).
SOURCES = {
    "bk_api.cu": [],
    "bk_append.cu": ["--fmad=false"],
    "bk_kvq.cu": ["--fmad=false"],
    "bk_decode.cu": [],
    "bk_decode_mma.cu": [],
    "bk_decode_f16.cu": [],
    "bk_noalloc.cu": [],
    "bk_layer.cu": ["--fmad=false"],
    "bk_pq2.cu": [],
    "bk_prefill.cu": [],
    "bk_prefill_umma.cu": [],
    "bk_p2p.cu": [],
    "bk_host_tables.cpp": [],
    "bk_snapshot.cpp": [],
}
HEADERS = ["bk_internal.h", "bk_device.cuh", "bk_decode_common.cuh", "bk_mma_common.cuh", "bk_umma.cuh", os.path.join(ROOT, "include", "bonsai_kv.h")]


def nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _newest_header():
    return max(os.path.getmtime(h if os.path.isabs(h) else os.path.join(CSRC, h)) for h in HEADERS)


def _compile(src, extra, force, verbose):
    path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    stamp = max(os.path.getmtime(path), _newest_header(), os.path.getmtime(os.path.abspath(__file__)))
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= stamp:
        return obj, ""
    cmd = [nvcc(), *ARCH, *COMMON, *extra, "-c", path, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        futs = [ex.submit(_compile, s, e, force, verbose) for s, e in SOURCES.items()]
        results = [f.result() for f in futs]
    objs = [o for o, _ in results]  # (a compile error has raised above, before any stale link)
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [nvcc(), *ARCH, "-shared", "-o", LIB, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
