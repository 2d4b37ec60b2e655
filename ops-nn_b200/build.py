"""Builds lib/libopsnn_b200.so (host C++ + CUDA kernels for sm_100a) in-tree with nvcc.

Usage:  python ops-nn_b200/build.py [--force] [--verbose]

The library links the CUDA runtime statically and resolves the driver's tensor-map encoder at run time, so it loads
(and phase 1 of every aclnn entry point runs) on a machine without a GPU or libcuda.
"""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "libopsnn_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
COMMON = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CSRC, "host"), "-I" + os.path.join(CSRC, "cuda"),
    "--expt-relaxed-constexpr", "-diag-suppress", "177,550",
]
for _m in ("OPSNN_DECODE_PF", "OPSNN_DECODE_MINB"):  # tuning knobs of the decode kernel, unset in normal builds
    if os.environ.get(_m):
        COMMON.append("-D%s=%s" % (_m, os.environ[_m]))
for _d in filter(None, os.environ.get("OPSNN_EXTRA_DEFS", "").split(",")):  # extra -D switches for tuning experiments
    COMMON.append("-D" + _d)


def sources():
    out = []
    for sub in ("host", "cuda"):
        d = os.path.join(CSRC, sub)
        for f in sorted(os.listdir(d)):
            if f.endswith((".cpp", ".cu")):
                out.append(os.path.join(d, f))
    return out


def _headers_digest():
    h = hashlib.sha1()
    for base in (os.path.join(ROOT, "include"), CSRC):
        for dp, _, fs in sorted(os.walk(base)):
            for f in sorted(fs):
                if f.endswith((".h", ".cuh", ".hpp")):
                    with open(os.path.join(dp, f), "rb") as fh:
                        h.update(fh.read())
    h.update(" ".join(COMMON).encode())
    return h.hexdigest()


def _compile(src, hdr_digest, force, verbose):
    with open(src, "rb") as fh:
        digest = hashlib.sha1(fh.read() + hdr_digest.encode()).hexdigest()
    obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
    stamp = obj + ".sha1"
    if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest:
        return obj, False
    cmd = [NVCC] + COMMON + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, res.stdout, res.stderr))
    if verbose or res.stderr.strip():
        sys.stderr.write(res.stderr)
    with open(stamp, "w") as fh:
        fh.write(digest)
    return obj, True


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr = _headers_digest()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, hdr, force, verbose), srcs))
    objs = [o for o, _ in results]
    if any(changed for _, changed in results) or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
