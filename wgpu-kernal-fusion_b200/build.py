"""Builds libwgf.so (C ABI in include/wgf.h) from csrc/ with nvcc for sm_100a.

Usage: python build.py [--force] [--verbose]
Objects go to csrc/_obj/, the library next to this file.  Only files newer than their
object are recompiled.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libwgf.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
         "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _newer(src, dst, headers):
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src] + headers)


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith((".cpp", ".cu")))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".hpp", ".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "wgf.h"))
    jobs = []
    for f in sources:
        src = os.path.join(CSRC, f)
        obj = os.path.join(OBJ, f + ".o")
        if force or _newer(src, obj, headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [NVCC, "-x", "cu", "-c", src, "-o", obj] + ARCH + FLAGS
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(compile_one, jobs):
            out = (r.stdout + r.stderr).strip()
            if r.returncode != 0:
                failed = True
                print(f"[build] FAILED {os.path.basename(src)}\n{out}", file=sys.stderr)
            elif verbose and out:
                print(f"[build] {os.path.basename(src)}\n{out}")
            if out:
                with open(os.path.join(OBJ, os.path.basename(src) + ".log"), "w") as fh:
                    fh.write(out + "\n")
    if failed:
        raise RuntimeError("libwgf.so: compilation failed")
    objs = [os.path.join(OBJ, f + ".o") for f in sources]
    if jobs or not os.path.exists(LIB):
        # linked under another name and moved into place, so that the library is never seen half written
        tmp = LIB + ".tmp"
        cmd = [NVCC, "-shared", "-o", tmp] + objs + ARCH + ["-cudart", "static", "-ldl", "-lpthread", "-Xlinker",
                                                             "--version-script=" + os.path.join(CSRC, "exports.map")]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("libwgf.so: link failed\n" + r.stdout + r.stderr)
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
