"""Build the sm_100a shared library in-tree.

`python -m operators_b200.build` compiles every file under csrc/ with nvcc for
compute_100a/sm_100a (cross-compiles without a GPU) and links
operators_b200/lib/libinfiniop.so, the path open_lib() falls back to when
INFINI_ROOT is not set.  `--install DIR` additionally copies the library to
DIR/lib/libinfiniop.so, the layout the reference's wrapper expects under
$INFINI_ROOT (reference operatorspy/liboperators.py:11, xmake.lua:236-238).
"""
import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "lib", "obj")
LIB = os.path.join(OUT_DIR, "libinfiniop.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put /usr/local/cuda/bin on PATH)")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    inc = os.path.join(HERE, "..", "include")
    headers += [os.path.join(inc, f) for f in ("infiniop.h", "infiniop_ext.h")]
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s%s" % (" ".join(cmd), r.stdout, r.stderr))
        return r.stdout + r.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for out in pool.map(run, jobs):
            if verbose and out:
                sys.stderr.write(out)
    if jobs or not os.path.exists(LIB):
        # cudart is linked statically: the library then only needs the driver.
        run([nvcc, "-shared", "-o", LIB] + objs + ["-cudart", "static"])
    return LIB


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--install", metavar="DIR", help="copy the library to DIR/lib (use as INFINI_ROOT)")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true", help="print ptxas register / spill report")
    args = ap.parse_args()
    lib = build(verbose=args.verbose, force=args.force)
    print(lib)
    if args.install:
        dst = os.path.join(args.install, "lib")
        os.makedirs(dst, exist_ok=True)
        shutil.copy2(lib, os.path.join(dst, "libinfiniop.so"))
        print(os.path.join(dst, "libinfiniop.so"))


if __name__ == "__main__":
    main()
