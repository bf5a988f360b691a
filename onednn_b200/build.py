"""Builds the CUDA library in-tree with nvcc for sm_100a.

    python -m onednn_b200.build [--force] [--verbose]

Output: ``onednn_b200/lib/libdnnl.so.3`` (plus the ``libdnnl.so`` link name a
linker looks for).  Every ``csrc/*.cu`` is one translation unit; objects are
cached under ``onednn_b200/lib/obj`` and rebuilt when a source or header is
newer.
"""
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIBNAME = "libdnnl.so.3"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def nvcc():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def lib_path():
    return os.path.join(LIBDIR, LIBNAME)


def _compile(args):
    src, obj, verbose, extra = args
    cmd = [nvcc()] + NVCC_FLAGS + extra + ["-c", src, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force=False, verbose=False, ptxas_info=False):
    os.makedirs(os.path.join(LIBDIR, "obj"), exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.hpp")) \
        + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    newest_hdr = max(os.path.getmtime(h) for h in headers)
    jobs, objs = [], []
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    for s in sources:
        o = os.path.join(LIBDIR, "obj", os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        stale = force or ptxas_info or not os.path.exists(o) \
            or os.path.getmtime(o) < max(os.path.getmtime(s), newest_hdr)
        if stale:
            jobs.append((s, o, verbose, extra))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, rc, out in ex.map(_compile, jobs):
                if (ptxas_info or rc != 0) and out:
                    print("---- %s\n%s" % (os.path.basename(src), out), flush=True)
                if rc != 0:
                    raise RuntimeError("nvcc failed on %s" % src)
    out = lib_path()
    if jobs or not os.path.exists(out):
        cmd = [nvcc(), "-shared", "-o", out] + objs + ["-Xlinker", "-soname," + LIBNAME,
                                                       "-Xlinker", "--exclude-libs,ALL"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        link = os.path.join(LIBDIR, "libdnnl.so")
        if os.path.lexists(link):
            os.remove(link)
        shutil.copy2(out, link)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                ptxas_info="--ptxas" in sys.argv))
