"""Builds the CPU oracle (test infrastructure, never part of the product).

* ``libqmm_oracle.so``   -- the plain-C restatement in ``qmm_oracle.c``.
* ``_ref/libdnnl_ref.so`` and ``_ref/libref_runner.so`` -- the reference
  library compiled from a oneDNN checkout by ``Makefile.ref`` (g++ on the
  sources where they lie, no CMake) plus the small driver in
  ``ref_runner.cpp``.  Only built when the checkout is present; on a machine
  without it the prebuilt files are used as they are.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
try:
    from .refdir import reference_dir
except ImportError:  # run as a script
    from refdir import reference_dir
REF_DEFAULT = reference_dir() or ""


def _gxx():
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"


def _gcc():
    return "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"


def _newer(target, *sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_port(verbose=False):
    out = os.path.join(HERE, "libqmm_oracle.so")
    src = os.path.join(HERE, "qmm_oracle.c")
    hdr = os.path.join(HERE, "qmm_oracle.h")
    if _newer(out, src, hdr):
        cmd = [_gcc(), "-O2", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared",
               "-Wall", "-o", out, src, "-lm"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return out


def build_ref(ref_dir=REF_DEFAULT, jobs=None, verbose=False):
    """Returns the path of libref_runner.so, or None when neither a checkout
    nor prebuilt files are available."""
    out_dir = os.path.join(HERE, "_ref")
    lib = os.path.join(out_dir, "libdnnl_ref.so")
    runner = os.path.join(out_dir, "libref_runner.so")
    have_src = os.path.isdir(os.path.join(ref_dir, "src", "cpu", "matmul"))
    if not have_src:
        return runner if os.path.exists(runner) else None
    if not os.path.exists(lib):
        jobs = jobs or os.cpu_count() or 4
        cmd = ["make", "-f", os.path.join(HERE, "Makefile.ref"), "REF=" + ref_dir,
               "-j%d" % jobs]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd, stdout=None if verbose else subprocess.DEVNULL)
    rsrc = os.path.join(HERE, "ref_runner.cpp")
    if _newer(runner, rsrc, os.path.join(HERE, "qmm_oracle.h"), lib):
        cmd = [_gxx(), "-std=c++17", "-O2", "-fPIC", "-shared", rsrc,
               "-I" + HERE, "-I" + os.path.join(out_dir, "include"),
               "-I" + os.path.join(ref_dir, "include"),
               "-L" + out_dir, "-ldnnl_ref", "-Wl,-rpath,$ORIGIN",
               "-Wl,-Bsymbolic", "-o", runner]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return runner


if __name__ == "__main__":
    print(build_port(verbose=True))
    print(build_ref(verbose=True))
