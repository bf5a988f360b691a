"""Compiles the C++ drop-in programs of this folder against the reference's
unchanged dnnl.hpp and links them with the in-tree libdnnl.so.3.  The
executables go beside the library (onednn_b200/lib/, not under version control)
so that they travel with it to a GPU machine that has no reference checkout."""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_INC = os.path.join(os.environ.get("ONEDNN_REFERENCE_DIR", "/root/reference"), "include")
GEN_INC = os.path.join(ROOT, "oracle", "_ref", "include")
LIBDIR = os.path.join(ROOT, "onednn_b200", "lib")


def exe_path(name):
    return os.path.join(LIBDIR, "dropin_" + name)


def available():
    return os.path.exists(os.path.join(REF_INC, "oneapi", "dnnl", "dnnl.hpp")) \
        and os.path.exists(os.path.join(GEN_INC, "oneapi", "dnnl", "dnnl_config.h")) \
        and os.path.exists(os.path.join(LIBDIR, "libdnnl.so.3"))


def build(name="exec_int8"):
    """Returns the executable's path, or None where the reference headers are absent."""
    if not available():
        return exe_path(name) if os.path.exists(exe_path(name)) else None
    src, out = os.path.join(HERE, name + ".cpp"), exe_path(name)
    lib = os.path.join(LIBDIR, "libdnnl.so.3")
    if os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(src), os.path.getmtime(lib)):
        return out
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    subprocess.check_call([gxx, "-std=c++17", "-O1", src, "-I" + REF_INC, "-I" + GEN_INC, "-L" + LIBDIR, "-ldnnl",
                           "-Wl,-rpath,$ORIGIN", "-o", out])
    return out


if __name__ == "__main__":
    print(build())
