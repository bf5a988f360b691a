"""Compiles the C++ drop-in programs of this folder against the reference's
unchanged dnnl.hpp and links them with the in-tree libdnnl.so.3.  The
executables go beside the library (onednn_b200/lib/, not under version control)
so that they travel with it to a GPU machine that has no reference checkout."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle.refdir import reference_dir  # noqa: E402

REF_INC = os.path.join(reference_dir() or "/nonexistent", "include")
# dnnl_config.h, dnnl_version.h, dnnl_version_hash.h as this library's build writes them
GEN_INC = os.path.join(ROOT, "onednn_b200", "lib", "include")
LIBDIR = os.path.join(ROOT, "onednn_b200", "lib")


def exe_path(name):
    return os.path.join(LIBDIR, "dropin_" + name)


def available():
    return os.path.exists(os.path.join(REF_INC, "oneapi", "dnnl", "dnnl.hpp")) \
        and os.path.exists(os.path.join(GEN_INC, "oneapi", "dnnl", "dnnl_config.h")) \
        and os.path.exists(os.path.join(LIBDIR, "libdnnl.so.3"))


# The reference's own example programs, compiled UNCHANGED from the checkout
# where it lies (nothing of them is kept in this repository): file below
# <checkout>/examples -> executable name.  example_utils.hpp includes
# dnnl_ocl.hpp for a GPU runtime, hence the checkout's CL/cl.h on the path.
REFERENCE_EXAMPLES = {
    "matmul_grouped.cpp": "ref_example_matmul_grouped",
    "matmul_f8_quantization.cpp": "ref_example_matmul_f8_quantization",
    "tutorials/matmul/matmul_with_weight_only_quantization.cpp": "ref_example_matmul_woq",
    "tutorials/matmul/inference_int8_matmul.cpp": "ref_example_inference_int8_matmul",
}


def build_reference_examples():
    """Returns {executable name: path} of what is built (or was built earlier and still lies there)."""
    out = {}
    ref = reference_dir()
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    lib = os.path.join(LIBDIR, "libdnnl.so.3")
    for rel, name in REFERENCE_EXAMPLES.items():
        exe = os.path.join(LIBDIR, name)
        src = os.path.join(ref, "examples", rel) if ref else None
        if available() and src and os.path.exists(src):
            if not os.path.exists(exe) or os.path.getmtime(exe) < max(os.path.getmtime(src), os.path.getmtime(lib)):
                subprocess.check_call([gxx, "-std=c++17", "-O1", src, "-I" + REF_INC, "-I" + os.path.join(ref, "examples"),
                                       "-I" + os.path.join(ref, "third_party", "opencl"), "-I" + GEN_INC,
                                       "-L" + LIBDIR, "-ldnnl", "-Wl,-rpath,$ORIGIN", "-o", exe])
        if os.path.exists(exe):
            out[name] = exe
    return out


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
    print(build_reference_examples())
    print(build())
