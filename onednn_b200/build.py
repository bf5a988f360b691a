"""Builds the CUDA library in-tree with nvcc for sm_100a.

    python -m onednn_b200.build [--force] [--verbose] [--ptxas]

Extra compiler flags can be given in the environment, e.g. the kernels' timing
switches for a profiling build: ``QMM_NVCC_EXTRA=-DQMM_PROFILE python -m
onednn_b200.build --force`` (a later plain ``--force`` build restores the
shipped library).

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


# The three headers oneDNN's build generates (include/oneapi/dnnl/dnnl_config.h.in,
# dnnl_version.h.in, dnnl_version_hash.h.in).  A program compiled against the
# unchanged dnnl.h / dnnl.hpp needs them next to those headers: pass
# -I<oneDNN>/include -I<this package>/lib/include.  The configuration they
# state is this library's: no CPU engine code is pulled into dnnl.hpp
# (sequential CPU runtime, the smallest the header's checks accept); grouped
# memory descriptors and stream profiling on.  DNNL_GPU_RUNTIME has no value
# for CUDA in the unchanged headers (dnnl_config.h.in:96-105 rejects anything
# but NONE / OCL / SYCL / ZE), and oneDNN's examples use it at compile time to
# pick how GPU memory is filled (examples/example_utils.hpp:247-254, 307-314:
# map_data / unmap_data for OCL and ZE).  This library fills GPU memory through
# map / unmap, so the header states OCL; nothing of OpenCL is called, the
# dnnl_ocl_interop_* functions are exported as stubs that return
# dnnl_unimplemented, and dnnl_version()->gpu_runtime reports
# DNNL_RUNTIME_CUDA.  Programs that include dnnl_ocl.hpp through
# example_utils.hpp need a CL/cl.h on their include path (oneDNN carries one
# under third_party/opencl).
GENERATED_HEADERS = {
    "dnnl_config.h": """#ifndef ONEAPI_DNNL_DNNL_CONFIG_H
#define ONEAPI_DNNL_DNNL_CONFIG_H
/* written by onednn_b200.build for the CUDA (B200) library */
#if defined(__GNUC__) && __GNUC__ >= 4
#define DNNL_HELPER_DLL_IMPORT __attribute__((visibility("default")))
#define DNNL_HELPER_DLL_EXPORT __attribute__((visibility("default")))
#else
#define DNNL_HELPER_DLL_IMPORT
#define DNNL_HELPER_DLL_EXPORT
#endif
#define DNNL_API
#if defined(__GNUC__)
#define DNNL_DEPRECATED __attribute__((deprecated))
#else
#define DNNL_DEPRECATED
#endif
#define DNNL_RUNTIME_NONE 0u
#define DNNL_RUNTIME_SEQ 1u
#define DNNL_RUNTIME_OMP 2u
#define DNNL_RUNTIME_TBB 4u
#define DNNL_RUNTIME_THREADPOOL 8u
#define DNNL_RUNTIME_OCL 256u
#define DNNL_RUNTIME_SYCL 512u
#define DNNL_RUNTIME_DPCPP DNNL_RUNTIME_SYCL
#define DNNL_RUNTIME_ZE 1024u
#define DNNL_VENDOR_NONE 0u
#define DNNL_VENDOR_INTEL 1u
#define DNNL_VENDOR_NVIDIA 2u
#define DNNL_VENDOR_AMD 4u
#define DNNL_VENDOR_GENERIC 8u
#define DNNL_CPU_THREADING_RUNTIME DNNL_RUNTIME_SEQ
#define DNNL_CPU_RUNTIME DNNL_RUNTIME_SEQ
#define DNNL_GPU_RUNTIME DNNL_RUNTIME_OCL
#define DNNL_GPU_VENDOR DNNL_VENDOR_NVIDIA
#define DNNL_EXPERIMENTAL_GROUPED_MEMORY 1
#define DNNL_EXPERIMENTAL_PROFILING
#define BUILD_TRAINING 0
#define BUILD_INFERENCE 1
#define BUILD_PRIMITIVE_ALL 0
#define BUILD_MATMUL 1
#define BUILD_REORDER 1
#endif
""",
    "dnnl_version.h": """#ifndef ONEAPI_DNNL_DNNL_VERSION_H
#define ONEAPI_DNNL_DNNL_VERSION_H
/* the API level this library implements */
#define DNNL_VERSION_MAJOR 3
#define DNNL_VERSION_MINOR 14
#define DNNL_VERSION_PATCH 0
#endif
""",
    "dnnl_version_hash.h": """#ifndef ONEAPI_DNNL_DNNL_VERSION_HASH_H
#define ONEAPI_DNNL_DNNL_VERSION_HASH_H
#define DNNL_VERSION_HASH "b200-native"
#endif
""",
}


def generated_include_dir():
    return os.path.join(LIBDIR, "include")


def write_generated_headers():
    d = os.path.join(generated_include_dir(), "oneapi", "dnnl")
    os.makedirs(d, exist_ok=True)
    for name, text in GENERATED_HEADERS.items():
        path = os.path.join(d, name)
        if not os.path.exists(path) or open(path).read() != text:
            with open(path, "w") as f:
                f.write(text)
    return generated_include_dir()


def _compile(args):
    src, obj, verbose, extra = args
    cmd = [nvcc()] + NVCC_FLAGS + extra + ["-c", src, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force=False, verbose=False, ptxas_info=False):
    os.makedirs(os.path.join(LIBDIR, "obj"), exist_ok=True)
    write_generated_headers()
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.hpp")) \
        + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    newest_hdr = max(os.path.getmtime(h) for h in headers)
    jobs, objs = [], []
    extra = (["-Xptxas", "-v"] if ptxas_info else []) + os.environ.get("QMM_NVCC_EXTRA", "").split()
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
