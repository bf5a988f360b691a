"""Drop-in check on the host: a C++ program written against the reference's
unchanged dnnl.hpp compiles, links against this library and gets the CUDA
implementations from the primitive descriptors (device-less engine, nothing
executes).  Needs the reference's headers; skipped where they are absent."""
import os
import shutil
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
from oracle.refdir import reference_dir  # noqa: E402

REF_INC = os.path.join(reference_dir() or "/nonexistent", "include")
# dnnl_config.h, dnnl_version.h, dnnl_version_hash.h as this library's build writes them
GEN_INC = os.path.join(ROOT, "onednn_b200", "lib", "include")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_INC, "oneapi", "dnnl", "dnnl.hpp")),
                    reason="reference headers not present")
def test_unchanged_dnnl_hpp_program_builds_and_dispatches(tmp_path):
    from onednn_b200 import api
    if not os.path.exists(os.path.join(GEN_INC, "oneapi", "dnnl", "dnnl_config.h")):
        pytest.skip("generated dnnl_config.h not built (python -m onednn_b200.build)")
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    libdir = os.path.dirname(api.lib_path())
    exe = str(tmp_path / "probe")
    cmd = [gxx, "-std=c++17", "-O1", os.path.join(HERE, "dropin", "probe.cpp"), "-I" + REF_INC, "-I" + GEN_INC,
           "-L" + libdir, "-ldnnl", "-Wl,-rpath," + libdir, "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    env = dict(os.environ, DNNL_B200_NO_DEVICE="1")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60, env=env)
    assert r.returncode == 0, (r.stdout, r.stderr)
    out = dict(line.split(" ", 1) for line in r.stdout.strip().splitlines())
    assert out["int8_zp"] == "cuda:tcgen05:int8"
    assert out["fp8"] == "cuda:tcgen05:fp8"
    assert out["int4"] == "cuda:tcgen05:woq4"
    assert out["int4_last"] == "cuda:ref:any"
    assert out["int8_postops"] == "cuda:tcgen05:int8"
    assert out["grouped"] == "cuda:tcgen05:grouped"


@pytest.mark.gpu
def test_dnnl_hpp_program_executes_on_the_gpu():
    """engine / stream / memory (map, unmap) / attr / primitive_desc / execute / wait through dnnl.hpp,
    checked inside the program against a scalar loop: s32 bit-exact, f32 within 1e-5."""
    import sys
    sys.path.insert(0, os.path.join(HERE, "dropin"))
    import build_dropin
    exe = build_dropin.build("exec_int8")
    if exe is None:
        pytest.skip("drop-in executable not built (reference headers absent at build time)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.stdout, r.stderr)
    assert "s32 cuda:tcgen05:int8 ok" in r.stdout and "f32 cuda:tcgen05:int8 ok" in r.stdout, r.stdout
    assert "reorder cuda:ref:reorder ok" in r.stdout, r.stdout


# The reference's own example programs (compiled unchanged by build_dropin.build_reference_examples),
# run with `gpu` as their engine argument.  matmul_with_weight_only_quantization returns before doing
# anything on a non-CPU engine (its own main), so it proves linking only; inference_int8_matmul uses
# DNNL_RUNTIME_DIM_VAL for M.
@pytest.mark.gpu
@pytest.mark.parametrize("name", ["ref_example_matmul_grouped", "ref_example_matmul_f8_quantization",
                                  "ref_example_inference_int8_matmul", "ref_example_matmul_woq"])
def test_reference_example_passes_on_the_gpu(name):
    sys.path.insert(0, os.path.join(HERE, "dropin"))
    import build_dropin
    exe = build_dropin.build_reference_examples().get(name)
    if exe is None:
        pytest.skip("example not built (no oneDNN checkout at build time)")
    r = subprocess.run([exe, "gpu"], capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    if name != "ref_example_matmul_woq":
        assert "Example passed on GPU." in r.stdout, r.stdout[-2000:]
