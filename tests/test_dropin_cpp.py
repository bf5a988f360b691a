"""Drop-in check on the host: a C++ program written against the reference's
unchanged dnnl.hpp compiles, links against this library and gets the CUDA
implementations from the primitive descriptors (device-less engine, nothing
executes).  Needs the reference's headers; skipped where they are absent."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_INC = os.path.join(os.environ.get("ONEDNN_REFERENCE_DIR", "/root/reference"), "include")
GEN_INC = os.path.join(ROOT, "oracle", "_ref", "include")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_INC, "oneapi", "dnnl", "dnnl.hpp")),
                    reason="reference headers not present")
def test_unchanged_dnnl_hpp_program_builds_and_dispatches(tmp_path):
    from onednn_b200 import api
    if not os.path.exists(os.path.join(GEN_INC, "oneapi", "dnnl", "dnnl_config.h")):
        pytest.skip("generated dnnl_config.h not built (oracle/build_oracle.py)")
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
