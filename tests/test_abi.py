"""The C-ABI library loads without a GPU and exports every entry point that
include/dnnl_b200.h declares; its enum values equal those of the reference
headers when a oneDNN checkout is at hand."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dnnl_b200.h")
sys.path.insert(0, ROOT)
from oracle.refdir import reference_dir  # noqa: E402

REF_INC = os.path.join(reference_dir() or "/nonexistent", "include")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = re.findall(r"\b(dnnl_[a-z0-9_]+)\s*\(", src)
    return sorted(set(n for n in names if not n.endswith("_t")))


def test_library_exports_every_declared_symbol():
    from onednn_b200 import api
    lib = ctypes.CDLL(api.lib_path())
    fns = declared_functions()
    assert len(fns) > 90
    missing = [f for f in fns if not hasattr(lib, f)]
    assert not missing, missing


def test_no_cpu_engine_and_version():
    from onednn_b200 import api
    assert api.engine.get_count(api.engine.kind.cpu) == 0
    with pytest.raises(api.error) as ei:
        api.engine(api.engine.kind.cpu, 0)
    assert ei.value.status == api.invalid_arguments

    class V(ctypes.Structure):
        _fields_ = [("major", ctypes.c_int), ("minor", ctypes.c_int), ("patch", ctypes.c_int),
                    ("hash", ctypes.c_char_p), ("cpu_runtime", ctypes.c_uint), ("gpu_runtime", ctypes.c_uint)]
    v = ctypes.cast(api.lib().dnnl_version(), ctypes.POINTER(V)).contents
    assert (v.major, v.minor) == (3, 14) and v.cpu_runtime == 0 and v.gpu_runtime == 2048


@pytest.mark.skipif(not os.path.isdir(REF_INC), reason="no oneDNN checkout")
def test_enum_values_equal_the_reference_headers(tmp_path):
    """Compiles two tiny programs, one against each header, printing every
    enumerator / macro our header defines, and compares the outputs."""
    src = open(HEADER).read()
    body = src[src.index("#ifndef ONEAPI_DNNL_DNNL_H"):src.index("#endif /* ONEAPI_DNNL_DNNL_H */")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = set(re.findall(r"^\s+(dnnl_[a-z0-9_]+)\s*(?:=|,|\})", body, flags=re.M))
    names |= set(re.findall(r"\{\s*(dnnl_[a-z0-9_]+),", body))
    for m in re.finditer(r"typedef enum \{([^}]*)\}", body):
        names |= set(re.findall(r"(dnnl_[a-z0-9_]+)", m.group(1)))
    names |= set(re.findall(r"#define (DNNL_ARG_[A-Z0-9_]+) ", body))
    names -= {"DNNL_ARG_ATTR_MULTIPLE_POST_OP"}
    names = sorted(names)
    assert len(names) > 120
    prints = "\n".join('printf("%s %%lld\\n", (long long)(%s));' % (n, n) for n in names)
    prog = "#include <stdio.h>\n#include INC\nint main(){%s\nprintf(\"po1 %%d\\n\", DNNL_ARG_ATTR_MULTIPLE_POST_OP(1));" \
           "printf(\"sz %%zu\\n\", sizeof(dnnl_exec_arg_t));return 0;}" % prints
    (tmp_path / "p.c").write_text(prog)
    # the reference's dnnl.h next to the three configured headers this library's build writes
    from onednn_b200 import build as B
    gen = B.write_generated_headers()
    outs = []
    for inc, flags in (('"dnnl_b200.h"', ["-I" + os.path.join(ROOT, "include")]),
                       ('"oneapi/dnnl/dnnl.h"', ["-I" + REF_INC, "-I" + gen])):
        exe = str(tmp_path / ("a%d" % len(outs)))
        subprocess.check_call(["gcc", "-DINC=" + inc, str(tmp_path / "p.c"), "-o", exe] + flags)
        outs.append(subprocess.check_output([exe]).decode())
    assert outs[0] == outs[1]
