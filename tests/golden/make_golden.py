"""Regenerates golden.npz: the dst of every case in cases.py as computed by
the UNMODIFIED reference library (oracle/_ref, pinned to its scalar ref*
implementation).  Needs the oneDNN checkout to build oracle/_ref:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from oracle import build_oracle, oracle as O  # noqa: E402
from cases import CASES  # noqa: E402

if __name__ == "__main__":
    assert build_oracle.build_ref() is not None, "reference checkout not available"
    out = {}
    for name, make in sorted(CASES.items()):
        p = make()
        dst, impl, _ = O.run_ref(p, pin_ref=True)
        assert impl.startswith("ref"), impl
        out[name] = dst.view(np.uint8).reshape(-1).copy()
        out[name + "__impl"] = np.frombuffer(impl.encode(), np.uint8)
        print("%-16s %-18s %d bytes" % (name, impl, out[name].size))
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
