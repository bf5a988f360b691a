"""Regenerates reorder.npz: the dst of every case in tests/reorder_cases.py as
computed by the UNMODIFIED reference library (oracle/_ref), whatever reorder
implementation it dispatches.  Needs the oneDNN checkout to build oracle/_ref:

    python tests/golden/make_golden_reorder.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from oracle import build_oracle, oracle as O  # noqa: E402
from reorder_cases import CASES  # noqa: E402

if __name__ == "__main__":
    assert build_oracle.build_ref() is not None, "reference checkout not available"
    out = {}
    for name, make in sorted(CASES.items()):
        dst, impl = O.run_ref_reorder(make())
        out[name] = dst.view(np.uint8).reshape(-1).copy()
        out[name + "__impl"] = np.frombuffer(impl.encode(), np.uint8)
        print("%-32s %-20s %d bytes" % (name, impl, out[name].size))
    np.savez_compressed(os.path.join(HERE, "reorder.npz"), **out)
