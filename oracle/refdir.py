"""Where the oneDNN checkout lies, for the recipes and tests that build or compile against it: the directory named by ONEDNN_REFERENCE_DIR,
else a sibling `reference/` of the repository when there is one.  None: they skip."""
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_dir():
    cands = [os.environ.get("ONEDNN_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "include", "oneapi", "dnnl", "dnnl.h")):
            return c
    return None
