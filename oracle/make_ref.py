"""Stage the reference's own Triton GCA file for use as a SECOND oracle on a GPU box.
TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [reference checkout; default: $GCA_REFERENCE, else a `reference` directory beside this repository]

The reference project ships its GCA operator as one Triton file, ``ltriton/gca.py`` (public
callables ``attention`` = ``_attention.apply`` at line 844 and ``gca_kv_cache`` at line 846).  That
file needs a CUDA driver at import time, so it can neither be imported nor run where this
repository is built; a GPU box, on the other hand, has no reference checkout.  This script copies
the file, byte for byte, into ``oracle/_ref/ltriton_gca.py``.  ``oracle/_ref/`` is ignored by git
(no reference source enters the history) but travels with the working tree to the GPU box, where
``tests/test_vs_reference_triton_gpu.py`` imports it and ``bench.py`` times it as the
"reference Triton on this box" anchor.  Nothing in the product imports it.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST_DIR = os.path.join(HERE, "_ref")
DEST = os.path.join(DEST_DIR, "ltriton_gca.py")


def stage(reference_root: str | None = None) -> str | None:
    """Copy ``<reference_root>/ltriton/gca.py`` to ``oracle/_ref/ltriton_gca.py``.
    Returns the destination path, or None when no reference checkout is present."""
    root = reference_root or os.environ.get("GCA_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    src = os.path.join(root, "ltriton", "gca.py")
    if not os.path.isfile(src):
        return None
    os.makedirs(DEST_DIR, exist_ok=True)
    if not os.path.isfile(DEST) or open(src, "rb").read() != open(DEST, "rb").read():
        shutil.copyfile(src, DEST)
    return DEST


def load():
    """Import the staged file as a module (needs a CUDA device: the file queries the Triton driver
    while it is being imported).  Raises FileNotFoundError when it was never staged."""
    import importlib.util
    if not os.path.isfile(DEST):
        raise FileNotFoundError(DEST)
    name = "_reference_ltriton_gca"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, DEST)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    try:
        spec.loader.exec_module(mod)       # runs to the end of the file: the module-global `causal`
    except BaseException:                  # that gca_kv_cache reads (line 859) is set at line 1026
        del sys.modules[name]
        raise
    return mod


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "no reference checkout found: nothing staged")
