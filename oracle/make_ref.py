"""Install the reference's own Python files for this path into oracle/_ref/ (git-ignored).

TEST INFRASTRUCTURE ONLY.  The reference implementation of the selection path is pure Python:
there is nothing to compile, "building" it means placing its unmodified files where the timed CPU
baseline, the reference arm of the benchmark and the tests can import them on a machine that has no
checkout of TransArch.  Nothing under oracle/_ref/ is tracked by git and nothing in the shipped
package imports it.

    python -m oracle.make_ref [/path/to/TransArch]      (default: $TRANSARCH_ROOT, else DEFAULT_ROOT below)

Installed:
  oracle/_ref/opendsa/ops/{topk_select,sparse_mla,flashkl_warmup}.py   <- OpenDSA/opendsa/ops/
      indexer_select_topk, sparse_attend_absorbed_chunked, prepare_ks_ke[_cp]: what the CPU baseline times
  oracle/_ref/opendsa/{modeling,dist}/*.py                             <- OpenDSA/opendsa/{modeling,dist}/
      the attention module that binds the two ops by name (the target of patch_opendsa()) and the
      LightningIndexer module (torch only)
  oracle/_ref/misa_vllm_patch/{misa_ops,block_ops}.py                  <- MISA_preprint/misa_vllm_patch_2stage/
      the TileLang kernels (torch + tilelang only), for a GPU-side comparator where TileLang can run them
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
DEFAULT_ROOT = os.environ.get("TRANSARCH_ROOT", os.path.join(os.sep, "root", "reference"))

FILES = [
    ("OpenDSA/opendsa/ops/topk_select.py", "opendsa/ops/topk_select.py"),
    ("OpenDSA/opendsa/ops/sparse_mla.py", "opendsa/ops/sparse_mla.py"),
    ("OpenDSA/opendsa/ops/flashkl_warmup.py", "opendsa/ops/flashkl_warmup.py"),
    ("OpenDSA/opendsa/ops/__init__.py", "opendsa/ops/__init__.py"),
    ("OpenDSA/opendsa/__init__.py", "opendsa/__init__.py"),
    # the modules that bind the two ops by name at import (what patch_opendsa() rebinds) and the indexer module
    ("OpenDSA/opendsa/modeling/__init__.py", "opendsa/modeling/__init__.py"),
    ("OpenDSA/opendsa/modeling/dsa_attention.py", "opendsa/modeling/dsa_attention.py"),
    ("OpenDSA/opendsa/modeling/indexer.py", "opendsa/modeling/indexer.py"),
    ("OpenDSA/opendsa/modeling/patch_deepseek.py", "opendsa/modeling/patch_deepseek.py"),
    ("OpenDSA/opendsa/modeling/ep_moe.py", "opendsa/modeling/ep_moe.py"),
    ("OpenDSA/opendsa/dist/__init__.py", "opendsa/dist/__init__.py"),
    ("OpenDSA/opendsa/dist/pg.py", "opendsa/dist/pg.py"),
    ("MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py", "misa_vllm_patch/misa_ops.py"),
    ("MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/block_ops.py", "misa_vllm_patch/block_ops.py"),
]


def make_ref(reference_root: str = DEFAULT_ROOT) -> bool:
    """Copy the files; returns False (and leaves oracle/_ref/ as it is) when the checkout is absent."""
    if not os.path.isdir(reference_root):
        return False
    for src, dst in FILES:
        s = os.path.join(reference_root, src)
        d = os.path.join(REF_DIR, dst)
        os.makedirs(os.path.dirname(d), exist_ok=True)
        shutil.copyfile(s, d)
    # the MISA package's own __init__ imports its vLLM model code; the two kernel files need none of it
    with open(os.path.join(REF_DIR, "misa_vllm_patch", "__init__.py"), "w") as f:
        f.write("")
    return True


def reference_ops():
    """The reference's opendsa.ops module from oracle/_ref/, or None when it was never installed."""
    if not os.path.exists(os.path.join(REF_DIR, "opendsa", "ops", "topk_select.py")):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import importlib
    return importlib.import_module("opendsa.ops")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else DEFAULT_ROOT
    ok = make_ref(root)
    print(f"oracle/_ref {'installed from ' + root if ok else 'NOT installed: ' + root + ' is missing'}")
