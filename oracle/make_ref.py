"""Builds the reference's own self-contained CUDA extensions for sm_100 into oracle/_ref/ (test infrastructure).

    python oracle/make_ref.py [--reference /path/to/tailquant-kernel] [--force]

The only executable pieces of the reference are its `load_inline` kernels; two of them cover stages of the split
linear path end to end and need nothing outside the reference tree:

    tools/fused_threshold_topr_pack_ext_v57.py   threshold_topr_pack   (select + scales + INT4 pack, fp16 input)
    tools/fused_sparse_epilogue_ext_v58.py       scale_sparse_epilogue_quad / _oct   (dequant + INT4 tail correction)

This script imports those two files where they lie and calls THEIR loader functions unchanged (their sources, their
compiler flags, --use_fast_math included), with TORCH_CUDA_ARCH_LIST=10.0 -- the loaders honour that variable, and
nvcc cross-compiles without a GPU.  The build happens in a temporary directory; only the two resulting shared
objects are copied to oracle/_ref/, which is not tracked (no reference source enters the repository).  The GPU test
tests/test_reference_kernels.py loads them as an independent checker of the reference-compatible (T4) entry points
and skips itself when they are absent.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# reference file -> (loader function in it, extension name it builds)
TARGETS = {
    "tools/fused_threshold_topr_pack_ext_v57.py": ("load_threshold_topr_pack_ext", "threshold_topr_pack_v57_ext"),
    "tools/fused_sparse_epilogue_ext_v58.py": ("load_fused_sparse_epilogue_ext", "fused_sparse_epilogue_v58_ext"),
}


def built() -> bool:
    return all(os.path.exists(os.path.join(OUT, name + ".so")) for _, name in TARGETS.values())


def build(reference: str, force: bool = False) -> bool:
    """Returns True when oracle/_ref/ holds both extensions afterwards."""
    if built() and not force:
        return True
    if not os.path.isdir(os.path.join(reference, "tools")):
        return False
    os.makedirs(OUT, exist_ok=True)
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    with tempfile.TemporaryDirectory(prefix="tq_ref_build_") as tmp:
        os.environ["TORCH_EXTENSIONS_DIR"] = tmp
        for rel, (loader, name) in TARGETS.items():
            spec = importlib.util.spec_from_file_location("_ref_" + name, os.path.join(reference, rel))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            getattr(mod, loader)(verbose=False)  # the reference's own loader: builds (and imports) the extension
            so = os.path.join(tmp, name, name + ".so")
            if not os.path.exists(so):
                raise RuntimeError(f"{name}: the build produced no {so}")
            shutil.copyfile(so, os.path.join(OUT, name + ".so"))
    return built()


def load(name: str):
    """Imports one of the built extensions from oracle/_ref/ (None when it is not there)."""
    path = os.path.join(OUT, name + ".so")
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    ok = build(a.reference, a.force)
    print("oracle/_ref:", "built" if ok else "reference tree not found, nothing built")
    sys.exit(0 if ok else 1)
