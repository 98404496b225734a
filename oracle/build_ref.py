#!/usr/bin/env python3
"""Compiles the reference's own native module (torchbiggraph/util.cpp: randperm, reverse_permutation,
shuffle, sub_bucket) from the sources where they lie in a PyTorch-BigGraph checkout, into oracle/_ref/.

    python oracle/build_ref.py --reference /path/to/PyTorch-BigGraph

Test infrastructure only: the compiled module pins oracle/pbg_edges.py (tests/golden/make_edges_golden.py
records its outputs); nothing of the product loads it.  No reference source is copied: the compiler reads
util.cpp in place and writes objects and the .so under oracle/_ref/ (git-ignored).  The module name must be
`_C` (PYBIND11_MODULE(_C, m), util.cpp:425)."""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build(reference: str, verbose: bool = False):
    from torch.utils.cpp_extension import load
    src = os.path.join(reference, "torchbiggraph", "util.cpp")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(OUT, exist_ok=True)
    return load(name="_C", sources=[src], build_directory=OUT, extra_cflags=["-O2"], verbose=verbose)


def load_built():
    """The module built earlier, or None."""
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    path = os.path.join(OUT, "_C.so")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location("_C", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    m = build(args.reference, verbose=True)
    print("built", os.path.join(OUT, "_C.so"), [n for n in dir(m) if not n.startswith("_")])
