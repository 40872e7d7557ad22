"""Build recipe for the reference's own CUDA extension (TEST INFRASTRUCTURE, not product code).

Compiles the reference project's three extension sources
(opentad/models/bricks/2d_sparse_v3_bind.cpp, 2d_sparse_v3.cu, implicit_gemm_v2.cu;
the same list as the reference's setup.py:10-14) for sm_100a, straight from the
reference checkout, into ``oracle/_ref/``.  Nothing is copied into this repository:
only the built shared object lands in ``oracle/_ref/`` (git-ignored).

The result is used only by tests and by the benchmark's reference legs, as the
"reference CUDA path" checker / baseline.  The product never imports it.

Usage:  python oracle/build_ref.py [--reference /path/to/reference]
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "opentad_sparse_ops_ref"


def built_path():
    p = os.path.join(OUT, NAME + ".so")
    return p if os.path.exists(p) else None


def build(reference_root, verbose=False):
    bricks = os.path.join(reference_root, "opentad", "models", "bricks")
    sources = [os.path.join(bricks, f) for f in
               ("2d_sparse_v3_bind.cpp", "2d_sparse_v3.cu", "implicit_gemm_v2.cu")]
    for s in sources:
        if not os.path.exists(s):
            raise FileNotFoundError(s)
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    load(name=NAME, sources=sources, build_directory=OUT,
         extra_cflags=["-O3"],
         extra_cuda_cflags=["-O3", "-gencode", "arch=compute_100a,code=sm_100a"],
         verbose=verbose, is_python_module=False)
    return built_path()


def load_built():
    """Import the prebuilt extension (needs a CUDA-capable torch at call time)."""
    p = built_path()
    if p is None:
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location(NAME, p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("-v", action="store_true")
    a = ap.parse_args()
    if not os.path.isdir(a.reference):
        print("reference checkout not found; nothing built", file=sys.stderr)
        sys.exit(0)
    print(build(a.reference, a.v))
