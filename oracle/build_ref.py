"""Build recipe for the reference's own CUDA extension (TEST INFRASTRUCTURE, not product code).

Compiles the reference project's three extension sources
(opentad/models/bricks/2d_sparse_v3_bind.cpp, 2d_sparse_v3.cu, implicit_gemm_v2.cu;
the same list as the reference's setup.py:10-14) for sm_100a, straight from the
reference checkout, into ``oracle/_ref/``, and byte-compiles the reference's Python wrapper
(opentad/models/bricks/sparse_conv_layer.py) next to it.  Nothing is copied into this
repository: only the built shared object and the compiled bytecode file land in ``oracle/_ref/``
(git-ignored).

The result is used only by tests and by the benchmark's reference legs, as the
"reference CUDA path" checker / baseline.  The product never imports it.

Usage:  python oracle/build_ref.py --reference /path/to/reference     (or SVTAD_REFERENCE_ROOT)
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "opentad_sparse_ops_ref"
WRAPPER_PYC = os.path.join(OUT, "ref_sparse_conv_layer.bytecode")


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
    build_wrapper(reference_root)
    return built_path()


def build_wrapper(reference_root):
    """Byte-compiles the reference's ``sparse_conv_layer.py`` (its SparseConv2d / SparseConv2dFunction) into
    ``oracle/_ref/``: the compiled module is what the "untouched reference wrapper on top of this library" test
    loads on a machine that has no reference checkout."""
    import py_compile
    src = os.path.join(reference_root, "opentad", "models", "bricks", "sparse_conv_layer.py")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(OUT, exist_ok=True)
    py_compile.compile(src, cfile=WRAPPER_PYC, doraise=True)
    return WRAPPER_PYC


def load_wrapper(sparse_ops_module):
    """Executes the compiled reference wrapper with ``sparse_ops_module`` answering its
    ``import opentad_sparse_ops``; returns the module object, or None when it has not been built."""
    if not os.path.exists(WRAPPER_PYC):
        return None
    import importlib.machinery
    import importlib.util
    saved = sys.modules.get("opentad_sparse_ops")
    sys.modules["opentad_sparse_ops"] = sparse_ops_module
    try:
        loader = importlib.machinery.SourcelessFileLoader("ref_sparse_conv_layer", WRAPPER_PYC)
        spec = importlib.util.spec_from_loader("ref_sparse_conv_layer", loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
    finally:
        if saved is None:
            sys.modules.pop("opentad_sparse_ops", None)
        else:
            sys.modules["opentad_sparse_ops"] = saved
    return mod


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
    ap.add_argument("--reference", default=os.environ.get("SVTAD_REFERENCE_ROOT"),
                    help="root of the reference checkout (default: $SVTAD_REFERENCE_ROOT)")
    ap.add_argument("-v", action="store_true")
    a = ap.parse_args()
    if not a.reference:
        ap.error("give --reference or set SVTAD_REFERENCE_ROOT")
    if not os.path.isdir(a.reference):
        print("reference checkout not found; nothing built", file=sys.stderr)
        sys.exit(0)
    print(build(a.reference, a.v))
