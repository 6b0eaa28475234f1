"""Compile the reference's own extension sources into oracle/_ref/ -- TEST INFRASTRUCTURE ONLY.

The reference path (core/wrapper/*.cu|cpp + core/include/*.cuh + core/helper/*.h) is compiled
from the sources where they lie in the read-only reference checkout; nothing is copied into
this repository and only built objects land in oracle/_ref/ (git-ignored, but shipped to the
GPU machine next to the product's own built library).  The result, ``core_lib.so``, exposes the
reference's five operators (core/wrapper/bind.cpp:78-161):

  csr_to_bcsr_cpu  -- CPU, used to generate tests/golden/ and to pin the layout oracle;
  spmm_tc, spmm_transpose, reindex_bcsr -- CUDA, compared against on the GPU when present;
  sample_all_layers -- built but never called (a different, deterministic top-K algorithm).

Usage: python oracle/build_ref.py [reference_root]
"""
import glob
import os
import sys


def default_reference_root() -> str:
    """GRWS_REFERENCE_ROOT, else a checkout named `reference` next to this repository."""
    here = os.path.dirname(os.path.abspath(__file__))
    return os.environ.get("GRWS_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(here)), "reference")


def build(ref_root: str = None, verbose: bool = False):
    ref_root = ref_root or default_reference_root()
    import torch  # noqa: F401
    from torch.utils import cpp_extension

    here = os.path.dirname(os.path.abspath(__file__))
    out = os.path.join(here, "_ref")
    os.makedirs(out, exist_ok=True)
    wrap = os.path.join(ref_root, "core", "wrapper")
    sources = sorted(glob.glob(os.path.join(wrap, "*.cu")) + glob.glob(os.path.join(wrap, "*.cpp")))
    if not sources:
        raise FileNotFoundError(f"no reference sources under {wrap}")
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    gomp_dir = "/usr/lib/gcc/x86_64-linux-gnu/13"
    ldflags = ["-lgomp"] + ([f"-L{gomp_dir}"] if os.path.isdir(gomp_dir) else [])
    cpp_extension.load(
        name="core_lib",
        sources=sources,
        extra_cflags=["-O3", "-fopenmp"],
        extra_cuda_cflags=["-O3", "-std=c++17", "--expt-relaxed-constexpr", "--expt-extended-lambda"],
        extra_ldflags=ldflags,
        build_directory=out,
        verbose=verbose,
        is_python_module=False,
    )
    return os.path.join(out, "core_lib.so")


def load():
    """Import oracle/_ref/core_lib.so if it was built; returns the module or None."""
    here = os.path.dirname(os.path.abspath(__file__))
    so = os.path.join(here, "_ref", "core_lib.so")
    if not os.path.exists(so):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location("core_lib", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True))
