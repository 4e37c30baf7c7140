"""Builds the reference's own CUDA operators, unmodified, from the reference tree into
oracle/_ref/ (git-ignored; nothing is copied from the reference, the sources are
compiled where they lie).  TEST INFRASTRUCTURE ONLY: tests/test_ref_ops.py loads these
modules on a GPU to pin the CPU oracle and the B200 kernels against the reference's
real outputs.  The recipe is what the reference's operators/*.py do at import time
(torch.utils.cpp_extension.load, e.g. operators/fused_gat.py:9-25), with the arch
fixed to sm_100a and the build directory redirected.

    python -m oracle.build_ref            # build everything that is missing
"""
from __future__ import annotations

import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REFERENCE = os.environ.get("GNN_REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))

# module name (as bound by the reference) -> sources relative to <reference>/src
MODULES = {
    "fused_gat_SM": ["fused_gat/fused_gat_SM.cpp", "fused_gat/fused_gat_SM.cu"],
    "fused_edgeconv": ["fused_edgeconv/fused_edgeconv.cpp", "fused_edgeconv/fused_edgeconv.cu"],
    "gmmconv": ["fused_gmmconv/gmmconv.cc", "fused_gmmconv/gmmconv.cu"],
    "mhsddmm": ["sddmm/mhsddmm.cc", "sddmm/mhsddmm.cu"],
    "mhspmm": ["spmm/mhspmm.cc", "spmm/mhspmm.cu"],
    "mhtranspose": ["csr2csc/mhtranspose.cc", "csr2csc/mhtranspose.cu"],
    "csrtocsc": ["csr2csc/csr2csc.cc", "csr2csc/csr2csc.cu"],
    "edge_softmax": ["edge_softmax/edge_softmax.cc", "edge_softmax/edge_softmax.cu"],
    "u_add_v": ["u_add_v/u_add_v.cpp", "u_add_v/u_add_v.cu"],
}


def reference_present() -> bool:
    return os.path.isdir(os.path.join(REFERENCE, "src"))


def so_path(name: str) -> str:
    return os.path.join(OUT, name, name + ".so")


def available(name: str) -> bool:
    return os.path.exists(so_path(name))


def build_one(name: str, verbose: bool = False) -> str:
    if available(name):
        return so_path(name)
    from torch.utils.cpp_extension import load

    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    bdir = os.path.join(OUT, name)
    os.makedirs(bdir, exist_ok=True)
    srcs = [os.path.join(REFERENCE, "src", s) for s in MODULES[name]]
    load(name=name, sources=srcs, build_directory=bdir, verbose=verbose,
         extra_ldflags=["-lcusparse"] if name == "csrtocsc" else [])
    return so_path(name)


def build_all(verbose: bool = False) -> None:
    for name in MODULES:
        build_one(name, verbose)


def load_module(name: str):
    """Imports a built reference module (needs torch's shared libraries, no GPU)."""
    import torch  # noqa: F401  (libtorch must be loaded first)

    spec = importlib.util.spec_from_file_location(name, so_path(name))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    if not reference_present():
        sys.exit(f"reference tree not found at {REFERENCE}")
    build_all(verbose="-v" in sys.argv)
    print("built:", ", ".join(n for n in MODULES if available(n)))
