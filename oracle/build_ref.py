"""Builds the reference's own CUDA extension sources for sm_100 into ``oracle/_ref/`` (test infrastructure).

The sources are compiled where they lie in a checkout of the reference (``--ref``, or the environment variable
``DYLLM_REFERENCE_ROOT``); nothing is copied.  The flags are those of the reference's ``setup.py:46-67`` with
``TORCH_CUDA_ARCH_LIST=10.0`` (``setup.py:12-17``: ``-gencode=arch=compute_100,code=sm_100``), ``-DDYLLM_NO_H100``
(``setup.py:83-87``: no Hopper sources without ``compute_90a``) and without the head_dim-512 files (no
configuration of this package uses that head size).  The result is the reference's ``mma.sync`` kernel
(``dyllm/csrc/attention/attention_ops_kernels_sm80.cu``) and its cache kernels, as they run on a B200.

Two modules are produced, importable with :func:`load_ref`:

* ``dyllm_ref_attention_ops``  (``attention_sparse_varlen``, ``fused_offset_launch``, ``attention_kernel_info``)
* ``dyllm_ref_cache``          (``get_seqs_cuda``, ``get_block_cuda``, ``reset_full_cuda``, ``reset_block_cuda``,
  ``scatter_update_cuda``)

They are used by ``tests/golden/make_ref_golden.py`` to produce golden vectors from the reference's own
kernels and by the kernel-to-beat timing; the product never loads them.

    python oracle/build_ref.py [--ref /path/to/reference]
"""

from __future__ import annotations

import argparse
import glob
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-DNDEBUG", "-D_USE_MATH_DEFINES", "-Wno-deprecated-declarations",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math",
    "-gencode=arch=compute_100,code=sm_100",
]
CXX_FLAGS = ["-O3", "-std=c++17"]


def build(ref_root: str, verbose: bool = False) -> None:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    from torch.utils.cpp_extension import load

    attn = os.path.join(ref_root, "dyllm", "csrc", "attention")
    cache = os.path.join(ref_root, "dyllm", "csrc", "cache")
    jobs = [
        ("dyllm_ref_attention_ops",
         [os.path.join(attn, f) for f in ("attention.cpp", "attention_aux_kernels.cu", "attention_ops_kernels_sm80.cu")],
         [attn], ["-DDYLLM_NO_H100"]),
        ("dyllm_ref_cache", [os.path.join(cache, f) for f in ("cache_kernels.cu", "cache.cpp")], [cache], []),
    ]
    for name, sources, includes, defines in jobs:
        bdir = os.path.join(OUT, "build_" + name)
        os.makedirs(bdir, exist_ok=True)
        load(name=name, sources=sources, extra_include_paths=includes, extra_cflags=CXX_FLAGS + defines,
             extra_cuda_cflags=NVCC_FLAGS + defines, build_directory=bdir, verbose=verbose, is_python_module=False)
        so = os.path.join(bdir, name + ".so")
        dst = os.path.join(OUT, name + ".so")
        if os.path.exists(dst):
            os.unlink(dst)
        os.link(so, dst)
        print("built", dst)


def available() -> bool:
    return all(os.path.exists(os.path.join(OUT, n + ".so")) for n in ("dyllm_ref_attention_ops", "dyllm_ref_cache"))


def load_ref(name: str):
    """Imports ``oracle/_ref/<name>.so`` (a pybind11 torch extension) as a Python module."""
    import torch  # noqa: F401  (the extension links against libtorch)

    path = os.path.join(OUT, name + ".so")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} is missing: run `python oracle/build_ref.py` where the reference is checked out")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("DYLLM_REFERENCE_ROOT", "/root/reference"))
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(a.ref, "dyllm", "csrc")):
        sys.exit(f"no reference checkout at {a.ref}")
    build(a.ref, a.verbose)
    for f in glob.glob(os.path.join(OUT, "*.so")):
        print(f, os.path.getsize(f))
