"""Custom-mask extension point: a user CUDA functor compiled into a private copy of the kernels.

A custom mask is a ``ChillMask`` subclass with two class attributes:

    cuda_functor_header = "/path/to/my_mask.h"   # defines `struct MyMask` in namespace chill
    cuda_functor        = "MyMask"

The header is included at the end of csrc/masks.cuh; the struct must provide the static
members listed at the top of that file (``mask``, ``k_range_for_q``, ``q_range_for_k``,
``k_full_range_for_q``, ``q_full_range_for_k``, ``is_full_block`` and the five constexpr
flags).  ``register_chill_mask`` calls ``build_custom_library`` once per (header, functor)
and registers the mask's ops against the resulting library, in which the functor is mask id
``CHILL_MASK_CUSTOM``.  This is the counterpart of the reference's JIT inlining of a
subclass's Triton functions (chill_attention/chill.py:45-52).
"""
from __future__ import annotations

import hashlib
import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


def _build_module():
    path = os.path.join(os.path.dirname(_HERE), "build.py")
    spec = importlib.util.spec_from_file_location("chill_b200_build", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build_custom_library(header: str, functor: str) -> str:
    header = os.path.abspath(header)
    with open(header, "rb") as f:
        tag = hashlib.sha256(f.read() + functor.encode()).hexdigest()[:16]
    out = os.path.join(_HERE, "_lib", f"libchill_b200_{functor}_{tag}.so")
    return _build_module().build_library(out_path=out, custom_header=header, custom_functor=functor)
