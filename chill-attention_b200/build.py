"""Build the CUDA library for sm_100a with nvcc (no other toolchain needed).

    python chill-attention_b200/build.py            # -> chill_attention/_lib/libchill_b200.so

Each mask functor's tensor-core kernels are a translation unit of their own
(csrc/tc_inst.cu with -DCHILL_INST_MASK=<functor>), compiled in parallel.
``build_library`` is also what ``chill_attention.custom`` calls to produce a private
library for a user-defined mask functor.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB_DIR = os.path.join(HERE, "chill_attention", "_lib")
BUILTIN_FUNCTORS = ("FullMask", "CausalMask", "SlidingWindowMask", "ChunkwiseMask", "PrefixLMMask")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC,
    # several builds of these sources can live in one process (the main library and custom-mask libraries): keep
    # their function-local statics apart instead of merging them as process-wide unique symbols
    "-Xcompiler", "-fno-gnu-unique",
]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found")
    return nvcc


def _sources_digest(extra=()):
    h = hashlib.sha256()
    names = sorted(os.listdir(CSRC)) + [os.path.join(INCLUDE, "chill_b200.h")]
    for name in names:
        path = name if os.path.isabs(name) else os.path.join(CSRC, name)
        if os.path.isfile(path):
            h.update(name.encode())
            with open(path, "rb") as f:
                h.update(f.read())
    for e in extra:
        h.update(str(e).encode())
    return h.hexdigest()


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_library(out_path=None, custom_header=None, custom_functor=None, verbose=False, force=False):
    """Compile and link the library; returns its path.  Skips work when sources are unchanged."""
    out_path = out_path or os.path.join(LIB_DIR, "libchill_b200.so")
    os.makedirs(os.path.dirname(out_path), exist_ok=True)
    # CHILL_B200_NVCC_FLAGS: extra compiler flags, e.g. "-DCHILL_FWD_POLY_NUM=1 -DCHILL_FWD_POLY_DEN=4"
    defines, functors = os.environ.get("CHILL_B200_NVCC_FLAGS", "").split(), list(BUILTIN_FUNCTORS)
    extra = tuple(defines)
    if custom_header is not None:
        custom_header = os.path.abspath(custom_header)
        with open(custom_header, "rb") as f:
            extra = extra + (custom_functor, hashlib.sha256(f.read()).hexdigest())
        defines = defines + [f'-DCHILL_CUSTOM_MASK_HEADER="{custom_header}"', f"-DCHILL_CUSTOM_MASK={custom_functor}"]
        functors.append(custom_functor)
    digest = _sources_digest(extra)
    stamp = out_path + ".stamp"
    if not force and os.path.exists(out_path) and os.path.exists(stamp) and open(stamp).read() == digest:
        return out_path
    obj_dir = os.path.join(os.path.dirname(out_path), "obj_" + os.path.basename(out_path))
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    jobs = [([nvcc] + NVCC_FLAGS + defines + ["-c", os.path.join(CSRC, src + ".cu"), "-o",
                                               os.path.join(obj_dir, src + ".o")]) for src in ("chill_abi", "host_pipeline")]
    for fn in functors:
        jobs.append([nvcc] + NVCC_FLAGS + defines + [f"-DCHILL_INST_MASK={fn}", "-c", os.path.join(CSRC, "tc_inst.cu"),
                                                      "-o", os.path.join(obj_dir, f"tc_{fn}.o")])
    if verbose:
        jobs = [j[:1] + ["-Xptxas", "-v"] + j[1:] for j in jobs]
    with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        outs = list(ex.map(_run, jobs))
    if verbose:
        print("\n".join(outs))
    objs = [j[j.index("-o") + 1] for j in jobs]
    _run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out_path] + objs)
    with open(stamp, "w") as f:
        f.write(digest)
    shutil.rmtree(obj_dir, ignore_errors=True)  # objects are not needed once linked
    return out_path


if __name__ == "__main__":
    path = build_library(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
