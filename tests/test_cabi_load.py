"""The C-ABI library builds, loads without a GPU and exports what include/chill_b200.h declares."""
import ctypes

import torch
import os
import re

import pytest

from helpers import ROOT, ensure_built


@pytest.fixture(scope="module")
def lib():
    ensure_built()
    from chill_attention import _cabi

    return _cabi.load_library()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "chill_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(chill_[a-z_0-9]+)\s*\(", text)))


def test_header_exports(lib):
    names = declared_functions()
    assert {"chill_fwd", "chill_bwd", "chill_bwd_delta", "chill_mask_tabulate"} <= set(names)
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    from chill_attention import _cabi

    assert set(_cabi.EXPORTS) <= set(names)


def test_struct_sizes_match_header(lib):
    # sizes computed by hand from the header's field list (LP64)
    from chill_attention import _cabi

    assert ctypes.sizeof(_cabi.MaskDesc) == 8 + 64 + 64
    assert ctypes.sizeof(_cabi.Shape) == 56 + 136
    assert ctypes.sizeof(_cabi.FwdArgs) == 192 + 5 * 8 + 4 * 32 + 24
    assert ctypes.sizeof(_cabi.BwdArgs) == 192 + 10 * 8 + 8 * 32 + 24 + 8 + 8 + 24 + 16 + 24 + 8
    # last: dq_accum, d_lse + strides, dk_part / dv_part, part_strides, part_head / part_tail


def test_host_only_entry_points(lib):
    assert lib.chill_abi_version() == 5
    assert lib.chill_status_string(0) == b"ok"
    assert b"invalid" in lib.chill_status_string(-1)
    # bit0 k full range, bit1 q full range, bit2/3 continuous limits, bit4 guaranteed safe
    assert lib.chill_mask_traits(0) == 31 and lib.chill_mask_traits(1) == 31
    assert lib.chill_mask_traits(2) == 15 and lib.chill_mask_traits(3) == 15 and lib.chill_mask_traits(4) == 31
    assert lib.chill_mask_traits(9) == -2


def test_invalid_arguments_are_rejected_without_a_gpu(lib):
    from chill_attention import _cabi

    a = _cabi.FwdArgs()
    assert lib.chill_fwd(ctypes.byref(a), None) == -1          # all-zero shape
    a.s.B, a.s.H, a.s.H_kv, a.s.Lq, a.s.Lk, a.s.D, a.s.seq_len = 1, 3, 2, 8, 8, 16, 8
    assert lib.chill_fwd(ctypes.byref(a), None) == -1          # H % H_kv != 0
    a.s.H = 4
    a.s.dtype = 7
    assert lib.chill_fwd(ctypes.byref(a), None) == -2          # unknown dtype
    a.s.dtype = 0
    a.s.mask.id = 5
    assert lib.chill_fwd(ctypes.byref(a), None) == -2          # custom functor not in this build
    a.s.mask.id = 1
    assert lib.chill_fwd(ctypes.byref(a), None) == -1          # null pointers
    s = _cabi.Shape()
    s.B, s.H, s.Lq = 2, 3, 5
    assert lib.chill_bwd_scratch_bytes(ctypes.byref(s)) == 2 * 3 * 5 * 4
    s.D, s.dtype = 64, 2
    assert lib.chill_bwd_dq_accum_bytes(ctypes.byref(s)) == 2 * 3 * 128 * 64 * 4  # whole query tiles
    s.dtype = 0
    assert lib.chill_bwd_dq_accum_bytes(ctypes.byref(s)) == 0  # fp32 data never takes that path


def test_missing_library_fails_loudly(tmp_path):
    from chill_attention import _cabi

    with pytest.raises(_cabi.ChillLibraryError):
        _cabi.load_library(str(tmp_path / "nope.so"))


def test_no_cuda_means_error_not_fallback(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    from chill_attention import CausalChillMask, chill_attention

    q = torch.randn(1, 1, 8, 16)
    with pytest.raises(Exception):
        chill_attention(q, q, q, mask=CausalChillMask())


def test_host_pipeline_chunk_schedule():
    """Every (batch row, kv-head group) exactly once, in order, no chunk above the limit."""
    import chill_attention as ca
    from chill_attention.host import chunk_schedule

    mask = ca.CausalChillMask()
    for B, H, Hkv, heads in [(8, 16, 16, 8), (1, 32, 32, 4), (2, 8, 4, 4), (1, 2, 2, 1), (3, 10, 5, 4), (1, 1, 1, 1),
                             (4, 7, 7, 16), (8, 16, 16, None)]:
        q = torch.empty(B, H, 4096, 128, dtype=torch.bfloat16, device="meta")
        k = torch.empty(B, Hkv, 4096, 128, dtype=torch.bfloat16, device="meta")
        sch = chunk_schedule(q, k, mask, heads)
        big = Hkv if heads is None else max(1, min(Hkv, heads // (H // Hkv)))
        covered = sorted((b, g) for b, g0, n in sch for g in range(g0, g0 + n))
        assert covered == [(b, g) for b in range(B) for g in range(Hkv)]
        assert all(1 <= n <= big for _, _, n in sch)
        assert [b for b, _, _ in sch] == sorted(b for b, _, _ in sch)
    # default: about 40 MB of input per chunk -> C2 (4.2 MB per head) gets 8 heads per full-size chunk
    assert max(n for _, _, n in sch) == 8


def test_header_is_plain_c(tmp_path):
    """include/chill_b200.h is what a C / cgo / JNI host includes: it must compile as C99 without CUDA headers, and a
    C program that takes the address of every declared entry point must link against the library."""
    import shutil
    import subprocess

    from chill_attention import _cabi

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    inc = os.path.join(ROOT, "include")
    src = tmp_path / "use_abi.c"
    calls = "\n".join(f"  p[{i}] = (void*)&{name};" for i, name in enumerate(_cabi.EXPORTS))
    src.write_text('#include "chill_b200.h"\n#include <stdio.h>\nint main(void) {\n'
                   f"  void* p[{len(_cabi.EXPORTS)}];\n{calls}\n"
                   '  chill_host_args a = {0};\n  chill_bwd_args b = {0};\n  (void)a; (void)b;\n'
                   '  printf("%d %d\\n", chill_abi_version(), p[0] != 0);\n  return 0;\n}\n')
    exe = tmp_path / "use_abi"
    lib_dir = os.path.dirname(_cabi.DEFAULT_LIB)
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", inc, str(src), "-o", str(exe), "-L", lib_dir,
                        "-l:libchill_b200.so", f"-Wl,-rpath,{lib_dir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.split() == [str(_cabi.ABI_VERSION), "1"], out.stdout + out.stderr
