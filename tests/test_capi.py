"""The C-ABI library loads without a GPU and exports every symbol include/natten_b200.h declares;
argument validation that happens before any CUDA call returns the documented codes."""
import ctypes
import os
import re
import shutil
import subprocess

import pytest

import natten_b200._lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "natten_b200.h")).read()
    return sorted(set(re.findall(r"B200NA_API\s+[\w\s\*]+?\b(b200na_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    declared = _declared_symbols()
    assert len(declared) >= 9
    lib = ctypes.CDLL(L.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert sorted(L.SYMBOLS) == declared


@pytest.mark.parametrize("compiler,flags", [("gcc", ["-std=c99", "-x", "c"]),
                                            ("g++", ["-std=c++11", "-x", "c++"])])
def test_header_is_plain_c_and_cxx(tmp_path, compiler, flags):
    """The boundary is a C ABI: the header must compile on its own as C99 and as C++ (no torch or
    CUDA headers, plain pointers and sizes)."""
    if shutil.which(compiler) is None:
        pytest.skip(f"{compiler} not installed")
    src = tmp_path / "use_header.c"
    src.write_text('#include "natten_b200.h"\nint main(void) { return b200na_version() < 0; }\n')
    subprocess.run([compiler, *flags, "-Wall", "-Wextra", "-Werror", "-pedantic",
                    "-I", os.path.join(ROOT, "include"), "-fsyntax-only", str(src)], check=True)


def test_version_and_strerror():
    assert L.lib.b200na_version() >= 100
    assert L.strerror(0) == "ok"
    for code in (-1, -2, -3, -4, -5, -6, -99):
        assert len(L.strerror(code)) > 0


def test_tokperm_rejects_bad_arguments_before_touching_cuda():
    f = L.lib.b200na_token_permute
    one = ctypes.c_void_p(16)
    assert f(None, one, 1, L.ints([4]), L.ints([2]), None, 1, 1, 1, 2, 1, None) == L.ERR_INVALID_ARGUMENT
    assert f(one, one, 4, L.ints([4, 4, 4, 4]), L.ints([2, 2, 2, 2]), None, 1, 1, 1, 2, 1, None) == L.ERR_INVALID_ARGUMENT
    assert f(one, one, 1, L.ints([4]), L.ints([0]), None, 1, 1, 1, 2, 1, None) == L.ERR_INVALID_ARGUMENT
    assert f(one, one, 1, L.ints([4]), L.ints([2]), None, 1, 1, 1, 3, 1, None) == L.ERR_INVALID_ARGUMENT


def _fna(**kw):
    a = dict(q=ctypes.c_void_p(1024), k=ctypes.c_void_p(1024), v=ctypes.c_void_p(1024),
             o=ctypes.c_void_p(1024), lse=None, ndim=1, qkv=[512], qs=[512], kvs=[512], ker=[64],
             st=[1], di=[1], ca=[0], qt=[256], kvt=[128], Bp=1, Hq=1, Hkv=1, D=128, dtype=L.BF16,
             scale=0.1)
    a.update(kw)
    return L.lib.b200na_fna_forward(a["q"], a["k"], a["v"], a["o"], a["lse"], a["ndim"],
                                    L.ints(a["qkv"]), L.ints(a["qs"]), L.ints(a["kvs"]),
                                    L.ints(a["ker"]), L.ints(a["st"]), L.ints(a["di"]),
                                    L.ints(a["ca"]), L.ints(a["qt"]), L.ints(a["kvt"]), a["Bp"],
                                    a["Hq"], a["Hkv"], a["D"], a["dtype"], a["scale"], None)


def test_fna_rejects_bad_arguments_before_touching_cuda():
    assert _fna(q=None) == L.ERR_INVALID_ARGUMENT
    assert _fna(dtype=L.F32) == L.ERR_UNSUPPORTED           # fp32 goes through the CUDA-core entry
    assert _fna(D=100) == L.ERR_UNSUPPORTED                  # head dim must be a multiple of 8
    assert _fna(D=136) == L.ERR_UNSUPPORTED                  # ... and at most 128
    assert _fna(D=96, dtype=L.E4M3) != L.ERR_UNSUPPORTED     # 8-bit floats: multiples of 16
    assert _fna(D=24, dtype=L.E4M3) == L.ERR_UNSUPPORTED
    assert _fna(ker=[1]) == L.ERR_INVALID_ARGUMENT           # kernel_size >= 2
    assert _fna(ker=[600]) == L.ERR_INVALID_ARGUMENT         # kernel * dilation <= extent
    assert _fna(ker=[8], st=[9]) == L.ERR_INVALID_ARGUMENT   # stride <= kernel
    assert _fna(qt=[64]) == L.ERR_INVALID_ARGUMENT           # q tile must hold 256 or 128 tokens
    assert _fna(qt=[512]) == L.ERR_INVALID_ARGUMENT
    assert _fna(kvt=[64]) == L.ERR_INVALID_ARGUMENT          # kv tile must hold 128 tokens
    assert _fna(qs=[500]) == L.ERR_INVALID_ARGUMENT          # tile must divide the padded shape
    assert _fna(qs=[256]) == L.ERR_INVALID_ARGUMENT          # padded shape must cover the layout
    assert _fna(Hq=3, Hkv=2) == L.ERR_INVALID_ARGUMENT
    assert _fna(di=[2], Bp=1) == L.ERR_INVALID_ARGUMENT      # Bp must be a multiple of prod(dilation)
    assert _fna(scale=-1.0) == L.ERR_INVALID_ARGUMENT


def test_merge_and_simt_reject_bad_arguments():
    one = ctypes.c_void_p(16)
    assert L.lib.b200na_merge(None, one, one, one, one, one, 4, 8, L.F32, None) == L.ERR_INVALID_ARGUMENT
    assert L.lib.b200na_merge(one, one, one, one, one, one, 4, 8, 7, None) == L.ERR_INVALID_ARGUMENT
    two = ctypes.c_void_p(32)
    assert L.lib.b200na_merge(one, one, one, one, one, two, 0, 8, L.F32, None) == L.OK
    # the merged LSE must be a buffer of its own (the merged output may overwrite an input)
    assert L.lib.b200na_merge(one, one, one, two, one, one, 4, 8, L.F32, None) == L.ERR_INVALID_ARGUMENT
    assert L.lib.b200na_merge(one, one, one, two, one, two, 4, 8, L.F32, None) == L.ERR_INVALID_ARGUMENT
    f = L.lib.b200na_na_forward_simt
    assert f(one, one, one, one, None, 1, L.ints([8]), L.ints([9]), None, None, None, 1, 1, 1, 8,
             L.F32, 1.0, None, None, 0, None) == L.ERR_INVALID_ARGUMENT
    assert f(one, one, one, one, None, 1, L.ints([8]), L.ints([3]), None, None, None, 1, 1, 1, 512,
             L.F32, 1.0, None, None, 0, None) == L.ERR_UNSUPPORTED
    assert f(one, one, one, one, None, 1, L.ints([8]), L.ints([3]), None, None, None, 1, 1, 1, 8,
             L.F32, 1.0, None, None, 3, None) == L.ERR_INVALID_ARGUMENT  # extra KV without tensors
