"""ctypes binding of libnatten_b200.so (the C ABI declared in include/natten_b200.h).

The product path has no fallback: if the library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
# NATTEN_B200_LIB overrides the library path (e.g. an instrumented build of the same sources).
LIB_PATH = os.environ.get("NATTEN_B200_LIB") or os.path.join(_HERE, "lib", "libnatten_b200.so")

OK = 0
ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_DEVICE, ERR_KERNEL_TIMEOUT = (
    -1, -2, -3, -4, -5, -6)
ERR_WORKSPACE_LIMIT = -7
STATIC_WORKSPACE_BYTES = 32 * 1024 * 1024
F32, F16, BF16, E4M3, E5M2 = 0, 1, 2, 3, 4

# Every symbol include/natten_b200.h declares.
SYMBOLS = (
    "b200na_strerror", "b200na_version", "b200na_token_permute", "b200na_token_unpermute",
    "b200na_fna_forward", "b200na_fna_forward_sharded", "b200na_na_forward_direct_sharded", "b200na_fna_forward_extra_kv", "b200na_na_forward_direct", "b200na_na_forward_direct_strided",
    "b200na_fmha_forward",
    "b200na_na_forward", "b200na_na_forward_workspace_bytes", "b200na_na_forward_static", "b200na_na_forward_simt", "b200na_na_backward_simt", "b200na_na_backward_direct", "b200na_merge",
    "b200na_device_status",
)


class NattenB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, where: str, text: str):
        super().__init__(f"{where} failed with code {code}: {text}")
        self.code = code


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. natten_b200 has no fallback path: build the CUDA library first "
            "with `python natten_b200/build.py` (needs nvcc; targets sm_100a).")
    lib = ctypes.CDLL(LIB_PATH)
    c_int, c_void_p, c_float, c_i64 = ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_int64
    ip = ctypes.POINTER(c_int)
    lib.b200na_strerror.restype = ctypes.c_char_p
    lib.b200na_strerror.argtypes = [c_int]
    lib.b200na_version.restype = c_int
    lib.b200na_version.argtypes = []
    for name in ("b200na_token_permute", "b200na_token_unpermute"):
        fn = getattr(lib, name)
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_int, ip, ip, ip, c_int, c_int, c_int, c_int, c_int,
                       c_void_p]
    lib.b200na_fna_forward.restype = c_int
    lib.b200na_fna_forward.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                       ip, ip, ip, ip, ip, ip, ip, ip, ip,
                                       c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200na_fna_forward_extra_kv.restype = c_int
    lib.b200na_fna_forward_extra_kv.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_int, c_void_p, c_void_p, c_int,
                                                ip, ip, ip, ip, ip, ip, ip, ip, ip,
                                                c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200na_na_forward_direct.restype = c_int
    lib.b200na_na_forward_direct.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int, c_void_p, c_void_p, c_int,
                                             ip, ip, ip, ip, ip, ip, ip,
                                             c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200na_na_forward_direct_strided.restype = c_int
    lib.b200na_na_forward_direct_strided.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
        ip, ip, ip, ip, ip, ip, ip, c_int, c_int, c_int, c_int, c_int, c_float, c_i64, c_i64, c_i64,
        c_void_p]
    lib.b200na_na_backward_simt.restype = c_int
    lib.b200na_na_backward_simt.argtypes = [c_void_p] * 8 + [c_int] + [c_void_p] * 6 + [
        c_int, ip, ip, ip, ip, ip, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200na_na_backward_direct.restype = c_int
    lib.b200na_na_backward_direct.argtypes = [c_void_p] * 8 + [c_int] + [c_void_p] * 6 + [
        c_int, ip, ip, ip, ip, ip, ip, ip, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200na_na_forward_direct_sharded.restype = c_int
    lib.b200na_na_forward_direct_sharded.argtypes = [c_void_p] * 5 + [c_int, c_void_p, c_void_p,
                                                     c_int] + [ip] * 10 + [
        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    lib.b200na_fna_forward_sharded.restype = c_int
    lib.b200na_fna_forward_sharded.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_int, ip, ip, ip, ip, ip, ip, ip, ip, ip,
                                               c_int, c_int, c_int, c_int, c_int, c_float,
                                               ip, ip, ip, c_void_p]
    lib.b200na_na_forward_workspace_bytes.restype = c_i64
    lib.b200na_na_forward_workspace_bytes.argtypes = [c_int, ip, ip, ip, ip, c_int, c_int, c_int,
                                                      c_int, c_int]
    lib.b200na_na_forward.restype = c_int
    lib.b200na_na_forward.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                      ip, ip, ip, ip, ip, ip, ip, c_int, c_int, c_int, c_int,
                                      c_int, c_float, c_void_p, c_i64, c_void_p]
    lib.b200na_na_forward_static.restype = c_int
    lib.b200na_na_forward_static.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                             ip, ip, ip, ip, ip, ip, ip, c_int, c_int, c_int,
                                             c_int, c_int, c_float, c_void_p]
    lib.b200na_fmha_forward.restype = c_int
    lib.b200na_fmha_forward.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                        c_void_p]
    lib.b200na_na_forward_simt.restype = c_int
    lib.b200na_na_forward_simt.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                           ip, ip, ip, ip, ip, c_int, c_int, c_int, c_int, c_int,
                                           c_float, c_void_p, c_void_p, c_int, c_void_p]
    lib.b200na_merge.restype = c_int
    lib.b200na_merge.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_i64,
                                 c_int, c_int, c_void_p]
    lib.b200na_device_status.restype = c_int
    lib.b200na_device_status.argtypes = [ip]
    return lib


lib = _load()


def ints(x: Optional[Sequence[int]]):
    if x is None:
        return None
    return (ctypes.c_int * len(x))(*[int(v) for v in x])


def strerror(code: int) -> str:
    return lib.b200na_strerror(int(code)).decode()


# Kernel launches issued through this binding since it was last reset (each successful
# kernel-launching C-ABI call counts one); read by the benchmark.
launches = 0


def check(code: int, where: str, kernel_launches: int = 1) -> None:
    global launches
    if code != OK:
        raise NattenB200Error(code, where, strerror(code))
    launches += kernel_launches
    if CHECK_STATUS and kernel_launches > 0:
        raise_on_kernel_timeout(where)


def device_status() -> int:
    """Synchronises the current device and returns (and clears) the kernels' status word: 0, or
    (role << 8 | barrier) of the first bounded wait that expired since the last call."""
    st = ctypes.c_int(0)
    code = lib.b200na_device_status(ctypes.byref(st))
    if code not in (OK, ERR_KERNEL_TIMEOUT):
        check(code, "b200na_device_status", kernel_launches=0)
    return st.value


# NATTEN_B200_CHECK_STATUS=1: every operator call is followed by a device synchronisation and a
# look at the status word, and raises if a bounded wait expired inside a kernel (debugging aid;
# it serialises host and device).
CHECK_STATUS = os.environ.get("NATTEN_B200_CHECK_STATUS", "0") not in ("", "0")


def raise_on_kernel_timeout(where: str) -> None:
    if CHECK_STATUS:
        word = device_status()
        if word != 0:
            raise NattenB200Error(ERR_KERNEL_TIMEOUT, where,
                                  f"{strerror(ERR_KERNEL_TIMEOUT)} (status word {word:#x})")
