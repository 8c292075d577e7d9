"""Loaders for the fixtures under tests/golden/ (outputs of the reference package itself)."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Exact only for values that are already bf16-representable."""
    return (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


class NaCase:
    def __init__(self, name, meta, z):
        self.name = name
        self.shape = tuple(meta["shape"])
        self.kernel_size = tuple(meta["kernel_size"])
        self.stride = tuple(meta["stride"])
        self.dilation = tuple(meta["dilation"])
        self.is_causal = tuple(bool(c) for c in meta["is_causal"])
        self.n_extra = meta["n_extra"]
        self.bf16_exact = meta["bf16_exact"]

        def load(key):
            a = z[f"{name}/{key}"]
            return bf16_bits_to_f32(a) if a.dtype == np.int16 else a

        self.q, self.k, self.v = load("q"), load("k"), load("v")
        self.add_k = load("add_k") if self.n_extra else None
        self.add_v = load("add_v") if self.n_extra else None
        self.out, self.lse = z[f"{name}/out"], z[f"{name}/lse"]

    def __repr__(self):
        return f"NaCase({self.name})"


_na_cache = None


def na_cases():
    global _na_cache
    if _na_cache is None:
        z = np.load(os.path.join(GOLDEN, "na_cases.npz"))
        meta = json.loads(bytes(z["__meta__"]).decode())
        _na_cache = {n: NaCase(n, m, z) for n, m in meta.items()}
    return _na_cache


def na_case_names():
    z = np.load(os.path.join(GOLDEN, "na_cases.npz"))
    return list(json.loads(bytes(z["__meta__"]).decode()).keys())


def attn_cases():
    z = np.load(os.path.join(GOLDEN, "attn_cases.npz"))
    meta = json.loads(bytes(z["__meta__"]).decode())
    return z, meta


def tokperm_cases():
    with open(os.path.join(GOLDEN, "tokperm_cases.json")) as f:
        return json.load(f)["cases"]


def pattern(n: int, bits: int) -> np.ndarray:
    """The machine-independent input bit pattern the token-permute fixtures were made from."""
    i = np.arange(n, dtype=np.uint64)
    v = (i * np.uint64(40503) + np.uint64(12345)) % np.uint64(1 << bits)
    if bits == 16:
        return v.astype(np.uint16) & np.uint16(0xBFFF)
    return v.astype(np.uint32) & np.uint32(0xBFFFFFFF)
