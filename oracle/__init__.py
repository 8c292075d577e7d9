"""CPU oracle for the neighborhood-attention forward path (test infrastructure, NOT product code).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py``
may import this package. The product (``natten_b200``) never imports it and has no CPU fallback.

Contents
--------
* ``na_forward`` / ``dense_attention`` / ``merge`` : ctypes front-ends of ``na_oracle.c`` (plain C +
  OpenMP restatement of the reference's mask and naive forward kernel; citations in that file).
* ``token_permute`` / ``token_unpermute`` : numpy index-map restatement of the reference's token
  permutation (src/natten/token_permute/torch_impl.py:40-187, 190-306), bit-exact on any dtype.
* ``window`` helpers used by host-logic tests.

Parity pin: ``tests/golden/*.npz`` hold outputs of the reference package itself (imported from its
source tree, CPU flex path / torch token permute) on seeded inputs; ``tests/test_oracle.py`` checks
every function here against them.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, "_build")
_LIB_PATH = os.path.join(_BUILD, "libna_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile na_oracle.c with gcc (-O3, OpenMP) into oracle/_build/libna_oracle.so."""
    srcs = [os.path.join(_HERE, "na_oracle.c"), os.path.join(_HERE, "na_oracle_body.inc")]
    if not force and os.path.exists(_LIB_PATH):
        if all(os.path.getmtime(_LIB_PATH) >= os.path.getmtime(s) for s in srcs):
            return _LIB_PATH
    os.makedirs(_BUILD, exist_ok=True)
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-std=c11",
           "-o", _LIB_PATH, srcs[0], "-lm"]
    subprocess.run(cmd, check=True, cwd=_HERE)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.na_oracle_forward.restype = ctypes.c_int
        _lib.na_oracle_dense.restype = ctypes.c_int
        _lib.na_oracle_merge.restype = ctypes.c_int
        _lib.na_oracle_backward.restype = ctypes.c_int
        _lib.na_oracle_set_threads.restype = ctypes.c_int
    return _lib


def set_threads(n: int) -> int:
    """Bound the OpenMP threads of the calls that follow; returns the number in effect."""
    return int(_load().na_oracle_set_threads(ctypes.c_int(int(n))))


def _ints(x: Sequence[int]):
    return (ctypes.c_int * len(x))(*[int(v) for v in x])


def _fptr(a: Optional[np.ndarray]):
    if a is None:
        return ctypes.c_void_p(0)
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32c(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _tup(x, n, cast=int):
    if isinstance(x, (list, tuple)):
        assert len(x) == n
        return tuple(cast(v) for v in x)
    return tuple(cast(x) for _ in range(n))


def na_forward(q, k, v, kernel_size, stride=1, dilation=1, is_causal=False, scale=None,
               add_k=None, add_v=None, tok_idx=None, acc64: bool = True
               ) -> Tuple[np.ndarray, np.ndarray]:
    """Neighborhood attention forward on fp32 numpy arrays ``[B, *shape, H, D]``.

    Returns ``(out [B, *shape | n_tok, Hq, Dv], lse [B, *shape | n_tok, Hq])``. With ``tok_idx`` (flat
    row-major token indices) only those query rows are computed and the token axes collapse to one.
    """
    lib = _load()
    q, k, v = _f32c(q), _f32c(k), _f32c(v)
    nd = q.ndim - 3
    shape = q.shape[1:1 + nd]
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    Hkv, Dv = k.shape[-2], v.shape[-1]
    ks, st, di = _tup(kernel_size, nd), _tup(stride, nd), _tup(dilation, nd)
    ca = _tup(is_causal, nd, lambda c: 1 if c else 0)
    scale = float(scale) if scale else float(D) ** -0.5
    n_extra = 0
    if add_k is not None:
        add_k, add_v = _f32c(add_k), _f32c(add_v)
        n_extra = add_k.shape[1]
    if tok_idx is not None:
        tok = np.ascontiguousarray(np.asarray(tok_idx, dtype=np.int64))
        n_tok = tok.shape[0]
        oshape = (B, n_tok)
    else:
        tok, n_tok, oshape = None, math.prod(shape), (B, *shape)
    out = np.empty((*oshape, Hq, Dv), dtype=np.float32)
    lse = np.empty((*oshape, Hq), dtype=np.float32)
    rc = lib.na_oracle_forward(
        _fptr(q), _fptr(k), _fptr(v), _fptr(out), _fptr(lse), ctypes.c_int(nd), _ints(shape),
        ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(D), ctypes.c_int(Dv),
        _ints(ks), _ints(st), _ints(di), _ints(ca), ctypes.c_float(scale), _fptr(add_k),
        _fptr(add_v), ctypes.c_int(n_extra), _fptr(tok), ctypes.c_int64(n_tok),
        ctypes.c_int(1 if acc64 else 0))
    if rc != 0:
        raise ValueError(f"na_oracle_forward rejected its arguments (code {rc})")
    return out, lse


def na_backward(q, k, v, d_out, kernel_size, stride=1, dilation=1, is_causal=False, scale=None,
                add_k=None, add_v=None):
    """Gradients of neighborhood attention w.r.t. q, k, v (and the extra tokens) for the output
    gradient ``d_out [B, *shape, Hq, Dv]``; fp32 numpy in and out, double accumulation inside.

    Returns ``(dq, dk, dv)`` or, with extra tokens, ``(dq, dk, dv, d_add_k, d_add_v)``."""
    lib = _load()
    q, k, v, d_out = _f32c(q), _f32c(k), _f32c(v), _f32c(d_out)
    nd = q.ndim - 3
    shape = q.shape[1:1 + nd]
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    Hkv, Dv = k.shape[-2], v.shape[-1]
    ks, st, di = _tup(kernel_size, nd), _tup(stride, nd), _tup(dilation, nd)
    ca = _tup(is_causal, nd, lambda c: 1 if c else 0)
    scale = float(scale) if scale else float(D) ** -0.5
    n_extra = 0
    dak = dav = None
    if add_k is not None:
        add_k, add_v = _f32c(add_k), _f32c(add_v)
        n_extra = add_k.shape[1]
        dak, dav = np.empty_like(add_k), np.empty_like(add_v)
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    rc = lib.na_oracle_backward(
        _fptr(q), _fptr(k), _fptr(v), _fptr(d_out), _fptr(dq), _fptr(dk), _fptr(dv),
        ctypes.c_int(nd), _ints(shape), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(Hkv),
        ctypes.c_int(D), ctypes.c_int(Dv), _ints(ks), _ints(st), _ints(di), _ints(ca),
        ctypes.c_float(scale), _fptr(add_k), _fptr(add_v), _fptr(dak), _fptr(dav),
        ctypes.c_int(n_extra))
    if rc != 0:
        raise ValueError(f"na_oracle_backward rejected its arguments (code {rc})")
    return (dq, dk, dv, dak, dav) if n_extra else (dq, dk, dv)


def dense_attention(q, k, v, scale=None, is_causal=False) -> Tuple[np.ndarray, np.ndarray]:
    """Dense attention on fp32 ``[B, N, H, D]`` arrays; returns ``(out, lse)``."""
    lib = _load()
    q, k, v = _f32c(q), _f32c(k), _f32c(v)
    B, Nq, Hq, D = q.shape
    Nk, Hkv, Dv = k.shape[1], k.shape[2], v.shape[-1]
    scale = float(scale) if scale else float(D) ** -0.5
    out = np.empty((B, Nq, Hq, Dv), dtype=np.float32)
    lse = np.empty((B, Nq, Hq), dtype=np.float32)
    rc = lib.na_oracle_dense(_fptr(q), _fptr(k), _fptr(v), _fptr(out), _fptr(lse), ctypes.c_int(B),
                             ctypes.c_int(Nq), ctypes.c_int(Nk), ctypes.c_int(Hq),
                             ctypes.c_int(Hkv), ctypes.c_int(D), ctypes.c_int(Dv),
                             ctypes.c_float(scale), ctypes.c_int(1 if is_causal else 0))
    if rc != 0:
        raise ValueError(f"na_oracle_dense rejected its arguments (code {rc})")
    return out, lse


def merge(o0, l0, o1, l1) -> Tuple[np.ndarray, np.ndarray]:
    """Two-way LSE merge in fp32 (src/natten/attn_merge.py:75-98)."""
    lib = _load()
    o0, o1, l0, l1 = _f32c(o0), _f32c(o1), _f32c(l0), _f32c(l1)
    D = o0.shape[-1]
    rows = l0.size
    o = np.empty_like(o0)
    l = np.empty_like(l0)
    lib.na_oracle_merge(_fptr(o0), _fptr(l0), _fptr(o1), _fptr(l1), _fptr(o), _fptr(l),
                        ctypes.c_int64(rows), ctypes.c_int(D))
    return o, l


# ----------------------------------------------------------------------------------------------
# Token permute / unpermute: index-map restatement of src/natten/token_permute/torch_impl.py.
# out[b*G + lin(g), lin(r)*|T| + lin(t), h, :] = in[b, (r_a*T_a + t_a)*d_a + g_a ..., h, :]
# (zero where a source coordinate falls outside the token layout). lin() is colexicographic
# (axis 0 fastest) when flip_tiled_dims, else lexicographic (last axis fastest).
# ----------------------------------------------------------------------------------------------

def rest_shape(shape, tile, dilation):
    """R_a = ceil(ceil(X_a / T_a) / d_a) (src/natten/token_permute/frontend.py:73)."""
    return tuple(-(-(-(-x // t)) // d) for x, t, d in zip(shape, tile, dilation))


def _source_index(shape, tile, dilation, flip):
    """For every permuted slot (group-major) the flat source token index, or -1 for padding."""
    n = len(shape)
    R = rest_shape(shape, tile, dilation)
    order = list(range(n)) if flip else list(range(n))[::-1]  # order[0] = fastest axis

    def axes_grid(ext):
        # decode a linear index over `ext` (fastest = order[0]) into per-axis coords
        size = math.prod(ext)
        idx = np.arange(size, dtype=np.int64)
        coords = [None] * n
        for a in order:
            coords[a] = idx % ext[a]
            idx = idx // ext[a]
        return coords

    g = axes_grid(dilation)
    r = axes_grid(R)
    t = axes_grid(tile)
    G, NR, NT = math.prod(dilation), math.prod(R), math.prod(tile)
    src = np.zeros((G, NR, NT), dtype=np.int64)
    valid = np.ones((G, NR, NT), dtype=bool)
    for a in range(n):
        ca = ((r[a][None, :, None] * tile[a] + t[a][None, None, :]) * dilation[a]
              + g[a][:, None, None])
        valid &= ca < shape[a]
        src = src * shape[a] + np.minimum(ca, shape[a] - 1)
    src[~valid] = -1
    return src.reshape(G, NR * NT)


def token_permute(x: np.ndarray, tile, dilation=None, flip: bool = True) -> np.ndarray:
    """``[B, *shape, H, D]`` -> ``[B * prod(d), prod(R*T), H, D]`` (bit copy, zero padding)."""
    n = x.ndim - 3
    shape = x.shape[1:1 + n]
    dilation = tuple(dilation) if dilation is not None else (1,) * n
    B, H, D = x.shape[0], x.shape[-2], x.shape[-1]
    src = _source_index(shape, tuple(tile), dilation, flip)  # [G, L]
    G, L = src.shape
    flat = x.reshape(B, math.prod(shape), H, D)
    out = np.zeros((B, G, L, H, D), dtype=x.dtype)
    ok = src >= 0
    for gi in range(G):
        out[:, gi, ok[gi]] = flat[:, src[gi, ok[gi]]]
    return out.reshape(B * G, L, H, D)


def token_unpermute(y: np.ndarray, shape, tile, dilation=None, flip: bool = True) -> np.ndarray:
    """Inverse of :func:`token_permute`, dropping padding: ``-> [B, *shape, H, D]``."""
    n = len(shape)
    dilation = tuple(dilation) if dilation is not None else (1,) * n
    src = _source_index(tuple(shape), tuple(tile), dilation, flip)
    G, L = src.shape
    Bp, Ly, H, D = y.shape
    assert Bp % G == 0 and Ly == L
    B = Bp // G
    yv = y.reshape(B, G, L, H, D)
    out = np.zeros((B, math.prod(shape), H, D), dtype=y.dtype)
    ok = src >= 0
    for gi in range(G):
        out[:, src[gi, ok[gi]]] = yv[:, gi, ok[gi]]
    return out.reshape(B, *shape, H, D)
