"""Op layer: one torch custom op per kernel-launching entry of the C ABI.

The reference wraps its native symbols in ``torch.library.custom_op`` with a ``register_fake``
twin so that its operators trace under ``torch.compile`` without graph breaks and allocate their
outputs in one place (src/natten/_libnatten/torch_wrappers.py:98-103, 665-742, 1385-1503). This
module does the same for ``libnatten_b200.so``: every function below takes contiguous CUDA tensors
plus plain ints / lists, allocates the outputs, makes the tensor's device current, passes the
current stream and raises on a non-zero status. Argument validation lives in ``functional.py``.

``NATTEN_B200_DISABLE_TORCH_OPS=1`` turns the registration off (the functions are then called
directly), like the reference's ``NATTEN_DISABLE_TORCH_OPS`` (src/natten/utils/environment.py:67-69).
Autograd formulas are registered for `na_forward` (functional.py) and `fmha_forward`; the other
ops have none, so differentiating through them raises.
"""
import ctypes
import math
import os
from typing import Callable, List, Optional, Tuple

import torch
from torch import Tensor

from . import _lib

USE_TORCH_OPS = os.environ.get("NATTEN_B200_DISABLE_TORCH_OPS", "0") != "1"
NAMESPACE = "natten_b200"
DTYPE_CODE = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16,
              torch.float8_e4m3fn: _lib.E4M3, torch.float8_e5m2: _lib.E5M2}


def _ptr(t: Optional[Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(t: Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _flags(xs) -> List[int]:
    return [1 if x else 0 for x in xs]


def _op(name: str, fake: Callable):
    """Registers ``fn`` as ``natten_b200::<name>`` with ``fake`` as its shape/dtype twin."""
    def wrap(fn):
        if not USE_TORCH_OPS:
            return fn
        op = torch.library.custom_op(f"{NAMESPACE}::{name}", fn, mutates_args=(),
                                     device_types="cuda")
        op.register_fake(fake)
        # the plain function, for callers that already run inside another op's body (a second
        # trip through the dispatcher would only add host time)
        op.raw = fn
        return op
    return wrap


def _rest(shape, tile, dilation):
    return [-(-(-(-x // t)) // d) for x, t, d in zip(shape, tile, dilation)]


# ---- token permute / unpermute ------------------------------------------------------------------

def _token_permute_fake(tensor, layout, tile_shape, dilation, flip_tiled_dims):
    post = [r * t for r, t in zip(_rest(layout, tile_shape, dilation), tile_shape)]
    return tensor.new_empty((tensor.shape[0] * math.prod(dilation), math.prod(post),
                             tensor.shape[-2], tensor.shape[-1]))


@_op("token_permute", _token_permute_fake)
def token_permute(tensor: Tensor, layout: List[int], tile_shape: List[int], dilation: List[int],
                  flip_tiled_dims: bool) -> Tensor:
    """``[B, *X, H, D] -> [B * prod(d), prod(R*T), H, D]`` (never the identity case)."""
    out = _token_permute_fake(tensor, layout, tile_shape, dilation, flip_tiled_dims)
    with torch.cuda.device(tensor.device):
        _lib.check(_lib.lib.b200na_token_permute(
            _ptr(tensor), _ptr(out), len(layout), _lib.ints(layout), _lib.ints(tile_shape),
            _lib.ints(dilation), tensor.shape[0], tensor.shape[-2], tensor.shape[-1],
            tensor.element_size(), 1 if flip_tiled_dims else 0, _stream(tensor)),
            "b200na_token_permute")
    return out


def _token_unpermute_fake(tensor, layout, tile_shape, dilation, flip_tiled_dims):
    return tensor.new_empty((tensor.shape[0] // math.prod(dilation), *layout, tensor.shape[-2],
                             tensor.shape[-1]))


@_op("token_unpermute", _token_unpermute_fake)
def token_unpermute(tensor: Tensor, layout: List[int], tile_shape: List[int], dilation: List[int],
                    flip_tiled_dims: bool) -> Tensor:
    """``[B * prod(d), prod(R*T), H, D] -> [B, *X, H, D]`` (never the identity case)."""
    out = _token_unpermute_fake(tensor, layout, tile_shape, dilation, flip_tiled_dims)
    with torch.cuda.device(tensor.device):
        _lib.check(_lib.lib.b200na_token_unpermute(
            _ptr(tensor), _ptr(out), len(layout), _lib.ints(layout), _lib.ints(tile_shape),
            _lib.ints(dilation), out.shape[0], tensor.shape[-2], tensor.shape[-1],
            tensor.element_size(), 1 if flip_tiled_dims else 0, _stream(tensor)),
            "b200na_token_unpermute")
    return out


# ---- LSE merge -----------------------------------------------------------------------------------

def _merge_fake(out0, lse0, out1, lse1):
    return torch.empty_like(out0), torch.empty_like(lse0)


@_op("merge", _merge_fake)
def merge(out0: Tensor, lse0: Tensor, out1: Tensor, lse1: Tensor) -> Tuple[Tensor, Tensor]:
    """Merges two attention results ``[B, N, H, D]`` / fp32 ``[B, N, H]`` over one query set."""
    out, lse = _merge_fake(out0, lse0, out1, lse1)
    rows = out0.shape[0] * out0.shape[1] * out0.shape[2]
    with torch.cuda.device(out0.device):
        _lib.check(_lib.lib.b200na_merge(_ptr(out0), _ptr(lse0), _ptr(out1), _ptr(lse1), _ptr(out),
                                         _ptr(lse), rows, out0.shape[3], DTYPE_CODE[out0.dtype],
                                         _stream(out0)), "b200na_merge")
    return out, lse


# ---- attention kernels ---------------------------------------------------------------------------

def _attn_fake(query, *_args):
    return (query.new_empty(query.shape),   # contiguous, also for a strided query view
            query.new_empty(query.shape[:-1], dtype=torch.float32))


def token_stride(t: Tensor) -> int:
    """Elements between consecutive tokens of a heads-last ``[B, *X, H, D]`` tensor whose tokens
    (batch entries included) are evenly spaced and whose ``[H, D]`` block is contiguous - true for
    contiguous tensors and for q / k / v sliced out of a fused ``[B, *X, 3, H, D]`` projection.
    -1 when the tensor is not of that form (or not aligned for a tensor map)."""
    H, D = t.shape[-2], t.shape[-1]
    if t.stride(-1) != 1 or t.stride(-2) != D:
        return -1
    ts = t.stride(-3)
    expected = ts
    for i in range(t.dim() - 3, -1, -1):
        if t.shape[i] != 1 and t.stride(i) != expected:
            return -1
        expected *= t.shape[i]
    if ts < H * D or (ts * t.element_size()) % 16 != 0 or t.data_ptr() % 16 != 0:
        return -1
    return int(ts)


def _fmha_fake(query, key, value, is_causal, scale):
    return _attn_fake(query)


@_op("fmha_forward", _fmha_fake)
def fmha_forward(query: Tensor, key: Tensor, value: Tensor, is_causal: bool,
                 scale: float) -> Tuple[Tensor, Tensor]:
    """Dense attention on ``[B, N, H, D]``; fp16/bf16 with head dim 64/128 run on tensor cores,
    everything else on CUDA cores (the library picks the kernel)."""
    out, lse = _attn_fake(query)
    B, Nq, Hq, D = query.shape
    with torch.cuda.device(query.device):
        _lib.check(_lib.lib.b200na_fmha_forward(
            _ptr(query), _ptr(key), _ptr(value), _ptr(out), _ptr(lse), B, Nq, key.shape[1], Hq,
            key.shape[2], D, DTYPE_CODE[query.dtype], float(scale), 1 if is_causal else 0,
            _stream(query)), "b200na_fmha_forward")
    return out, lse


def _na_direct_fake(query, key, value, additional_keys, additional_values, kernel_size, stride,
                    dilation, is_causal, scale, q_tile_shape, kv_tile_shape):
    return _attn_fake(query)


@_op("na_forward_direct", _na_direct_fake)
def na_forward_direct(query: Tensor, key: Tensor, value: Tensor,
                      additional_keys: Optional[Tensor], additional_values: Optional[Tensor],
                      kernel_size: List[int], stride: List[int], dilation: List[int],
                      is_causal: List[bool], scale: float, q_tile_shape: List[int],
                      kv_tile_shape: List[int]) -> Tuple[Tensor, Tensor]:
    """The fused tensor-core kernel on the caller's ``[B, *X, H, D]`` layout (one launch).
    query / key / value may be evenly token-strided views (see `token_stride`): the kernel's
    tensor maps absorb the stride, nothing is copied."""
    strides = [token_stride(t) for t in (query, key, value)]
    if min(strides) < 0:
        query, key, value = (t if s >= 0 else t.contiguous()
                             for t, s in zip((query, key, value), strides))
        strides = [token_stride(t) for t in (query, key, value)]
    out, lse = _attn_fake(query)
    na_dim = query.dim() - 3
    n_extra = additional_keys.shape[1] if additional_keys is not None else 0
    with torch.cuda.device(query.device):
        _lib.check(_lib.lib.b200na_na_forward_direct_strided(
            _ptr(query), _ptr(key), _ptr(value), _ptr(additional_keys), _ptr(additional_values),
            n_extra, _ptr(out), _ptr(lse), na_dim, _lib.ints(query.shape[1:1 + na_dim]),
            _lib.ints(kernel_size), _lib.ints(stride), _lib.ints(dilation),
            _lib.ints(_flags(is_causal)), _lib.ints(q_tile_shape), _lib.ints(kv_tile_shape),
            query.shape[0], query.shape[-2], key.shape[-2], query.shape[-1],
            DTYPE_CODE[query.dtype], float(scale), strides[0], strides[1], strides[2],
            _stream(query)), "b200na_na_forward_direct_strided")
    return out, lse


def _fna_permuted_fake(q_perm, k_perm, v_perm, additional_keys, additional_values, qkv_shape,
                       q_shape, kv_shape, kernel_size, stride, dilation, is_causal, scale,
                       q_tile_shape, kv_tile_shape):
    return _attn_fake(q_perm)


@_op("fna_forward_permuted", _fna_permuted_fake)
def fna_forward_permuted(q_perm: Tensor, k_perm: Tensor, v_perm: Tensor,
                         additional_keys: Optional[Tensor], additional_values: Optional[Tensor],
                         qkv_shape: List[int], q_shape: List[int], kv_shape: List[int],
                         kernel_size: List[int], stride: List[int], dilation: List[int],
                         is_causal: List[bool], scale: float, q_tile_shape: List[int],
                         kv_tile_shape: List[int]) -> Tuple[Tensor, Tensor]:
    """The fused tensor-core kernel on token-permuted ``[B', S, H, D]`` operands; extra key/value
    tokens stay in the original ``[B, M, Hkv, D]`` layout."""
    out, lse = _attn_fake(q_perm)
    bp, _, hq, d = q_perm.shape
    n_extra = additional_keys.shape[1] if additional_keys is not None else 0
    with torch.cuda.device(q_perm.device):
        _lib.check(_lib.lib.b200na_fna_forward_extra_kv(
            _ptr(q_perm), _ptr(k_perm), _ptr(v_perm), _ptr(additional_keys),
            _ptr(additional_values), n_extra, _ptr(out), _ptr(lse), len(qkv_shape),
            _lib.ints(qkv_shape), _lib.ints(q_shape), _lib.ints(kv_shape), _lib.ints(kernel_size),
            _lib.ints(stride), _lib.ints(dilation), _lib.ints(_flags(is_causal)),
            _lib.ints(q_tile_shape), _lib.ints(kv_tile_shape), bp, hq, k_perm.shape[2], d,
            DTYPE_CODE[q_perm.dtype], float(scale), _stream(q_perm)),
            "b200na_fna_forward_extra_kv")
    return out, lse


def _na_simt_fake(query, key, value, additional_keys, additional_values, kernel_size, stride,
                  dilation, is_causal, scale):
    return _attn_fake(query)


@_op("na_forward_simt", _na_simt_fake)
def na_forward_simt(query: Tensor, key: Tensor, value: Tensor, additional_keys: Optional[Tensor],
                    additional_values: Optional[Tensor], kernel_size: List[int], stride: List[int],
                    dilation: List[int], is_causal: List[bool],
                    scale: float) -> Tuple[Tensor, Tensor]:
    """The CUDA-core kernel on the caller's layout: fp32 operands and head dims other than 64/128."""
    out, lse = _attn_fake(query)
    na_dim = query.dim() - 3
    n_extra = additional_keys.shape[1] if additional_keys is not None else 0
    with torch.cuda.device(query.device):
        _lib.check(_lib.lib.b200na_na_forward_simt(
            _ptr(query), _ptr(key), _ptr(value), _ptr(out), _ptr(lse), na_dim,
            _lib.ints(query.shape[1:1 + na_dim]), _lib.ints(kernel_size), _lib.ints(stride),
            _lib.ints(dilation), _lib.ints(_flags(is_causal)), query.shape[0], query.shape[-2],
            key.shape[-2], query.shape[-1], DTYPE_CODE[query.dtype], float(scale),
            _ptr(additional_keys), _ptr(additional_values), n_extra, _stream(query)),
            "b200na_na_forward_simt")
    return out, lse


# ---- backward --------------------------------------------------------------------------------------

def _na_backward_fake(query, key, value, out, d_out, lse, additional_keys, additional_values,
                      kernel_size, stride, dilation, is_causal, scale):
    extra = additional_keys if additional_keys is not None else key.new_empty((0,))
    return (torch.empty_like(query), torch.empty_like(key), torch.empty_like(value),
            torch.empty_like(extra), torch.empty_like(extra))


@_op("na_backward_simt", _na_backward_fake)
def na_backward_simt(query: Tensor, key: Tensor, value: Tensor, out: Tensor, d_out: Tensor,
                     lse: Tensor, additional_keys: Optional[Tensor],
                     additional_values: Optional[Tensor], kernel_size: List[int],
                     stride: List[int], dilation: List[int], is_causal: List[bool],
                     scale: float) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Gradients of neighborhood attention w.r.t. query, key, value and the extra tokens (empty
    tensors when there are none) on the caller's layout, CUDA-core kernels, any supported dtype."""
    dq, dk, dv, dak, dav = _na_backward_fake(query, key, value, out, d_out, lse, additional_keys,
                                             additional_values, kernel_size, stride, dilation,
                                             is_causal, scale)
    na_dim = query.dim() - 3
    n_extra = additional_keys.shape[1] if additional_keys is not None else 0
    delta = torch.empty(query.shape[:-1], dtype=torch.float32, device=query.device)
    with torch.cuda.device(query.device):
        _lib.check(_lib.lib.b200na_na_backward_simt(
            _ptr(query), _ptr(key), _ptr(value), _ptr(out), _ptr(d_out), _ptr(lse),
            _ptr(additional_keys), _ptr(additional_values), n_extra, _ptr(dq), _ptr(dk), _ptr(dv),
            _ptr(dak) if n_extra else None, _ptr(dav) if n_extra else None, _ptr(delta), na_dim,
            _lib.ints(query.shape[1:1 + na_dim]), _lib.ints(kernel_size), _lib.ints(stride),
            _lib.ints(dilation), _lib.ints(_flags(is_causal)), query.shape[0], query.shape[-2],
            key.shape[-2], query.shape[-1], DTYPE_CODE[query.dtype], float(scale),
            _stream(query)), "b200na_na_backward_simt", kernel_launches=4 if n_extra else 3)
    return dq, dk, dv, dak, dav


def _na_backward_direct_fake(query, key, value, out, d_out, lse, additional_keys,
                             additional_values, kernel_size, stride, dilation, is_causal, scale,
                             q_tile_shape, kv_tile_shape):
    extra = additional_keys if additional_keys is not None else key.new_empty((0,))
    return (torch.empty_like(query), torch.empty_like(key), torch.empty_like(value),
            torch.empty_like(extra), torch.empty_like(extra))


@_op("na_backward_direct", _na_backward_direct_fake)
def na_backward_direct(query: Tensor, key: Tensor, value: Tensor, out: Tensor, d_out: Tensor,
                       lse: Tensor, additional_keys: Optional[Tensor],
                       additional_values: Optional[Tensor], kernel_size: List[int],
                       stride: List[int], dilation: List[int], is_causal: List[bool], scale: float,
                       q_tile_shape: List[int], kv_tile_shape: List[int]
                       ) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """dQ, dK, dV and the extra tokens' gradients (empty tensors when there are none) on tensor
    cores (fp16/bf16, head dim 64/128), caller's layout."""
    dq, dk, dv, dak, dav = _na_backward_direct_fake(
        query, key, value, out, d_out, lse, additional_keys, additional_values, kernel_size,
        stride, dilation, is_causal, scale, q_tile_shape, kv_tile_shape)
    na_dim = query.dim() - 3
    n_extra = additional_keys.shape[1] if additional_keys is not None else 0
    delta = torch.empty(query.shape[:-1], dtype=torch.float32, device=query.device)
    with torch.cuda.device(query.device):
        _lib.check(_lib.lib.b200na_na_backward_direct(
            _ptr(query), _ptr(key), _ptr(value), _ptr(out), _ptr(d_out), _ptr(lse),
            _ptr(additional_keys), _ptr(additional_values), n_extra, _ptr(dq), _ptr(dk), _ptr(dv),
            _ptr(dak) if n_extra else None, _ptr(dav) if n_extra else None, _ptr(delta), na_dim,
            _lib.ints(query.shape[1:1 + na_dim]), _lib.ints(kernel_size), _lib.ints(stride),
            _lib.ints(dilation), _lib.ints(_flags(is_causal)), _lib.ints(q_tile_shape),
            _lib.ints(kv_tile_shape), query.shape[0], query.shape[-2], key.shape[-2],
            query.shape[-1], DTYPE_CODE[query.dtype], float(scale), _stream(query)),
            "b200na_na_backward_direct", kernel_launches=4 if n_extra else 3)
    return dq, dk, dv, dak, dav


def _fmha_setup_context(ctx, inputs, output):
    query, key, value, is_causal, scale = inputs
    out, lse = output
    ctx.save_for_backward(query, key, value, out, lse)
    ctx.is_causal, ctx.scale = is_causal, scale


def _fmha_backward(ctx, d_out, d_lse):
    # Self attention is neighborhood attention whose window is the whole sequence, so its
    # gradients come from the same kernels; d_lse is ignored like in the reference's backward
    # (src/natten/backends/blackwell_fna.py:185-318 returns gradients of the output only).
    query, key, value, out, lse = ctx.saved_tensors
    if query.shape[1] != key.shape[1]:
        raise NotImplementedError("natten_b200: backward of attention() needs equal query and "
                                  "key/value lengths.")
    n = query.shape[1]
    dq, dk, dv, _, _ = na_backward_simt(query, key, value, out, d_out.contiguous(), lse, None,
                                        None, [n], [1], [1], [bool(ctx.is_causal)], ctx.scale)
    return dq, dk, dv, None, None


if USE_TORCH_OPS:
    fmha_forward.register_autograd(_fmha_backward, setup_context=_fmha_setup_context)
