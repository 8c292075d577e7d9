"""Host-side operators of the B200 neighborhood-attention forward path.

Mirrors the reference's operator interface for this path — same names, argument meaning and error
behaviour (src/natten/functional.py:74-99, 354-564, 567-1151; src/natten/attn_merge.py:193-289;
src/natten/token_permute/frontend.py:42-137) — and calls the CUDA kernels through the C ABI in
``include/natten_b200.h``. PyTorch is used for device memory and streams only. There is no CPU or
library fallback: tensors must live on a CUDA device of compute capability 10.x.

Autograd: `na1d/na2d/na3d` (extra tokens fused) and self-attention `attention()` are
differentiable - their backward runs the CUDA-core gradient kernels; `merge_attentions` and the
unfused extra-token composition register no formula, so differentiating through them raises.
"""
from __future__ import annotations

import bisect
import ctypes
import functools
import math
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
from torch import Tensor

from . import _lib, ops
from .log import get_logger
from .checks import (CausalArgType, DimensionType, additional_kv_tensor_checks, check_all_args,
                     check_args_against_input, check_tile_shape, fmha_tensor_checks,
                     is_self_attention, na_tensor_checks)

logger = get_logger("natten_b200.functional")

BACKEND_NAME = "b200-fna"
FMHA_BACKEND_NAME = "b200-fmha"
# The reference's names for the backends this library replaces are accepted as aliases, so that
# code written against it (backend="blackwell-fna") runs unchanged.
BACKEND_ALIASES = (None, BACKEND_NAME, "blackwell-fna")
FMHA_BACKEND_ALIASES = (None, FMHA_BACKEND_NAME, "blackwell-fmha")
Q_TILE_SIZE = 256
KV_TILE_SIZE = 128
# A query tile holds 256 tokens (one CTA per SM, two 128-row halves sharing every key/value tile)
# or 128 (two CTAs per SM, each walking the key/value box of its own 128 queries): the smaller
# tile wins when windows are small, because the union of the windows of 128 queries is much
# smaller than that of 256. It pays with twice the key/value tile loads per query row and a
# shallower load ring, so its tile count is charged this factor in the tile-shape choice.
Q_TILE_SIZES = (256, 128)
SMALL_Q_TILE_PENALTY = 1.15
TENSOR_CORE_HEAD_DIMS = (64, 128)

_DTYPE_CODE = ops.DTYPE_CODE
FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)
FP8_HEAD_DIM = 128


def _padded_head_dim(dtype: torch.dtype, head_dim: int) -> int:
    """Head dim the operands are zero-padded to so that the tensor-core kernels take them:
    fp16 / bf16 below 128 go to 64 or 128; everything else is left alone."""
    if dtype in (torch.float16, torch.bfloat16) and head_dim < 128 and head_dim not in (64,):
        return 64 if head_dim < 64 else 128
    # 8-bit floats: the reference's Blackwell kernels take every multiple of 16
    # (csrc/src/blackwell_fna_forward.cu:178-191); the kernel here is built for 128
    if dtype in FP8_DTYPES and head_dim < FP8_HEAD_DIM and head_dim % 16 == 0:
        return FP8_HEAD_DIM
    return head_dim


def _pad_head_dim(t: Tensor, padded_dim: int) -> Tensor:
    """`t` with its last axis zero-padded to `padded_dim` (8-bit floats have no pad kernel in
    torch: zeros + copy)."""
    if t.dtype in FP8_DTYPES:
        out = torch.zeros(t.shape[:-1] + (padded_dim,), dtype=t.dtype, device=t.device)
        out[..., :t.shape[-1]].copy_(t)
        return out
    return torch.nn.functional.pad(t, (0, padded_dim - t.shape[-1]))


def _reads_natively(dtype: torch.dtype, head_dim: int) -> bool:
    """Head dims the forward kernels read without a padded copy: the kernels are built for 64 and
    128 (8-bit floats: 128), and a smaller head dim that keeps rows 16-byte aligned (a multiple of
    8, or 16 for 8-bit floats - the reference's rule, csrc/src/blackwell_fna_forward.cu:123-138,
    178-191) is read through tensor-map boxes that return zeros for the missing channels."""
    if dtype in (torch.float16, torch.bfloat16):
        return 8 <= head_dim <= 128 and head_dim % 8 == 0
    return dtype in FP8_DTYPES and 16 <= head_dim <= FP8_HEAD_DIM and head_dim % 16 == 0


MAX_3D_EXTENT = 65536   # 3-D problems with a longer axis run on the CUDA-core kernel


def _tensor_core_supported(dtype: torch.dtype, head_dim: int) -> bool:
    """Operands the tcgen05 forward kernels take as they are (see `_reads_natively`)."""
    return _reads_natively(dtype, head_dim)


def _wants_grad(*tensors: Optional[Tensor]) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


def _ptr(t: Optional[Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(t: Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda(*tensors: Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "natten_b200 runs on CUDA tensors only (no CPU path); got a tensor on "
                f"{t.device}.")


# ------------------------------------------------------------------------------------------------
# Window arithmetic on the host (same integer semantics as the kernels; reference:
# csrc/include/natten/cuda/reference/mask.hpp:47-89, 220-225). Used for tile-shape selection and
# for the multi-GPU halo computation.
# ------------------------------------------------------------------------------------------------

def window_start(i: int, k: int, s: int, L: int, causal: bool) -> int:
    wl, wr = k // 2, k // 2 + (k % 2 - 1)
    if causal:
        lead = min((i // s) * s + s - 1, L - 1)
        return max(lead - wl - wr, 0)
    lead = min((i // s) * s + s // 2, L - 1)
    return max(lead - wl, 0) + ((L - wr - lead - 1) if lead + wr >= L else 0)


def window_end(i: int, start: int, k: int, L: int, causal: bool) -> int:
    return min(i + 1, L) if causal else start + k


def group_extent(X: int, d: int, g: int) -> int:
    return X // d + (1 - ((g + (d - (X % d))) // d))


def _axis_tile_cost(X: int, k: int, s: int, d: int, causal: bool, tq: int, tkv: int,
                    aligned: bool = False) -> int:
    """KV tiles visited along one axis, summed over that axis' query tiles (largest group).
    `aligned`: the tile walk of a query tile starts at the first key its queries attend (tiles
    gathered from the caller's layout); otherwise key/value tiles lie on a grid from 0."""
    L = group_extent(X, d, 0)
    total = 0
    for q_lo in range(0, L, tq):
        q_hi = q_lo + tq - 1
        st = window_start(q_lo, k, s, L, causal)
        s_hi = window_start(q_hi, k, s, L, causal)
        en = window_end(q_hi, s_hi, k, L, causal)
        total += -(-(en - st) // tkv) if aligned else -(-en // tkv) - st // tkv
    return total


def _axis_inverse_tile_cost(X: int, k: int, s: int, d: int, causal: bool, tq: int,
                            tkv: int) -> int:
    """Query tiles visited along one axis, summed over that axis' key tiles (largest group), by a
    pass whose stationary tile holds keys: the walk of a key tile starts at the first query that
    attends one of its keys and ends after the last one."""
    L = group_extent(X, d, 0)
    starts = [window_start(i, k, s, L, causal) for i in range(L)]
    ends = [window_end(i, starts[i], k, L, causal) for i in range(L)]
    total = 0
    for k_lo in range(0, L, tkv):
        k_hi = min(k_lo + tkv, L) - 1
        first = bisect.bisect_right(ends, k_lo)       # first query whose window ends beyond k_lo
        last = bisect.bisect_right(starts, k_hi)      # first query whose window starts beyond k_hi
        total += max(1, -(-(last - first) // tq))
    return total


def _pow2_compositions(total_log2: int, n: int):
    if n == 1:
        yield (1 << total_log2,)
        return
    for e in range(total_log2 + 1):
        for rest in _pow2_compositions(total_log2 - e, n - 1):
            yield (1 << e,) + rest


def choose_tile_shapes(shape: DimensionType, kernel_size: DimensionType, stride: DimensionType,
                       dilation: DimensionType, is_causal: CausalArgType
                       ) -> Tuple[DimensionType, DimensionType]:
    """Cached front of :func:`_choose_tile_shapes` (normalises its arguments to hashable tuples)."""
    return _choose_tile_shapes(tuple(int(x) for x in shape), tuple(int(x) for x in kernel_size),
                               tuple(int(x) for x in stride), tuple(int(x) for x in dilation),
                               tuple(bool(x) for x in is_causal))


@functools.lru_cache(maxsize=256)
def _choose_tile_shapes(shape: DimensionType, kernel_size: DimensionType, stride: DimensionType,
                        dilation: DimensionType, is_causal: CausalArgType
                        ) -> Tuple[DimensionType, DimensionType]:
    """Picks (q_tile_shape, kv_tile_shape) - 256 or 128 query tokens, 128 key/value tokens - that
    minimise the tile products the kernel has to compute (the reference instead offers a fixed list:
    src/natten/backends/configs/cutlass_blackwell/__init__.py:45-64)."""
    n = len(shape)
    if n == 1:
        return (Q_TILE_SIZE,), (KV_TILE_SIZE,)
    cost: Dict[Tuple[int, int, int, bool], int] = {}
    for a in range(n):
        for eq in range(9):
            for ek in range(8):
                for aligned in (False, True):
                    cost[(a, 1 << eq, 1 << ek, aligned)] = _axis_tile_cost(
                        shape[a], kernel_size[a], stride[a], dilation[a], is_causal[a], 1 << eq,
                        1 << ek, aligned)
    best = None
    for q_log2, weight in ((8, 2.0), (7, SMALL_Q_TILE_PENALTY)):
        # cost in 128-row x 128-key products: a 256-token query tile makes two per key/value tile
        for tq in _pow2_compositions(q_log2, n):
            for tkv in _pow2_compositions(7, n):
                # tiles the kernel can gather from the caller's layout start at the window; tile
                # shapes that need token-permuted copies are tied to the tile grid
                aligned = direct_layout_supported(tq, tkv, dilation)
                c = weight
                for a in range(n):
                    c *= cost[(a, tq[a], tkv[a], aligned)]
                # ties: prefer tiles that are long along the last (memory-contiguous) axis
                key = (c, -tq[-1], -tkv[-1])
                if best is None or key < best[0]:
                    best = (key, tq, tkv)
    assert best is not None
    return best[1], best[2]


# ------------------------------------------------------------------------------------------------
# Token permute / unpermute (reference: src/natten/token_permute/frontend.py:42-137)
# ------------------------------------------------------------------------------------------------

def _rest(shape, tile, dilation):
    return tuple(-(-(-(-x // t)) // d) for x, t, d in zip(shape, tile, dilation))


def token_permute_operation(tensor: Tensor, tile_shape: DimensionType,
                            dilation: Optional[DimensionType] = None,
                            flip_tiled_dims: bool = True
                            ) -> Tuple[Tensor, DimensionType, DimensionType]:
    """``[B, *X, H, D] -> [B * prod(d), prod(R*T), H, D]``; returns (output, X, R*T)."""
    if tensor.dim() not in [4, 5, 6]:
        raise ValueError("Expected 4D, 5D, or 6D tensor (corresponding to NA1D, 2D, 3D), "
                         f"got {tensor.dim()}D input.")
    na_dim = tensor.dim() - 3
    if len(tile_shape) != na_dim:
        raise ValueError(f"Expected {na_dim}D tiler for NA{na_dim}D, got {tile_shape=}.")
    if dilation is not None and len(dilation) != na_dim:
        raise ValueError(f"Expected {na_dim}D dilation for NA{na_dim}D, got {dilation=}.")
    _require_cuda(tensor)
    dil = tuple(dilation) if dilation is not None else tuple(1 for _ in range(na_dim))
    tensor = tensor.contiguous()
    batch, *layout, heads, dim = tensor.shape
    layout = tuple(layout)
    rest = _rest(layout, tile_shape, dil)
    post = tuple(r * t for r, t in zip(rest, tile_shape))
    # 1-D, undilated, already a tile multiple: the permutation is the identity
    if na_dim == 1 and dil[0] == 1 and post[0] == layout[0]:
        return tensor, layout, post
    out = ops.token_permute(tensor, list(layout), list(tile_shape), list(dil),
                            bool(flip_tiled_dims))
    return out, layout, post


def token_unpermute_operation(tensor: Tensor, token_layout_shape: DimensionType,
                              tile_shape: DimensionType,
                              dilation: Optional[DimensionType] = None,
                              flip_tiled_dims: bool = True) -> Tensor:
    """Inverse of :func:`token_permute_operation`: ``[B * prod(d), prod(R*T), H, D] -> [B, *X, H, D]``."""
    if tensor.dim() != 4:
        raise ValueError(f"Expected flattened 4D tensor, got {tensor.dim()}D input.")
    na_dim = len(token_layout_shape)
    if len(tile_shape) != na_dim:
        raise ValueError(f"Expected {na_dim}D tiler for NA{na_dim}D, got {tile_shape=}.")
    if dilation is not None and len(dilation) != na_dim:
        raise ValueError(f"Expected {na_dim}D dilation for NA{na_dim}D, got {dilation=}.")
    _require_cuda(tensor)
    dil = tuple(dilation) if dilation is not None else tuple(1 for _ in range(na_dim))
    layout = tuple(int(x) for x in token_layout_shape)
    tensor = tensor.contiguous()
    bp, seq, heads, dim = tensor.shape
    groups = math.prod(dil)
    rest = _rest(layout, tile_shape, dil)
    post = tuple(r * t for r, t in zip(rest, tile_shape))
    if bp % groups != 0 or seq != math.prod(post):
        raise ValueError(f"Permuted tensor of shape {tuple(tensor.shape)} does not match token "
                         f"layout {layout}, {tile_shape=}, dilation={dil}.")
    batch = bp // groups
    if na_dim == 1 and dil[0] == 1 and post[0] == layout[0]:
        return tensor.reshape(batch, *layout, heads, dim)
    out = ops.token_unpermute(tensor, list(layout), list(tile_shape), list(dil),
                              bool(flip_tiled_dims))
    return out


# ------------------------------------------------------------------------------------------------
# merge_attentions (reference: src/natten/attn_merge.py:193-289)
# ------------------------------------------------------------------------------------------------

def merge_attentions(outputs: List[Tensor], lse_tensors: List[Tensor], torch_compile: bool = True,
                     use_autograd_fix: bool = True) -> Tuple[Tensor, Tensor]:
    """Merges attention outputs that share a query as if their KV sets had been concatenated.

    ``torch_compile`` and ``use_autograd_fix`` are accepted for source compatibility and ignored:
    the merge is one CUDA kernel per pair and this build is forward only."""
    if len(outputs) < 2:
        raise ValueError("`merge_attentions` expects at least two tensors.")
    if len(outputs) != len(lse_tensors):
        raise ValueError("`merge_attentions` expected number of outputs and LSE tensors to match, "
                         f"got {len(outputs)=} != {len(lse_tensors)}.")
    shape = outputs[0].shape
    for i, (output, lse) in enumerate(zip(outputs, lse_tensors)):
        if output.dim() != 4:
            raise ValueError("Output tensors must be rank-4 tensors with (batch, seq, heads, dim), "
                             f"but got output {i} with rank={output.dim()}.")
        if output.shape != shape:
            raise ValueError(f"Output tensors must must match in shape, but got output {i} "
                             f"with shape={output.shape}.")
        if lse.dim() != 3:
            raise ValueError("LSE tensors must be rank-3 tensors with (batch, seq, heads)"
                             f"but got LSE {i} with rank={lse.dim()}.")
        if lse.shape != shape[:3]:
            raise ValueError("LSE tensors must must match outputs in shape except last dim "
                             f"({shape=}), but got LSE {i} with shape={lse.shape}.")
        if output.dtype != outputs[0].dtype:
            raise ValueError("Output tensors must share one dtype.")
    _require_cuda(*outputs, *lse_tensors)
    dtype = outputs[0].dtype
    if dtype not in _DTYPE_CODE or dtype in FP8_DTYPES:
        raise NotImplementedError(f"merge_attentions does not support dtype {dtype}.")
    acc_o = outputs[0].contiguous()
    acc_l = lse_tensors[0].to(torch.float32).contiguous()
    for i in range(1, len(outputs)):
        acc_o, acc_l = ops.merge(acc_o, acc_l, outputs[i].contiguous(),
                                 lse_tensors[i].to(torch.float32).contiguous())
    out, out_l = acc_o, acc_l
    return out, out_l


# ------------------------------------------------------------------------------------------------
# attention (reference: src/natten/functional.py:74-348) — dense, non-varlen
# ------------------------------------------------------------------------------------------------

def attention(query: Tensor, key: Tensor, value: Tensor, is_causal: bool = False,
              scale: Optional[float] = None, seqlens_Q: Optional[Tensor] = None,
              seqlens_KV: Optional[Tensor] = None, cumulative_seqlen_Q: Optional[Tensor] = None,
              cumulative_seqlen_KV: Optional[Tensor] = None, max_seqlen_Q: Optional[int] = None,
              max_seqlen_KV: Optional[int] = None, backend: Optional[str] = None,
              q_tile_size: Optional[int] = None, kv_tile_size: Optional[int] = None,
              backward_q_tile_size: Optional[int] = None,
              backward_kv_tile_size: Optional[int] = None,
              backward_kv_splits: Optional[int] = None, backward_use_pt_reduction: bool = False,
              run_persistent_kernel: bool = True, kernel_schedule: Any = None,
              torch_compile: bool = False, return_lse: bool = False
              ) -> Union[Tensor, Tuple[Tensor, Tensor]]:
    """Dense dot-product attention on heads-last ``[B, N, H, D]`` tensors."""
    fmha_tensor_checks(query, key, value)
    if any(x is not None for x in (seqlens_Q, seqlens_KV, cumulative_seqlen_Q,
                                   cumulative_seqlen_KV, max_seqlen_Q, max_seqlen_KV)):
        raise NotImplementedError("natten_b200.attention does not implement variable-length "
                                  "(varlen) attention.")
    if backend not in FMHA_BACKEND_ALIASES:
        raise NotImplementedError(f"Unrecognized NATTEN FMHA backend {backend}; natten_b200 "
                                  f"provides '{FMHA_BACKEND_NAME}' only.")
    if q_tile_size not in (None, Q_TILE_SIZE) or kv_tile_size not in (None, KV_TILE_SIZE):
        raise ValueError(f"'{FMHA_BACKEND_NAME}' uses q/kv tile sizes {Q_TILE_SIZE}/{KV_TILE_SIZE}.")
    _require_cuda(query, key, value)
    scale = scale or query.shape[-1] ** -0.5
    B, Nq, Hq, D = query.shape
    Nk, Hkv = key.shape[1], key.shape[2]
    if is_causal and Nq != Nk:
        raise NotImplementedError("Causal attention needs equal query and key lengths here.")
    if query.dtype not in _DTYPE_CODE:
        raise NotImplementedError(f"natten_b200.attention does not support dtype {query.dtype}.")
    q, k, v = (t.contiguous() for t in (query, key, value))
    padded_dim = _padded_head_dim(query.dtype, D)   # see neighborhood_attention_generic
    if padded_dim != D and _reads_natively(query.dtype, D) and not _wants_grad(query, key, value):
        padded_dim = D
    if padded_dim != D:
        q, k, v = (_pad_head_dim(t, padded_dim) for t in (q, k, v))
    out, lse = ops.fmha_forward(q, k, v, bool(is_causal), float(scale))
    if padded_dim != D:
        out = out[..., :D].contiguous()
    return (out, lse) if return_lse else out


# ------------------------------------------------------------------------------------------------
# neighborhood attention (reference: src/natten/functional.py:354-564)
# ------------------------------------------------------------------------------------------------

def neighborhood_attention_generic(
        query: Tensor, key: Tensor, value: Tensor, kernel_size: Any, stride: Any = 1,
        dilation: Any = 1, is_causal: Any = False, scale: Optional[float] = None,
        additional_keys: Optional[Tensor] = None, additional_values: Optional[Tensor] = None,
        attention_kwargs: Optional[Dict] = None, backend: Optional[str] = None,
        q_tile_shape: Optional[DimensionType] = None, kv_tile_shape: Optional[DimensionType] = None,
        backward_q_tile_shape: Optional[DimensionType] = None,
        backward_kv_tile_shape: Optional[DimensionType] = None,
        backward_kv_splits: Optional[DimensionType] = None, backward_use_pt_reduction: bool = False,
        run_persistent_kernel: bool = True, kernel_schedule: Any = None,
        torch_compile: bool = False, return_lse: bool = False
) -> Union[Tensor, Tuple[Tensor, Tensor]]:
    na_tensor_checks(query, key, value)
    additional_kv_tensor_checks(query, key, value, additional_keys, additional_values)
    na_dim = query.dim() - 3
    kernel_size, stride, dilation, is_causal = check_all_args(na_dim, kernel_size, stride,
                                                              dilation, is_causal)
    check_args_against_input(query, kernel_size, stride, dilation, is_causal)
    if backend not in BACKEND_ALIASES:
        raise NotImplementedError(f"Unrecognized NATTEN backend {backend}; natten_b200 provides "
                                  f"'{BACKEND_NAME}' only.")
    _require_cuda(query, key, value, additional_keys, additional_values)
    has_extra = additional_keys is not None and additional_values is not None

    # A window that covers the whole layout is plain attention (the reference takes the same
    # shortcut, src/natten/functional.py:423-447). With extra tokens attached the reference
    # concatenates them to K/V first; here that case stays on the neighborhood kernel, which
    # attends the extra tokens in the same softmax without a copy and - unlike dense attention
    # with more keys than queries - has a backward, so the call stays trainable.
    if is_self_attention(query, kernel_size, is_causal, has_extra) and not has_extra:
        query_shape = query.shape
        q = query.flatten(1, na_dim)
        k = key.flatten(1, na_dim)
        v = value.flatten(1, na_dim)
        fmha_kwargs = {kk: vv for kk, vv in (attention_kwargs or {}).items()
                       if kk not in ("unfused_extra_kv", "permuted_layout")}
        out, lse = attention(q, k, v, is_causal=is_causal[0], scale=scale, return_lse=True,
                             **fmha_kwargs)
        out = out.reshape(*query_shape[:-1], value.shape[-1])
        lse = lse.reshape(*query_shape[:-1])
        return (out, lse) if return_lse else out

    scale = scale or query.shape[-1] ** -0.5
    if query.dtype not in _DTYPE_CODE:
        raise NotImplementedError(f"natten_b200 does not support dtype {query.dtype}.")
    if q_tile_shape is not None:
        q_tile_shape = check_tile_shape(na_dim, q_tile_shape, "q_tile_shape", Q_TILE_SIZES)
    if kv_tile_shape is not None:
        kv_tile_shape = check_tile_shape(na_dim, kv_tile_shape, "kv_tile_shape", KV_TILE_SIZE)
    fuse_extra = has_extra and not (attention_kwargs or {}).get("unfused_extra_kv", False)
    want_permuted = bool((attention_kwargs or {}).get("permuted_layout", False))
    # no .contiguous() here: evenly token-strided views (q / k / v sliced out of a fused
    # projection) reach the kernel as they are - its tensor maps absorb the stride; the op makes
    # anything else contiguous itself
    q, k, v = query, key, value
    ak = additional_keys.contiguous() if fuse_extra else None
    av = additional_values.contiguous() if fuse_extra else None
    # fp16 / bf16 with a head dim below 128 that the tensor-core kernels do not take as is (the
    # reference's Blackwell kernels accept every multiple of 8, blackwell_fna_forward.cu:123-138;
    # e.g. 32 in NAT-style models): zero-pad the head dim to 64 or 128. Zeros change neither q.k
    # nor the real columns of P.V, the scale is already fixed, and autograd differentiates through
    # the pad and the slice - far faster than the CUDA-core kernel despite the wasted columns.
    head_dim = query.shape[-1]
    padded_dim = _padded_head_dim(query.dtype, head_dim)
    # Without gradients no copy is needed at all: the kernel reads the narrow rows through
    # tensor-map boxes that fill the missing channels with zeros and writes narrow output rows
    # (three layout axes leave the tensor map no room for a batch axis, so 3-D needs batch 1).
    # The backward kernels are built for the padded head dims only, so a call that will be
    # differentiated keeps the pad / slice pair, which autograd differentiates through.
    if (padded_dim != head_dim and _reads_natively(query.dtype, head_dim)
            and not _wants_grad(query, key, value, additional_keys, additional_values)
            and (na_dim < 3 or query.shape[0] == 1)):
        padded_dim = head_dim
    if padded_dim != head_dim:
        logger.debug("head dim %d zero-padded to %d for the tensor-core kernels", head_dim,
                     padded_dim)
        q, k, v = (_pad_head_dim(t, padded_dim) for t in (q, k, v))
        if fuse_extra:
            ak, av = _pad_head_dim(ak, padded_dim), _pad_head_dim(av, padded_dim)
    if backward_q_tile_shape is not None:
        backward_q_tile_shape = check_tile_shape(na_dim, backward_q_tile_shape,
                                                 "backward_q_tile_shape", BACKWARD_TILE_SIZE)
    if backward_kv_tile_shape is not None:
        backward_kv_tile_shape = check_tile_shape(na_dim, backward_kv_tile_shape,
                                                  "backward_kv_tile_shape", BACKWARD_TILE_SIZE)
    output, lse = na_forward_op(q, k, v, ak, av, list(kernel_size), list(stride), list(dilation),
                                [bool(c) for c in is_causal], float(scale),
                                list(q_tile_shape or ()), list(kv_tile_shape or ()), want_permuted,
                                list(backward_q_tile_shape or ()),
                                list(backward_kv_tile_shape or ()))
    if padded_dim != head_dim:
        output = output[..., :head_dim].contiguous()
    if has_extra and not fuse_extra:
        # the reference's composition: a second (dense) attention over the extra tokens, then
        # an LSE merge (src/natten/functional.py:524-559); kept for comparison
        kwargs = dict(attention_kwargs or {})
        kwargs.pop("unfused_extra_kv", None)
        kwargs.pop("permuted_layout", None)
        kwargs.pop("torch_compile", None)
        add_out, add_lse = attention(query.flatten(1, na_dim), additional_keys, additional_values,
                                     is_causal=False, scale=scale, return_lse=True, **kwargs)
        m_out, m_lse = merge_attentions([output.flatten(1, na_dim), add_out],
                                        [lse.flatten(1, na_dim), add_lse])
        output = m_out.reshape(output.shape)
        lse = m_lse.reshape(output.shape[:-1])
    return (output, lse) if return_lse else output


def _na_forward_fake(query, key, value, additional_keys, additional_values, kernel_size, stride,
                     dilation, is_causal, scale, q_tile_shape, kv_tile_shape, permuted_layout,
                     backward_q_tile_shape, backward_kv_tile_shape):
    return (torch.empty_like(query), query.new_empty(query.shape[:-1], dtype=torch.float32))


@ops._op("na_forward", _na_forward_fake)
def na_forward_op(query: Tensor, key: Tensor, value: Tensor, additional_keys: Optional[Tensor],
                  additional_values: Optional[Tensor], kernel_size: List[int], stride: List[int],
                  dilation: List[int], is_causal: List[bool], scale: float,
                  q_tile_shape: List[int], kv_tile_shape: List[int], permuted_layout: bool,
                  backward_q_tile_shape: List[int],
                  backward_kv_tile_shape: List[int]) -> Tuple[Tensor, Tensor]:
    """Neighborhood attention forward on validated, contiguous ``[B, *X, H, D]`` operands: the
    one node `na1d/na2d/na3d` leave in a torch.compile graph. Everything that depends on concrete
    sizes happens in here, at run time: kernel choice (tensor cores for fp16/bf16 with head dim
    64/128, CUDA cores otherwise), tile shapes (empty lists = choose), and whether the kernel
    can read this layout directly or needs token-permuted copies. The backward tile shapes
    (128 tokens each, empty = choose) only matter when the result is differentiated."""
    na_dim = query.dim() - 3
    shape = tuple(int(x) for x in query.shape[1:1 + na_dim])
    kernel_size, stride, dilation = tuple(kernel_size), tuple(stride), tuple(dilation)
    is_causal = tuple(bool(c) for c in is_causal)
    tensor_core = _tensor_core_supported(query.dtype, query.shape[-1])
    if na_dim == 3 and max(shape) >= MAX_3D_EXTENT and query.dtype not in FP8_DTYPES:
        tensor_core = False     # the 3-D tensor-core kernel keeps window bounds in 16 bits
    if not tensor_core and query.dtype in FP8_DTYPES:
        raise NotImplementedError("natten_b200: 8-bit operands need a head dim that is a multiple "
                                  f"of 16 and at most {FP8_HEAD_DIM}, got {query.shape[-1]}.")
    if not tensor_core:
        # fp32 operands (and other head dims): CUDA-core kernel on the original layout, extra KV
        # tokens fused into the same softmax.
        logger.debug("na%dd %s: CUDA-core kernel (dtype %s, head dim %d), shape %s kernel %s "
                     "stride %s dilation %s causal %s", na_dim, BACKEND_NAME, query.dtype,
                     query.shape[-1], shape, kernel_size, stride, dilation, is_causal)
        query, key, value = query.contiguous(), key.contiguous(), value.contiguous()
        return ops.na_forward_simt(query, key, value, additional_keys, additional_values,
                                   list(kernel_size), list(stride), list(dilation),
                                   list(is_causal), scale)
    if not q_tile_shape or not kv_tile_shape:
        auto_q, auto_kv = choose_tile_shapes(shape, kernel_size, stride, dilation, is_causal)
        q_tile_shape = tuple(q_tile_shape) or auto_q
        kv_tile_shape = tuple(kv_tile_shape) or auto_kv
    q_tile_shape, kv_tile_shape = tuple(q_tile_shape), tuple(kv_tile_shape)
    direct = not permuted_layout and direct_layout_supported(q_tile_shape, kv_tile_shape, dilation)
    if logger.debug_enabled:
        tiles = math.prod(_axis_tile_cost(shape[a], kernel_size[a], stride[a], dilation[a],
                                          is_causal[a], q_tile_shape[a], kv_tile_shape[a], direct)
                          for a in range(na_dim))
        items = math.prod(-(-group_extent(shape[a], dilation[a], 0) // q_tile_shape[a])
                          for a in range(na_dim))
        logger.debug("na%dd %s: tensor-core kernel on %s, dtype %s head dim %d, shape %s kernel "
                     "%s stride %s dilation %s causal %s, q_tile %s kv_tile %s, %.1f kv tiles per "
                     "query tile (+%d extra-token tiles), %d extra tokens", na_dim, BACKEND_NAME,
                     "the caller's layout (one launch)" if direct else "token-permuted copies",
                     query.dtype, query.shape[-1], shape, kernel_size, stride, dilation, is_causal,
                     q_tile_shape, kv_tile_shape, tiles / max(1, items),
                     0 if additional_keys is None else -(-additional_keys.shape[1] // 128),
                     0 if additional_keys is None else additional_keys.shape[1])
    if direct:
        # one kernel on the caller's layout: no permuted copies of Q/K/V/O/LSE at all
        return fna_forward_direct(query, key, value, kernel_size, stride, dilation, is_causal,
                                  scale, q_tile_shape, kv_tile_shape, additional_keys,
                                  additional_values, _inside_op=True)
    return fna_forward_permuted(query.contiguous(), key.contiguous(), value.contiguous(),
                                kernel_size, stride, dilation, is_causal, scale, q_tile_shape,
                                kv_tile_shape, additional_keys, additional_values)


def _na_setup_context(ctx, inputs, output):
    (query, key, value, additional_keys, additional_values, kernel_size, stride, dilation,
     is_causal, scale, _q_tile, _kv_tile, _permuted, bwd_q_tile, bwd_kv_tile) = inputs
    ctx.bwd_tiles = (tuple(bwd_q_tile), tuple(bwd_kv_tile))
    out, lse = output
    ctx.has_extra = additional_keys is not None
    saved = [query, key, value, out, lse]
    if ctx.has_extra:
        saved += [additional_keys, additional_values]
    ctx.save_for_backward(*saved)
    ctx.na_args = (list(kernel_size), list(stride), list(dilation), list(is_causal), scale)


def _na_backward(ctx, d_out, d_lse):
    """Gradients of the output w.r.t. query, key, value and the fused extra tokens. d_lse is
    ignored, as in the reference's backward (src/natten/backends/blackwell_fna.py:185-318)."""
    query, key, value, out, lse = ctx.saved_tensors[:5]
    query, key, value = query.contiguous(), key.contiguous(), value.contiguous()
    ak, av = ctx.saved_tensors[5:] if ctx.has_extra else (None, None)
    kernel_size, stride, dilation, is_causal, scale = ctx.na_args
    na_dim = query.dim() - 3
    tensor_core = (query.dtype in (torch.float16, torch.bfloat16)
                   and query.shape[-1] in TENSOR_CORE_HEAD_DIMS
                   and not BACKWARD_ON_CUDA_CORES)
    if tensor_core:
        q_tile, kv_tile = choose_backward_tile_shapes(
            tuple(int(x) for x in query.shape[1:1 + na_dim]), kernel_size, stride, dilation,
            is_causal)
        q_tile = ctx.bwd_tiles[0] or q_tile      # the caller's choice wins
        kv_tile = ctx.bwd_tiles[1] or kv_tile
        tensor_core = backward_layout_supported(q_tile, kv_tile, dilation)
    if tensor_core:
        dq, dk, dv, dak, dav = ops.na_backward_direct(
            query, key, value, out, d_out.contiguous(), lse, ak, av, kernel_size, stride, dilation,
            is_causal, scale, list(q_tile), list(kv_tile))
        if not ctx.has_extra:
            dak = dav = None
        return (dq, dk, dv, dak, dav) + (None,) * 10
    # fp32 operands, other head dims, boxes a tensor map cannot express
    dq, dk, dv, dak, dav = ops.na_backward_simt(query, key, value, out, d_out.contiguous(), lse,
                                                ak, av, kernel_size, stride, dilation, is_causal,
                                                scale)
    if not ctx.has_extra:
        dak = dav = None
    return (dq, dk, dv, dak, dav) + (None,) * 10


BACKWARD_TILE_SIZE = 128
# set True to force the CUDA-core gradient kernels (used by the tests to compare the two)
BACKWARD_ON_CUDA_CORES = False


def backward_layout_supported(q_tile_shape: DimensionType, kv_tile_shape: DimensionType,
                              dilation: DimensionType) -> bool:
    """Whether the tensor-core backward can address the caller's layout with these 128-token tiles
    (a tile of one dilation group must fit a tensor-map box)."""
    return all(d <= MAX_TMA_ELEMENT_STRIDE and tq * d <= MAX_TMA_BOX and tkv * d <= MAX_TMA_BOX
               for tq, tkv, d in zip(q_tile_shape, kv_tile_shape, dilation))


def choose_backward_tile_shapes(shape: DimensionType, kernel_size: DimensionType,
                                stride: DimensionType, dilation: DimensionType,
                                is_causal: CausalArgType) -> Tuple[DimensionType, DimensionType]:
    """(q_tile_shape, kv_tile_shape), 128 tokens each, for the backward kernels: the pair that
    minimises the tile products of both passes - key/value tiles visited per query tile (dQ) plus
    query tiles visited per key/value tile (dK, dV). Both walks start at the first token the
    stationary tile interacts with, not on a tile grid."""
    return _choose_backward_tile_shapes(
        tuple(int(x) for x in shape), tuple(int(x) for x in kernel_size),
        tuple(int(x) for x in stride), tuple(int(x) for x in dilation),
        tuple(bool(x) for x in is_causal))


@functools.lru_cache(maxsize=256)
def _choose_backward_tile_shapes(shape, kernel_size, stride, dilation, is_causal):
    n = len(shape)
    if n == 1:
        return (BACKWARD_TILE_SIZE,), (BACKWARD_TILE_SIZE,)
    cost: Dict[Tuple[int, int, int], Tuple[int, int]] = {}
    for a in range(n):
        for eq in range(8):
            for ek in range(8):
                args = (shape[a], kernel_size[a], stride[a], dilation[a], is_causal[a], 1 << eq,
                        1 << ek)
                cost[(a, 1 << eq, 1 << ek)] = (_axis_tile_cost(*args, True),
                                               _axis_inverse_tile_cost(*args))
    best = None
    for tq in _pow2_compositions(7, n):
        for tkv in _pow2_compositions(7, n):
            if not backward_layout_supported(tq, tkv, dilation):
                continue
            c_dq = c_dkdv = 1
            for a in range(n):
                c_dq *= cost[(a, tq[a], tkv[a])][0]
                c_dkdv *= cost[(a, tq[a], tkv[a])][1]
            c = c_dq + c_dkdv
            key = (c, -tq[-1], -tkv[-1])
            if best is None or key < best[0]:
                best = (key, tq, tkv)
    if best is None:  # no 128-token box fits: the caller falls back to the CUDA-core kernels
        return (BACKWARD_TILE_SIZE,) + (1,) * (n - 1), (BACKWARD_TILE_SIZE,) + (1,) * (n - 1)
    return best[1], best[2]


if ops.USE_TORCH_OPS:
    na_forward_op.register_autograd(_na_backward, setup_context=_na_setup_context)


def can_run_b200_fna(query: Tensor, key: Tensor, value: Tensor, raise_error: bool = False) -> bool:
    """Whether the tensor-core kernels take these operands (the reference's per-backend predicate,
    src/natten/backends/configs/checks.py:143-248): CUDA tensors on a compute-capability-10 GPU,
    fp16 / bf16 with head dim 64 or 128, or 8-bit floats with head dim 128."""
    def fail(msg: str) -> bool:
        if raise_error:
            raise ValueError(msg)
        return False
    if not (query.is_cuda and key.is_cuda and value.is_cuda):
        return fail("natten_b200 needs CUDA tensors.")
    if torch.cuda.get_device_capability(query.device)[0] != 10:
        return fail("natten_b200's tensor-core kernels need compute capability 10.x (B200).")
    if not _tensor_core_supported(query.dtype, query.shape[-1]):
        return fail(f"Unsupported dtype / head dim for the tensor-core kernels: {query.dtype}, "
                    f"{query.shape[-1]}.")
    return True


def _all_tile_shapes(na_dim: int, q_log2: int, kv_log2: int):
    return [(tq, tkv) for tq in _pow2_compositions(q_log2, na_dim)
            for tkv in _pow2_compositions(kv_log2, na_dim)]


def get_configs_for_b200_fna(query: Tensor, key: Tensor, value: Tensor):
    """Forward tile-shape pairs `(q_tile_shape, kv_tile_shape)` the kernel accepts for these
    operands - every power-of-two factorisation of 256 / 128 tokens (any factorisation works; the
    list is what `choose_tile_shapes` searches). Counterpart of the reference's
    `get_configs_for_cutlass_blackwell_fna` (src/natten/backends/configs/__init__.py:159-188)."""
    if not can_run_b200_fna(query, key, value):
        return []
    return _all_tile_shapes(query.dim() - 3, 8, 7) + _all_tile_shapes(query.dim() - 3, 7, 7)


def get_bwd_configs_for_b200_fna(query: Tensor, key: Tensor, value: Tensor):
    """Backward tile-shape pairs (128 tokens each) for the tensor-core backward; empty for 8-bit
    operands (no backward). Counterpart of `get_bwd_configs_for_cutlass_blackwell_fna`
    (src/natten/backends/configs/__init__.py:191-220)."""
    if not can_run_b200_fna(query, key, value) or query.dtype in FP8_DTYPES:
        return []
    return _all_tile_shapes(query.dim() - 3, 7, 7)


def get_configs_for_b200_fmha(query: Tensor, key: Tensor, value: Tensor):
    """Forward `(q_tile_size, kv_tile_size)` pairs of the dense-attention mode: one, the kernel's
    256-row query tile and 128-row key/value tile. Counterpart of the reference's
    `get_configs_for_cutlass_blackwell_fmha` (src/natten/backends/configs/__init__.py:97-125)."""
    if not query.is_cuda or query.dtype not in (torch.float16, torch.bfloat16) + tuple(FP8_DTYPES):
        return []
    return [(Q_TILE_SIZE, KV_TILE_SIZE)]


def get_bwd_configs_for_b200_fmha(query: Tensor, key: Tensor, value: Tensor):
    """Backward `(q_tile_size, kv_tile_size)` pairs of the dense-attention mode (128-token tiles);
    empty for 8-bit operands. Counterpart of `get_bwd_configs_for_cutlass_blackwell_fmha`
    (src/natten/backends/configs/__init__.py:128-156)."""
    if not query.is_cuda or query.dtype not in (torch.float16, torch.bfloat16):
        return []
    return [(128, 128)]


# The reference's names for the same queries, so that code written against its Blackwell backend
# keeps working after the import is switched (src/natten/__init__.py:66-106).
get_configs_for_cutlass_blackwell_fna = get_configs_for_b200_fna
get_bwd_configs_for_cutlass_blackwell_fna = get_bwd_configs_for_b200_fna
get_configs_for_cutlass_blackwell_fmha = get_configs_for_b200_fmha
get_bwd_configs_for_cutlass_blackwell_fmha = get_bwd_configs_for_b200_fmha


MAX_TMA_BOX = 256      # positions a tensor-map box may span per axis
MAX_TMA_ELEMENT_STRIDE = 8


def direct_layout_supported(q_tile_shape: DimensionType, kv_tile_shape: DimensionType,
                            dilation: DimensionType) -> bool:
    """Whether the fused kernel can read the caller's ``[B, *X, H, D]`` layout directly: a tile of
    one dilation group must fit a tensor-map box (tile * dilation <= 256 positions per axis,
    dilation <= 8). A 256-token query tile is fetched as two halves split along its last non-unit
    axis, a 128-token one whole."""
    q_box = list(q_tile_shape)
    if math.prod(q_box) != KV_TILE_SIZE:
        split = 0
        for a, t in enumerate(q_box):
            if t > 1:
                split = a
        if q_box[split] % 2:
            return False
        q_box[split] //= 2
    return all(d <= MAX_TMA_ELEMENT_STRIDE and tq * d <= MAX_TMA_BOX and tkv * d <= MAX_TMA_BOX
               for tq, tkv, d in zip(q_box, kv_tile_shape, dilation))


def fna_forward_direct(query: Tensor, key: Tensor, value: Tensor, kernel_size: DimensionType,
                       stride: DimensionType, dilation: DimensionType, is_causal: CausalArgType,
                       scale: float, q_tile_shape: DimensionType, kv_tile_shape: DimensionType,
                       additional_keys: Optional[Tensor] = None,
                       additional_values: Optional[Tensor] = None,
                       _inside_op: bool = False) -> Tuple[Tensor, Tensor]:
    """The fused kernel on the original heads-last layout: what the reference does as
    permute -> kernel -> unpermute (src/natten/backends/blackwell_fna.py:111-165) in one launch,
    the tile gathers (dilation included) done by the kernel's tensor-map loads."""
    q, k, v = query, key, value   # token-strided views are fine, see ops.na_forward_direct
    ak = additional_keys.contiguous() if additional_keys is not None else None
    av = additional_values.contiguous() if additional_values is not None else None
    op = getattr(ops.na_forward_direct, "raw", ops.na_forward_direct) if _inside_op \
        else ops.na_forward_direct
    out, lse = op(q, k, v, ak, av, list(kernel_size), list(stride), list(dilation),
                  [bool(c) for c in is_causal], float(scale), list(q_tile_shape),
                  list(kv_tile_shape))
    return out, lse


def fna_forward_permuted(query: Tensor, key: Tensor, value: Tensor, kernel_size: DimensionType,
                         stride: DimensionType, dilation: DimensionType, is_causal: CausalArgType,
                         scale: float, q_tile_shape: DimensionType, kv_tile_shape: DimensionType,
                         additional_keys: Optional[Tensor] = None,
                         additional_values: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """permute Q/K/V -> fused kernel -> unpermute O/LSE, the flow of the reference's
    src/natten/backends/blackwell_fna.py:91-181. Extra key/value tokens ``[B, M, Hkv, D]``, when
    given, are attended by every query inside the same kernel (no second attention, no merge)."""
    na_dim = query.dim() - 3
    q_perm, qkv_shape, q_shape = token_permute_operation(query, q_tile_shape, dilation, True)
    k_perm, _, kv_shape = token_permute_operation(key, kv_tile_shape, dilation, True)
    v_perm, _, _ = token_permute_operation(value, kv_tile_shape, dilation, True)
    q_perm = q_perm.reshape(-1, math.prod(q_shape), *q_perm.shape[-2:])
    k_perm = k_perm.reshape(-1, math.prod(kv_shape), *k_perm.shape[-2:])
    v_perm = v_perm.reshape(-1, math.prod(kv_shape), *v_perm.shape[-2:])
    o_perm, lse_perm = fna_forward_op(q_perm, k_perm, v_perm, qkv_shape, q_shape, kv_shape,
                                      kernel_size, stride, dilation, is_causal, scale,
                                      q_tile_shape, kv_tile_shape, additional_keys,
                                      additional_values)
    output = token_unpermute_operation(o_perm, qkv_shape, q_tile_shape, dilation, True)
    lse = token_unpermute_operation(lse_perm.unsqueeze(-1), qkv_shape, q_tile_shape, dilation,
                                    True).squeeze(-1)
    return output, lse


def fna_forward_op(q_perm: Tensor, k_perm: Tensor, v_perm: Tensor, qkv_shape: DimensionType,
                   q_shape: DimensionType, kv_shape: DimensionType, kernel_size: DimensionType,
                   stride: DimensionType, dilation: DimensionType, is_causal: CausalArgType,
                   scale: float, q_tile_shape: DimensionType, kv_tile_shape: DimensionType,
                   additional_keys: Optional[Tensor] = None,
                   additional_values: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """The fused kernel on token-permuted ``[B', S, H, D]`` operands; allocates O and LSE like the
    reference's op wrapper (src/natten/_libnatten/torch_wrappers.py:670-714). Extra key/value
    tokens stay in the original ``[B, M, Hkv, D]`` layout."""
    ak = additional_keys.contiguous() if additional_keys is not None else None
    av = additional_values.contiguous() if additional_values is not None else None
    out, lse = ops.fna_forward_permuted(
        q_perm.contiguous(), k_perm.contiguous(), v_perm.contiguous(), ak, av, list(qkv_shape),
        list(q_shape), list(kv_shape), list(kernel_size), list(stride), list(dilation),
        [bool(c) for c in is_causal], float(scale), list(q_tile_shape), list(kv_tile_shape))
    return out, lse


def fused_workspace_bytes(shape: DimensionType, dilation: DimensionType, q_tile_shape: DimensionType,
                          kv_tile_shape: DimensionType, batch: int, heads_q: int, heads_kv: int,
                          head_dim: int, want_lse: bool = True) -> int:
    """Scratch bytes `na_forward_fused` needs (0 when the layout needs no permutation)."""
    n = _lib.lib.b200na_na_forward_workspace_bytes(
        len(shape), _lib.ints(shape), _lib.ints(dilation), _lib.ints(q_tile_shape),
        _lib.ints(kv_tile_shape), batch, heads_q, heads_kv, head_dim, 1 if want_lse else 0)
    if n < 0:
        _lib.check(int(n), "b200na_na_forward_workspace_bytes", kernel_launches=0)
    return int(n)


def na_forward_fused(query: Tensor, key: Tensor, value: Tensor, kernel_size, stride=1, dilation=1,
                     is_causal=False, scale: Optional[float] = None, q_tile_shape=None,
                     kv_tile_shape=None, workspace: Optional[Tensor] = None
                     ) -> Tuple[Tensor, Tensor]:
    """Neighborhood attention forward through the single-call C entry `b200na_na_forward`
    (permute -> attention -> unpermute inside the library, permuted copies in `workspace`).
    Same results as `na1d/na2d/na3d(..., return_lse=True)` for fp16/bf16 and head dim 64/128;
    `workspace` is a uint8 CUDA tensor of at least `fused_workspace_bytes(...)` bytes (allocated
    here when omitted)."""
    na_tensor_checks(query, key, value)
    na_dim = query.dim() - 3
    kernel_size, stride, dilation, is_causal = check_all_args(na_dim, kernel_size, stride,
                                                              dilation, is_causal)
    check_args_against_input(query, kernel_size, stride, dilation, is_causal)
    _require_cuda(query, key, value)
    shape = tuple(query.shape[1:1 + na_dim])
    B, Hq, D = query.shape[0], query.shape[-2], query.shape[-1]
    Hkv = key.shape[-2]
    if query.dtype not in (torch.float16, torch.bfloat16) or D not in TENSOR_CORE_HEAD_DIMS:
        raise NotImplementedError("na_forward_fused needs fp16/bf16 operands and head dim 64 or 128.")
    if q_tile_shape is None or kv_tile_shape is None:
        auto_q, auto_kv = choose_tile_shapes(shape, kernel_size, stride, dilation, is_causal)
        q_tile_shape = q_tile_shape or auto_q
        kv_tile_shape = kv_tile_shape or auto_kv
    q_tile_shape = check_tile_shape(na_dim, q_tile_shape, "q_tile_shape", Q_TILE_SIZES)
    kv_tile_shape = check_tile_shape(na_dim, kv_tile_shape, "kv_tile_shape", KV_TILE_SIZE)
    need = fused_workspace_bytes(shape, dilation, q_tile_shape, kv_tile_shape, B, Hq, Hkv, D)
    if workspace is None and need > 0:
        workspace = torch.empty(need, dtype=torch.uint8, device=query.device)
    q, k, v = (t.detach().contiguous() for t in (query, key, value))
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device)
    scale = scale or D ** -0.5
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib.b200na_na_forward(
            _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), na_dim, _lib.ints(shape),
            _lib.ints(kernel_size), _lib.ints(stride), _lib.ints(dilation),
            _lib.ints([1 if c else 0 for c in is_causal]), _lib.ints(q_tile_shape),
            _lib.ints(kv_tile_shape), B, Hq, Hkv, D, _DTYPE_CODE[q.dtype], float(scale),
            _ptr(workspace) if need > 0 else None, workspace.numel() if need > 0 else 0,
            _stream(q)), "b200na_na_forward", kernel_launches=1 if need == 0 else 6)
    return out, lse


def _na(na_dim: int, query: Tensor, *args, **kwargs):
    if query.dim() != na_dim + 3:
        raise ValueError(f"NA{na_dim}D requires {na_dim + 3}-D input tensors, got {query.dim()=}.")
    return neighborhood_attention_generic(query, *args, **kwargs)


def na1d(query: Tensor, key: Tensor, value: Tensor, kernel_size, stride=1, dilation=1,
         is_causal=False, scale: Optional[float] = None, additional_keys: Optional[Tensor] = None,
         additional_values: Optional[Tensor] = None, attention_kwargs: Optional[Dict] = None,
         backend: Optional[str] = None, q_tile_shape=None, kv_tile_shape=None,
         backward_q_tile_shape=None, backward_kv_tile_shape=None, backward_kv_splits=None,
         backward_use_pt_reduction: bool = False, run_persistent_kernel: bool = True,
         kernel_schedule=None, torch_compile: bool = False, return_lse: bool = False):
    """1-D neighborhood attention on ``[batch, seqlen, heads, head_dim]`` tensors
    (reference: src/natten/functional.py:567-753)."""
    return _na(1, query, key, value, kernel_size, stride, dilation, is_causal, scale,
               additional_keys, additional_values, attention_kwargs, backend, q_tile_shape,
               kv_tile_shape, backward_q_tile_shape, backward_kv_tile_shape, backward_kv_splits,
               backward_use_pt_reduction, run_persistent_kernel, kernel_schedule, torch_compile,
               return_lse)


def na2d(query: Tensor, key: Tensor, value: Tensor, kernel_size, stride=1, dilation=1,
         is_causal=False, scale: Optional[float] = None, additional_keys: Optional[Tensor] = None,
         additional_values: Optional[Tensor] = None, attention_kwargs: Optional[Dict] = None,
         backend: Optional[str] = None, q_tile_shape=None, kv_tile_shape=None,
         backward_q_tile_shape=None, backward_kv_tile_shape=None, backward_kv_splits=None,
         backward_use_pt_reduction: bool = False, run_persistent_kernel: bool = True,
         kernel_schedule=None, torch_compile: bool = False, return_lse: bool = False):
    """2-D neighborhood attention on ``[batch, X, Y, heads, head_dim]`` tensors
    (reference: src/natten/functional.py:756-952)."""
    return _na(2, query, key, value, kernel_size, stride, dilation, is_causal, scale,
               additional_keys, additional_values, attention_kwargs, backend, q_tile_shape,
               kv_tile_shape, backward_q_tile_shape, backward_kv_tile_shape, backward_kv_splits,
               backward_use_pt_reduction, run_persistent_kernel, kernel_schedule, torch_compile,
               return_lse)


def na3d(query: Tensor, key: Tensor, value: Tensor, kernel_size, stride=1, dilation=1,
         is_causal=False, scale: Optional[float] = None, additional_keys: Optional[Tensor] = None,
         additional_values: Optional[Tensor] = None, attention_kwargs: Optional[Dict] = None,
         backend: Optional[str] = None, q_tile_shape=None, kv_tile_shape=None,
         backward_q_tile_shape=None, backward_kv_tile_shape=None, backward_kv_splits=None,
         backward_use_pt_reduction: bool = False, run_persistent_kernel: bool = True,
         kernel_schedule=None, torch_compile: bool = False, return_lse: bool = False):
    """3-D neighborhood attention on ``[batch, X, Y, Z, heads, head_dim]`` tensors
    (reference: src/natten/functional.py:955-1151)."""
    return _na(3, query, key, value, kernel_size, stride, dilation, is_causal, scale,
               additional_keys, additional_values, attention_kwargs, backend, q_tile_shape,
               kv_tile_shape, backward_q_tile_shape, backward_kv_tile_shape, backward_kv_splits,
               backward_use_pt_reduction, run_persistent_kernel, kernel_schedule, torch_compile,
               return_lse)
