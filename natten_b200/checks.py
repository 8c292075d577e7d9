"""Argument and tensor validation with the reference's rules and exception types
(src/natten/utils/checks.py:49-82, 85-182, 185-277, 278-370, 383-526)."""
from __future__ import annotations

from typing import Any, Optional, Sequence, Tuple

from torch import Tensor

DimensionType = Tuple[int, ...]
CausalArgType = Tuple[bool, ...]


def _universal_tensor_checks(query: Tensor, key: Tensor, value: Tensor) -> None:
    if query.is_sparse or key.is_sparse or value.is_sparse:
        raise NotImplementedError("natten_b200 does not support sparse tensors.")
    if query.is_nested or key.is_nested or value.is_nested:
        raise NotImplementedError("natten_b200 does not support nested tensors.")
    if query.device != key.device or query.device != value.device:
        raise ValueError("Query, key, and value must be on the same device, "
                         f"got {query.device=}, {key.device=}, {value.device=}.")
    if query.dtype != key.dtype or query.dtype != value.dtype:
        raise ValueError("Query, key, and value must assume the same data type, "
                         f"got {query.dtype=}, {key.dtype=}, {value.dtype=}.")


def _gqa_checks(query: Tensor, key: Tensor, value: Tensor) -> None:
    if key.shape[-2] != value.shape[-2]:
        raise ValueError("Key and value must always have the same number of heads, got "
                         f"{key.shape[-2]=}, {value.shape[-2]=}.")
    heads_q, heads_kv = query.shape[-2], key.shape[-2]
    if heads_q < heads_kv or heads_q % heads_kv != 0:
        raise ValueError("Key/value heads must evenly divide query heads, got "
                         f"{heads_q=}, {heads_kv=}.")


def na_tensor_checks(query: Tensor, key: Tensor, value: Tensor) -> None:
    _universal_tensor_checks(query, key, value)
    if query.dim() != key.dim() or query.dim() != value.dim():
        raise ValueError("Query, key, and value must have the same rank, "
                         f"got {query.dim()=}, {key.dim()=}, {value.dim()=}.")
    if query.dim() not in [4, 5, 6]:
        raise ValueError("Expected 4-D, 5-D, or 6-D tensors as inputs (corresponding to NA1D, "
                         f"NA2D, and NA3D), got {query.dim()=}.")
    na_dim = query.dim() - 3
    if query.shape[-1] != key.shape[-1]:
        raise ValueError(f"Q and K head dims must match, got {query.shape[-1]=}, {key.shape[-1]=}.")
    if query.shape[-1] != value.shape[-1]:
        raise ValueError("natten_b200 does not support different head dims for QK and V, got "
                         f"{query.shape[-1]=}, {value.shape[-1]=}.")
    if query.shape[0] != key.shape[0] or query.shape[0] != value.shape[0]:
        raise ValueError("Q, K, and V must match in batch size, got "
                         f"{query.shape[0]=}, {key.shape[0]=}, {value.shape[0]=}.")
    if (query.shape[1:na_dim + 1] != key.shape[1:na_dim + 1]
            or query.shape[1:na_dim + 1] != value.shape[1:na_dim + 1]):
        raise ValueError("Neighborhood Attention operations require Q, K, and V to match in their "
                         f"token layouts, got {query.shape[1:na_dim+1]=}, "
                         f"{key.shape[1:na_dim+1]=}, {value.shape[1:na_dim+1]=}.")
    _gqa_checks(query, key, value)


def fmha_tensor_checks(query: Tensor, key: Tensor, value: Tensor) -> None:
    _universal_tensor_checks(query, key, value)
    if query.dim() != key.dim() or query.dim() != value.dim():
        raise ValueError("Query, key, and value must have the same rank, "
                         f"got {query.dim()=}, {key.dim()=}, {value.dim()=}.")
    if query.dim() != 4:
        raise ValueError(f"Expected 4-D tensors as inputs to FMHA, got {query.dim()=}.")
    if query.shape[-1] != key.shape[-1]:
        raise ValueError(f"Q and K head dims must match, got {query.shape[-1]=}, {key.shape[-1]=}.")
    if query.shape[-1] != value.shape[-1]:
        raise ValueError("natten_b200 does not support different head dims for QK and V, got "
                         f"{query.shape[-1]=}, {value.shape[-1]=}.")
    if query.shape[0] != key.shape[0] or query.shape[0] != value.shape[0]:
        raise ValueError("Q, K, and V must match in batch size, got "
                         f"{query.shape[0]=}, {key.shape[0]=}, {value.shape[0]=}.")
    if key.shape[1] != value.shape[1]:
        raise ValueError("K and V must match in sequence length, got "
                         f"{key.shape[1]=}, {value.shape[1]=}.")
    _gqa_checks(query, key, value)


def additional_kv_tensor_checks(query: Tensor, key: Tensor, value: Tensor,
                                add_key: Optional[Tensor], add_value: Optional[Tensor]) -> None:
    if (add_key is not None) ^ (add_value is not None):
        raise ValueError(
            "`additional_keys` and `additional_values` must be either both Tensors or None.")
    if add_key is None:
        return
    assert add_value is not None
    _universal_tensor_checks(query, add_key, add_value)
    if add_key.dim() != 4 or add_value.dim() != 4:
        raise ValueError("Additional keys/values must be 4-D [batch, tokens, heads, head_dim], got "
                         f"{add_key.dim()=}, {add_value.dim()=}.")
    if query.shape[-1] != add_key.shape[-1]:
        raise ValueError(
            f"Q and K head dims must match, got {query.shape[-1]=}, {add_key.shape[-1]=}.")
    if query.shape[0] != add_key.shape[0] or query.shape[0] != add_value.shape[0]:
        raise ValueError("Q, additional K, and additional V must match in batch size, got "
                         f"{query.shape[0]=}, {add_key.shape[0]=}, {add_value.shape[0]=}.")
    if add_key.shape[1] != add_value.shape[1]:
        raise ValueError("Additional K and V must match in sequence length, got "
                         f"{add_key.shape[1]=}, {add_value.shape[1]=}.")
    if key.shape[-2] != add_key.shape[-2] or value.shape[-2] != add_value.shape[-2]:
        raise ValueError("Additional key/value tokens must match the self attention key/value "
                         f"tokens in number of heads, got {key.shape[-2]=} != "
                         f"{add_key.shape[-2]=}, and {value.shape[-2]=} != {add_value.shape[-2]=}.")
    if key.shape[-1] != add_key.shape[-1] or value.shape[-1] != add_value.shape[-1]:
        raise ValueError("Additional key/value tokens must match the self attention key/value "
                         f"tokens in head dim, got {key.shape[-1]=} != {add_key.shape[-1]=}, and "
                         f"{value.shape[-1]=} != {add_value.shape[-1]=}.")


def _dim_arg(na_dim: int, x: Any, name: str, minimum: int, default: Optional[int]) -> DimensionType:
    assert 0 < na_dim < 4
    if x is None and default is not None:
        return tuple(default for _ in range(na_dim))
    if (isinstance(x, Sequence) and len(x) == na_dim
            and all(isinstance(v, int) and not isinstance(v, bool) and v >= minimum for v in x)):
        return tuple(int(v) for v in x)
    if isinstance(x, int) and not isinstance(x, bool) and x >= minimum:
        return tuple(x for _ in range(na_dim))
    raise ValueError(f"Invalid value for `{name}`; expected an integer or iterable of {na_dim} "
                     f"integers, all >= {minimum}, got {type(x)=}, {x=}.")


def check_causal_arg(na_dim: int, is_causal: Any) -> CausalArgType:
    if is_causal is None:
        return tuple(False for _ in range(na_dim))
    if (isinstance(is_causal, Sequence) and len(is_causal) == na_dim
            and all(isinstance(c, bool) for c in is_causal)):
        return tuple(bool(c) for c in is_causal)
    if isinstance(is_causal, bool):
        return tuple(is_causal for _ in range(na_dim))
    raise ValueError("Invalid value for `is_causal`; expected a boolean or tuple of booleans, "
                     f"got {type(is_causal)=}, {is_causal=}.")


def check_all_args(na_dim: int, kernel_size: Any, stride: Any, dilation: Any, is_causal: Any):
    return (_dim_arg(na_dim, kernel_size, "kernel_size", 2, None),
            _dim_arg(na_dim, stride, "stride", 1, 1),
            _dim_arg(na_dim, dilation, "dilation", 1, 1),
            check_causal_arg(na_dim, is_causal))


def check_args_against_input(input_tensor: Tensor, kernel_size: DimensionType,
                             stride: DimensionType, dilation: DimensionType,
                             is_causal: CausalArgType) -> None:
    na_dim = input_tensor.dim() - 3
    input_size = tuple(input_tensor.shape[1:1 + na_dim])
    if any(k * d > x for x, k, d in zip(input_size, kernel_size, dilation)):
        raise ValueError("The product of kernel size and dilation cannot be larger than input size "
                         f"along any dimension, got {input_size=} ({input_tensor.shape=}), "
                         f"{kernel_size=}, {dilation=}.")
    if any(s > k for k, s in zip(kernel_size, stride)):
        raise ValueError("Stride cannot be larger than kernel size along any dimension, got "
                         f"{kernel_size=}, {stride=}.")


def is_self_attention(input_tensor: Tensor, kernel_size: DimensionType, is_causal: CausalArgType,
                      has_additional_attention: bool) -> bool:
    na_dim = input_tensor.dim() - 3
    input_size = tuple(input_tensor.shape[1:1 + na_dim])
    # 1-D with a full window equals plain (causal) attention unless extra context is attached
    if na_dim == 1 and not has_additional_attention:
        return kernel_size[0] == input_size[0]
    return all(k == x and not c for x, k, c in zip(input_size, kernel_size, is_causal))


def check_tile_shape(na_dim: int, tile_shape: Any, name: str, product) -> DimensionType:
    """`product`: the number of tokens the tile must hold, or a tuple of allowed numbers."""
    allowed = tuple(product) if isinstance(product, (tuple, list)) else (int(product),)
    if (not isinstance(tile_shape, Sequence) or len(tile_shape) != na_dim
            or not all(isinstance(v, int) and v >= 1 for v in tile_shape)):
        raise ValueError(f"`{name}` must be a tuple of {na_dim} positive integers, got {tile_shape=}.")
    prod = 1
    for v in tile_shape:
        prod *= v
    if prod not in allowed:
        raise ValueError(f"`{name}` must have {' or '.join(str(a) for a in allowed)} elements for "
                         f"this backend, got {tile_shape=} ({prod} elements).")
    return tuple(int(v) for v in tile_shape)
