"""Neighborhood-attention layers on top of the B200 operators.

Drop-in counterparts of the reference's ``NeighborhoodAttention1D/2D/3D``
(src/natten/modules.py:42-122): same constructor arguments, same parameter names (``qkv``,
``proj``), so a reference checkpoint loads unchanged. Trainable: the operator underneath is
differentiable.
"""
from typing import Any, Optional

from torch import Tensor, nn

from .checks import check_all_args
from .functional import neighborhood_attention_generic


class NeighborhoodAttentionGeneric(nn.Module):
    """QKV projection -> neighborhood attention over ``na_dim`` token axes -> output projection.

    Input and output are ``[batch, *token_layout, embed_dim]``."""

    def __init__(self, na_dim: int, embed_dim: int, num_heads: int, kernel_size: Any,
                 stride: Any = 1, dilation: Any = 1, is_causal: Any = False, qkv_bias: bool = True,
                 qk_scale: Optional[float] = None, proj_drop: float = 0.0):
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError("Number of attention heads must evenly divide embedding dimension, "
                             f"got {embed_dim=}, {num_heads=}.")
        self.kernel_size, self.stride, self.dilation, self.is_causal = check_all_args(
            na_dim, kernel_size, stride, dilation, is_causal)
        self.na_dim = na_dim
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        self.scale = qk_scale or self.head_dim ** -0.5
        self.qkv = nn.Linear(embed_dim, 3 * embed_dim, bias=qkv_bias)
        self.proj = nn.Linear(embed_dim, embed_dim)
        self.proj_drop = nn.Dropout(proj_drop)

    def forward(self, x: Tensor) -> Tensor:
        if x.dim() != self.na_dim + 2:
            raise ValueError(f"NeighborhoodAttention{self.na_dim}D expected a tensor with rank "
                             f"{self.na_dim + 2} (batch, {self.na_dim} token axes, embedding), "
                             f"got {x.dim()=}.")
        if x.shape[-1] != self.embed_dim:
            raise ValueError(f"Expected embedding dimension {self.embed_dim}, got {x.shape[-1]} "
                             f"({x.shape=}).")
        lead = x.shape[:-1]
        # [..., 3, heads, head_dim]: q, k, v are strided views of one projection output
        q, k, v = self.qkv(x).unflatten(-1, (3, self.num_heads, self.head_dim)).unbind(-3)
        out = neighborhood_attention_generic(q, k, v, kernel_size=self.kernel_size,
                                             stride=self.stride, dilation=self.dilation,
                                             is_causal=self.is_causal, scale=self.scale)
        return self.proj_drop(self.proj(out.reshape(*lead, self.embed_dim)))

    def extra_repr(self) -> str:
        return (f"head_dim={self.head_dim}, num_heads={self.num_heads}, "
                f"kernel_size={self.kernel_size}, stride={self.stride}, "
                f"dilation={self.dilation}, is_causal={self.is_causal}")


class NeighborhoodAttention1D(NeighborhoodAttentionGeneric):
    """1-D neighborhood attention layer on ``[batch, length, embed_dim]``."""

    def __init__(self, embed_dim: int, num_heads: int, kernel_size: Any, stride: Any = 1,
                 dilation: Any = 1, is_causal: Any = False, qkv_bias: bool = True,
                 qk_scale: Optional[float] = None, proj_drop: float = 0.0):
        super().__init__(1, embed_dim, num_heads, kernel_size, stride, dilation, is_causal,
                         qkv_bias, qk_scale, proj_drop)


class NeighborhoodAttention2D(NeighborhoodAttentionGeneric):
    """2-D neighborhood attention layer on ``[batch, X, Y, embed_dim]``."""

    def __init__(self, embed_dim: int, num_heads: int, kernel_size: Any, stride: Any = 1,
                 dilation: Any = 1, is_causal: Any = False, qkv_bias: bool = True,
                 qk_scale: Optional[float] = None, proj_drop: float = 0.0):
        super().__init__(2, embed_dim, num_heads, kernel_size, stride, dilation, is_causal,
                         qkv_bias, qk_scale, proj_drop)


class NeighborhoodAttention3D(NeighborhoodAttentionGeneric):
    """3-D neighborhood attention layer on ``[batch, X, Y, Z, embed_dim]``."""

    def __init__(self, embed_dim: int, num_heads: int, kernel_size: Any, stride: Any = 1,
                 dilation: Any = 1, is_causal: Any = False, qkv_bias: bool = True,
                 qk_scale: Optional[float] = None, proj_drop: float = 0.0):
        super().__init__(3, embed_dim, num_heads, kernel_size, stride, dilation, is_causal,
                         qkv_bias, qk_scale, proj_drop)
