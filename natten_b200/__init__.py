"""natten_b200 — B200 (sm_100a) neighborhood-attention forward path.

Public surface mirrors the reference's for this path (src/natten/__init__.py:66-106):
``na1d``, ``na2d``, ``na3d``, ``attention``, ``merge_attentions`` plus the token permute
operators. Importing the package loads ``lib/libnatten_b200.so`` and raises if it is missing.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is not built)
from .log import get_logger  # noqa: F401
from .functional import (BACKEND_NAME, FMHA_BACKEND_NAME, attention, choose_tile_shapes,
                         fna_forward_op, fna_forward_permuted, fna_forward_direct, direct_layout_supported,
                         can_run_b200_fna, get_configs_for_b200_fna, get_bwd_configs_for_b200_fna,
                         get_configs_for_b200_fmha, get_bwd_configs_for_b200_fmha,
                         get_configs_for_cutlass_blackwell_fna,
                         get_bwd_configs_for_cutlass_blackwell_fna,
                         get_configs_for_cutlass_blackwell_fmha,
                         get_bwd_configs_for_cutlass_blackwell_fmha,
                         fused_workspace_bytes, merge_attentions,
                         na1d, na2d, na3d, na_forward_fused,
                         neighborhood_attention_generic, token_permute_operation,
                         token_unpermute_operation)

from .host_io import na_forward_from_host  # noqa: E402
from .modules import (NeighborhoodAttention1D, NeighborhoodAttention2D,  # noqa: E402
                      NeighborhoodAttention3D)

__version__ = "0.1.0"
__all__ = [
    "na1d", "na2d", "na3d", "attention", "merge_attentions", "neighborhood_attention_generic",
    "NeighborhoodAttention1D", "NeighborhoodAttention2D", "NeighborhoodAttention3D",
    "na_forward_from_host", "can_run_b200_fna", "get_configs_for_b200_fna",
    "get_bwd_configs_for_b200_fna", "get_configs_for_b200_fmha", "get_bwd_configs_for_b200_fmha",
    "get_configs_for_cutlass_blackwell_fna", "get_bwd_configs_for_cutlass_blackwell_fna",
    "get_configs_for_cutlass_blackwell_fmha", "get_bwd_configs_for_cutlass_blackwell_fmha",
    "token_permute_operation", "token_unpermute_operation", "fna_forward_op",
    "fna_forward_permuted", "fna_forward_direct", "direct_layout_supported", "na_forward_fused", "fused_workspace_bytes", "choose_tile_shapes", "BACKEND_NAME", "FMHA_BACKEND_NAME",
]
