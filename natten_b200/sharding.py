"""Multi-GPU partitioning of the neighborhood-attention forward path (one process per GPU).

The reference has no distributed code; its only hint is that `merge_attentions` "can also be used
for distributed setups" (src/natten/attn_merge.py:199-204). Two partitionings are provided:

* **(batch x heads) units** — no term of the computation couples different (batch, head) pairs
  (problem shape of the reference kernel: csrc/include/natten/cuda/fna_blackwell/fna_forward.cuh:75-84),
  so ranks take disjoint unit ranges and run the ordinary operators; no collective.
* **Spatial slabs of axis 0** — a rank owns token coordinates ``[t0, t1)`` of the outermost axis
  for Q, K, V and O. A query only needs the keys inside its window, so each rank receives the
  key/value frames its queries' windows reach outside its own slab (the *halo*) from the owning
  ranks with point-to-point sends (NCCL over NVLink on GPUs, gloo on CPU), into its own memory,
  and then runs the kernel in layout coordinates (`b200na_fna_forward_sharded`). The output stays
  sharded. The halo follows from the window functions (reference semantics:
  csrc/include/natten/cuda/reference/mask.hpp:59-89): e.g. a causal axis with kernel 16, stride 1
  needs the 15 frames before the slab and nothing after it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from .functional import window_end, window_start
from .log import get_logger

logger = get_logger("natten_b200.sharding")


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous range of (batch x head) units of `rank`; sizes differ by at most one."""
    base, rem = divmod(n_units, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch_heads(B: int, H: int, world: int, rank: int) -> Tuple[slice, slice]:
    """Slices of the batch and head axes for `rank` when B*H units are split over `world` ranks.
    Splits the batch first and heads within a batch entry, so a rank's slice is one block."""
    if (B * H) % world != 0:
        raise ValueError(f"{B * H} (batch x heads) units do not divide over {world} ranks")
    per = B * H // world
    if per >= H:
        if per % H != 0:
            raise ValueError("a rank's share must be whole batch entries or a divisor of the heads")
        nb = per // H
        return slice(rank * nb, (rank + 1) * nb), slice(0, H)
    if H % per != 0:
        raise ValueError("a rank's share must be whole batch entries or a divisor of the heads")
    ranks_per_b = H // per
    b, r = divmod(rank, ranks_per_b)
    return slice(b, b + 1), slice(r * per, (r + 1) * per)


def slab_bounds(extent: int, world: int) -> List[Tuple[int, int]]:
    """Near-equal contiguous slabs of axis 0, one per rank."""
    return [unit_range(extent, world, r) for r in range(world)]


def kv_range_for_slab(t0: int, t1: int, extent: int, kernel: int, stride: int, causal: bool
                      ) -> Tuple[int, int]:
    """Key coordinates ``[lo, hi)`` along the sharded axis that queries ``[t0, t1)`` attend to.
    Window start and end are monotone in the query index, so the first and last query bound it."""
    lo = window_start(t0, kernel, stride, extent, causal)
    s_last = window_start(t1 - 1, kernel, stride, extent, causal)
    hi = window_end(t1 - 1, s_last, kernel, extent, causal)
    return lo, hi


@dataclass
class HaloPlan:
    """Who sends which frames of axis 0 to whom. All ranks compute the same plan."""
    world: int
    slabs: List[Tuple[int, int]]                 # owned [t0, t1) per rank
    needs: List[Tuple[int, int]]                 # key range [lo, hi) per rank
    # transfers[(src, dst)] = (a, b): frames [a, b) owned by src and needed by dst
    transfers: dict

    def recv_list(self, rank: int):
        return sorted((src, rng) for (src, dst), rng in self.transfers.items() if dst == rank)

    def send_list(self, rank: int):
        return sorted((dst, rng) for (src, dst), rng in self.transfers.items() if src == rank)

    def halo_frames(self, rank: int) -> int:
        return sum(b - a for _, (a, b) in self.recv_list(rank))


def balanced_slab_bounds(extent: int, world: int, kernel: int, stride: int, causal: bool,
                         align: int = 1) -> List[Tuple[int, int]]:
    """Contiguous slabs of axis 0 with near-equal attention work instead of near-equal length: a
    frame costs as many key frames as its window holds, which on a causal axis grows over the
    first `kernel` frames. Boundaries are multiples of `align` (the query tile's extent)."""
    cost = []
    for t in range(extent):
        st = window_start(t, kernel, stride, extent, causal)
        cost.append(window_end(t, st, kernel, extent, causal) - st)
    total = float(sum(cost))
    bounds, acc, t = [0], 0.0, 0
    for r in range(1, world):
        target = total * r / world
        while t < extent and acc + cost[t] / 2 < target:
            acc += cost[t]
            t += 1
        b = int(round(t / align)) * align
        b = min(max(b, bounds[-1] + align), extent - (world - r) * align)
        bounds.append(b)
        # keep the running sum consistent with the boundary actually chosen
        acc, t = float(sum(cost[:b])), b
    bounds.append(extent)
    return [(bounds[i], bounds[i + 1]) for i in range(world)]


def make_halo_plan(extent: int, world: int, kernel: int, stride: int, causal: bool,
                   balanced: bool = False, align: int = 1) -> HaloPlan:
    """`balanced`: slabs of near-equal work (see balanced_slab_bounds) instead of equal length."""
    slabs = (balanced_slab_bounds(extent, world, kernel, stride, causal, align) if balanced
             else slab_bounds(extent, world))
    if any(t1 <= t0 for t0, t1 in slabs):
        raise ValueError(f"axis of extent {extent} cannot be split over {world} ranks")
    needs = [kv_range_for_slab(t0, t1, extent, kernel, stride, causal) for t0, t1 in slabs]
    transfers = {}
    for dst, (lo, hi) in enumerate(needs):
        for src, (a, b) in enumerate(slabs):
            if src == dst:
                continue
            x, y = max(lo, a), min(hi, b)
            if x < y:
                transfers[(src, dst)] = (x, y)
    return HaloPlan(world, slabs, needs, transfers)


def exchange_halo(k_local: Tensor, v_local: Tensor, plan: HaloPlan, rank: int,
                  group: Optional[dist.ProcessGroup] = None) -> Tuple[Tensor, Tensor, int]:
    """Builds this rank's key/value slabs ``[B, hi - lo, ...]`` (own frames + received halo).

    `k_local` / `v_local` are ``[B, t1 - t0, *rest, H, D]``. Returns ``(k_slab, v_slab, lo)``. Works
    on CPU tensors with gloo and on CUDA tensors with NCCL (remote frames always land in this
    rank's own memory before any kernel reads them)."""
    t0, t1 = plan.slabs[rank]
    lo, hi = plan.needs[rank]
    assert k_local.shape[1] == t1 - t0 and v_local.shape[1] == t1 - t0
    shape = list(k_local.shape)
    shape[1] = hi - lo
    k_slab = torch.empty(shape, dtype=k_local.dtype, device=k_local.device)
    v_slab = torch.empty(shape, dtype=v_local.dtype, device=v_local.device)
    ops = []
    for dst, (a, b) in plan.send_list(rank):
        ops.append(dist.P2POp(dist.isend, k_local[:, a - t0:b - t0].contiguous(), dst, group))
        ops.append(dist.P2POp(dist.isend, v_local[:, a - t0:b - t0].contiguous(), dst, group))
    recv_bufs = []
    for src, (a, b) in plan.recv_list(rank):
        # batch 1 makes the destination slice contiguous; otherwise receive into a staging buffer
        kd, vd = k_slab[:, a - lo:b - lo], v_slab[:, a - lo:b - lo]
        if kd.is_contiguous():
            ops.append(dist.P2POp(dist.irecv, kd, src, group))
            ops.append(dist.P2POp(dist.irecv, vd, src, group))
        else:
            ks, vs = torch.empty_like(kd), torch.empty_like(vd)
            recv_bufs.append((kd, ks, vd, vs))
            ops.append(dist.P2POp(dist.irecv, ks, src, group))
            ops.append(dist.P2POp(dist.irecv, vs, src, group))
    reqs = dist.batch_isend_irecv(ops) if ops else []
    # own frames are copied while the transfers are in flight
    k_slab[:, t0 - lo:t1 - lo].copy_(k_local)
    v_slab[:, t0 - lo:t1 - lo].copy_(v_local)
    for r in reqs:
        r.wait()
    for kd, ks, vd, vs in recv_bufs:
        kd.copy_(ks)
        vd.copy_(vs)
    return k_slab, v_slab, lo


def exchange_halo_parts(k_local: Tensor, v_local: Tensor, plan: HaloPlan, rank: int,
                        group: Optional[dist.ProcessGroup] = None):
    """Starts the halo exchange and returns without waiting for it: ``(parts, requests, keep)``.
    `parts` is a list of ``(k_part, v_part, first_frame)`` - contiguous buffers in this rank's
    own memory holding received frames from `first_frame` on; they are valid once every request
    in `requests` has been waited for (on CUDA tensors ``wait()`` orders the current stream after
    the transfer, it does not block the host). `keep` holds the send buffers, which must stay
    alive until then. Own frames are not copied anywhere."""
    t0, t1 = plan.slabs[rank]
    ops, parts, keep = [], [], []
    for dst, (a, b) in plan.send_list(rank):
        ks, vs = k_local[:, a - t0:b - t0].contiguous(), v_local[:, a - t0:b - t0].contiguous()
        keep += [ks, vs]
        ops.append(dist.P2POp(dist.isend, ks, dst, group))
        ops.append(dist.P2POp(dist.isend, vs, dst, group))
    lo, hi = plan.needs[rank]
    recvs = plan.recv_list(rank)
    if k_local.shape[0] == 1:
        # batch 1: a frame range is one contiguous block, so everything before the slab lands in
        # one buffer and everything after it in another (at most two partial calls later)
        for first, last in ((lo, t0), (t1, hi)):
            if last <= first:
                continue
            shape = list(k_local.shape)
            shape[1] = last - first
            kp = torch.empty(shape, dtype=k_local.dtype, device=k_local.device)
            vp = torch.empty(shape, dtype=v_local.dtype, device=v_local.device)
            parts.append((kp, vp, first))
            for src, (a, b) in recvs:
                if first <= a and b <= last:
                    ops.append(dist.P2POp(dist.irecv, kp[:, a - first:b - first], src, group))
                    ops.append(dist.P2POp(dist.irecv, vp[:, a - first:b - first], src, group))
    else:
        for src, (a, b) in recvs:
            shape = list(k_local.shape)
            shape[1] = b - a
            kp = torch.empty(shape, dtype=k_local.dtype, device=k_local.device)
            vp = torch.empty(shape, dtype=v_local.dtype, device=v_local.device)
            parts.append((kp, vp, a))
            ops.append(dist.P2POp(dist.irecv, kp, src, group))
            ops.append(dist.P2POp(dist.irecv, vp, src, group))
    reqs = dist.batch_isend_irecv(ops) if ops else []
    return parts, reqs, keep


def fna_forward_slab(q_local: Tensor, k_slab: Tensor, v_slab: Tensor,
                     global_shape: Sequence[int], q_origin0: int, kv_origin0: int,
                     kernel_size: Sequence[int], stride: Sequence[int],
                     is_causal: Sequence[bool], scale: Optional[float] = None,
                     q_tile_shape=None, kv_tile_shape=None, clip: bool = False,
                     permuted: bool = False, out: Optional[Tensor] = None,
                     lse: Optional[Tensor] = None, additional_keys: Optional[Tensor] = None,
                     additional_values: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """Attention for query coordinates ``[q_origin0, q_origin0 + q_local.shape[1])`` of axis 0
    against a key/value slab that starts at coordinate ``kv_origin0`` (no communication here).
    One launch on the slabs as they lie (`b200na_na_forward_direct_sharded`); tile shapes a
    tensor-map box cannot express, or ``permuted=True``, take permute ->
    `b200na_fna_forward_sharded` -> unpermute. ``clip=True``: partial attention over the keys the
    slab holds (windows cut to it; a query with no key there gets O = 0, LSE = -inf), to be
    combined with the other parts by `merge_attentions`. `out` / `lse` (contiguous, the slab's
    shape) receive the result when given, `additional_keys` / `additional_values`
    ``[B, M, Hkv, D]`` are attended by every query (both: direct launch only)."""
    import ctypes

    from . import _lib
    from .functional import (_DTYPE_CODE, _ptr, _stream, choose_tile_shapes,
                             direct_layout_supported)

    nd = len(global_shape)
    global_shape = tuple(int(x) for x in global_shape)
    n_local = q_local.shape[1]
    if q_tile_shape is None or kv_tile_shape is None:
        # tile shapes are chosen for the slab (axis 0 is only n_local long here)
        local = (max(n_local, int(kernel_size[0])),) + global_shape[1:]
        q_tile_shape, kv_tile_shape = choose_tile_shapes(
            local, tuple(int(k) for k in kernel_size), tuple(int(s) for s in stride), (1,) * nd,
            tuple(bool(c) for c in is_causal))
    dil = (1,) * nd
    if permuted or not direct_layout_supported(q_tile_shape, kv_tile_shape, dil):
        if clip or additional_keys is not None or out is not None:
            raise NotImplementedError("partial (clipped) slab attention, extra tokens and "
                                      "caller-provided outputs need tile shapes the kernel can "
                                      "gather from the slabs directly")
        return _fna_forward_slab_permuted(q_local, k_slab, v_slab, global_shape, q_origin0,
                                          kv_origin0, kernel_size, stride, is_causal, scale,
                                          q_tile_shape, kv_tile_shape)
    q_local, k_slab, v_slab = q_local.contiguous(), k_slab.contiguous(), v_slab.contiguous()
    B, Hq, D = q_local.shape[0], q_local.shape[-2], q_local.shape[-1]
    Hkv = k_slab.shape[-2]
    if out is None:
        out = torch.empty_like(q_local)
    if lse is None:
        lse = torch.empty(q_local.shape[:-1], dtype=torch.float32, device=q_local.device)
    if not (out.is_contiguous() and lse.is_contiguous() and out.shape == q_local.shape):
        raise ValueError("out / lse must be contiguous tensors of the query slab's shape")
    scale = float(scale) if scale else float(D) ** -0.5
    q_origin = (int(q_origin0),) + (0,) * (nd - 1)
    kv_origin = (int(kv_origin0),) + (0,) * (nd - 1)
    with torch.cuda.device(q_local.device):
        _lib.check(_lib.lib.b200na_na_forward_direct_sharded(
            _ptr(q_local), _ptr(k_slab), _ptr(v_slab),
            _ptr(additional_keys.contiguous()) if additional_keys is not None else None,
            _ptr(additional_values.contiguous()) if additional_keys is not None else None,
            0 if additional_keys is None else int(additional_keys.shape[1]),
            _ptr(out), _ptr(lse), nd,
            _lib.ints(global_shape), _lib.ints(kernel_size), _lib.ints(stride),
            _lib.ints([1 if c else 0 for c in is_causal]), _lib.ints(q_tile_shape),
            _lib.ints(kv_tile_shape), _lib.ints(q_origin), _lib.ints(q_local.shape[1:1 + nd]),
            _lib.ints(kv_origin), _lib.ints(k_slab.shape[1:1 + nd]), 1 if clip else 0, B, Hq, Hkv,
            D, _DTYPE_CODE[q_local.dtype], ctypes.c_float(scale), _stream(q_local)),
            "b200na_na_forward_direct_sharded")
    return out, lse


def _fna_forward_slab_permuted(q_local: Tensor, k_slab: Tensor, v_slab: Tensor,
                               global_shape, q_origin0: int, kv_origin0: int, kernel_size,
                               stride, is_causal, scale, q_tile_shape, kv_tile_shape
                               ) -> Tuple[Tensor, Tensor]:
    """The slab through token-permuted copies: permute -> `b200na_fna_forward_sharded` ->
    unpermute."""
    import ctypes

    from . import _lib
    from .functional import (_DTYPE_CODE, _ptr, _stream, token_permute_operation,
                             token_unpermute_operation)

    nd = len(global_shape)
    dil = (1,) * nd
    q_perm, q_local_shape, q_shape = token_permute_operation(q_local, q_tile_shape, dil)
    k_perm, _, kv_shape = token_permute_operation(k_slab, kv_tile_shape, dil)
    v_perm, _, _ = token_permute_operation(v_slab, kv_tile_shape, dil)
    B, Hq, D = q_local.shape[0], q_local.shape[-2], q_local.shape[-1]
    Hkv = k_slab.shape[-2]
    q_perm = q_perm.reshape(B, math.prod(q_shape), Hq, D)
    k_perm = k_perm.reshape(B, math.prod(kv_shape), Hkv, D)
    v_perm = v_perm.reshape(B, math.prod(kv_shape), Hkv, D)
    out = torch.empty_like(q_perm)
    lse = torch.empty((B, q_perm.shape[1], Hq), dtype=torch.float32, device=q_perm.device)
    scale = float(scale) if scale else float(D) ** -0.5
    q_origin = (int(q_origin0),) + (0,) * (nd - 1)
    kv_origin = (int(kv_origin0),) + (0,) * (nd - 1)
    with torch.cuda.device(q_perm.device):
        _lib.check(_lib.lib.b200na_fna_forward_sharded(
            _ptr(q_perm), _ptr(k_perm), _ptr(v_perm), _ptr(out), _ptr(lse), nd,
            _lib.ints(global_shape), _lib.ints(q_shape), _lib.ints(kv_shape),
            _lib.ints(kernel_size), _lib.ints(stride), _lib.ints(dil),
            _lib.ints([1 if c else 0 for c in is_causal]), _lib.ints(q_tile_shape),
            _lib.ints(kv_tile_shape), B, Hq, Hkv, D, _DTYPE_CODE[q_perm.dtype],
            ctypes.c_float(scale), _lib.ints(q_origin), _lib.ints(q_local_shape),
            _lib.ints(kv_origin), _stream(q_perm)), "b200na_fna_forward_sharded")
    o_local = token_unpermute_operation(out, q_local_shape, q_tile_shape, dil)
    lse_local = token_unpermute_operation(lse.unsqueeze(-1), q_local_shape, q_tile_shape,
                                          dil).squeeze(-1)
    return o_local, lse_local


def na_forward_spatial_shard(q_local: Tensor, k_local: Tensor, v_local: Tensor,
                             global_shape: Sequence[int], kernel_size: Sequence[int],
                             stride: Sequence[int], is_causal: Sequence[bool],
                             scale: Optional[float] = None, rank: Optional[int] = None,
                             world: Optional[int] = None,
                             group: Optional[dist.ProcessGroup] = None,
                             q_tile_shape=None, kv_tile_shape=None,
                             overlap: bool = True, plan: Optional[HaloPlan] = None
                             ) -> Tuple[Tensor, Tensor]:
    """Neighborhood attention forward for this rank's slab of axis 0 (dilation 1). Inputs are
    ``[B, t1 - t0, *rest, H, D]`` (fp16/bf16, head dim 64 or 128); returns the rank's slab of the
    output and logsumexp, equal to the same rows of the unsharded result up to rounding.

    ``overlap=True`` (default): the halo transfers are started first, the rank then attends its
    OWN key/value frames (windows cut to the slab) while the frames of the other ranks are in
    flight, attends each received block once it has landed, and folds the partial results
    together with the LSE merge - the use the reference's `merge_attentions` hints at
    (src/natten/attn_merge.py:199-204). ``overlap=False``: exchange, then one kernel over the
    assembled key/value slab. `plan`: the halo plan the inputs were sliced by (default: slabs of
    equal length; `make_halo_plan(..., balanced=True)` gives slabs of equal work)."""
    from .functional import merge_attentions

    rank = dist.get_rank(group) if rank is None else rank
    world = dist.get_world_size(group) if world is None else world
    if plan is None:
        plan = make_halo_plan(int(global_shape[0]), world, int(kernel_size[0]), int(stride[0]),
                              bool(is_causal[0]))
    t0, t1 = plan.slabs[rank]
    if q_local.shape[1] != t1 - t0:
        raise ValueError(f"rank {rank} owns frames [{t0}, {t1}) but got {q_local.shape[1]} frames")
    if not overlap or not plan.recv_list(rank):
        k_slab, v_slab, lo = exchange_halo(k_local, v_local, plan, rank, group)
        return fna_forward_slab(q_local, k_slab, v_slab, global_shape, t0, lo, kernel_size, stride,
                                is_causal, scale, q_tile_shape, kv_tile_shape)
    nd = len(global_shape)
    logger.debug("rank %d/%d: frames [%d, %d) of %d, halo %s, exchange overlapped with the "
                 "attention over the rank's own frames", rank, world, t0, t1, int(global_shape[0]),
                 [(src, rng) for src, rng in plan.recv_list(rank)])
    parts, reqs, keep = exchange_halo_parts(k_local, v_local, plan, rank, group)
    out, lse = fna_forward_slab(q_local, k_local, v_local, global_shape, t0, t0, kernel_size,
                                stride, is_causal, scale, q_tile_shape, kv_tile_shape, clip=True)
    for r in reqs:
        r.wait()      # orders the current stream after the transfers
    flat_o, flat_l = out.flatten(1, nd), lse.flatten(1, nd)
    for kp, vp, first in parts:
        o2, l2 = fna_forward_slab(q_local, kp, vp, global_shape, t0, first, kernel_size, stride,
                                  is_causal, scale, q_tile_shape, kv_tile_shape, clip=True)
        flat_o, flat_l = merge_attentions([flat_o, o2.flatten(1, nd)], [flat_l, l2.flatten(1, nd)])
    del keep
    return flat_o.reshape(out.shape), flat_l.reshape(lse.shape)
