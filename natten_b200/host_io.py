"""Neighborhood attention on operands that live in host memory.

The reference's operators take device tensors only; a caller whose data sits in (pinned) host
memory pays host -> device copies of Q, K, V and a device -> host copy of the result around every
call. This helper pipelines the three: while one piece is being computed, the next piece's
operands are already crossing PCIe in one direction and the previous piece's result in the other
(separate copy streams; the link is full duplex). Pieces are slabs of the outermost token axis
where the problem allows it (undilated fp16 / bf16) - a slab of queries only
needs the key/value frames its windows reach, which for all but its last frames have arrived with
earlier slabs - and whole batch entries otherwise.
"""
from typing import Any, Optional, Tuple

import torch
from torch import Tensor

from .checks import check_all_args
from .functional import (TENSOR_CORE_HEAD_DIMS, choose_tile_shapes, direct_layout_supported,
                         neighborhood_attention_generic)


def na_forward_from_host(query: Tensor, key: Tensor, value: Tensor, kernel_size: Any,
                         stride: Any = 1, dilation: Any = 1, is_causal: Any = False,
                         scale: Optional[float] = None, additional_keys: Optional[Tensor] = None,
                         additional_values: Optional[Tensor] = None, out: Optional[Tensor] = None,
                         lse: Optional[Tensor] = None, device: Optional[torch.device] = None,
                         batch_chunk: int = 1) -> Tuple[Tensor, Tensor]:
    """``na1d/na2d/na3d(..., return_lse=True)`` for host tensors ``[B, *X, H, D]``.

    Operands should be pinned (``tensor.pin_memory()``) for the copies to be asynchronous. `out`
    / `lse` are pinned host tensors to fill (allocated when omitted). The work is enqueued on the
    current stream of `device` (default: the current CUDA device) and two internal copy streams;
    on return the current stream is ordered after everything, so synchronising it makes `out` and
    `lse` valid. Batch entries are processed `batch_chunk` at a time."""
    if query.is_cuda or key.is_cuda or value.is_cuda:
        raise ValueError("na_forward_from_host expects host tensors; call na1d/na2d/na3d directly "
                         "for device tensors.")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B = query.shape[0]
    if out is None:
        out = torch.empty(query.shape, dtype=query.dtype).pin_memory()
    if lse is None:
        lse = torch.empty(query.shape[:-1], dtype=torch.float32).pin_memory()
    has_extra = additional_keys is not None and additional_values is not None
    if batch_chunk == 1:
        plan = _slab_plan(query, key, kernel_size, stride, dilation, is_causal)
        if plan is not None:
            return _stream_slabs(query, key, value, plan, scale, out, lse, dev,
                                 additional_keys if has_extra else None,
                                 additional_values if has_extra else None)
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = _copy_streams(dev)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    step = max(1, int(batch_chunk))
    for b0 in range(0, B, step):
        b1 = min(B, b0 + step)
        with torch.cuda.stream(s_in):
            ops = [t[b0:b1].to(dev, non_blocking=True) for t in (query, key, value)]
            if has_extra:
                ops += [t[b0:b1].to(dev, non_blocking=True)
                        for t in (additional_keys, additional_values)]
            arrived = s_in.record_event()
        cur.wait_event(arrived)
        for t in ops:
            t.record_stream(cur)  # allocated on the copy stream, consumed on the compute stream
        o, l = neighborhood_attention_generic(
            ops[0], ops[1], ops[2], kernel_size, stride, dilation, is_causal, scale,
            ops[3] if has_extra else None, ops[4] if has_extra else None, return_lse=True)
        done = cur.record_event()
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            out[b0:b1].copy_(o, non_blocking=True)
            lse[b0:b1].copy_(l, non_blocking=True)
            o.record_stream(s_out)
            l.record_stream(s_out)
    cur.wait_stream(s_out)
    return out, lse


_streams = {}


def _copy_streams(dev: torch.device):
    key = (dev.type, dev.index)
    if key not in _streams:
        _streams[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _streams[key]


def _slab_plan(query: Tensor, key: Tensor, kernel_size, stride, dilation, is_causal):
    """Slabs of axis 0 to stream the problem in, or None when it has to go whole: needs fp16 /
    bf16 operands with a tensor-core head dim, no dilation, tile shapes the kernel gathers from
    the caller's layout, and an axis 0 long enough for at least four slabs."""
    from .sharding import kv_range_for_slab
    na_dim = query.dim() - 3
    if query.dtype not in (torch.float16, torch.bfloat16) or query.shape[-1] not in TENSOR_CORE_HEAD_DIMS:
        return None
    ks, st, di, ca = check_all_args(na_dim, kernel_size, stride, dilation, is_causal)
    if any(d != 1 for d in di) or key.shape[1:1 + na_dim] != query.shape[1:1 + na_dim]:
        return None
    shape = tuple(int(x) for x in query.shape[1:1 + na_dim])
    tq, tkv = choose_tile_shapes(shape, ks, st, di, ca)
    if not direct_layout_supported(tq, tkv, di):
        return None
    # slabs of about 1/8 of the axis, whole query tiles each
    step = max(tq[0], -(-shape[0] // 8 // tq[0]) * tq[0])
    if shape[0] < 4 * step:
        return None
    slabs = []
    for a in range(0, shape[0], step):
        b = min(shape[0], a + step)
        lo, hi = kv_range_for_slab(a, b, shape[0], ks[0], st[0], ca[0])
        slabs.append((a, b, lo, hi))
    return dict(shape=shape, ks=ks, st=st, ca=ca, tq=tq, tkv=tkv, slabs=slabs)


def _stream_slabs(query, key, value, plan, scale, out, lse, dev, add_k=None, add_v=None):
    from .sharding import fna_forward_slab
    shape, slabs = plan["shape"], plan["slabs"]
    B = query.shape[0]
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = _copy_streams(dev)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    # Device buffers for one batch entry, two sets used in turn. They are allocated on the
    # current stream and every use on the copy streams is ordered before the end of this call
    # (the two wait_stream calls at the bottom), so the caching allocator may hand them out again
    # right away: no allocation - and no device synchronisation - in steady state.
    with torch.cuda.device(dev):
        sets = []
        for _ in range(min(2, B)):
            qd, kd, vd = (torch.empty((1,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
                          for t in (query, key, value))
            sets.append((qd, kd, vd, torch.empty_like(qd),
                         torch.empty(qd.shape[:-1], dtype=torch.float32, device=dev)))
        with torch.cuda.stream(s_in):
            # extra tokens are small: all batch entries at once, ahead of everything else
            akd = add_k.to(dev, non_blocking=True) if add_k is not None else None
            avd = add_v.to(dev, non_blocking=True) if add_v is not None else None
    drained = [None, None]   # per set: event after the last D2H copy that read it
    for b in range(B):
        qd, kd, vd, od, ld = sets[b % 2]
        if drained[b % 2] is not None:
            s_in.wait_event(drained[b % 2])   # entry b - 2 has left these buffers
        have = 0      # key/value frames of this batch entry already on their way to the device
        for a, e, lo, hi in slabs:
            with torch.cuda.stream(s_in):
                if hi > have:
                    kd[:, have:hi].copy_(key[b:b + 1, have:hi], non_blocking=True)
                    vd[:, have:hi].copy_(value[b:b + 1, have:hi], non_blocking=True)
                    have = hi
                qd[:, a:e].copy_(query[b:b + 1, a:e], non_blocking=True)
                arrived = s_in.record_event()
            cur.wait_event(arrived)
            fna_forward_slab(qd[:, a:e], kd[:, lo:hi], vd[:, lo:hi], shape, a, lo, plan["ks"],
                             plan["st"], plan["ca"], scale, plan["tq"], plan["tkv"],
                             out=od[:, a:e], lse=ld[:, a:e],
                             additional_keys=akd[b:b + 1] if akd is not None else None,
                             additional_values=avd[b:b + 1] if avd is not None else None)
            done = cur.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                out[b:b + 1, a:e].copy_(od[:, a:e], non_blocking=True)
                lse[b:b + 1, a:e].copy_(ld[:, a:e], non_blocking=True)
        drained[b % 2] = s_out.record_event()
    cur.wait_stream(s_out)
    cur.wait_stream(s_in)
    return out, lse
