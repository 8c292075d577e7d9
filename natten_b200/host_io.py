"""Neighborhood attention on operands that live in host memory.

The reference's operators take device tensors only; a caller whose data sits in (pinned) host
memory pays host -> device copies of Q, K, V and a device -> host copy of the result around every
call. Batch entries are independent, so this helper pipelines them: while one batch chunk is
being computed, the next chunk's operands are already crossing PCIe in one direction and the
previous chunk's result in the other (separate copy streams; the link is full duplex).
"""
from typing import Any, Optional, Tuple

import torch
from torch import Tensor

from .functional import neighborhood_attention_generic


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
