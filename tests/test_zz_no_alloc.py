"""b200na_na_forward_static: the whole operator through the C ABI with no allocation anywhere.

Some hosts cannot ask CUDA for memory at the moment they need attention (a plug-in whose host owns
the device-memory budget, a serving loop that must stay off the allocator, a process that gave its
memory to a pool at start-up). For them the library carries a fixed 32 MiB scratch array; this
file checks that the entry built on it returns exactly what the ordinary workspace entry returns,
on two consecutive calls (the second one sees the first one's left-overs in the array), and that a
problem too large for the array is refused with its own error code.

The file name sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes

import pytest
import torch

import natten_b200 as nb
import natten_b200._lib as L

pytestmark = pytest.mark.gpu


def _call_static(q, k, v, shape, ks, st, di, ca, tq, tkv, scale, watch_memory=False):
    """Straight through ctypes: outputs are the only tensors created here, the entry itself gets
    nothing but pointers to inputs and outputs. With `watch_memory` the driver's free-byte count
    and torch's allocator statistics are read right before and right after the call (and again
    once the kernels have run) and must not have moved."""
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device)
    torch.cuda.synchronize()
    before = (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(),
              torch.cuda.memory_reserved())
    rc = _static_entry(q, k, v, out, lse, shape, ks, st, di, ca, tq, tkv, scale)
    if watch_memory:
        after_call = (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(),
                      torch.cuda.memory_reserved())
        torch.cuda.synchronize()
        after_run = (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(),
                     torch.cuda.memory_reserved())
        assert after_call == before and after_run == before, (before, after_call, after_run)
    return rc, out, lse


def _static_entry(q, k, v, out, lse, shape, ks, st, di, ca, tq, tkv, scale):
    rc = L.lib.b200na_na_forward_static(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), ctypes.c_void_p(v.data_ptr()),
        ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(lse.data_ptr()), len(shape),
        L.ints(shape), L.ints(ks), L.ints(st), L.ints(di), L.ints([1 if c else 0 for c in ca]),
        L.ints(tq), L.ints(tkv), q.shape[0], q.shape[-2], k.shape[-2], q.shape[-1],
        {torch.float16: L.F16, torch.bfloat16: L.BF16}[q.dtype], ctypes.c_float(scale),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc


def test_static_workspace_entry_matches_the_workspace_entry_twice_in_a_row():
    torch.manual_seed(31)
    problems = [
        # a large first problem leaves the array full of data the smaller second one must ignore
        ((48, 56), (9, 7), (1, 2), (2, 1), (False, True), torch.bfloat16, 128),
        ((5, 12, 20), (3, 5, 6), (1, 1, 2), (1, 1, 1), (True, False, False), torch.float16, 64),
    ]
    for shape, ks, st, di, ca, dtype, D in problems:
        q, k, v = (torch.randn(2, *shape, 2, D, device="cuda").to(dtype) for _ in range(3))
        tq, tkv = nb.choose_tile_shapes(shape, ks, st, di, ca)
        need = nb.fused_workspace_bytes(shape, di, tq, tkv, 2, 2, 2, D)
        assert 0 < need <= L.STATIC_WORKSPACE_BYTES
        want_o, want_l = nb.na_forward_fused(q, k, v, ks, st, di, ca, q_tile_shape=tq,
                                             kv_tile_shape=tkv)
        # first call for this dtype / head dim: the driver may still load kernel code now
        rc, _, _ = _call_static(q, k, v, shape, ks, st, di, ca, tq, tkv, D ** -0.5)
        assert rc == L.OK, L.strerror(rc)
        torch.cuda.synchronize()
        # from here on the entry must leave device memory exactly as it finds it: neither the
        # driver's free-byte count nor torch's allocator may move across the call itself
        # (_call_static creates the two output tensors before it takes its readings)
        rc, out, lse = _call_static(q, k, v, shape, ks, st, di, ca, tq, tkv, D ** -0.5,
                                    watch_memory=True)
        assert rc == L.OK, L.strerror(rc)
        assert L.device_status() == 0
        # same kernels on the same data: bit-identical, well inside the 2e-2 the other tests allow
        assert torch.equal(out, want_o)
        assert torch.equal(lse, want_l)
        assert (out.float() - want_o.float()).abs().max().item() <= 2e-2


def test_static_workspace_entry_refuses_problems_beyond_its_array():
    shape, ks, tq, tkv = (512, 512), (7, 7), (16, 16), (16, 8)
    need = nb.fused_workspace_bytes(shape, (1, 1), tq, tkv, 1, 8, 8, 128)
    assert need > L.STATIC_WORKSPACE_BYTES
    q = torch.zeros(1, *shape, 8, 128, device="cuda", dtype=torch.bfloat16)
    rc, _, _ = _call_static(q, q, q, shape, ks, (1, 1), (1, 1), (False, False), tq, tkv, 0.1)
    assert rc == L.ERR_WORKSPACE_LIMIT
    assert "32 MiB" in L.strerror(rc)
