"""torch op registration and layers on the GPU: opcheck, torch.compile without graph breaks,
layer output against the oracle."""
import numpy as np
import pytest
import torch

import natten_b200 as nb
import natten_b200._lib as L
import oracle
from natten_b200 import ops

pytestmark = pytest.mark.gpu


def test_opcheck_schema_and_fake_implementations():
    torch.manual_seed(2)
    q = torch.randn(1, 24, 20, 2, 64, device="cuda").bfloat16()
    ak = torch.randn(1, 9, 2, 64, device="cuda").bfloat16()
    tests = ("test_schema", "test_faketensor")
    import natten_b200.functional as F
    torch.library.opcheck(F.na_forward_op,
                          (q, q, q, ak, ak, [5, 7], [1, 2], [2, 1], [False, True], 0.125, [], [],
                           False, [], []), test_utils=tests)
    torch.library.opcheck(ops.na_forward_direct,
                          (q, q, q, ak, ak, [5, 7], [1, 2], [2, 1], [False, True], 0.125,
                           [16, 16], [16, 8]), test_utils=tests)
    torch.library.opcheck(ops.na_forward_simt,
                          (q.float(), q.float(), q.float(), None, None, [5, 7], [1, 2], [2, 1],
                           [False, True], 0.125), test_utils=tests)
    torch.library.opcheck(ops.token_permute, (q, [24, 20], [8, 4], [2, 1], True), test_utils=tests)
    a = q.flatten(1, 2)
    torch.library.opcheck(ops.fmha_forward, (a, a, a, False, 0.125), test_utils=tests)
    o, l = ops.fmha_forward(a, a, a, False, 0.125)
    torch.library.opcheck(ops.merge, (o, l, o, l), test_utils=tests)
    assert L.device_status() == 0


def test_operator_compiles_without_graph_breaks():
    torch.manual_seed(3)
    q, k, v = (torch.randn(2, 32, 40, 2, 128, device="cuda").bfloat16() for _ in range(3))
    ak, av = (torch.randn(2, 40, 2, 128, device="cuda").bfloat16() for _ in range(2))

    def f(q, k, v, ak, av):
        o, l = nb.na2d(q * 1.0, k, v, (7, 9), (1, 2), (2, 1), (False, True), additional_keys=ak,
                       additional_values=av, return_lse=True)
        return o.float() * 2.0, l + 1.0

    want = f(q, k, v, ak, av)
    got = torch.compile(f, fullgraph=True)(q, k, v, ak, av)
    assert L.device_status() == 0
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])


@pytest.mark.parametrize("cls,shape,ks,di,ca", [
    (nb.NeighborhoodAttention1D, (300,), 33, 2, True),
    (nb.NeighborhoodAttention2D, (24, 28), (5, 7), (1, 2), (False, False)),
    (nb.NeighborhoodAttention3D, (6, 10, 12), (3, 4, 5), 1, (True, False, False)),
])
def test_layers_match_projections_around_the_oracle(cls, shape, ks, di, ca):
    torch.manual_seed(5)
    heads, dim = 2, 64
    layer = cls(heads * dim, heads, ks, dilation=di, is_causal=ca).cuda().bfloat16().eval()
    x = torch.randn(2, *shape, heads * dim, device="cuda").bfloat16()
    with torch.no_grad():
        got = layer(x)
        compiled = torch.compile(layer, fullgraph=True)(x)
        qkv = layer.qkv(x).unflatten(-1, (3, heads, dim))
    assert L.device_status() == 0
    assert torch.equal(got, compiled)
    q, k, v = (qkv.select(-3, i).float().cpu().numpy() for i in range(3))
    want_attn, _ = oracle.na_forward(q, k, v, layer.kernel_size, layer.stride, layer.dilation,
                                     layer.is_causal)
    with torch.no_grad():
        want = layer.proj(torch.from_numpy(want_attn).cuda().bfloat16().reshape(x.shape))
    # attention tolerance (2e-2) carried through the output projection of O(1) weights
    assert np.abs(got.float().cpu().numpy() - want.float().cpu().numpy()).max() <= 2e-2


def test_ops_without_a_formula_refuse_to_differentiate():
    o = torch.randn(1, 64, 2, 64, device="cuda").bfloat16().requires_grad_()
    l = torch.randn(1, 64, 2, device="cuda")
    m, _ = nb.merge_attentions([o, o], [l, l])
    with pytest.raises(RuntimeError):
        m.float().sum().backward()


def test_host_operand_entry_point_matches_the_device_call():
    torch.manual_seed(9)
    q, k, v = (torch.randn(5, 20, 24, 2, 64).bfloat16().pin_memory() for _ in range(3))
    ak, av = (torch.randn(5, 33, 2, 64).bfloat16().pin_memory() for _ in range(2))
    args = dict(kernel_size=(5, 7), stride=(1, 2), dilation=(2, 1), is_causal=(False, True))
    want_o, want_l = nb.na2d(q.cuda(), k.cuda(), v.cuda(), additional_keys=ak.cuda(),
                             additional_values=av.cuda(), return_lse=True, **args)
    for chunk in (1, 2, 8):
        out, lse = nb.na_forward_from_host(q, k, v, additional_keys=ak, additional_values=av,
                                           batch_chunk=chunk, **args)
        torch.cuda.current_stream().synchronize()
        assert L.device_status() == 0
        assert out.is_pinned() and not out.is_cuda
        assert torch.equal(out, want_o.cpu()) and torch.equal(lse, want_l.cpu())
    with pytest.raises(ValueError):
        nb.na_forward_from_host(q.cuda(), k, v, **args)


@pytest.mark.gpu
def test_host_operand_entry_point_streams_slabs_of_the_outermost_axis():
    """Undilated 16-bit problems go through the GPU slab by slab along axis 0 (the copies of one
    slab overlap the kernel of another), extra tokens included; same result as the device call."""
    from natten_b200 import host_io
    torch.manual_seed(10)
    for shape, ks, st, ca, n_extra in [((64, 24), (9, 7), (1, 2), (True, False), 0),
                                       ((48, 8, 8), (5, 4, 4), (1, 2, 2), (False, False, False), 40),
                                       ((4096,), (300,), (1,), (False,), 0)]:
        q, k, v = (torch.randn(3, *shape, 2, 64).half().pin_memory() for _ in range(3))
        ak = av = None
        if n_extra:
            ak, av = (torch.randn(3, n_extra, 2, 64).half().pin_memory() for _ in range(2))
        assert host_io._slab_plan(q, k, ks, st, 1, ca) is not None
        fn = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[len(shape)]
        want_o, want_l = fn(q.cuda(), k.cuda(), v.cuda(), kernel_size=ks, stride=st, is_causal=ca,
                            additional_keys=ak.cuda() if n_extra else None,
                            additional_values=av.cuda() if n_extra else None, return_lse=True)
        for _ in range(2):      # the second call reuses the first one's device buffers
            out, lse = nb.na_forward_from_host(q, k, v, ks, st, 1, ca, additional_keys=ak,
                                               additional_values=av)
            torch.cuda.current_stream().synchronize()
            assert L.device_status() == 0
            assert (out.float() - want_o.cpu().float()).abs().max().item() <= 1e-2
            assert (lse - want_l.cpu()).abs().max().item() <= 2e-3


def test_reference_backend_names_and_config_listing():
    q = torch.randn(1, 20, 24, 2, 64, device="cuda").half()
    a = nb.na2d(q, q, q, 5, backend="blackwell-fna")          # the reference's name is an alias
    b = nb.na2d(q, q, q, 5, backend="b200-fna")
    assert torch.equal(a, b)
    with pytest.raises(NotImplementedError):
        nb.na2d(q, q, q, 5, backend="hopper-fna")
    assert nb.can_run_b200_fna(q, q, q)
    cfgs = nb.get_configs_for_b200_fna(q, q, q)
    assert ((16, 16), (16, 8)) in cfgs and ((8, 16), (16, 8)) in cfgs and all(
        qt[0] * qt[1] in (256, 128) and kt[0] * kt[1] == 128 for qt, kt in cfgs)
    bwd = nb.get_bwd_configs_for_b200_fna(q, q, q)
    assert ((8, 16), (16, 8)) in bwd
    assert not nb.can_run_b200_fna(q.float(), q.float(), q.float())
    assert nb.get_configs_for_b200_fna(q.float(), q.float(), q.float()) == []
    with pytest.raises(ValueError):
        nb.can_run_b200_fna(q.cpu(), q.cpu(), q.cpu(), raise_error=True)
    # every listed forward pair gives the same result up to rounding; so does a caller-chosen
    # backward pair
    want = nb.na2d(q, q, q, 5).float()
    for qt, kt in cfgs[::7]:
        got = nb.na2d(q, q, q, 5, q_tile_shape=qt, kv_tile_shape=kt).float()
        assert (got - want).abs().max().item() <= 2e-2
    grads = []
    for bq, bk in (None, None), ((4, 32), (32, 4)):
        x = q.clone().requires_grad_()
        nb.na2d(x, q, q, 5, backward_q_tile_shape=bq, backward_kv_tile_shape=bk).float().sum().backward()
        grads.append(x.grad.float())
    assert L.device_status() == 0
    assert (grads[0] - grads[1]).abs().max().item() <= 2e-2 * max(1.0, grads[0].abs().max().item())
    with pytest.raises(ValueError):
        nb.na2d(q, q, q, 5, backward_q_tile_shape=(16, 16))


def test_fused_projection_views_are_read_in_place():
    """q, k, v sliced out of a fused [B, *X, 3, H, D] projection go to the kernel without copies
    (the tensor maps absorb the token stride) and give the bits of the contiguous call."""
    torch.manual_seed(12)
    qkv = torch.randn(2, 24, 28, 3, 2, 128, device="cuda").bfloat16()
    q, k, v = qkv.unbind(-3)
    assert not q.is_contiguous() and ops.token_stride(q) == 3 * 2 * 128
    args = dict(kernel_size=(7, 5), stride=(1, 2), dilation=(2, 1), is_causal=(False, True),
                return_lse=True)
    o_v, l_v = nb.na2d(q, k, v, **args)
    o_c, l_c = nb.na2d(q.contiguous(), k.contiguous(), v.contiguous(), **args)
    assert L.device_status() == 0
    assert o_v.is_contiguous() and torch.equal(o_v, o_c) and torch.equal(l_v, l_c)
    # a view the maps cannot express (transposed heads) is copied by the op, not refused
    qt = torch.randn(2, 24, 28, 128, 2, device="cuda").bfloat16().transpose(-1, -2)
    assert ops.token_stride(qt) < 0
    o_t = nb.na2d(qt, qt, qt, kernel_size=5)
    assert torch.equal(o_t, nb.na2d(qt.contiguous(), qt.contiguous(), qt.contiguous(), kernel_size=5))
    # gradients flow back into the fused tensor
    qkv2 = qkv.clone().requires_grad_()
    q2, k2, v2 = qkv2.unbind(-3)
    nb.na2d(q2, k2, v2, kernel_size=(7, 5)).float().square().mean().backward()
    assert qkv2.grad is not None and torch.isfinite(qkv2.grad).all() and qkv2.grad.abs().max() > 0
