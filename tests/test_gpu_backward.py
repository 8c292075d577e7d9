"""Backward of neighborhood attention through autograd, against the CPU oracle
(oracle.na_backward: double accumulation, tied to the reference's forward by tests/test_oracle.py).

Tolerances: fp32 operands 2e-4 relative to the largest gradient entry; fp16/bf16 operands 2e-2
(the forward's tolerance) - gradients are rounded to the operand dtype."""
import numpy as np
import pytest
import torch

import natten_b200 as nb
import natten_b200._lib as L
import oracle
from golden_io import na_cases

pytestmark = pytest.mark.gpu

CASES = ["c2s_na1d_1024_k128_causal", "na1d_300_k33", "na1d_257_k9_s3_d4_causal", "na2d_33x30_k3x5_s1x2_d3x2_causal01",
         "na2d_16x16_k5_gqa", "c3s_na2d_32x32_k13_d2", "c4s_na2d_32x32_k8_s4_extra24",
         "c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT", "na3d_6x9x11_k3x3x5_s1x1x2_d2x1x1_causalW",
         "na1d_96_k17_causal_extra7", "na2d_8x8_k8_selfattn"]


def _grads(c, dtype):
    fn = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[len(c.shape)]
    leaves = [torch.from_numpy(t).cuda().to(dtype).requires_grad_() for t in (c.q, c.k, c.v)]
    if c.n_extra:
        leaves += [torch.from_numpy(t).cuda().to(dtype).requires_grad_() for t in (c.add_k, c.add_v)]
    out = fn(leaves[0], leaves[1], leaves[2], kernel_size=c.kernel_size, stride=c.stride,
             dilation=c.dilation, is_causal=c.is_causal,
             additional_keys=leaves[3] if c.n_extra else None,
             additional_values=leaves[4] if c.n_extra else None)
    torch.manual_seed(11)
    d_out = torch.randn(out.shape, device="cuda").to(dtype)
    out.backward(d_out)
    assert L.device_status() == 0
    want = oracle.na_backward(c.q, c.k, c.v, d_out.float().cpu().numpy(), c.kernel_size, c.stride,
                              c.dilation, c.is_causal, add_k=c.add_k, add_v=c.add_v)
    return [t.grad for t in leaves], want


@pytest.mark.parametrize("name", CASES)
def test_fp32_gradients_match_the_oracle(name):
    got, want = _grads(na_cases()[name], torch.float32)
    for g, w in zip(got, want):
        assert g.dtype == torch.float32 and tuple(g.shape) == w.shape
        assert np.abs(g.cpu().numpy() - w).max() <= 2e-4 * max(1.0, np.abs(w).max())


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_16bit_gradients_match_the_oracle(name, dtype):
    got, want = _grads(na_cases()[name], dtype)
    for g, w in zip(got, want):
        assert g.dtype == dtype
        assert np.abs(g.float().cpu().numpy() - w).max() <= 2e-2 * max(1.0, np.abs(w).max())


def test_layer_trains():
    torch.manual_seed(1)
    layer = nb.NeighborhoodAttention2D(128, 2, (5, 5), dilation=(1, 2)).cuda()
    x = torch.randn(2, 12, 14, 128, device="cuda", requires_grad=True)
    layer(x).square().mean().backward()
    assert L.device_status() == 0
    for p in list(layer.parameters()) + [x]:
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().max() > 0


@pytest.mark.parametrize("shape,ks,st,di,ca,hq,hkv,D,n_extra", [
    ((700,), (65,), (3,), (1,), (True,), 2, 2, 128, 0),
    ((1000,), (33,), (1,), (2,), (False,), 4, 2, 64, 0),            # dilation groups, GQA
    ((40, 44), (7, 9), (1, 2), (2, 3), (False, True), 2, 1, 128, 0),
    ((64, 64), (16, 16), (8, 8), (1, 1), (False, False), 1, 1, 128, 0),   # block-sparse windows
    ((37, 51), (5, 5), (1, 1), (4, 8), (False, False), 2, 2, 64, 0),
    ((6, 20, 24), (3, 5, 8), (1, 1, 4), (1, 2, 1), (True, False, False), 2, 2, 128, 0),
    ((9, 11, 13), (3, 3, 3), (1, 1, 1), (3, 2, 4), (False, True, False), 4, 2, 64, 0),
    ((32, 32), (8, 8), (4, 4), (1, 1), (False, False), 2, 2, 128, 256),   # config 4 scaled
    ((30, 26), (5, 7), (1, 1), (2, 3), (False, True), 4, 2, 64, 130),     # ragged extras, GQA
    ((700,), (65,), (3,), (1,), (True,), 2, 1, 128, 7),
    ((6, 10, 12), (3, 4, 5), (1, 2, 1), (1, 1, 1), (True, False, False), 1, 1, 64, 300),
    ((33, 30), (3, 5), (1, 2), (3, 2), (False, True), 4, 2, 32, 0),       # head dim 32: zero-padded
    ((500,), (21,), (1,), (1,), (True,), 2, 2, 96, 19),                   # head dim 96 -> 128
    # more work items than CTAs: every CTA carries its ring positions, barrier phases and the
    # parity of its S / dP regions from one row tile to the next
    ((12000,), (129,), (1,), (1,), (True,), 2, 2, 128, 0),
    ((9000,), (200,), (7,), (1,), (False,), 4, 2, 64, 40),
    ((96, 96), (9, 9), (1, 1), (1, 1), (False, True), 2, 2, 128, 0),
    ((10, 40, 48), (3, 5, 8), (1, 1, 4), (1, 1, 1), (True, False, False), 2, 1, 128, 130),
    # window = whole layout with extra tokens attached: stays on the neighborhood kernels (dense
    # attention with more keys than queries has no backward)
    ((12, 20), (12, 20), (1, 1), (1, 1), (False, False), 2, 2, 64, 50),
    ((300,), (300,), (1,), (1,), (False,), 2, 1, 128, 33),
])
def test_tensor_core_backward_against_oracle_and_cuda_core_kernels(shape, ks, st, di, ca, hq, hkv,
                                                                   D, n_extra):
    """The tcgen05 backward (two passes of one kernel) against the oracle, and against the
    CUDA-core gradient kernels on the same inputs (independent implementations)."""
    import natten_b200.functional as F
    torch.manual_seed(23)
    fn = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[len(shape)]
    q = torch.randn(2, *shape, hq, D).bfloat16()
    k, v = (torch.randn(2, *shape, hkv, D).bfloat16() for _ in range(2))
    d_out = torch.randn(2, *shape, hq, D).bfloat16()
    extras = [torch.randn(2, n_extra, hkv, D).bfloat16() for _ in range(2)] if n_extra else []
    assert F.backward_layout_supported(*F.choose_backward_tile_shapes(shape, ks, st, di, ca), di)
    grads = {}
    for mode in (False, True):
        F.BACKWARD_ON_CUDA_CORES = mode
        try:
            leaves = [t.cuda().requires_grad_() for t in [q, k, v] + extras]
            out = fn(leaves[0], leaves[1], leaves[2], kernel_size=ks, stride=st, dilation=di,
                     is_causal=ca, additional_keys=leaves[3] if n_extra else None,
                     additional_values=leaves[4] if n_extra else None)
            out.backward(d_out.cuda())
            assert L.device_status() == 0
            grads[mode] = [t.grad.float().cpu().numpy() for t in leaves]
        finally:
            F.BACKWARD_ON_CUDA_CORES = False
    want = oracle.na_backward(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                              d_out.float().numpy(), ks, st, di, ca,
                              add_k=extras[0].float().numpy() if n_extra else None,
                              add_v=extras[1].float().numpy() if n_extra else None)
    assert len(want) == len(grads[False]) == (5 if n_extra else 3)
    for tc, cc, w in zip(grads[False], grads[True], want):
        tol = 2e-2 * max(1.0, np.abs(w).max())
        assert np.isfinite(tc).all()
        assert np.abs(tc - w).max() <= tol
        assert np.abs(cc - w).max() <= tol


def test_compiled_training_step_matches_eager():
    """torch.compile (AOT autograd) traces the registered backward too: gradients of a compiled
    layer equal the eager ones."""
    torch.manual_seed(3)
    layer = nb.NeighborhoodAttention2D(128, 2, (7, 5), stride=(1, 2), is_causal=(False, True)).cuda().bfloat16()
    x = torch.randn(2, 20, 24, 128, device="cuda").bfloat16()
    grads = []
    for fn in (layer, torch.compile(layer, fullgraph=True)):
        layer.zero_grad()
        xi = x.clone().requires_grad_()
        fn(xi).float().square().mean().backward()
        grads.append([xi.grad.float()] + [p.grad.float().clone() for p in layer.parameters()])
    assert L.device_status() == 0
    for a, b in zip(*grads):
        assert torch.allclose(a, b, rtol=1e-2, atol=1e-3 * max(1.0, a.abs().max().item()))
