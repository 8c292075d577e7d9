"""8-bit float operands (e4m3 / e5m2, head dim 128) on the tensor-core kernel against the oracle
fed the same (already rounded) inputs.

The reference's own test accepts 5e-1 (e4m3) / 9e-1 (e5m2) absolute error for this path
(tests/test_blackwell_fna.py:104-109). The bounds here are tighter and follow from the arithmetic:
logits and LSE are exact products of 8-bit values accumulated in fp32 (2e-2 like the 16-bit
paths); P is rounded to e4m3 before P.V and O to the operand type, so the output carries one
rounding of its own magnitude (2^-4 relative for e4m3, 2^-3 for e5m2)."""
import numpy as np
import pytest
import torch

import natten_b200 as nb
import natten_b200._lib as L
import oracle

pytestmark = pytest.mark.gpu

# per element: |error| <= rel * |expected| + floor (rel = half a unit in the last place of the
# output type; floor covers the e4m3 rounding of P); plus a bound on the mean error
OUT_TOL = {torch.float8_e4m3fn: (2.0 ** -4, 0.08, 0.02), torch.float8_e5m2: (2.0 ** -3, 0.12, 0.04)}


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("shape,ks,st,di,ca,n_extra,hq,hkv,layout", [
    ((1024,), (128,), (1,), (1,), (True,), 0, 2, 2, "direct"),
    ((700,), (65,), (3,), (2,), (False,), 40, 4, 2, "direct"),
    ((40, 44), (7, 9), (1, 2), (2, 3), (False, True), 0, 2, 1, "direct"),
    ((40, 44), (7, 9), (1, 2), (2, 3), (False, True), 130, 2, 2, "permuted"),
    ((64, 64), (16, 16), (8, 8), (1, 1), (False, False), 0, 1, 1, "direct"),
    ((6, 20, 24), (3, 5, 8), (1, 1, 4), (1, 2, 1), (True, False, False), 0, 2, 2, "direct"),
    ((256,), (256,), (1,), (1,), (False,), 0, 2, 2, "direct"),          # self-attention path
])
def test_fp8_forward_matches_oracle(dtype, shape, ks, st, di, ca, n_extra, hq, hkv, layout):
    torch.manual_seed(41)
    D = 128
    fn = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[len(shape)]
    q = torch.randn(2, *shape, hq, D).to(dtype)
    k, v = (torch.randn(2, *shape, hkv, D).to(dtype) for _ in range(2))
    ak = av = None
    if n_extra:
        ak, av = (torch.randn(2, n_extra, hkv, D).to(dtype) for _ in range(2))
    out, lse = fn(q.cuda(), k.cuda(), v.cuda(), kernel_size=ks, stride=st, dilation=di,
                  is_causal=ca, additional_keys=ak.cuda() if n_extra else None,
                  additional_values=av.cuda() if n_extra else None, return_lse=True,
                  attention_kwargs={"permuted_layout": True} if layout == "permuted" else None)
    assert L.device_status() == 0
    assert out.dtype == dtype and lse.dtype == torch.float32
    want_o, want_l = oracle.na_forward(
        q.float().numpy(), k.float().numpy(), v.float().numpy(), ks, st, di, ca,
        add_k=ak.float().numpy() if n_extra else None, add_v=av.float().numpy() if n_extra else None)
    err = np.abs(out.float().cpu().numpy() - want_o)
    assert np.isfinite(err).all()
    rel, floor, mean = OUT_TOL[dtype]
    assert (err <= rel * np.abs(want_o) + floor).all() and err.mean() <= mean
    assert np.abs(lse.cpu().numpy() - want_l).max() <= 2e-2


@pytest.mark.parametrize("D", [16, 64, 96])
def test_fp8_head_dims_below_128_run_zero_padded(D):
    """The reference's Blackwell kernels take 8-bit operands with every head dim that is a multiple
    of 16 (csrc/src/blackwell_fna_forward.cu:178-191); here they are zero-padded to 128."""
    torch.manual_seed(42)
    dtype = torch.float8_e4m3fn
    shape, ks, st, ca = (24, 40), (7, 9), (1, 2), (False, True)
    q, k, v = (torch.randn(1, *shape, 2, D).to(dtype) for _ in range(3))
    out, lse = nb.na2d(q.cuda(), k.cuda(), v.cuda(), kernel_size=ks, stride=st, is_causal=ca,
                       return_lse=True)
    assert L.device_status() == 0
    assert out.shape == q.shape and out.dtype == dtype
    want_o, want_l = oracle.na_forward(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                                       ks, st, 1, ca)
    err = np.abs(out.float().cpu().numpy() - want_o)
    rel, floor, mean = OUT_TOL[dtype]
    assert (err <= rel * np.abs(want_o) + floor).all() and err.mean() <= mean
    assert np.abs(lse.cpu().numpy() - want_l).max() <= 2e-2


def test_fp8_head_dim_must_be_a_multiple_of_16():
    q = torch.randn(1, 64, 2, 40, device="cuda").to(torch.float8_e4m3fn)
    with pytest.raises(NotImplementedError):
        nb.na1d(q, q, q, kernel_size=9)
