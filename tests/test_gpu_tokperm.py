"""Token permute / unpermute kernels through the C ABI: bit-exact against the reference's own
outputs (tests/golden/tokperm_cases.json) and against the numpy oracle on further shapes."""
import hashlib

import numpy as np
import pytest
import torch

import natten_b200 as nb
import oracle
from golden_io import pattern, tokperm_cases

pytestmark = pytest.mark.gpu

_TORCH_INT = {16: torch.int16, 32: torch.int32}
_TORCH_FLT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def _input(case):
    bits = 32 if case["dtype"] == "fp32" else 16
    n = case["B"] * int(np.prod(case["shape"])) * case["H"] * case["D"]
    raw = pattern(n, bits)
    t = torch.from_numpy(raw.view(np.int16 if bits == 16 else np.int32).copy())
    x = t.view(_TORCH_FLT[case["dtype"]]).reshape(case["B"], *case["shape"], case["H"], case["D"])
    return x.cuda(), bits


@pytest.mark.parametrize("idx", range(len(tokperm_cases())))
def test_tokperm_matches_reference_bits(idx):
    case = tokperm_cases()[idx]
    x, bits = _input(case)
    y, layout, post = nb.token_permute_operation(x, tuple(case["tile"]), tuple(case["dilation"]),
                                                 flip_tiled_dims=case["flip"])
    assert list(y.shape) == case["out_shape"]
    assert list(post) == case["post_dilation"] and list(layout) == list(case["shape"])
    yb = y.contiguous().view(_TORCH_INT[bits]).cpu().numpy()
    assert hashlib.sha256(yb.tobytes()).hexdigest() == case["sha256"]
    back = nb.token_unpermute_operation(y, tuple(case["shape"]), tuple(case["tile"]),
                                        tuple(case["dilation"]), flip_tiled_dims=case["flip"])
    assert torch.equal(back.view(_TORCH_INT[bits]), x.view(_TORCH_INT[bits]))


@pytest.mark.parametrize("shape,tile,dil,H,D,dtype", [
    ((128, 128), (16, 16), (2, 2), 4, 128, torch.bfloat16),     # config-3 tiling, fewer heads
    ((64, 64), (8, 16), (1, 1), 3, 128, torch.float16),         # config-4 tiling
    ((8, 48, 80), (2, 8, 8), (1, 1, 1), 2, 128, torch.bfloat16),  # config-5 tiling, fewer frames
    ((37, 29), (4, 64), (1, 1), 2, 24, torch.float32),          # ragged, heavy padding
    ((1000,), (256,), (1,), 5, 1, torch.float32),               # LSE-like rows (D = 1), 20-byte rows
    ((33, 17), (16, 16), (2, 3), 3, 1, torch.float32),          # 12-byte rows: 4-byte vectors
    ((50,), (128,), (3,), 1, 7, torch.bfloat16),                # 14-byte rows: 2-byte vectors
])
def test_tokperm_matches_oracle(shape, tile, dil, H, D, dtype):
    torch.manual_seed(0)
    B = 2
    x = torch.randn(B, *shape, H, D).to(dtype)
    ibits = torch.int16 if dtype != torch.float32 else torch.int32
    xn = x.view(ibits).numpy()
    want = oracle.token_permute(xn, tile, dil, flip=True)
    y, _, _ = nb.token_permute_operation(x.cuda(), tile, dil)
    got = y.view(ibits).cpu().numpy()
    assert got.shape == want.shape
    assert np.array_equal(got, want)
    back = nb.token_unpermute_operation(y, shape, tile, dil)
    assert np.array_equal(back.view(ibits).cpu().numpy(), xn)


def test_permute_1d_identity_is_a_view():
    x = torch.randn(2, 512, 3, 8, device="cuda")
    y, _, post = nb.token_permute_operation(x, (256,), (1,))
    assert y.data_ptr() == x.data_ptr() and post == (512,)


def test_full_size_config3_round_trip_and_padding_is_zero():
    """BASELINE config 3 shape (bf16, 8 x 128 x 128 x 16 x 128): size-independent properties."""
    torch.manual_seed(1)
    x = torch.randn(8, 128, 128, 16, 128, device="cuda", dtype=torch.bfloat16)
    y, _, post = nb.token_permute_operation(x, (16, 16), (2, 2))
    assert y.shape == (32, 64 * 64, 16, 128)
    # a permutation without padding preserves the multiset of elements: compare checksums
    assert torch.equal(y.view(torch.int16).to(torch.int64).sum(), x.view(torch.int16).to(torch.int64).sum())
    back = nb.token_unpermute_operation(y, (128, 128), (16, 16), (2, 2))
    assert torch.equal(back.view(torch.int16), x.view(torch.int16))
    # spot check the index map: group (1, 0), tile (2, 3), in-tile (5, 7), flip => axis 0 fastest
    b, g0, g1, r0, r1, t0, t1 = 3, 1, 0, 2, 3, 5, 7
    bp = b * 4 + (g0 + 2 * g1)
    s = (r0 + 4 * r1) * 256 + (t0 + 16 * t1)
    src = x[b, (r0 * 16 + t0) * 2 + g0, (r1 * 16 + t1) * 2 + g1]
    assert torch.equal(y[bp, s].view(torch.int16), src.view(torch.int16))
