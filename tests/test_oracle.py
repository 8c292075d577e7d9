"""Pins the CPU oracle against outputs of the reference package itself (tests/golden/)."""
import hashlib

import numpy as np
import pytest

import oracle
from golden_io import attn_cases, na_case_names, na_cases, pattern, tokperm_cases

# fp32 flex path of the reference vs the double-accumulating oracle
ATOL_OUT = 2e-6
ATOL_LSE = 4e-6


@pytest.mark.parametrize("name", na_case_names())
def test_na_oracle_matches_reference(name):
    c = na_cases()[name]
    out, lse = oracle.na_forward(c.q, c.k, c.v, c.kernel_size, c.stride, c.dilation, c.is_causal,
                                 add_k=c.add_k, add_v=c.add_v)
    assert out.shape == c.out.shape and lse.shape == c.lse.shape
    assert np.abs(out - c.out).max() <= ATOL_OUT
    assert np.abs(lse - c.lse).max() <= ATOL_LSE


def test_na_oracle_fp32_accumulation_and_row_sample():
    c = na_cases()["c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT"]
    tok = np.array([0, 1, 19, 20, 239, 240, 1000, 1919], dtype=np.int64)
    out, lse = oracle.na_forward(c.q, c.k, c.v, c.kernel_size, c.stride, c.dilation, c.is_causal,
                                 tok_idx=tok, acc64=False)
    ref_o = c.out.reshape(1, -1, *c.out.shape[-2:])[:, tok]
    ref_l = c.lse.reshape(1, -1, c.lse.shape[-1])[:, tok]
    assert np.abs(out - ref_o).max() <= 1e-5
    assert np.abs(lse - ref_l).max() <= 1e-5


def test_na_oracle_rejects_bad_args():
    q = np.zeros((1, 8, 1, 8), np.float32)
    with pytest.raises(ValueError):
        oracle.na_forward(q, q, q, kernel_size=9)       # k*d > X
    with pytest.raises(ValueError):
        oracle.na_forward(q, q, q, kernel_size=3, stride=4)  # s > k
    with pytest.raises(ValueError):
        oracle.na_forward(q, q, q, kernel_size=1)       # k < 2


def test_dense_oracle_matches_reference_attention():
    z, meta = attn_cases()
    for name, m in meta.items():
        q, k, v = (z[f"attn/{name}/{t}"] for t in "qkv")
        out, lse = oracle.dense_attention(q, k, v, is_causal=m["is_causal"])
        assert np.abs(out - z[f"attn/{name}/out"]).max() <= ATOL_OUT
        assert np.abs(lse - z[f"attn/{name}/lse"]).max() <= ATOL_LSE


def test_merge_oracle_matches_reference():
    z, _ = attn_cases()
    o, l = oracle.merge(z["merge/merge2/o0"], z["merge/merge2/l0"], z["merge/merge2/o1"],
                        z["merge/merge2/l1"])
    assert np.abs(o - z["merge/merge2/out"]).max() <= 1e-6
    assert np.abs(l - z["merge/merge2/lse"]).max() <= 1e-6
    # three-way: the reference folds inputs left to right (attn_merge.py:89-95)
    o, l = oracle.merge(z["merge/merge3/o0"], z["merge/merge3/l0"], z["merge/merge3/o1"],
                        z["merge/merge3/l1"])
    o, l = oracle.merge(o, l, z["merge/merge3/o2"], z["merge/merge3/l2"])
    assert np.abs(o - z["merge/merge3/out"]).max() <= 1e-6
    assert np.abs(l - z["merge/merge3/lse"]).max() <= 1e-6


def test_extra_kv_equals_na_plus_dense_plus_merge():
    """The reference composes extra KV as FNA + dense attention + merge
    (src/natten/functional.py:524-559); the oracle's fused rule must agree with that."""
    c = na_cases()["c4s_na2d_32x32_k8_s4_extra24"]
    o1, l1 = oracle.na_forward(c.q, c.k, c.v, c.kernel_size, c.stride, c.dilation, c.is_causal)
    B, H, D = c.q.shape[0], c.q.shape[-2], c.q.shape[-1]
    o2, l2 = oracle.dense_attention(c.q.reshape(B, -1, H, D), c.add_k, c.add_v)
    o, l = oracle.merge(o1.reshape(B, -1, H, D), l1.reshape(B, -1, H), o2, l2)
    assert np.abs(o.reshape(c.out.shape) - c.out).max() <= 5e-6
    assert np.abs(l.reshape(c.lse.shape) - c.lse).max() <= 5e-6


def _pattern_input(case):
    bits = 32 if case["dtype"] == "fp32" else 16
    n = case["B"] * int(np.prod(case["shape"])) * case["H"] * case["D"]
    return pattern(n, bits).reshape(case["B"], *case["shape"], case["H"], case["D"])


@pytest.mark.parametrize("idx", range(len(tokperm_cases())))
def test_tokperm_oracle_matches_reference(idx):
    case = tokperm_cases()[idx]
    x = _pattern_input(case)
    y = oracle.token_permute(x, case["tile"], case["dilation"], flip=case["flip"])
    assert list(y.shape) == case["out_shape"]
    assert hashlib.sha256(np.ascontiguousarray(y).tobytes()).hexdigest() == case["sha256"]
    back = oracle.token_unpermute(y, case["shape"], case["tile"], case["dilation"],
                                  flip=case["flip"])
    assert np.array_equal(back, x)


# ---- backward -----------------------------------------------------------------------------------
# The reference's CPU-capable path refuses to differentiate ("FlexAttention does not support
# backward on CPU"), so no gradient fixtures can be generated from it. The backward oracle is tied
# to the pinned forward instead: a dense masked attention in torch (float64) whose forward matches
# the reference's own outputs in tests/golden/ is differentiated by torch.autograd, and the
# oracle's gradients must agree with it.

def _dense_twin(c):
    """torch float64 restatement of one golden case as dense attention under an explicit mask."""
    import torch
    from natten_b200.functional import group_extent, window_end, window_start
    shape = c.shape
    n = int(np.prod(shape))
    mask = torch.zeros(n, n + c.n_extra, dtype=torch.bool)
    mask[:, n:] = True
    coords = np.stack(np.unravel_index(np.arange(n), shape), axis=1)
    for qi, qc in enumerate(coords):
        axes = []
        for x, k, s, d, ca, X in zip(qc, c.kernel_size, c.stride, c.dilation, c.is_causal, shape):
            g, i = int(x) % d, int(x) // d
            L = group_extent(X, d, g)
            st = window_start(i, k, s, L, ca)
            axes.append([j * d + g for j in range(st, window_end(i, st, k, L, ca))])
        grid = np.stack(np.meshgrid(*axes, indexing="ij"), axis=-1).reshape(-1, len(shape))
        mask[qi, np.ravel_multi_index(tuple(grid.T), shape)] = True
    leaves = [torch.from_numpy(t).double().requires_grad_() for t in (c.q, c.k, c.v)]
    if c.n_extra:
        leaves += [torch.from_numpy(t).double().requires_grad_() for t in (c.add_k, c.add_v)]
    q, k, v = (t.flatten(1, len(shape)) for t in leaves[:3])
    if c.n_extra:
        k, v = torch.cat([k, leaves[3]], 1), torch.cat([v, leaves[4]], 1)
    rep = q.shape[2] // k.shape[2]
    k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * q.shape[-1] ** -0.5
    s = s.masked_fill(~mask, float("-inf"))
    out = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), v).reshape(c.out.shape)
    return leaves, out


@pytest.mark.parametrize("name", [
    "na1d_300_k33", "na1d_257_k9_s3_d4_causal", "na2d_33x30_k3x5_s1x2_d3x2_causal01",
    "na2d_16x16_k5_gqa", "c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT",
    "na3d_6x9x11_k3x3x5_s1x1x2_d2x1x1_causalW", "na1d_96_k17_causal_extra7"])
def test_backward_oracle_is_the_derivative_of_the_pinned_forward(name):
    import torch
    c = na_cases()[name]
    leaves, out = _dense_twin(c)
    # the twin's forward is the reference's forward ...
    assert np.abs(out.detach().numpy() - c.out).max() <= 4e-6
    torch.manual_seed(7)
    d_out = torch.randn(out.shape, dtype=torch.float64)
    out.backward(d_out)
    # ... so its autograd gradients are what the backward oracle must return
    got = oracle.na_backward(c.q, c.k, c.v, d_out.float().numpy(), c.kernel_size, c.stride,
                             c.dilation, c.is_causal, add_k=c.add_k, add_v=c.add_v)
    assert len(got) == len(leaves)
    for g, leaf in zip(got, leaves):
        want = leaf.grad.numpy()
        assert np.abs(g - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
