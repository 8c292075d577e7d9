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
