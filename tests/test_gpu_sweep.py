"""Seeded random sweep over problem parameters, forward and backward against the oracle - the
counterpart of the reference's randomized sweep (tests/test_blackwell_fna.py:445-503): random
rank, token layout, window, stride, dilation, causal flags, head counts (GQA), head dim, operand
type and extra tokens. Tolerances: 2e-2 for output, logsumexp and gradients (relative to the
largest gradient entry), as everywhere for 16-bit operands.

A second sweep runs the forward alone (no gradient: the operands are then read as they lie) on
head dims the kernels are not built for - multiples of 8 below 128 - and on 8-bit operands (head
dims that are multiples of 16), with the 8-bit tolerances of tests/test_gpu_fp8.py.

NATTEN_B200_SWEEP_CASES (default 48 and 32) and NATTEN_B200_SWEEP_SEED (default 1000) scale the
two sweeps for an occasional long run; 1000 + 600 cases from seeds 7000 / 9000 took six minutes
and found nothing."""
import os
import random

import numpy as np
import pytest
import torch

import natten_b200 as nb
import natten_b200._lib as L
import oracle

pytestmark = pytest.mark.gpu


def _random_problem(rng: random.Random):
    nd = rng.choice([1, 1, 2, 2, 3])
    budget = rng.choice([600, 1500, 3000])                  # tokens, keeps the oracle fast
    side = max(4, int(round(budget ** (1.0 / nd))))
    shape, ks, st, di, ca = [], [], [], [], []
    for _ in range(nd):
        x = rng.randint(max(4, side // 2), side * 2 if nd > 1 else budget)
        d = rng.choice([1, 1, 1, 2, 3]) if x >= 12 else 1
        k = rng.randint(2, max(2, min(x // d, 2 * side)))
        s = rng.randint(1, k) if rng.random() < 0.4 else 1
        shape.append(x); ks.append(k); st.append(s); di.append(d)
        ca.append(rng.random() < 0.3)
    if all(k * d == x for k, d, x in zip(ks, di, shape)) and nd == 1 and not any(ca):
        ks[0] = max(2, ks[0] - 1)                             # keep it off the dense fast path
    hkv = rng.choice([1, 2])
    hq = hkv * rng.choice([1, 1, 2])
    return dict(shape=tuple(shape), ks=tuple(ks), st=tuple(st), di=tuple(di), ca=tuple(ca), hq=hq,
                hkv=hkv, D=rng.choice([64, 128]), dtype=rng.choice([torch.bfloat16, torch.float16]),
                n_extra=rng.choice([0, 0, 0, rng.randint(1, 200)]), B=rng.choice([1, 2]))


N_CASES = int(os.environ.get("NATTEN_B200_SWEEP_CASES", "0"))
SEED = int(os.environ.get("NATTEN_B200_SWEEP_SEED", "1000"))
PROBLEMS = [_random_problem(random.Random(SEED + i)) for i in range(N_CASES or 48)]


@pytest.mark.parametrize("idx", range(len(PROBLEMS)))
def test_random_problem_forward_and_backward(idx):
    pr = PROBLEMS[idx]
    torch.manual_seed(500 + idx)
    fn = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[len(pr["shape"])]
    B, D, dt = pr["B"], pr["D"], pr["dtype"]
    q = torch.randn(B, *pr["shape"], pr["hq"], D).to(dt)
    k, v = (torch.randn(B, *pr["shape"], pr["hkv"], D).to(dt) for _ in range(2))
    ak = av = None
    if pr["n_extra"]:
        ak, av = (torch.randn(B, pr["n_extra"], pr["hkv"], D).to(dt) for _ in range(2))
    leaves = [t.cuda().requires_grad_() for t in (q, k, v)] + (
        [t.cuda().requires_grad_() for t in (ak, av)] if pr["n_extra"] else [])
    kwargs = dict(kernel_size=pr["ks"], stride=pr["st"], dilation=pr["di"], is_causal=pr["ca"],
                  additional_keys=leaves[3] if pr["n_extra"] else None,
                  additional_values=leaves[4] if pr["n_extra"] else None, return_lse=True)
    if idx % 3 == 2:
        kwargs["attention_kwargs"] = {"permuted_layout": True}   # the reference's flow as well
    out, lse = fn(leaves[0], leaves[1], leaves[2], **kwargs)
    d_out = torch.randn(out.shape).to(dt)
    out.backward(d_out.cuda())
    assert L.device_status() == 0
    f32 = [t.float().numpy() for t in (q, k, v)]
    ex = dict(add_k=ak.float().numpy(), add_v=av.float().numpy()) if pr["n_extra"] else {}
    want_o, want_l = oracle.na_forward(*f32, pr["ks"], pr["st"], pr["di"], pr["ca"], **ex)
    assert np.abs(out.detach().float().cpu().numpy() - want_o).max() <= 2e-2, pr
    assert np.abs(lse.detach().cpu().numpy() - want_l).max() <= 2e-2, pr
    want_g = oracle.na_backward(*f32, d_out.float().numpy(), pr["ks"], pr["st"], pr["di"], pr["ca"],
                                **ex)
    for leaf, w in zip(leaves, want_g):
        g = leaf.grad.float().cpu().numpy()
        assert np.isfinite(g).all(), pr
        assert np.abs(g - w).max() <= 2e-2 * max(1.0, np.abs(w).max()), pr


FP8_TOL = {torch.float8_e4m3fn: (2.0 ** -4, 0.08), torch.float8_e5m2: (2.0 ** -3, 0.12)}


def _narrow_problem(seed: int):
    rng = random.Random(seed)
    pr = _random_problem(rng)
    if rng.random() < 0.25:
        pr["D"] = rng.choice([16, 32, 64, 96, 128])
        pr["dtype"] = rng.choice([torch.float8_e4m3fn, torch.float8_e5m2])
    else:
        pr["D"] = rng.choice([8, 16, 24, 32, 40, 48, 56, 72, 88, 96, 104, 120])
    return pr


NARROW = [_narrow_problem(SEED + 50000 + i) for i in range(N_CASES or 32)]


@pytest.mark.parametrize("idx", range(len(NARROW)))
def test_random_problem_narrow_head_dim_or_8bit_forward(idx):
    pr = NARROW[idx]
    torch.manual_seed(900 + idx)
    fn = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[len(pr["shape"])]
    B, D, dt = pr["B"], pr["D"], pr["dtype"]
    f8 = dt in FP8_TOL

    def make(*shape):
        return (torch.randn(*shape) * (0.5 if f8 else 1.0)).to(dt)

    q = make(B, *pr["shape"], pr["hq"], D)
    k, v = (make(B, *pr["shape"], pr["hkv"], D) for _ in range(2))
    ak = av = None
    if pr["n_extra"]:
        ak, av = (make(B, pr["n_extra"], pr["hkv"], D) for _ in range(2))
    kwargs = dict(kernel_size=pr["ks"], stride=pr["st"], dilation=pr["di"], is_causal=pr["ca"],
                  additional_keys=ak.cuda() if pr["n_extra"] else None,
                  additional_values=av.cuda() if pr["n_extra"] else None, return_lse=True)
    if idx % 3 == 2:
        kwargs["attention_kwargs"] = {"permuted_layout": True}
    out, lse = fn(q.cuda(), k.cuda(), v.cuda(), **kwargs)
    assert L.device_status() == 0
    assert out.shape == q.shape and out.dtype == dt
    ex = dict(add_k=ak.float().numpy(), add_v=av.float().numpy()) if pr["n_extra"] else {}
    want_o, want_l = oracle.na_forward(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                                       pr["ks"], pr["st"], pr["di"], pr["ca"], **ex)
    got = out.float().cpu().numpy()
    err_l = np.abs(lse.cpu().numpy() - want_l).max()
    if f8:
        rel, floor = FP8_TOL[dt]
        assert (np.abs(got - want_o) - rel * np.abs(want_o)).max() <= floor, pr
        assert err_l <= 4e-2, pr
    else:
        assert np.abs(got - want_o).max() <= 2e-2, pr
        assert err_l <= 2e-2, pr
