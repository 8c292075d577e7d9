"""Attention kernels through the public operators / C ABI against the reference's own outputs
(tests/golden/) and the CPU oracle.

Tolerances (max-abs, on output and logsumexp): 1e-4 for fp32 operands, 2e-2 for fp16/bf16."""
import ctypes

import numpy as np
import pytest
import torch

import natten_b200 as nb
import natten_b200._lib as L
import oracle
from golden_io import attn_cases, na_case_names, na_cases

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-4
TOL_16 = 2e-2


def _na_fn(nd):
    return {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[nd]


def _run(c, dtype, **kw):
    dev = "cuda"
    q, k, v = (torch.from_numpy(t).to(dev).to(dtype) for t in (c.q, c.k, c.v))
    ak = torch.from_numpy(c.add_k).to(dev).to(dtype) if c.n_extra else None
    av = torch.from_numpy(c.add_v).to(dev).to(dtype) if c.n_extra else None
    out, lse = _na_fn(len(c.shape))(q, k, v, kernel_size=c.kernel_size, stride=c.stride,
                                    dilation=c.dilation, is_causal=c.is_causal,
                                    additional_keys=ak, additional_values=av, return_lse=True,
                                    **kw)
    assert L.device_status() == 0
    assert out.dtype == dtype and lse.dtype == torch.float32
    return out.float().cpu().numpy(), lse.cpu().numpy()


@pytest.mark.parametrize("name", na_case_names())
def test_fp32_path_matches_reference(name):
    c = na_cases()[name]
    out, lse = _run(c, torch.float32)
    assert out.shape == c.out.shape and lse.shape == c.lse.shape
    assert np.abs(out - c.out).max() <= TOL_F32
    assert np.abs(lse - c.lse).max() <= TOL_F32


LAYOUTS = {"direct": None, "permuted": {"permuted_layout": True}}


@pytest.mark.parametrize("name", [n for n in na_case_names() if n != "c1_na2d_32x32_k7"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layout", list(LAYOUTS))
def test_16bit_path_matches_reference(name, dtype, layout):
    """bf16-exact operands on the tensor-core kernel (head dims other than 64/128 zero-padded).
    The tensor-core kernel is run both on the caller's layout (tensor-map gathers, the default)
    and on token-permuted copies (the reference's flow)."""
    c = na_cases()[name]
    out, lse = _run(c, dtype, attention_kwargs=LAYOUTS[layout])
    assert np.isfinite(out).all() and np.isfinite(lse).all()
    assert np.abs(out - c.out).max() <= TOL_16
    assert np.abs(lse - c.lse).max() <= TOL_16


@pytest.mark.parametrize("name,qt,kvt", [
    ("c3s_na2d_32x32_k13_d2", (16, 16), (16, 8)),
    ("c3s_na2d_32x32_k13_d2", (8, 32), (4, 32)),
    ("c3s_na2d_32x32_k13_d2", (64, 4), (2, 64)),
    ("c4s_na2d_32x32_k8_s4_extra24", (16, 16), (8, 16)),
    ("c4s_na2d_32x32_k8_s4_extra24", (256, 1), (1, 128)),
    ("c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT", (8, 4, 8), (4, 4, 8)),
    ("c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT", (2, 8, 16), (2, 8, 8)),
    ("c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT", (1, 16, 16), (1, 2, 64)),
    # 128-token query tiles: one 128-row tile per CTA, two CTAs per SM
    ("c3s_na2d_32x32_k13_d2", (8, 16), (4, 32)),
    ("c3s_na2d_32x32_k13_d2", (128, 1), (16, 8)),
    ("c4s_na2d_32x32_k8_s4_extra24", (8, 16), (8, 16)),
    ("c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT", (2, 8, 8), (2, 8, 8)),
    ("c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT", (1, 4, 32), (4, 4, 8)),
    ("c2s_na1d_1024_k128_causal", (128,), (128,)),
])
def test_tensor_core_kernel_with_explicit_tile_shapes(name, qt, kvt):
    c = na_cases()[name]
    for layout, kwargs in LAYOUTS.items():
        out, lse = _run(c, torch.bfloat16, q_tile_shape=qt, kv_tile_shape=kvt,
                        attention_kwargs=kwargs)
        assert np.abs(out - c.out).max() <= TOL_16, layout
        assert np.abs(lse - c.lse).max() <= TOL_16, layout


@pytest.mark.parametrize("shape,ks,st,di,ca,qt,kvt,n_extra,hq,hkv,D", [
    ((1000,), (33,), (1,), (2,), (False,), (256,), (128,), 0, 2, 2, 64),       # ragged, dilated 1-D
    ((777,), (100,), (7,), (1,), (True,), (256,), (128,), 50, 4, 2, 128),
    ((40, 44), (7, 9), (1, 2), (2, 3), (False, True), (16, 16), (16, 8), 0, 2, 1, 128),
    ((37, 51), (5, 5), (1, 1), (4, 8), (False, False), (8, 32), (4, 32), 130, 2, 2, 64),
    ((64, 64), (16, 16), (8, 8), (1, 1), (False, False), (2, 128), (1, 128), 0, 1, 1, 128),
    ((6, 20, 24), (3, 5, 8), (1, 1, 4), (1, 2, 1), (True, False, False), (2, 8, 16), (2, 8, 8), 0, 2, 2, 128),
    ((9, 11, 13), (3, 3, 3), (1, 1, 1), (3, 2, 4), (False, True, False), (4, 8, 8), (4, 4, 8), 17, 2, 2, 64),
    ((5, 7, 300), (2, 2, 31), (1, 1, 1), (1, 1, 2), (False, False, True), (1, 2, 128), (1, 1, 128), 0, 1, 1, 64),
])
def test_direct_layout_agrees_with_the_permuted_flow(shape, ks, st, di, ca, qt, kvt,
                                                     n_extra, hq, hkv, D):
    """The kernel reading the caller's layout through tensor maps (one launch, no scratch) against
    permute -> kernel -> unpermute with the same tile shapes; ragged extents, dilation groups of
    unequal size, GQA and extra tokens included. The two walk the keys in different tiles (gathered
    tiles start at the first attended key, permuted ones lie on the tile grid), so they agree to
    rounding, not bit for bit; both are checked against the oracle."""
    torch.manual_seed(33)
    q = torch.randn(2, *shape, hq, D).bfloat16()
    k, v = (torch.randn(2, *shape, hkv, D).bfloat16() for _ in range(2))
    ak = av = None
    if n_extra:
        ak, av = (torch.randn(2, n_extra, hkv, D).bfloat16() for _ in range(2))
    assert nb.direct_layout_supported(qt, kvt, di)
    args = (q.cuda(), k.cuda(), v.cuda(), ks, st, di, ca, D ** -0.5, qt, kvt,
            ak.cuda() if n_extra else None, av.cuda() if n_extra else None)
    o_d, l_d = nb.fna_forward_direct(*args)
    o_p, l_p = nb.fna_forward_permuted(*args)
    assert L.device_status() == 0
    assert (o_d.float() - o_p.float()).abs().max().item() <= TOL_16
    assert (l_d - l_p).abs().max().item() <= 1e-3
    want_o, want_l = oracle.na_forward(
        q.float().numpy(), k.float().numpy(), v.float().numpy(), ks, st, di, ca,
        add_k=ak.float().numpy() if n_extra else None, add_v=av.float().numpy() if n_extra else None)
    for o, l in ((o_d, l_d), (o_p, l_p)):
        assert np.abs(o.float().cpu().numpy() - want_o).max() <= TOL_16
        assert np.abs(l.cpu().numpy() - want_l).max() <= TOL_16


def test_direct_layout_limits():
    """A tile of one dilation group must fit a tensor-map box; beyond that the C entry refuses and
    the operator falls back to permuted copies."""
    assert not nb.direct_layout_supported((256,), (128,), (3,))
    assert nb.direct_layout_supported((256,), (128,), (2,))
    assert not nb.direct_layout_supported((16, 16), (16, 8), (1, 9))
    q = torch.randn(1, 1200, 2, 64, device="cuda").half()
    with pytest.raises(L.NattenB200Error) as e:
        nb.fna_forward_direct(q, q, q, (33,), (1,), (3,), (False,), 0.125, (256,), (128,))
    assert e.value.code == L.ERR_UNSUPPORTED
    out = nb.na1d(q, q, q, 33, dilation=3)     # permuted fallback
    assert L.device_status() == 0 and torch.isfinite(out.float()).all()


def test_dense_attention_matches_reference():
    z, meta = attn_cases()
    for name, m in meta.items():
        for dtype, tol in ((torch.float32, TOL_F32), (torch.bfloat16, TOL_16), (torch.float16, TOL_16)):
            q, k, v = (torch.from_numpy(z[f"attn/{name}/{t}"]).cuda().to(dtype) for t in "qkv")
            out, lse = nb.attention(q, k, v, is_causal=m["is_causal"], return_lse=True)
            assert L.device_status() == 0
            assert np.abs(out.float().cpu().numpy() - z[f"attn/{name}/out"]).max() <= tol, (name, dtype)
            assert np.abs(lse.cpu().numpy() - z[f"attn/{name}/lse"]).max() <= tol, (name, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_causal_attention_matches_oracle(dtype):
    """Causal dense attention is not runnable on the reference's CPU backend, so the pin here is
    the oracle (mask.hpp semantics for a full causal window)."""
    torch.manual_seed(5)
    q, k, v = (torch.randn(2, 300, 2, 64).bfloat16().float() for _ in range(3))
    want_o, want_l = oracle.dense_attention(q.numpy(), k.numpy(), v.numpy(), is_causal=True)
    out, lse = nb.attention(q.cuda().to(dtype), k.cuda().to(dtype), v.cuda().to(dtype),
                            is_causal=True, return_lse=True)
    tol = TOL_F32 if dtype == torch.float32 else TOL_16
    assert np.abs(out.float().cpu().numpy() - want_o).max() <= tol
    assert np.abs(lse.cpu().numpy() - want_l).max() <= tol
    # the 1-D full-window fast path of na1d takes the same route
    out2 = nb.na1d(q.cuda().to(dtype), k.cuda().to(dtype), v.cuda().to(dtype), kernel_size=300,
                   is_causal=True)
    assert torch.equal(out2, out)


def test_merge_matches_reference():
    z, _ = attn_cases()
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        outs = [torch.from_numpy(z[f"merge/merge3/o{i}"]).cuda().to(dtype) for i in range(3)]
        lses = [torch.from_numpy(z[f"merge/merge3/l{i}"]).cuda() for i in range(3)]
        if dtype == torch.float32:
            o2, l2 = nb.merge_attentions(
                [torch.from_numpy(z[f"merge/merge2/o{i}"]).cuda() for i in range(2)],
                [torch.from_numpy(z[f"merge/merge2/l{i}"]).cuda() for i in range(2)])
            assert np.abs(o2.cpu().numpy() - z["merge/merge2/out"]).max() <= tol
            assert np.abs(l2.cpu().numpy() - z["merge/merge2/lse"]).max() <= tol
        o3, l3 = nb.merge_attentions(outs, lses)
        assert np.abs(o3.float().cpu().numpy() - z["merge/merge3/out"]).max() <= max(tol, 2e-6) * 4
        assert np.abs(l3.cpu().numpy() - z["merge/merge3/lse"]).max() <= 4e-6


def test_merge_in_place_and_with_an_empty_input():
    """The merged output may overwrite one of its inputs (each element is read before it is
    written); an input without keys (LSE = -inf, O = 0) leaves the other one unchanged."""
    torch.manual_seed(4)
    o0, o1 = (torch.randn(3, 50, 2, 256, device="cuda") for _ in range(2))   # fp32, D = 256
    l0, l1 = (torch.randn(3, 50, 2, device="cuda") for _ in range(2))
    want_o, want_l = nb.merge_attentions([o0, o1], [l0, l1])
    got_l = torch.empty_like(l0)
    dst = o0.clone()
    L.check(L.lib.b200na_merge(ctypes.c_void_p(dst.data_ptr()), ctypes.c_void_p(l0.data_ptr()),
                               ctypes.c_void_p(o1.data_ptr()), ctypes.c_void_p(l1.data_ptr()),
                               ctypes.c_void_p(dst.data_ptr()), ctypes.c_void_p(got_l.data_ptr()),
                               l0.numel(), 256, L.F32,
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
            "b200na_merge")
    assert torch.equal(dst, want_o) and torch.equal(got_l, want_l)
    empty_l = torch.full_like(l1, float("-inf"))
    for order in (0, 1):
        outs = [o0, torch.zeros_like(o1)][::1 if order == 0 else -1]
        lses = [l0, empty_l][::1 if order == 0 else -1]
        m_o, m_l = nb.merge_attentions(outs, lses)
        assert torch.equal(m_o, o0) and torch.equal(m_l, l0)


def test_merge_equals_attention_over_concatenated_keys():
    """The property the reference's own merge test uses (tests/test_attn_merge.py:92-114)."""
    torch.manual_seed(2)
    q = torch.randn(1, 384, 2, 128, device="cuda").bfloat16()
    k = torch.randn(1, 640, 2, 128, device="cuda").bfloat16()
    v = torch.randn(1, 640, 2, 128, device="cuda").bfloat16()
    full, full_l = nb.attention(q, k, v, return_lse=True)
    parts = [nb.attention(q, k[:, a:b], v[:, a:b], return_lse=True) for a, b in ((0, 200), (200, 640))]
    m, ml = nb.merge_attentions([p[0] for p in parts], [p[1] for p in parts])
    assert (m.float() - full.float()).abs().max().item() <= TOL_16
    assert (ml - full_l).abs().max().item() <= 1e-2


FULL_CONFIGS = {
    # BASELINE configs 2-5 exactly as specified - full token layout, full batch and head counts on
    # the GPU (so every head offset of the tensor maps and every batch entry is exercised). The CPU
    # oracle computes a row sample of the first and the last head of every batch entry.
    # dtype, shape, batch, heads, kernel, stride, dilation, causal, extra tokens, input multiplier
    "c2_na1d": (torch.bfloat16, (32768,), 4, 16, (2048,), (1,), (1,), (True,), 0, 1.0),
    "c3_na2d": (torch.bfloat16, (128, 128), 8, 16, (13, 13), (1, 1), (2, 2), (False, False), 0, 1.0),
    "c4_na2d": (torch.float16, (256, 256), 1, 24, (32, 32), (16, 16), (1, 1), (False, False), 256, 0.5),
    "c5_na3d": (torch.bfloat16, (32, 48, 80), 1, 24, (16, 24, 24), (1, 8, 8), (1, 1, 1),
                (True, False, False), 0, 1.0),
}
FULL_ROWS = {"c2_na1d": 1024, "c3_na2d": 1024, "c4_na2d": 2048, "c5_na3d": 4096}


def _band_rows(shape, kernel, dilation, n_rows, seed):
    """Flat token indices: half uniform, half inside one (dilated) kernel size of an axis end,
    every axis and side in turn (windows clamped, shifted or cut by causality live there)."""
    rng = np.random.default_rng(seed)
    n_tok = int(np.prod(shape))
    picks = [rng.integers(0, n_tok, size=n_rows // 2), np.array([0, n_tok - 1])]
    nd = len(shape)
    per = max(1, (n_rows - n_rows // 2) // (2 * nd))
    for a in range(nd):
        band = min(kernel[a] * dilation[a], shape[a])
        for side in (0, 1):
            coords = [rng.integers(0, shape[b], size=per) for b in range(nd)]
            coords[a] = rng.integers(0, band, size=per) + (0 if side == 0 else shape[a] - band)
            picks.append(np.ravel_multi_index(coords, shape))
    return np.unique(np.concatenate(picks)).astype(np.int64)


@pytest.mark.parametrize("name", list(FULL_CONFIGS))
def test_full_size_configs_row_sample_against_oracle(name):
    dtype, shape, B, H, ks, st, di, ca, n_extra, mul = FULL_CONFIGS[name]
    D = 128
    nd = len(shape)
    g = torch.Generator(device="cuda").manual_seed(1000 + list(FULL_CONFIGS).index(name) + 1)
    q, k, v = ((torch.randn(B, *shape, H, D, generator=g, device="cuda") * mul).to(dtype)
               for _ in range(3))
    ak = av = None
    if n_extra:
        ak, av = (torch.randn(B, n_extra, H, D, generator=g, device="cuda").to(dtype)
                  for _ in range(2))
    out, lse = _na_fn(nd)(q, k, v, kernel_size=ks, stride=st, dilation=di, is_causal=ca,
                          additional_keys=ak, additional_values=av, return_lse=True)
    assert L.device_status() == 0
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    rows = _band_rows(shape, ks, di, FULL_ROWS[name], seed=7)
    idx = torch.from_numpy(rows).cuda()
    heads = sorted({0, H - 1})
    for b in range(B):
        qh, kh, vh = (t[b:b + 1][..., heads, :].float().cpu().numpy() for t in (q, k, v))
        akh = avh = None
        if n_extra:
            akh, avh = (t[b:b + 1][..., heads, :].float().cpu().numpy() for t in (ak, av))
        want_o, want_l = oracle.na_forward(qh, kh, vh, ks, st, di, ca, add_k=akh, add_v=avh,
                                           tok_idx=rows)
        got_o = out[b].flatten(0, nd - 1)[idx][:, heads].float().cpu().numpy()
        got_l = lse[b].flatten(0, nd - 1)[idx][:, heads].cpu().numpy()
        assert np.abs(got_o - want_o[0]).max() <= TOL_16, b
        assert np.abs(got_l - want_l[0]).max() <= TOL_16, b


def test_tensor_core_kernel_agrees_with_cuda_core_kernel_on_every_row():
    """Full-tensor cross-check of the two independent kernels at a mid-size 3-D problem with
    causal, strided and ragged axes (every query row, not a sample)."""
    torch.manual_seed(3)
    shape, ks, st, di, ca = (10, 27, 45), (4, 9, 12), (1, 3, 4), (1, 1, 2), (True, False, False)
    q, k, v = (torch.randn(1, *shape, 2, 128, device="cuda").bfloat16() for _ in range(3))
    o_tc, l_tc = nb.na3d(q, k, v, ks, st, di, ca, return_lse=True)
    o_cc, l_cc = nb.na3d(q.float(), k.float(), v.float(), ks, st, di, ca, return_lse=True)
    assert L.device_status() == 0
    assert (o_tc.float() - o_cc).abs().max().item() <= TOL_16
    assert (l_tc - l_cc).abs().max().item() <= TOL_16


@pytest.mark.parametrize("shape,ks,st,ca,world", [
    ((32, 12, 20), (16, 6, 6), (1, 2, 2), (True, False, False), 8),   # config 5 scaled, T sharded
    ((24, 16, 16), (7, 5, 5), (1, 1, 1), (False, False, False), 4),   # two-sided halo
    ((4096,), (512,), (64,), (False,), 4),
])
def test_spatial_slabs_reproduce_the_unsharded_result(shape, ks, st, ca, world):
    """Every rank's slab (ranks emulated one after the other on this GPU; the halo is sliced from
    the global tensors) equals the unsharded rows: one launch on the slabs as they lie, the same
    through token-permuted copies, and the overlapped form - partial attention over the rank's
    own frames and over each halo block (windows cut to the block), folded with the LSE merge."""
    from natten_b200 import sharding
    torch.manual_seed(11)
    q, k, v = (torch.randn(1, *shape, 2, 128, device="cuda").bfloat16() for _ in range(3))
    fn = _na_fn(len(shape))
    nd = len(shape)
    full_o, full_l = fn(q, k, v, ks, st, 1, ca, return_lse=True)
    plan = sharding.make_halo_plan(shape[0], world, ks[0], st[0], ca[0])
    for r in range(world):
        t0, t1 = plan.slabs[r]
        lo, hi = plan.needs[r]
        ql = q[:, t0:t1].contiguous()
        for permuted in (False, True):
            o, l = sharding.fna_forward_slab(ql, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(),
                                             shape, t0, lo, ks, st, ca, permuted=permuted)
            assert L.device_status() == 0
            # slab and unsharded call tile the keys differently: equal up to bf16 rounding of O
            assert (o.float() - full_o[:, t0:t1].float()).abs().max().item() <= 1e-2, (r, permuted)
            assert (l - full_l[:, t0:t1]).abs().max().item() <= 2e-3, (r, permuted)
        # own frames first, then the frames before and after the slab, merged
        o, l = sharding.fna_forward_slab(ql, k[:, t0:t1].contiguous(), v[:, t0:t1].contiguous(),
                                         shape, t0, t0, ks, st, ca, clip=True)
        o, l = o.flatten(1, nd), l.flatten(1, nd)
        for a, b in ((lo, t0), (t1, hi)):
            if b <= a:
                continue
            o2, l2 = sharding.fna_forward_slab(ql, k[:, a:b].contiguous(), v[:, a:b].contiguous(),
                                               shape, t0, a, ks, st, ca, clip=True)
            o, l = nb.merge_attentions([o, o2.flatten(1, nd)], [l, l2.flatten(1, nd)])
        assert L.device_status() == 0
        assert torch.isfinite(l).all()
        assert (o.float() - full_o[:, t0:t1].flatten(1, nd).float()).abs().max().item() <= 1.6e-2, r
        assert (l - full_l[:, t0:t1].flatten(1, nd)).abs().max().item() <= 2e-3, r
    # a slab that does not hold every needed key is refused, not silently wrong
    t0, t1 = plan.slabs[world - 1]
    lo, hi = plan.needs[world - 1]
    with pytest.raises(L.NattenB200Error):
        sharding.fna_forward_slab(q[:, t0:t1].contiguous(), k[:, lo + 1:hi].contiguous(),
                                  v[:, lo + 1:hi].contiguous(), shape, t0, lo + 1, ks, st, ca)


@pytest.mark.parametrize("shape,ks,st,di,ca", [
    ((40, 44), (7, 9), (1, 2), (2, 1), (False, True)),
    ((6, 20, 24), (3, 5, 8), (1, 1, 4), (1, 1, 1), (True, False, False)),
    ((1024,), (128,), (1,), (1,), (True,)),        # identity layout: no workspace needed
    ((1000,), (33,), (1,), (3,), (False,)),
])
def test_single_call_c_entry_equals_the_operator(shape, ks, st, di, ca):
    """b200na_na_forward (permute -> attention -> unpermute in one C call, caller workspace) agrees
    with na1d/na2d/na3d to rounding (the operator gathers its tiles from the caller's layout and
    starts them at the first attended key; the C call tiles permuted copies on a grid), and gives
    the same bits when the workspace is reused by a second call."""
    torch.manual_seed(21)
    q, k, v = (torch.randn(2, *shape, 2, 64, device="cuda").half() for _ in range(3))
    want_o, want_l = _na_fn(len(shape))(q, k, v, ks, st, di, ca, return_lse=True)
    tq, tkv = nb.choose_tile_shapes(shape, ks, st, di, ca)
    need = nb.fused_workspace_bytes(shape, di, tq, tkv, 2, 2, 2, 64)
    assert (need == 0) == (shape == (1024,))
    ws = torch.full((max(need, 1),), 0xAB, dtype=torch.uint8, device="cuda")
    first = None
    for _ in range(2):
        o, l = nb.na_forward_fused(q, k, v, ks, st, di, ca, workspace=ws)
        assert L.device_status() == 0
        assert (o.float() - want_o.float()).abs().max().item() <= TOL_16
        assert (l - want_l).abs().max().item() <= 1e-3
        if first is not None:
            assert torch.equal(o, first[0]) and torch.equal(l, first[1])
        first = (o.clone(), l.clone())
    if need:
        with pytest.raises(L.NattenB200Error):
            nb.na_forward_fused(q, k, v, ks, st, di, ca, workspace=ws[:need - 256])


@pytest.mark.parametrize("shape,ks,st,di,ca,n_extra,hq,hkv", [
    ((32, 32), (8, 8), (4, 4), (1, 1), (False, False), 256, 2, 2),   # config 4 scaled
    ((30, 26), (5, 7), (1, 1), (2, 3), (False, True), 77, 4, 2),     # dilation groups share the extra tokens; GQA
    ((700,), (65,), (3,), (1,), (True,), 130, 2, 2),
    ((6, 10, 12), (3, 4, 5), (1, 2, 1), (1, 1, 1), (True, False, False), 1, 1, 1),
])
def test_fused_extra_kv_equals_attention_plus_merge(shape, ks, st, di, ca, n_extra, hq, hkv):
    """Extra KV tokens fused into the neighborhood kernel vs the reference's composition
    (neighborhood attention, dense attention over the extra tokens, LSE merge) and vs the oracle."""
    torch.manual_seed(17)
    q = torch.randn(2, *shape, hq, 128).bfloat16()
    k, v = (torch.randn(2, *shape, hkv, 128).bfloat16() for _ in range(2))
    ak, av = (torch.randn(2, n_extra, hkv, 128).bfloat16() for _ in range(2))
    fn = _na_fn(len(shape))
    args = dict(kernel_size=ks, stride=st, dilation=di, is_causal=ca, return_lse=True,
                additional_keys=ak.cuda(), additional_values=av.cuda())
    o_f, l_f = fn(q.cuda(), k.cuda(), v.cuda(), **args)
    o_u, l_u = fn(q.cuda(), k.cuda(), v.cuda(), attention_kwargs={"unfused_extra_kv": True}, **args)
    assert L.device_status() == 0
    want_o, want_l = oracle.na_forward(q.float().numpy(), k.float().numpy(), v.float().numpy(), ks,
                                       st, di, ca, add_k=ak.float().numpy(), add_v=av.float().numpy())
    assert np.abs(o_f.float().cpu().numpy() - want_o).max() <= TOL_16
    assert np.abs(l_f.cpu().numpy() - want_l).max() <= TOL_16
    assert (o_f.float() - o_u.float()).abs().max().item() <= TOL_16
    assert (l_f - l_u).abs().max().item() <= TOL_16


def test_forward_is_deterministic():
    torch.manual_seed(4)
    q, k, v = (torch.randn(2, 40, 40, 2, 64, device="cuda").half() for _ in range(3))
    a = nb.na2d(q, k, v, 7, 1, 2, return_lse=True)
    b = nb.na2d(q, k, v, 7, 1, 2, return_lse=True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_unsupported_inputs_fail_loudly():
    q = torch.randn(1, 64, 2, 64, device="cuda", dtype=torch.float64)
    with pytest.raises(NotImplementedError):
        nb.na1d(q, q, q, kernel_size=5)
    q = torch.randn(1, 64, 2, 64, device="cuda").bfloat16()
    with pytest.raises(ValueError):
        nb.na1d(q, q, q, kernel_size=5, q_tile_shape=(64,))
    with pytest.raises(NotImplementedError):
        nb.attention(q, q, q, cumulative_seqlen_Q=torch.zeros(2, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("D", [8, 32, 48, 80, 96, 20])
def test_head_dims_the_kernels_are_not_built_for(D):
    """fp16/bf16 head dims below 128 other than 64 run on the 64 / 128-channel tensor-core kernels:
    multiples of 8 are read as they lie (zero-filled tensor-map boxes, narrow output rows; no
    copies) when no gradient is needed, the same inputs with a gradient - and head dims like 20 -
    go through a zero-padded copy. All of them match the oracle, for neighborhood and dense
    attention, on the caller's layout, on permuted copies, 1-D to 3-D."""
    torch.manual_seed(D)
    q, k, v = (torch.randn(2, 20, 28, 2, D).bfloat16() for _ in range(3))
    ks, st, di, ca = (5, 7), (1, 2), (2, 1), (False, True)
    want_o, want_l = oracle.na_forward(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                                       ks, st, di, ca)
    for kwargs in ({}, {"permuted_layout": True}):
        for grad in (False, True):
            qc = q.cuda().requires_grad_(grad)
            out, lse = nb.na2d(qc, k.cuda(), v.cuda(), ks, st, di, ca, return_lse=True,
                               attention_kwargs=kwargs)
            assert out.shape == q.shape and out.is_contiguous()
            assert np.abs(out.detach().float().cpu().numpy() - want_o).max() <= TOL_16
            assert np.abs(lse.detach().cpu().numpy() - want_l).max() <= TOL_16
    a, b, c = (t.flatten(1, 2)[:, :300] for t in (q, k, v))
    o2, l2 = nb.attention(a.cuda(), b.cuda(), c.cuda(), return_lse=True)
    w2, wl2 = oracle.dense_attention(a.float().numpy(), b.float().numpy(), c.float().numpy())
    assert L.device_status() == 0
    assert np.abs(o2.float().cpu().numpy() - w2).max() <= TOL_16
    assert np.abs(l2.cpu().numpy() - wl2).max() <= TOL_16
    # 1-D with extra tokens and 3-D (batch 1: read as it lies; batch 2: padded copy)
    q1, k1, v1 = (torch.randn(2, 500, 2, D).bfloat16() for _ in range(3))
    ak, av = (torch.randn(2, 37, 2, D).bfloat16() for _ in range(2))
    o1, l1 = nb.na1d(q1.cuda(), k1.cuda(), v1.cuda(), 33, 2, 1, True, additional_keys=ak.cuda(),
                     additional_values=av.cuda(), return_lse=True)
    w1, wl1 = oracle.na_forward(q1.float().numpy(), k1.float().numpy(), v1.float().numpy(), (33,),
                                (2,), (1,), (True,), add_k=ak.float().numpy(),
                                add_v=av.float().numpy())
    assert np.abs(o1.float().cpu().numpy() - w1).max() <= TOL_16
    assert np.abs(l1.cpu().numpy() - wl1).max() <= TOL_16
    for batch in (1, 2):
        q3, k3, v3 = (torch.randn(batch, 6, 10, 12, 2, D).bfloat16() for _ in range(3))
        o3, l3 = nb.na3d(q3.cuda(), k3.cuda(), v3.cuda(), (3, 4, 5), (1, 2, 1), 1,
                         (True, False, False), return_lse=True)
        w3, wl3 = oracle.na_forward(q3.float().numpy(), k3.float().numpy(), v3.float().numpy(),
                                    (3, 4, 5), (1, 2, 1), (1, 1, 1), (True, False, False))
        assert np.abs(o3.float().cpu().numpy() - w3).max() <= TOL_16
        assert np.abs(l3.cpu().numpy() - wl3).max() <= TOL_16
    assert L.device_status() == 0


def test_three_dimensional_problems_with_a_very_long_axis_run_on_the_cuda_core_kernel():
    """The 3-D tensor-core kernel keeps a row's window bounds in 16-bit halves, so the C entry
    refuses 3-D shapes with an axis of 65536 tokens or more; the Python operator sends them to the
    CUDA-core kernel, and the result still matches the oracle (checked on a sample of rows
    that includes both ends of the long axis)."""
    torch.manual_seed(21)
    shape, ks, st, di, ca = (65600, 2, 2), (9, 2, 2), (1, 1, 1), (1, 1, 1), (True, False, False)
    q, k, v = (torch.randn(1, *shape, 1, 64).half() for _ in range(3))
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    out, lse = nb.na3d(qc, kc, vc, ks, st, di, ca, return_lse=True)
    assert L.device_status() == 0
    rng = np.random.default_rng(3)
    n_tok = int(np.prod(shape))
    rows = np.unique(np.concatenate([np.arange(64), np.arange(n_tok - 64, n_tok),
                                     rng.integers(0, n_tok, size=512)])).astype(np.int64)
    want_o, want_l = oracle.na_forward(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                                       ks, st, di, ca, tok_idx=rows)
    got_o = out.flatten(1, 3).float().cpu().numpy()[:, rows]
    got_l = lse.flatten(1, 3).cpu().numpy()[:, rows]
    assert np.abs(got_o - want_o).max() <= TOL_16
    assert np.abs(got_l - want_l).max() <= TOL_16
    # the tensor-core entry itself says so
    with pytest.raises(L.NattenB200Error) as err:
        nb.fna_forward_direct(qc, kc, vc, ks, st, di, ca, 64 ** -0.5, (64, 2, 2), (32, 2, 2))
    assert err.value.code == L.ERR_UNSUPPORTED
