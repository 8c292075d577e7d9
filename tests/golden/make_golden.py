"""Generate the golden fixtures in this directory from the reference package itself.

Run where the reference source tree is mounted (it is not needed to *use* the fixtures):

    REFERENCE_SRC=/path/to/NATTEN/src python tests/golden/make_golden.py

The reference is imported from source without its compiled extension, so neighborhood attention
runs through its CPU-capable Flex backend in fp32 (src/natten/backends/__init__.py:103-105) and
token permutation through its torch implementation (src/natten/token_permute/torch_impl.py).
Inputs are seeded; everything needed to replay a case is stored next to the reference's outputs.

Files written:
  na_cases.npz       neighborhood attention (na1d/na2d/na3d, +extra KV, +self-attention path)
  attn_cases.npz     dense attention() and merge_attentions()
  tokperm_cases.json token permute / unpermute: parameters + SHA-256 of the reference's output bytes
"""
import hashlib
import json
import os
import sys

import numpy as np

REF = os.environ.get("REFERENCE_SRC")
if not REF:
    raise SystemExit("set REFERENCE_SRC to the `src` directory of a checkout of the reference "
                     "(the one that holds the `natten` package)")
sys.path.insert(0, REF)
os.environ.setdefault("NATTEN_LOG_LEVEL", "error")
sys.dont_write_bytecode = True

import torch  # noqa: E402
import natten  # noqa: E402
from natten.token_permute import token_permute_operation, token_unpermute_operation  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
torch.set_num_threads(max(1, os.cpu_count() or 1))


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


# name: (shape, B, Hq, Hkv, D, kernel, stride, dilation, causal, n_extra, round_to_bf16)
NA_CASES = {
    # BASELINE config 1, in full (fp32 operands)
    "c1_na2d_32x32_k7": ((32, 32), 1, 4, 4, 32, (7, 7), (1, 1), (1, 1), (False, False), 0, False),
    "na1d_300_k33": ((300,), 1, 2, 2, 32, (33,), (1,), (1,), (False,), 0, True),
    "na1d_512_k64_s8_causal": ((512,), 2, 2, 2, 64, (64,), (8,), (1,), (True,), 0, True),
    "na1d_257_k9_s3_d4_causal": ((257,), 1, 2, 2, 32, (9,), (3,), (4,), (True,), 0, True),
    # config 2 scaled down along the sequence
    "c2s_na1d_1024_k128_causal": ((1024,), 1, 1, 1, 128, (128,), (1,), (1,), (True,), 0, True),
    "na2d_20x24_k5x7": ((20, 24), 1, 2, 2, 32, (5, 7), (1, 1), (1, 1), (False, False), 0, True),
    "na2d_33x30_k3x5_s1x2_d3x2_causal01": ((33, 30), 1, 2, 2, 32, (3, 5), (1, 2), (3, 2),
                                           (False, True), 0, True),
    # config 3 scaled down 4x per axis
    "c3s_na2d_32x32_k13_d2": ((32, 32), 1, 2, 2, 64, (13, 13), (1, 1), (2, 2), (False, False), 0,
                              True),
    # config 4 scaled down (stride = k/2 block-sparse) with extra KV tokens
    "c4s_na2d_32x32_k8_s4_extra24": ((32, 32), 1, 1, 1, 128, (8, 8), (4, 4), (1, 1),
                                     (False, False), 24, True),
    "na2d_16x16_k5_gqa": ((16, 16), 1, 4, 2, 32, (5, 5), (1, 1), (1, 1), (False, False), 0, True),
    # config 5 scaled down 4x per axis
    "c5s_na3d_8x12x20_k4x6x6_s1x2x2_causalT": ((8, 12, 20), 1, 1, 1, 64, (4, 6, 6), (1, 2, 2),
                                               (1, 1, 1), (True, False, False), 0, True),
    "na3d_6x9x11_k3x3x5_s1x1x2_d2x1x1_causalW": ((6, 9, 11), 1, 2, 2, 32, (3, 3, 5), (1, 1, 2),
                                                 (2, 1, 1), (False, False, True), 0, True),
    "na3d_5x6x7_k2x3x4_allcausal": ((5, 6, 7), 1, 1, 1, 16, (2, 3, 4), (1, 2, 3), (1, 1, 1),
                                    (True, True, True), 0, True),
    "na1d_96_k17_causal_extra7": ((96,), 2, 2, 2, 32, (17,), (2,), (1,), (True,), 7, True),
    # self-attention fast path (src/natten/functional.py:404-444)
    "na1d_64_k64_selfattn": ((64,), 1, 2, 2, 32, (64,), (1,), (1,), (False,), 0, True),
    "na2d_8x8_k8_selfattn": ((8, 8), 1, 2, 2, 32, (8, 8), (1, 1), (1, 1), (False, False), 0, True),
}


def make_na():
    out = {}
    meta = {}
    for idx, (name, c) in enumerate(NA_CASES.items()):
        shape, B, Hq, Hkv, D, ks, st, di, ca, n_extra, rnd = c
        torch.manual_seed(1000 + idx)
        q = torch.randn(B, *shape, Hq, D)
        k = torch.randn(B, *shape, Hkv, D)
        v = torch.randn(B, *shape, Hkv, D)
        ak = av = None
        if n_extra:
            ak = torch.randn(B, n_extra, Hkv, D)
            av = torch.randn(B, n_extra, Hkv, D)
        if rnd:
            q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
            if n_extra:
                ak, av = bf16_round(ak), bf16_round(av)
        fn = {1: natten.na1d, 2: natten.na2d, 3: natten.na3d}[len(shape)]
        o, lse = fn(q, k, v, kernel_size=ks, stride=st, dilation=di, is_causal=ca,
                    additional_keys=ak, additional_values=av, return_lse=True)
        print(name, tuple(o.shape), float(o.abs().max()), float(lse.abs().max()), flush=True)
        ins = [("q", q), ("k", k), ("v", v)] + ([("add_k", ak), ("add_v", av)] if n_extra else [])
        for key, t in ins:
            # bf16-exact operands are stored as their 16-bit patterns (half the bytes)
            out[f"{name}/{key}"] = (t.to(torch.bfloat16).view(torch.int16).numpy() if rnd
                                    else t.contiguous().numpy())
        out[f"{name}/out"] = o.contiguous().numpy()
        out[f"{name}/lse"] = lse.contiguous().numpy()
        meta[name] = dict(shape=shape, kernel_size=ks, stride=st, dilation=di,
                          is_causal=[bool(x) for x in ca], n_extra=n_extra, bf16_exact=rnd)
    out["__meta__"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "na_cases.npz"), **out)


def make_attn():
    out = {}
    torch.manual_seed(77)
    # dense attention: cross-attention shapes (Nq != Nk), GQA. The reference's CPU-capable backend
    # has no causal dense attention (configs/checks.py: "Flex FMHA doesn't support causal mask"),
    # so causal dense attention cannot be pinned from here.
    cases = {"cross_100x37": (1, 100, 37, 2, 2, 32, False), "gqa_64x80": (2, 64, 80, 4, 1, 64, False),
             "self_128": (1, 128, 128, 2, 2, 128, False)}
    meta = {}
    for name, (B, Nq, Nk, Hq, Hkv, D, causal) in cases.items():
        q = bf16_round(torch.randn(B, Nq, Hq, D))
        k = bf16_round(torch.randn(B, Nk, Hkv, D))
        v = bf16_round(torch.randn(B, Nk, Hkv, D))
        o, lse = natten.attention(q, k, v, is_causal=causal, return_lse=True)
        for key, t in (("q", q), ("k", k), ("v", v), ("out", o), ("lse", lse)):
            out[f"attn/{name}/{key}"] = t.contiguous().numpy()
        meta[name] = dict(is_causal=causal)
        print("attention", name, tuple(o.shape), flush=True)
    # merge_attentions: two- and three-way (src/natten/attn_merge.py:75-98)
    for name, n_way in (("merge2", 2), ("merge3", 3)):
        outs = [torch.randn(2, 50, 3, 16) for _ in range(n_way)]
        lses = [torch.randn(2, 50, 3) * 3 for _ in range(n_way)]
        o, l = natten.merge_attentions(outs, lses, torch_compile=False, use_autograd_fix=False)
        for i in range(n_way):
            out[f"merge/{name}/o{i}"] = outs[i].numpy()
            out[f"merge/{name}/l{i}"] = lses[i].numpy()
        out[f"merge/{name}/out"] = o.numpy()
        out[f"merge/{name}/lse"] = l.numpy()
        print("merge", name, flush=True)
    out["__meta__"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "attn_cases.npz"), **out)


def pattern(n: int, bits: int) -> np.ndarray:
    """Machine-independent bit pattern: element i = (i * 40503 + 12345) mod 2^bits, no NaN/Inf
    exponents (the top exponent bit is cleared) so float views compare reliably."""
    i = np.arange(n, dtype=np.uint64)
    v = (i * np.uint64(40503) + np.uint64(12345)) % np.uint64(1 << bits)
    if bits == 16:
        return (v.astype(np.uint16) & np.uint16(0xBFFF))
    return (v.astype(np.uint32) & np.uint32(0xBFFFFFFF))


# (token layout, tile, dilation) — includes the padded / odd-dilation shapes the reference's own
# suite uses (tests/test_token_permute.py:78-109, 203-260) and the BASELINE configs' tilings.
TOKPERM_CASES = [
    ((19,), (3,), (7,)), ((256,), (128,), (1,)), ((300,), (64,), (2,)),
    ((16, 16), (8, 2), (2, 4)), ((17, 10), (4, 4), (1, 3)), ((48, 80), (16, 16), (11, 7)),
    ((48, 80), (16, 8), (1, 1)), ((32, 32), (16, 16), (2, 2)), ((33, 30), (8, 16), (3, 2)),
    ((5, 6, 7), (2, 2, 4), (2, 1, 1)), ((8, 8, 8), (2, 4, 2), (1, 1, 1)),
    ((57, 20, 88), (4, 4, 8), (2, 1, 1)), ((8, 12, 20), (4, 4, 16), (1, 1, 1)),
    ((6, 9, 11), (2, 8, 8), (2, 1, 1)),
]


def make_tokperm():
    cases = []
    for shape, tile, dil in TOKPERM_CASES:
        for flip in (True, False):
            for dt_name, tdt, bits in (("fp32", torch.float32, 32), ("bf16", torch.bfloat16, 16),
                                       ("fp16", torch.float16, 16)):
                if dt_name == "fp16" and len(shape) != 2:
                    continue
                B, H, D = (2, 3, 8) if int(np.prod(shape)) < 20000 else (1, 2, 16)
                n = B * int(np.prod(shape)) * H * D
                raw = pattern(n, bits)
                x = torch.from_numpy(raw.view(np.int16 if bits == 16 else np.int32).copy())
                x = x.view(tdt).reshape(B, *shape, H, D)
                y, _, post = token_permute_operation(x, tile_shape=tile, dilation=dil,
                                                     flip_tiled_dims=flip, use_torch=True)
                back = token_unpermute_operation(y, token_layout_shape=shape, tile_shape=tile,
                                                 dilation=dil, flip_tiled_dims=flip,
                                                 use_torch=True)
                assert torch.equal(back.view(torch.int16 if bits == 16 else torch.int32),
                                   x.view(torch.int16 if bits == 16 else torch.int32))
                yb = y.contiguous().view(torch.int16 if bits == 16 else torch.int32).numpy()
                cases.append(dict(shape=shape, tile=tile, dilation=dil, flip=flip, dtype=dt_name,
                                  B=B, H=H, D=D, out_shape=list(y.shape), post_dilation=list(post),
                                  sha256=hashlib.sha256(yb.tobytes()).hexdigest()))
        print("tokperm", shape, tile, dil, flush=True)
    with open(os.path.join(HERE, "tokperm_cases.json"), "w") as f:
        json.dump(dict(pattern="(i*40503+12345) mod 2^bits, bit 14 (16-bit) / bit 30 (32-bit) cleared",
                       cases=cases), f, indent=0)


if __name__ == "__main__":
    which = sys.argv[1:] or ["tokperm", "attn", "na"]
    if "tokperm" in which:
        make_tokperm()
    if "attn" in which:
        make_attn()
    if "na" in which:
        make_na()
