"""Op registration and layers, checked without a GPU: schemas, shape/dtype propagation through the
ops' fake implementations (what torch.compile traces with), layer parameter names."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import natten_b200 as nb
from natten_b200 import ops

OPS = ("token_permute", "token_unpermute", "merge", "fmha_forward", "na_forward",
       "na_forward_direct", "fna_forward_permuted", "na_forward_simt")


def test_every_kernel_entry_is_a_registered_torch_op():
    assert ops.USE_TORCH_OPS
    for name in OPS:
        op = getattr(torch.ops.natten_b200, name)
        schema = str(op.default._schema)
        assert schema.startswith(f"natten_b200::{name}(")
        assert "Tensor" in schema.split("->")[1]


def _fake_cuda(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, device="cuda", dtype=dtype)


def test_operators_propagate_shapes_through_fake_tensors():
    with FakeTensorMode():
        q = _fake_cuda(2, 16, 20, 4, 64)
        kv = _fake_cuda(2, 16, 20, 2, 64)
        out, lse = nb.na2d(q, kv, kv, 5, dilation=(2, 1), return_lse=True)   # direct layout
        assert out.shape == q.shape and out.dtype == q.dtype
        assert lse.shape == q.shape[:-1] and lse.dtype == torch.float32
        ak = _fake_cuda(2, 7, 2, 64)
        out = nb.na2d(q, kv, kv, 5, additional_keys=ak, additional_values=ak,
                      attention_kwargs={"unfused_extra_kv": True, "permuted_layout": True})
        assert out.shape == q.shape                     # permute, kernel, unpermute, fmha, merge
        q1 = _fake_cuda(1, 1000, 2, 128)
        assert nb.na1d(q1, q1, q1, 33, dilation=3).shape == q1.shape   # permuted fallback
        q32 = _fake_cuda(1, 32, 32, 4, 32, dtype=torch.float32)
        out, lse = nb.na2d(q32, q32, q32, 7, return_lse=True)          # CUDA-core kernel
        assert out.dtype == torch.float32 and lse.shape == (1, 32, 32, 4)
        q3 = _fake_cuda(1, 4, 6, 8, 2, 64, dtype=torch.float16)
        assert nb.na3d(q3, q3, q3, (4, 6, 8)).shape == q3.shape        # self-attention path
        a = _fake_cuda(2, 50, 2, 64)
        o, l = nb.attention(a, a, a, return_lse=True)
        assert o.shape == a.shape and l.shape == (2, 50, 2)
        mo, ml = nb.merge_attentions([o, o, o], [l, l, l])
        assert mo.shape == o.shape and ml.dtype == torch.float32
        p, layout, post = nb.token_permute_operation(q, (8, 8), (2, 1))
        assert p.shape == (4, 8 * 24, 4, 64) and layout == (16, 20) and post == (8, 24)
        assert nb.token_unpermute_operation(p, layout, (8, 8), (2, 1)).shape == q.shape


@pytest.mark.parametrize("cls,nd", [(nb.NeighborhoodAttention1D, 1), (nb.NeighborhoodAttention2D, 2),
                                    (nb.NeighborhoodAttention3D, 3)])
def test_layers_mirror_the_reference_modules(cls, nd):
    layer = cls(embed_dim=128, num_heads=2, kernel_size=3, stride=1, dilation=2, is_causal=True)
    # the reference's parameter names (src/natten/modules.py:80-82): its checkpoints load as they are
    assert set(layer.state_dict()) == {"qkv.weight", "qkv.bias", "proj.weight", "proj.bias"}
    assert layer.qkv.weight.shape == (384, 128) and layer.head_dim == 64
    assert layer.kernel_size == (3,) * nd and layer.dilation == (2,) * nd
    assert layer.is_causal == (True,) * nd
    assert "kernel_size=" in layer.extra_repr()
    with pytest.raises(ValueError):
        layer(torch.zeros(1, 8, 128) if nd != 1 else torch.zeros(1, 8, 8, 128))
    with pytest.raises(ValueError):
        layer(torch.zeros(1, *([8] * nd), 64))
    with pytest.raises(RuntimeError):          # CPU tensors: no CPU path
        layer(torch.zeros(1, *([8] * nd), 128))
    with pytest.raises(ValueError):
        cls(embed_dim=100, num_heads=3, kernel_size=3)


def test_layer_forward_shapes_with_fake_tensors():
    with FakeTensorMode(), torch.device("cuda"):
        torch.set_default_dtype(torch.bfloat16)
        try:
            layer = nb.NeighborhoodAttention3D(128, 2, (3, 3, 3))
        finally:
            torch.set_default_dtype(torch.float32)
        x = torch.empty(1, 4, 6, 8, 128, dtype=torch.bfloat16)
        assert layer(x).shape == x.shape


def _traced_ops(fn, *args, dynamic=False):
    gm, _ = torch._dynamo.export(fn, assume_static_by_default=not dynamic)(*args)
    return [n.target.name() for n in gm.graph.nodes
            if n.op == "call_function" and hasattr(n.target, "name")
            and n.target.name().startswith("natten_b200::")]


@pytest.mark.parametrize("dynamic", [False, True])
def test_operators_trace_into_one_graph_without_breaks(monkeypatch, dynamic):
    """Dynamo must see nothing it cannot trace (no ctypes call, no data-dependent Python), with
    static and with symbolic (dynamic) shapes: a neighborhood-attention call becomes the single
    node natten_b200::na_forward - kernel, tile shapes and layout are chosen inside it at run
    time. Traced here with CPU tensors and the device check patched out; nothing is executed."""
    import natten_b200.functional as F
    monkeypatch.setattr(F, "_require_cuda", lambda *a: None)
    q, k, v = (torch.randn(2, 32, 40, 2, 128).bfloat16() for _ in range(3))
    ak, av = (torch.randn(2, 40, 2, 128).bfloat16() for _ in range(2))

    def fused(q, k, v, ak, av):
        o, l = nb.na2d(q * 1.0, k, v, (7, 9), (1, 2), (2, 1), (False, True), additional_keys=ak,
                       additional_values=av, return_lse=True)
        return o.float() * 2.0, l + 1.0
    assert _traced_ops(fused, q, k, v, ak, av, dynamic=dynamic) == ["natten_b200::na_forward"]

    def unfused(q, k, v, ak, av):
        return nb.na2d(q, k, v, 5, additional_keys=ak, additional_values=av,
                       attention_kwargs={"unfused_extra_kv": True})
    assert _traced_ops(unfused, q, k, v, ak, av, dynamic=dynamic) == [
        "natten_b200::na_forward", "natten_b200::fmha_forward", "natten_b200::merge"]

    q1 = torch.randn(1, 1000, 2, 64).bfloat16()
    assert _traced_ops(lambda a: nb.na1d(a, a, a, 33, dilation=3), q1, dynamic=dynamic) == [
        "natten_b200::na_forward"]
    q32 = torch.randn(1, 16, 16, 2, 32)
    assert _traced_ops(lambda a: nb.na2d(a, a, a, 7), q32, dynamic=dynamic) == [
        "natten_b200::na_forward"]
    assert _traced_ops(lambda a: nb.na2d(a, a, a, 16), q32, dynamic=dynamic) == [
        "natten_b200::fmha_forward"]                      # window = whole layout: dense attention

    layer = nb.NeighborhoodAttention3D(128, 2, (3, 4, 5), is_causal=(True, False, False)).bfloat16()
    x = torch.randn(2, 6, 10, 12, 128).bfloat16()
    assert _traced_ops(layer, x, dynamic=dynamic) == ["natten_b200::na_forward"]

    def permute_roundtrip(t):
        p, layout, _ = nb.token_permute_operation(t, (8, 8), (2, 1))
        return nb.token_unpermute_operation(p, layout, (8, 8), (2, 1))
    assert _traced_ops(permute_roundtrip, q, dynamic=False) == [
        "natten_b200::token_permute", "natten_b200::token_unpermute"]
