"""Host-side logic that needs no GPU: argument rules (same exceptions as the reference),
window arithmetic against the oracle's C restatement, tile-shape selection."""

import numpy as np
import pytest
import torch

import natten_b200 as nb
from natten_b200 import functional as F
from natten_b200.checks import check_all_args, is_self_attention


def test_cpu_tensors_are_refused_loudly():
    q = torch.randn(1, 16, 2, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        nb.na1d(q, q, q, kernel_size=3)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        nb.attention(q, q, q)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        nb.token_permute_operation(q, (4,))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        nb.merge_attentions([q, q], [q[..., 0], q[..., 0]])


def test_argument_rules_match_the_reference():
    q = torch.randn(1, 16, 16, 2, 8)
    with pytest.raises(ValueError):
        nb.na2d(q, q, q, kernel_size=17)                 # k * d > X
    with pytest.raises(ValueError):
        nb.na2d(q, q, q, kernel_size=4, dilation=5)
    with pytest.raises(ValueError):
        nb.na2d(q, q, q, kernel_size=4, stride=5)        # s > k
    with pytest.raises(ValueError):
        nb.na2d(q, q, q, kernel_size=1)                  # k >= 2
    with pytest.raises(ValueError):
        nb.na2d(q, q, q, kernel_size=(3, 3, 3))
    with pytest.raises(ValueError):
        nb.na1d(q, q, q, kernel_size=3)                  # wrong rank for na1d
    with pytest.raises(ValueError):
        nb.na2d(q, q[:, :8], q, kernel_size=3)           # token layouts differ
    with pytest.raises(ValueError):
        nb.na2d(q, q.double(), q, kernel_size=3)         # dtypes differ
    with pytest.raises(ValueError):
        nb.na2d(q, q, q, kernel_size=3, additional_keys=q[:, 0])  # only one of the pair
    with pytest.raises(ValueError):
        nb.na2d(q, q[..., :1, :].expand(-1, -1, -1, 3, -1), q, kernel_size=3)  # 2 % 3 heads
    with pytest.raises(NotImplementedError):
        nb.na2d(q, q, q, kernel_size=3, backend="hopper-fna")
    assert check_all_args(2, 3, None, None, None) == ((3, 3), (1, 1), (1, 1), (False, False))
    assert check_all_args(2, (3, 5), 2, (1, 2), (True, False)) == ((3, 5), (2, 2), (1, 2), (True, False))


def test_self_attention_detection():
    q1 = torch.empty(1, 64, 1, 8)
    assert is_self_attention(q1, (64,), (True,), False)       # 1-D causal full window
    assert not is_self_attention(q1, (64,), (True,), True)    # ... unless extra KV is attached
    q2 = torch.empty(1, 8, 8, 1, 8)
    assert is_self_attention(q2, (8, 8), (False, False), True)
    assert not is_self_attention(q2, (8, 8), (True, False), False)
    assert not is_self_attention(q2, (8, 7), (False, False), False)


def test_merge_attentions_argument_rules():
    o = torch.randn(1, 4, 2, 8)
    l = torch.randn(1, 4, 2)
    with pytest.raises(ValueError):
        nb.merge_attentions([o], [l])
    with pytest.raises(ValueError):
        nb.merge_attentions([o, o], [l])
    with pytest.raises(ValueError):
        nb.merge_attentions([o, o[:, :2]], [l, l])
    with pytest.raises(ValueError):
        nb.merge_attentions([o, o], [l, l[..., 0]])


def test_window_arithmetic_matches_oracle_enumeration():
    """Host window functions vs a brute-force use of the oracle: a one-hot value tensor makes the
    attention output reveal exactly which keys each query attends."""
    import oracle
    for (L, k, s, d, causal) in [(23, 5, 1, 1, False), (23, 6, 3, 1, True), (29, 4, 2, 3, False),
                                 (31, 7, 7, 2, True)]:
        q = np.zeros((1, L, 1, 4), np.float32)
        v = np.eye(L, dtype=np.float32).reshape(1, L, 1, L)
        out, _ = oracle.na_forward(q, q, v, (k,), (s,), (d,), (causal,))
        attended = out[0, :, 0, :] > 0
        for x in range(L):
            g, i = x % d, x // d
            Lg = F.group_extent(L, d, g)
            st = F.window_start(i, k, s, Lg, causal)
            en = F.window_end(i, st, k, Lg, causal)
            expect = np.zeros(L, bool)
            expect[[j * d + g for j in range(st, en)]] = True
            assert np.array_equal(attended[x], expect), (L, k, s, d, causal, x)


def test_tile_shape_selection_is_valid_and_no_worse_than_reference_defaults():
    cases = [((128, 128), (13, 13), (1, 1), (2, 2), (False, False)),
             ((256, 256), (32, 32), (16, 16), (1, 1), (False, False)),
             ((32, 48, 80), (16, 24, 24), (1, 8, 8), (1, 1, 1), (True, False, False)),
             ((57, 20, 88), (3, 5, 7), (1, 2, 3), (2, 1, 1), (False, True, False))]
    ref_default = {2: ((16, 16), (16, 8)), 3: ((8, 4, 8), (4, 4, 8))}
    for shape, k, s, d, c in cases:
        tq, tkv = nb.choose_tile_shapes(shape, k, s, d, c)
        assert np.prod(tq) in (256, 128) and np.prod(tkv) == 128
        n = len(shape)

        def cost(tq_, tkv_):
            # 128-row x 128-key products per query token; gathered tiles start at the first
            # attended key, permuted ones lie on the tile grid
            aligned = nb.direct_layout_supported(tq_, tkv_, d)
            tiles = np.prod([F._axis_tile_cost(shape[a], k[a], s[a], d[a], c[a], tq_[a], tkv_[a],
                                               aligned) for a in range(n)], dtype=np.float64)
            return tiles * (2.0 if np.prod(tq_) == 256 else F.SMALL_Q_TILE_PENALTY)
        assert cost(tq, tkv) <= cost(*ref_default[n])
    # small windows take the 128-token query tile (two CTAs per SM), large ones the 256-token one
    assert np.prod(nb.choose_tile_shapes((128, 128), (13, 13), (1, 1), (2, 2), (False, False))[0]) == 128
    assert np.prod(nb.choose_tile_shapes((256, 256), (32, 32), (16, 16), (1, 1), (False, False))[0]) == 256
    assert np.prod(nb.choose_tile_shapes((32, 48, 80), (16, 24, 24), (1, 8, 8), (1, 1, 1),
                                         (True, False, False))[0]) == 256
    assert nb.choose_tile_shapes((4096,), (64,), (1,), (1,), (False,)) == ((256,), (128,))
    # a window that is a whole number of tiles wide costs exactly that many gathered tiles,
    # wherever it starts: 32 keys from 16 j - 8 are two 16-key tiles, three on the grid
    assert F._axis_tile_cost(256, 32, 16, 1, False, 16, 16, aligned=True) == 2 * 16
    assert F._axis_tile_cost(256, 32, 16, 1, False, 16, 16, aligned=False) == 3 * 16 - 2


def test_layout_predicates_and_backward_tile_choice():
    # a tile of one dilation group must fit a tensor-map box (256 positions, element stride <= 8);
    # the 256-token query tile is fetched as two halves split along its last non-unit axis
    assert nb.direct_layout_supported((256,), (128,), (1,))
    assert nb.direct_layout_supported((256,), (128,), (2,))           # halves of 128 * 2 = 256
    assert not nb.direct_layout_supported((256,), (128,), (3,))
    assert nb.direct_layout_supported((16, 16), (16, 8), (8, 8))
    assert not nb.direct_layout_supported((16, 16), (16, 8), (9, 1))  # stride > 8
    assert not nb.direct_layout_supported((4, 64), (2, 64), (1, 5))   # 32 * 5 fits, 64 * 5 does not
    assert F.backward_layout_supported((128,), (128,), (2,))
    assert not F.backward_layout_supported((128,), (128,), (3,))
    for shape, k, s, d, c in [((128, 128), (13, 13), (1, 1), (2, 2), (False, False)),
                              ((32, 48, 80), (16, 24, 24), (1, 8, 8), (1, 1, 1), (True, False, False)),
                              ((57, 20, 88), (3, 5, 7), (1, 2, 3), (2, 1, 4), (False, True, False))]:
        tq, tkv = F.choose_backward_tile_shapes(shape, k, s, d, c)
        assert np.prod(tq) == 128 and np.prod(tkv) == 128
        assert F.backward_layout_supported(tq, tkv, d)
    assert F.choose_backward_tile_shapes((5000,), (33,), (1,), (1,), (True,)) == ((128,), (128,))
    # nothing fits a box at dilation 9: the caller then uses the CUDA-core kernels
    tq, tkv = F.choose_backward_tile_shapes((90, 90), (3, 3), (1, 1), (9, 9), (False, False))
    assert not F.backward_layout_supported(tq, tkv, (9, 9))


def test_backend_names():
    assert "blackwell-fna" in F.BACKEND_ALIASES and "b200-fna" in F.BACKEND_ALIASES
    q = torch.zeros(1, 16, 2, 64)
    with pytest.raises(NotImplementedError):
        nb.na1d(q, q, q, 3, backend="hopper-fna")
    with pytest.raises(NotImplementedError):
        nb.attention(q, q, q, backend="cutlass-fmha")
    with pytest.raises(RuntimeError):             # accepted name, but CPU tensors
        nb.na1d(q, q, q, 3, backend="blackwell-fna")


def test_config_queries_answer_to_the_reference_names():
    """The tile-shape queries exist under the reference's Blackwell names too; on CPU tensors they
    answer "no configuration", like the reference's do for operands its backend cannot run."""
    q = torch.zeros(1, 16, 16, 2, 64, dtype=torch.bfloat16)
    assert nb.get_configs_for_cutlass_blackwell_fna is nb.get_configs_for_b200_fna
    assert nb.get_bwd_configs_for_cutlass_blackwell_fna is nb.get_bwd_configs_for_b200_fna
    for fn in (nb.get_configs_for_cutlass_blackwell_fna, nb.get_bwd_configs_for_cutlass_blackwell_fna,
               nb.get_configs_for_cutlass_blackwell_fmha, nb.get_bwd_configs_for_cutlass_blackwell_fmha):
        assert fn(q, q, q) == []
    # every forward pair the search considers is a 256 / 128-token factorisation
    for tq, tkv in F._all_tile_shapes(2, 8, 7):
        assert np.prod(tq) == 256 and np.prod(tkv) == 128
    for tq, tkv in F._all_tile_shapes(3, 7, 7):
        assert np.prod(tq) == 128 and np.prod(tkv) == 128


def test_logger_follows_the_reference_environment_variables(tmp_path):
    """NATTEN_LOG_LEVEL / NATTEN_LOG_PIPE as in the reference (src/natten/utils/log.py:43-134):
    debug lines reach the chosen file only at level debug."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("from natten_b200.log import get_logger; l = get_logger('natten_b200.test'); "
            "l.debug('tile %s', (4, 8, 8)); l.info('hello'); print(l.debug_enabled)")
    for level, expect_debug in (("debug", True), ("warning", False), ("", False)):
        pipe = tmp_path / f"log_{level or 'default'}.txt"
        env = dict(os.environ, NATTEN_LOG_LEVEL=level, NATTEN_LOG_PIPE=str(pipe), PYTHONPATH=root)
        res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                             check=True)
        text = pipe.read_text() if pipe.exists() else ""
        assert ("tile (4, 8, 8)" in text) == expect_debug
        assert ("hello" in text) == (level != "warning")
        assert res.stdout.strip() == str(expect_debug)
