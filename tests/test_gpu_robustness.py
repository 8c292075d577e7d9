"""Concurrency and failure handling of the tensor-core kernels: launches that overlap on different
streams and inside a replayed CUDA graph must not disturb each other's work counters; a bounded
wait that expires must end the kernel with a status word, not hang it, and leave the context
usable. No test here faults, traps or hangs the GPU: the expiring wait is made on purpose, short,
in a build of the library meant for this test only."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

import natten_b200 as nb
import natten_b200._lib as L

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_overlapping_launches_on_two_streams_and_a_graph_keep_their_work_counters_apart():
    """More launches than the old 64-entry counter pool held, issued alternately on two streams
    while a captured graph of a third problem replays on its own stream. Every result must equal
    the one the same call gives when it runs alone."""
    torch.manual_seed(5)
    problems = []
    for shape, ks, st, ca, heads in [((2048,), (256,), (1,), (True,), 6),
                                     ((48, 64), (9, 11), (1, 2), (False, False), 5),
                                     ((8, 16, 24), (4, 5, 7), (1, 1, 2), (True, False, False), 4)]:
        q, k, v = (torch.randn(1, *shape, heads, 128, device="cuda").bfloat16() for _ in range(3))
        fn = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[len(shape)]
        call = (lambda fn=fn, q=q, k=k, v=v, ks=ks, st=st, ca=ca:
                fn(q, k, v, kernel_size=ks, stride=st, is_causal=ca, return_lse=True))
        want = call()
        problems.append((call, want))
    torch.cuda.synchronize()
    s1, s2, s3 = (torch.cuda.Stream() for _ in range(3))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g_out = problems[2][0]()
    torch.cuda.synchronize()
    results = []
    for i in range(80):
        with torch.cuda.stream(s1):
            results.append((0, problems[0][0]()))
        with torch.cuda.stream(s2):
            results.append((1, problems[1][0]()))
        if i % 4 == 0:
            with torch.cuda.stream(s3):
                graph.replay()
    torch.cuda.synchronize()
    assert L.device_status() == 0
    for which, (o, l) in results:
        want_o, want_l = problems[which][1]
        assert torch.equal(o, want_o) and torch.equal(l, want_l)
    assert torch.equal(g_out[0], problems[2][1][0]) and torch.equal(g_out[1], problems[2][1][1])


HOOK_LIB = os.path.join(ROOT, "natten_b200", "lib", "libnatten_b200_testhooks.so")

CHILD = textwrap.dedent("""
    import ctypes, sys, torch
    import natten_b200 as nb, natten_b200._lib as L
    torch.manual_seed(3)
    q, k, v = (torch.randn(1, 2048, 2, 128, device="cuda").bfloat16() for _ in range(3))
    want_o, want_l = nb.na1d(q, k, v, 512, is_causal=True, return_lse=True)
    torch.cuda.synchronize()
    assert L.device_status() == 0
    # the load warp of every CTA keeps back the record of its second key/value tile: the softmax
    # threads wait for it, the wait (about a millisecond in this build) runs out
    L.lib.b200na_test_withhold_record(2)
    nb.na1d(q, k, v, 512, is_causal=True, return_lse=True)
    torch.cuda.synchronize()                 # the kernel must come back by itself
    st = ctypes.c_int(0)
    code = L.lib.b200na_device_status(ctypes.byref(st))
    assert code == L.ERR_KERNEL_TIMEOUT and st.value != 0, (code, st.value)
    role, barrier = st.value >> 8, st.value & 255
    assert role in (1, 2, 3), st.value
    L.lib.b200na_test_withhold_record(0)
    assert L.device_status() == 0            # the word was cleared
    # the context is usable and the next launch is right
    o, l = nb.na1d(q, k, v, 512, is_causal=True, return_lse=True)
    torch.cuda.synchronize()
    assert L.device_status() == 0
    assert torch.equal(o, want_o) and torch.equal(l, want_l)
    print("expired-wait ok", hex(st.value))
""")


def test_an_expired_wait_ends_the_kernel_with_a_status_word_and_the_next_launch_is_correct():
    """Runs in a child process against the test-hook build of the library (bounded waits of about
    a millisecond, one producer arrive can be held back from the host): the kernel returns, the
    status call reports B200NA_ERR_KERNEL_TIMEOUT with the role and barrier that gave up, and a
    normal launch afterwards gives the right result."""
    if not os.path.exists(HOOK_LIB):
        pytest.skip("test-hook build of the library not present (python natten_b200/build.py)")
    env = dict(os.environ, NATTEN_B200_LIB=HOOK_LIB, PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "expired-wait ok" in res.stdout
