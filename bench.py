#!/usr/bin/env python
"""Benchmark of the B200 neighborhood-attention forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl b200|reference]

One "step" is one forward call of the operator na1d/na2d/na3d on seeded synthetic inputs: one
launch of the fused attention kernel, which gathers its tiles from the caller's layout and
attends the extra KV tokens of a config in the same softmax (token-permuted copies are only made
for tile/dilation combinations a tensor-map box cannot express). The default workload is
BASELINE config 5 (na3d bf16, 32x48x80 tokens, 24 heads, kernel 16x24x24, stride 1x8x8, causal
in T): the largest single-GPU configuration and the class the throughput target is stated for.
`--config c1..c5` selects the other BASELINE configs, `--config ref1d|ref2d_na|ref2d_gna|
ref3d_na|ref3d_gna` the shapes the reference publishes B200 kernel times for (printed beside the
measurement as `published`). With N > 1 (launched by torchrun, one rank per GPU) the
(batch x heads) units of the same fixed problem are partitioned across ranks with no collective
("strong"); config 5 then also reports its T-axis slab partitioning as a `spatial` sub-record.

Prints ONE JSON line on rank 0: whole-job effective TFLOP/s (unmasked FLOPs / time) with inputs
resident in HBM (`value`: the median of three timed blocks of K steps), the same through host
buffers (`e2e`), the dominant kernel against its roofline (`roofline`), a row-sampled check of the
timed call's own output against the CPU oracle (`checked`; the run fails above the tolerance),
the bandwidth-bound kernels of the path at this config's shapes (`kernels`) and a CPU baseline of
the oracle on the host cores (`cpu_baseline`).

`--impl reference` times the CPU restatement of the reference's algorithm (oracle/) on all host
cores on a bounded row sample of the same workload and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name: (op, dtype, batch, heads, shape, head_dim, kernel, stride, dilation, causal, n_extra, input multiplier)
CONFIGS = {
    "c1": ("na2d", "fp32", 1, 4, (32, 32), 32, (7, 7), (1, 1), (1, 1), (False, False), 0, 1.0),
    "c2": ("na1d", "bf16", 4, 16, (32768,), 128, (2048,), (1,), (1,), (True,), 0, 1.0),
    "c3": ("na2d", "bf16", 8, 16, (128, 128), 128, (13, 13), (1, 1), (2, 2), (False, False), 0, 1.0),
    "c4": ("na2d", "fp16", 1, 24, (256, 256), 128, (32, 32), (16, 16), (1, 1), (False, False), 256, 0.5),
    "c5": ("na3d", "bf16", 1, 24, (32, 48, 80), 128, (16, 24, 24), (1, 8, 8), (1, 1, 1),
           (True, False, False), 0, 1.0),
    # the shapes the reference's documentation reports B200 kernel times for (fp16, batch 1)
    "ref1d": ("na1d", "fp16", 1, 1, (32768,), 128, (2048,), (1,), (1,), (False,), 0, 1.0),
    "ref2d_na": ("na2d", "fp16", 1, 24, (256, 256), 128, (80, 80), (1, 1), (1, 1),
                 (False, False), 0, 1.0),
    "ref2d_gna": ("na2d", "fp16", 1, 24, (256, 256), 128, (80, 80), (16, 16), (1, 1),
                  (False, False), 0, 1.0),
    "ref3d_na": ("na3d", "fp16", 1, 24, (30, 48, 80), 128, (18, 24, 24), (1, 1, 1), (1, 1, 1),
                 (False, False, False), 0, 1.0),
    "ref3d_gna": ("na3d", "fp16", 1, 24, (30, 48, 80), 128, (18, 24, 24), (16, 8, 8), (1, 1, 1),
                  (False, False, False), 0, 1.0),
}
# Kernel-only times the reference publishes for its Blackwell FNA backend on a B200 (forward,
# fp16, its own profiler): (ms, effective TFLOP/s derived as 4*D*pairs/time, file:line in the
# reference tree). They were measured on the authors' machine, not on this one.
PUBLISHED = {
    "ref1d": (0.058111, 591.0, "docs/sample-outputs/profiler-1d-32k-w2k-blackwell-fna-b200.txt:5"),
    "ref2d_na": (8.692, 593.0, "docs/sample-outputs/profiler-2d-flux-na-blackwell-fna-b200.txt:5"),
    "ref2d_gna": (4.114, 1253.0, "docs/sample-outputs/profiler-2d-flux-gna-blackwell-fna-b200.txt:5"),
    "ref3d_na": (42.243, 347.0, "docs/sample-outputs/profiler-3d-hunyuan-na-blackwell-fna-b200.txt:5"),
    "ref3d_gna": (13.010, 1128.0, "docs/sample-outputs/profiler-3d-hunyuan-gna-blackwell-fna-b200.txt:5"),
}
WORKLOAD_TEXT = {
    "c1": "BASELINE config 1: na2d fp32 B=1 H=4 32x32 D=32 kernel=7x7 (CUDA-core fp32 kernel)",
    "ref1d": "reference-published shape: na1d fp16 B=1 H=1 L=32768 D=128 kernel=2048",
    "ref2d_na": "reference-published shape: na2d fp16 B=1 H=24 256x256 D=128 kernel=80x80 stride=1",
    "ref2d_gna": "reference-published shape: na2d fp16 B=1 H=24 256x256 D=128 kernel=80x80 stride=16x16",
    "ref3d_na": "reference-published shape: na3d fp16 B=1 H=24 30x48x80 D=128 kernel=18x24x24 stride=1",
    "ref3d_gna": "reference-published shape: na3d fp16 B=1 H=24 30x48x80 D=128 kernel=18x24x24 stride=16x8x8",
    "c2": "BASELINE config 2: na1d bf16 B=4 H=16 L=32768 D=128 kernel=2048 stride=1 dilation=1 causal",
    "c3": "BASELINE config 3: na2d bf16 B=8 H=16 128x128 D=128 kernel=13x13 dilation=2x2",
    "c4": "BASELINE config 4: na2d fp16 B=1 H=24 256x256 D=128 kernel=32x32 stride=16x16 + 256 extra KV",
    "c5": "BASELINE config 5: na3d bf16 B=1 H=24 32x48x80 D=128 kernel=16x24x24 stride=1x8x8 causal=(T,F,F)",
}


def _win(i, k, s, L, causal):
    wl, wr = k // 2, k // 2 + (k % 2 - 1)
    if causal:
        lead = min((i // s) * s + s - 1, L - 1)
        st = max(lead - wl - wr, 0)
        return st, min(i + 1, L)
    lead = min((i // s) * s + s // 2, L - 1)
    st = max(lead - wl, 0) + ((L - wr - lead - 1) if lead + wr >= L else 0)
    return st, st + k


def attended_pairs(shape, kernel, stride, dilation, causal) -> int:
    """Sum over queries of the number of attended keys, per (batch, head)."""
    total = 1
    for X, k, s, d, c in zip(shape, kernel, stride, dilation, causal):
        axis = 0
        for x in range(X):
            g, i = x % d, x // d
            L = X // d + (1 - ((g + (d - (X % d))) // d))
            st, en = _win(i, k, s, L, c)
            axis += en - st
        total *= axis
    return total


def algorithmic_flops(cfg, units=None) -> float:
    """4 * D * attended pairs (QK^T and PV, multiply-add = 2) over `units` (batch x head) slices."""
    _, _, B, H, shape, D, ks, st, di, ca, n_extra, _ = cfg
    pairs = attended_pairs(shape, ks, st, di, ca) + n_extra * math.prod(shape)
    return 4.0 * D * pairs * (B * H if units is None else units)


# DRAM traffic of the attention kernel per (batch x head) unit, bytes, from ncu captures of reduced
# cases (dram__bytes_read.sum + dram__bytes_write.sum of one launch / units in that launch),
# summarised in profiles/fna_fwd_kernel_c2.md and profiles/fna_fwd_kernel_c5_c4_c3.md; scaled by
# the units of a launch.
NCU_TRAFFIC_PER_UNIT = {"c2": (202.29e6 + 48.23e6) / 8,
                        "c3": (408.15e6 + 118.48e6) / 32,
                        "c4": (203.21e6 + 46.08e6) / 4,
                        "c5": (429.39e6 + 118.13e6) / 4}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower() == "active":
                    reasons.add(n)
        return dict(sm_mhz=float(np.median(sm)) if sm else None,
                    sm_max_mhz=float(max(mx)) if mx else None, reasons=sorted(reasons),
                    samples=len(sm))


def shard_units(B, H, world, rank):
    """(batch, heads) of this rank's slice when B*H independent units are split over `world`."""
    from natten_b200.sharding import shard_batch_heads
    try:
        bs, hs = shard_batch_heads(B, H, world, rank)
    except ValueError as e:
        raise SystemExit(str(e))
    return bs.stop - bs.start, hs.stop - hs.start


def make_inputs(cfg, b_local, h_local, seed, device, slab=None):
    import torch
    _, dt, _, _, shape, D, _, _, _, _, n_extra, mul = cfg
    if slab is not None:
        shape = (slab[1] - slab[0],) + tuple(shape[1:])
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[dt]
    g = torch.Generator(device="cpu").manual_seed(seed)
    host = []
    for _ in range(3):
        t = torch.randn((b_local, *shape, h_local, D), generator=g, dtype=torch.float32)
        host.append((t * mul).to(dtype).pin_memory())
    extra = []
    if n_extra:
        for _ in range(2):
            t = torch.randn((b_local, n_extra, h_local, D), generator=g, dtype=torch.float32)
            extra.append(t.to(dtype).pin_memory())
    return host, extra


def host_threads():
    """Cores this process may really run on: the affinity mask, capped by the cgroup CPU quota
    (threads beyond the quota only add contention)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    for path in ("/sys/fs/cgroup/cpu.max", "/sys/fs/cgroup/cpu/cpu.cfs_quota_us"):
        try:
            with open(path) as f:
                parts = f.read().split()
            if path.endswith("cpu.max"):
                if parts[0] != "max":
                    n = min(n, max(1, math.ceil(int(parts[0]) / int(parts[1]))))
            else:
                quota = int(parts[0])
                if quota > 0:
                    with open("/sys/fs/cgroup/cpu/cpu.cfs_period_us") as f:
                        n = min(n, max(1, math.ceil(quota / int(f.read().split()[0]))))
            break
        except (OSError, ValueError, IndexError):
            continue
    return max(1, n)


def cpu_baseline(cfg, budget_s=12.0, acc64=False):
    """Times the oracle (fp32-accumulating port of the reference's naive kernel, OpenMP on all host
    cores) on a bounded sample of the workload: all query rows of `heads` (batch, head) slices, or
    a row sample of one slice when even one slice exceeds the budget. Returns effective TFLOP/s."""
    import oracle
    _, _, _, _, shape, D, ks, st, di, ca, n_extra, mul = cfg
    rng = np.random.default_rng(0)
    N = math.prod(shape)
    cores = oracle.set_threads(host_threads())
    pairs_per_row = (attended_pairs(shape, ks, st, di, ca) + n_extra * N) / N

    def run(heads, rows):
        q = rng.standard_normal((1, *shape, heads, D), dtype=np.float32) * mul
        k = rng.standard_normal((1, *shape, heads, D), dtype=np.float32) * mul
        v = rng.standard_normal((1, *shape, heads, D), dtype=np.float32) * mul
        ak = av = None
        if n_extra:
            ak = rng.standard_normal((1, n_extra, heads, D), dtype=np.float32)
            av = rng.standard_normal((1, n_extra, heads, D), dtype=np.float32)
        t0 = time.perf_counter()
        oracle.na_forward(q, k, v, ks, st, di, ca, add_k=ak, add_v=av, tok_idx=rows, acc64=acc64)
        return time.perf_counter() - t0

    n = min(N, 64 * cores)
    rows = np.sort(rng.choice(N, size=n, replace=False)).astype(np.int64)
    dt = run(1, rows)                      # calibration
    per_row = max(dt, 1e-4) / n
    want_rows = budget_s / per_row
    if want_rows <= N:
        heads, n2 = 1, int(max(n, min(N, want_rows)))
    else:
        heads, n2 = int(min(8, max(1, want_rows // N))), N
    rows = None if n2 == N else np.sort(rng.choice(N, size=n2, replace=False)).astype(np.int64)
    dt = run(heads, rows)
    flops = 4.0 * D * pairs_per_row * n2 * heads
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=cores, kind="port",
                sample=f"{n2} of {N} query rows of {heads} (batch, head) slice(s), fp32 "
                       f"accumulation, OpenMP on {cores} threads, {dt:.1f} s"), dt, n2 * heads


def run_reference_arm(args, cfg, rank):
    if rank != 0:
        return
    steps, warmup = args.steps, args.warmup
    per_step_budget = max(1.0, min(12.0, 120.0 / max(1, steps + warmup)))
    vals, times = [], []
    info = None
    for i in range(warmup + steps):
        info, dt, _ = cpu_baseline(cfg, budget_s=per_step_budget)
        if i >= warmup:
            vals.append(info["value"])
            times.append(dt)
    v = float(np.mean(vals))
    info["value"] = v
    line = dict(metric="FNA fwd effective TFLOPS (unmasked FLOPs)", value=v, unit="TFLOP/s",
                impl="reference", n_gpus=args.gpus, steps=steps, warmup=warmup,
                ms_per_step=float(np.mean(times)) * 1e3, higher_is_better=True, scaling="strong",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=WORKLOAD_TEXT[args.config], sample=info["sample"]),
                cpu_baseline=info,
                e2e=dict(value=v, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def row_sample(shape, kernel, n_rows, seed=0):
    """Flat token indices to check: half of them uniformly random, the other half forced into the
    border bands (coordinate within one kernel size of either end of an axis, each axis and side
    in turn), where windows are clamped, shifted or causal-truncated."""
    rng = np.random.default_rng(seed)
    N = math.prod(shape)
    n_rows = min(n_rows, N)
    picks = [rng.integers(0, N, size=n_rows // 2)]
    nd = len(shape)
    per = max(1, (n_rows - n_rows // 2) // (2 * nd))
    for a in range(nd):
        band = min(kernel[a], shape[a])
        for side in (0, 1):
            coords = [rng.integers(0, shape[b], size=per) for b in range(nd)]
            coords[a] = rng.integers(0, band, size=per) + (0 if side == 0 else shape[a] - band)
            picks.append(np.ravel_multi_index(coords, shape))
    return np.unique(np.concatenate(picks)).astype(np.int64)


def check_against_oracle(cfg, host, extra, out, lse, n_rows, tol):
    """Compares the timed call's own output with the CPU oracle on a row sample: every batch
    entry, the first and the last head, rows from row_sample(). Returns the `checked` record."""
    import oracle
    import torch
    _, _, _, _, shape, D, ks, st, di, ca, n_extra, _ = cfg
    oracle.set_threads(host_threads())
    B, H = host[0].shape[0], host[0].shape[-2]
    heads = sorted({0, H - 1})
    rows = row_sample(shape, ks, n_rows)
    nd = len(shape)
    idx = torch.from_numpy(rows)
    worst_o = worst_l = 0.0
    t0 = time.perf_counter()
    for b in range(B):
        q, k, v = (t[b:b + 1][..., heads, :].float().numpy() for t in host)
        ak = av = None
        if n_extra:
            ak, av = (t[b:b + 1][..., heads, :].float().numpy() for t in extra)
        want_o, want_l = oracle.na_forward(q, k, v, ks, st, di, ca, add_k=ak, add_v=av,
                                           tok_idx=rows)
        got_o = out[b].flatten(0, nd - 1)[idx.to(out.device)][:, heads].float().cpu().numpy()
        got_l = lse[b].flatten(0, nd - 1)[idx.to(lse.device)][:, heads].float().cpu().numpy()
        worst_o = max(worst_o, float(np.abs(got_o - want_o[0]).max()))
        worst_l = max(worst_l, float(np.abs(got_l - want_l[0]).max()))
    return dict(rows=int(len(rows)) * B * len(heads), rows_per_slice=int(len(rows)),
                batch_entries=B, heads=heads, max_abs_out=worst_o, max_abs_lse=worst_l, tol=tol,
                oracle_s=round(time.perf_counter() - t0, 2),
                ok=bool(worst_o <= tol and worst_l <= tol))


def time_cuda(fn, steps, warmup=3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def kernels_leg(cfg, nb, dq, dk, out, lse, q_tile, kv_tile, peaks, steps=10):
    """The bandwidth-bound kernels of the path, timed alone at this config's shapes and tile
    shapes: token permute (Q with the query tile, K with the key/value tile), token unpermute of
    O and of the LSE rows, and the LSE merge of two attention results. Algorithmic bytes = the
    unpadded elements, one read and one write each (merge: two reads and one write of O and
    LSE). Every operand is re-read from HBM: each call's working set (>= 2 x the tensor) is far
    larger than L2 for the BASELINE configs; small configs are marked."""
    import torch
    _, _, _, _, shape, D, _, _, di, _, _, _ = cfg
    res = {}
    nd = len(shape)
    hbm = peaks["hbm_gbs"]
    es = dq.element_size()

    def rec(ms, nbytes):
        return dict(ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / hbm,
                    bytes=int(nbytes), l2_cold=bool(nbytes > 2 * 126e6))

    if nd == 1 and di[0] == 1 and shape[0] % 256 == 0:
        res["token_permute"] = res["token_unpermute"] = res["lse_unpermute"] = dict(
            ms=0.0, note="identity layout: the operator makes no copy")
    else:
        qb = dq.numel() * es * 2
        res["token_permute"] = rec(time_cuda(lambda: nb.token_permute_operation(dq, q_tile, di), steps), qb)
        kb = dk.numel() * es * 2
        res["token_permute_kv"] = rec(time_cuda(lambda: nb.token_permute_operation(dk, kv_tile, di), steps), kb)
        o_perm, qkv_shape, q_shape = nb.token_permute_operation(out, q_tile, di)
        o_perm = o_perm.reshape(-1, math.prod(q_shape), *o_perm.shape[-2:])
        res["token_unpermute"] = rec(time_cuda(
            lambda: nb.token_unpermute_operation(o_perm, qkv_shape, q_tile, di), steps), qb)
        l_perm, _, _ = nb.token_permute_operation(lse.unsqueeze(-1).contiguous(), q_tile, di)
        l_perm = l_perm.reshape(-1, math.prod(q_shape), *l_perm.shape[-2:])
        res["lse_unpermute"] = rec(time_cuda(
            lambda: nb.token_unpermute_operation(l_perm, qkv_shape, q_tile, di), steps),
            lse.numel() * 4 * 2)
        del o_perm, l_perm
    o_flat, l_flat = out.flatten(1, nd), lse.flatten(1, nd)
    o2 = o_flat.clone()
    l2 = l_flat.clone()
    mb = 3 * o_flat.numel() * es + 3 * l_flat.numel() * 4
    res["merge"] = rec(time_cuda(lambda: nb.merge_attentions([o_flat, o2], [l_flat, l2]), steps), mb)
    del o2, l2
    torch.cuda.empty_cache()
    return res


def spatial_subrecord(cfg, world, rank, dev, barrier, steps):
    """Config 5 partitioned along T instead of by heads: every rank holds all heads of its slab
    of frames, receives the key/value frames its windows reach before the slab from their
    owners (NCCL point-to-point) while it already attends its own frames, and merges the two
    partial results. Returns ms per step (max over ranks is taken by the caller's reduction
    below), the aggregate effective TFLOP/s, the exchange alone and the halo bytes per rank."""
    import torch
    import torch.distributed as dist
    from natten_b200 import sharding
    _, dt, B, H, shape, D, ks, st, di, ca, _, _ = cfg
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16}[dt]
    import natten_b200 as nb
    q_tile, _ = nb.choose_tile_shapes(shape, ks, st, di, ca)
    # slabs of equal attention work (the first 15 frames of a causal axis have shorter windows)
    plan = sharding.make_halo_plan(shape[0], world, ks[0], st[0], ca[0], balanced=True,
                                   align=q_tile[0])
    t0, t1 = plan.slabs[rank]
    def frames(which, a, b):
        # frame t of tensor `which` is a function of (which, t) alone, so a rank can rebuild the
        # frames its neighbours own and check what the exchange delivered
        out = []
        for t in range(a, b):
            g = torch.Generator(device=dev).manual_seed(5000 + 100 * which + t)
            out.append(torch.randn((B, 1, *shape[1:], H, D), generator=g, device=dev,
                                   dtype=torch.float32).to(dtype))
        return torch.cat(out, dim=1)

    q, k, v = (frames(i, t0, t1) for i in range(3))

    def run():
        return sharding.na_forward_spatial_shard(q, k, v, shape, ks, st, ca, rank=rank, world=world,
                                                 plan=plan)

    def exchange_only():
        return sharding.exchange_halo(k, v, plan, rank)

    for _ in range(3):
        run()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    for _ in range(2):
        exchange_only()
    barrier()
    x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    x0.record()
    for _ in range(steps):
        exchange_only()
    x1.record()
    barrier()
    xms = x0.elapsed_time(x1) / steps
    # the overlapped result on real ranks against one kernel over locally rebuilt halo frames
    lo, hi = plan.needs[rank]
    got_o, got_l = run()
    ref_o, ref_l = sharding.fna_forward_slab(q, frames(1, lo, hi), frames(2, lo, hi), shape, t0, lo,
                                             ks, st, ca)
    err_o = float((got_o.float() - ref_o.float()).abs().max())
    err_l = float((got_l - ref_l).abs().max())
    del got_o, got_l, ref_o, ref_l
    t = torch.tensor([ms, xms, err_o, err_l], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, xms, err_o, err_l = (float(x) for x in t.tolist())
    if err_o > 2e-2 or err_l > 2e-2:
        raise SystemExit(f"spatial partitioning: slab differs from the local reference "
                         f"(out {err_o:.3e}, lse {err_l:.3e})")
    frame_bytes = math.prod(shape[1:]) * H * D * q.element_size() * B
    halo = [plan.halo_frames(r) * frame_bytes * 2 for r in range(world)]
    return dict(partition="slabs of axis 0 (T), all heads per rank; halo of K/V frames by NCCL "
                          "send/recv, overlapped with attention over the rank's own frames; "
                          "output stays sharded",
                ms_per_step=ms, value=algorithmic_flops(cfg) / (ms * 1e-3) / 1e12,
                unit="TFLOP/s", exchange_ms=xms,
                halo_bytes=int(max(halo)), halo_frames=int(max(plan.halo_frames(r) for r in range(world))),
                slabs=[list(x) for x in plan.slabs], steps=steps,
                checked=dict(against="one kernel over locally rebuilt halo frames, every row of "
                                     "every rank's slab", max_abs_out=err_o, max_abs_lse=err_l,
                             tol=2e-2))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c5", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--partition", default="units", choices=["units", "spatial"],
                    help="multi-GPU partitioning: (batch x heads) units, or slabs of the outermost "
                         "axis with a key/value halo exchange (config c5 only)")
    ap.add_argument("--units", type=int, default=0,
                    help="profiling aid: shrink the problem to this many (batch x head) units "
                         "(batch 1); the printed line is then NOT a benchmark value")
    ap.add_argument("--eager", action="store_true",
                    help="time eager operator calls instead of CUDA-graph replays of one call")
    ap.add_argument("--pass", dest="pass_", default="forward", choices=["forward", "backward"],
                    help="backward: time the gradient kernels (delta + dQ pass + dK/dV pass) "
                         "instead of the forward call; an extra, not the BASELINE metric")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the oracle check of the output")
    ap.add_argument("--no-kernels", action="store_true",
                    help="skip the permute / unpermute / merge bandwidth legs")
    ap.add_argument("--kernel-steps", type=int, default=10,
                    help="timed launches per bandwidth-bound kernel in the `kernels` legs")
    ap.add_argument("--check-rows", type=int, default=4608,
                    help="query rows per (batch, head) slice compared with the oracle")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    if args.units:
        cfg = cfg[:2] + (1, args.units) + cfg[4:]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, cfg, rank)
        return
    if args.warmup < 3 and not args.units:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    import natten_b200 as nb
    import natten_b200._lib as L

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    op, dt, B, H, shape, D, ks, st, di, ca, n_extra, _ = cfg
    spatial = args.partition == "spatial" and world > 1
    if args.partition == "spatial" and (n_extra or any(d != 1 for d in di)):
        raise SystemExit("--partition spatial needs an undilated config without extra KV (c5)")
    if spatial:
        from natten_b200 import sharding
        plan = sharding.make_halo_plan(shape[0], world, ks[0], st[0], ca[0])
        b_local, h_local = B, H
        host, extra = make_inputs(cfg, B, H, 1000 + rank, dev, slab=plan.slabs[rank])
        work_fraction = None  # FLOPs of this rank's rows are computed below
    else:
        b_local, h_local = shard_units(B, H, world, rank)
        host, extra = make_inputs(cfg, b_local, h_local, 1000 + rank, dev)
    fn = getattr(nb, op)

    def call(q, k, v, ak=None, av=None):
        if spatial:
            return sharding.na_forward_spatial_shard(q, k, v, shape, ks, st, ca, rank=rank,
                                                     world=world)
        return fn(q, k, v, kernel_size=ks, stride=st, dilation=di, is_causal=ca,
                  additional_keys=ak, additional_values=av, return_lse=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    dq, dk, dv = (t.to(dev, non_blocking=True) for t in host)
    dak, dav = (t.to(dev, non_blocking=True) for t in extra) if n_extra else (None, None)
    torch.cuda.synchronize()

    if args.pass_ == "backward":
        run_backward(args, cfg, nb, L, dq, dk, dv, dak, dav, b_local, h_local, rank, world, barrier)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- device-resident timing (inputs already in HBM; operands far exceed the 126 MB L2) ----
    for _ in range(args.warmup):
        out, lse = call(dq, dk, dv, dak, dav)
    # One operator call is captured into a CUDA graph and replayed per step, so that host-side
    # launch latency and OS jitter (8 ranks share the host's cores) do not open gaps between the
    # sub-millisecond steps of the multi-GPU runs. The graph holds exactly the kernels one call
    # launches; spatial mode (NCCL point-to-point inside the step) stays eager. The cost of an
    # eager call is reported beside it (`eager_ms_per_step`).
    graph = None
    launches_per_step = None
    if not spatial and not args.eager:
        try:
            torch.cuda.synchronize()
            L.launches = 0
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out, lse = call(dq, dk, dv, dak, dav)
            launches_per_step = L.launches
            for _ in range(2):
                graph.replay()
            torch.cuda.synchronize()
        except Exception as e:  # capture not possible here: time eager calls instead
            print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); eager steps",
                  file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def step():
        nonlocal out, lse
        if graph is not None:
            graph.replay()
        else:
            out, lse = call(dq, dk, dv, dak, dav)

    # Three blocks of exactly `steps` steps, each bracketed by a barrier and a device
    # synchronisation; the reported step time is the median block's (max over ranks per block).
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    L.launches = 0
    block_ms = []
    for _ in range(3):
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
        block_ms.append(ev0.elapsed_time(ev1))
    launches = (L.launches if graph is None else launches_per_step * args.steps * 3) // 3
    clocks = sampler.stop() if rank == 0 else None
    status = L.device_status()

    # ---- the same step as plain eager operator calls (host launch cost included) ----
    eager_ms = None
    if graph is not None:
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            call(dq, dk, dv, dak, dav)
        g1.record()
        barrier()
        eager_ms = g0.elapsed_time(g1) / args.steps

    # ---- the fused attention kernel alone (roofline of the dominant kernel) ----
    tensor_core = dt != "fp32"
    q_tile, kv_tile = nb.choose_tile_shapes(shape, ks, st, di, ca)
    kernel_alone = tensor_core and not spatial
    if kernel_alone:
        scale = D ** -0.5
        if nb.direct_layout_supported(q_tile, kv_tile, di):
            def kernel_call():
                nb.fna_forward_direct(dq, dk, dv, ks, st, di, ca, scale, q_tile, kv_tile)
        else:
            qp, qkv_shape, q_shape = nb.token_permute_operation(dq, q_tile, di)
            kp, _, kv_shape = nb.token_permute_operation(dk, kv_tile, di)
            vp, _, _ = nb.token_permute_operation(dv, kv_tile, di)
            qp = qp.reshape(-1, math.prod(q_shape), h_local, D)
            kp = kp.reshape(-1, math.prod(kv_shape), h_local, D)
            vp = vp.reshape(-1, math.prod(kv_shape), h_local, D)

            def kernel_call():
                nb.fna_forward_op(qp, kp, vp, qkv_shape, q_shape, kv_shape, ks, st, di, ca, scale,
                                  q_tile, kv_tile)
        kernel_ms = time_cuda(kernel_call, args.steps)
    else:
        kernel_ms = float(np.median(block_ms)) / args.steps

    # ---- the timed call's own output against the oracle (row sample) ----
    checked = None
    if not spatial and not args.no_check:
        tol = 1e-4 if dt == "fp32" else 2e-2
        checked = check_against_oracle(cfg, host, extra, out, lse, args.check_rows, tol)

    # ---- the bandwidth-bound kernels of the path at this config's shapes ----
    peaks = read_peaks()
    kernels = None
    if rank == 0 and tensor_core and not spatial and not args.no_kernels:
        kernels = kernels_leg(cfg, nb, dq, dk, out, lse, q_tile, kv_tile, peaks,
                              steps=args.kernel_steps)

    # ---- end to end through the public operator with HOST buffers ----
    e2e_ms = None
    h2d = sum(t.numel() * t.element_size() for t in host + extra)
    d2h = out.numel() * out.element_size() + lse.numel() * lse.element_size()
    if not args.no_e2e:
        out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        lse_h = torch.empty(lse.shape, dtype=lse.dtype).pin_memory()

        def e2e_step():
            # the repository's host-operand entry point: chunks of (batch, heads) are pipelined,
            # so the H2D copy of one chunk, the kernel of the previous and the D2H copy of the
            # one before overlap (spatial mode: plain copies around the sharded call)
            if spatial:
                tq, tk, tv = (t.to(dev, non_blocking=True) for t in host)
                o, l = call(tq, tk, tv, None, None)
                out_h.copy_(o, non_blocking=True)
                lse_h.copy_(l, non_blocking=True)
                return
            nb.na_forward_from_host(host[0], host[1], host[2], ks, st, di, ca,
                                    additional_keys=extra[0] if n_extra else None,
                                    additional_values=extra[1] if n_extra else None,
                                    out=out_h, lse=lse_h, device=dev)

        for _ in range(3):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, min(args.steps, 10))
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / n_e2e
        del out_h, lse_h

    # ---- config 5 on several GPUs: the T-axis slab partitioning beside the head partitioning ----
    spatial_rec = None
    if world > 1 and args.config == "c5" and not spatial and not args.units:
        del dq, dk, dv, out, lse, graph
        torch.cuda.empty_cache()
        spatial_rec = spatial_subrecord(cfg, world, rank, dev, barrier, max(3, args.steps // 2))

    # ---- max over ranks ----
    t = torch.tensor(block_ms + [kernel_ms, e2e_ms or 0.0, float(status), eager_ms or 0.0,
                                 0.0 if checked is None or checked["ok"] else 1.0,
                                 checked["max_abs_out"] if checked else 0.0,
                                 checked["max_abs_lse"] if checked else 0.0],
                     device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    vals = [float(x) for x in t.tolist()]
    block_ms = vals[:3]
    kernel_ms_max, e2e_ms_max, status_max, eager_ms_max, check_failed, worst_o, worst_l = vals[3:]
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        if check_failed:
            raise SystemExit(1)
        return
    if status_max != 0:
        raise SystemExit(f"device status word {int(status_max)}: a bounded wait expired in the kernel")

    flops_all = algorithmic_flops(cfg)
    fna_flops_rank = 4.0 * D * attended_pairs(shape, ks, st, di, ca) * b_local * h_local
    if spatial:
        fna_flops_rank /= world  # rows are split evenly; the roofline entry is then approximate
    ms_step = float(np.median(block_ms)) / args.steps
    value = flops_all / (ms_step * 1e-3) / 1e12
    achieved = fna_flops_rank / (kernel_ms_max * 1e-3) / 1e12
    if checked is not None:
        checked.update(max_abs_out=worst_o, max_abs_lse=worst_l, ok=not check_failed,
                       ranks=world)
    line = dict(
        metric="FNA fwd effective TFLOPS (unmasked FLOPs)", value=value, unit="TFLOP/s",
        n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms_step,
        higher_is_better=True, scaling="strong", vs_baseline=None, dtype=dt, data="synthetic",
        config=dict(workload=WORKLOAD_TEXT[args.config] + (
            f" [REDUCED to {args.units} (batch x head) units for profiling: not a benchmark value]"
            if args.units else ""),
                    partition=("slabs of axis 0 + NCCL halo exchange of K/V, output stays sharded"
                               if spatial else "batch x heads, no collective"),
                    units_per_gpu=b_local * h_local,
                    launch="cuda-graph replay of one operator call" if graph_used(launches_per_step)
                    else "eager operator calls", l2="inputs larger than L2 (no flush needed)"
                    if h2d > 2 * 126e6 else "inputs SMALLER than L2: latency figure, not bandwidth",
                    q_tile=list(q_tile), kv_tile=list(kv_tile)),
        blocks=dict(n=3, steps_each=args.steps, ms_per_step_median=ms_step,
                    ms_per_step_min=min(block_ms) / args.steps,
                    ms_per_step_max=max(block_ms) / args.steps),
        eager_ms_per_step=eager_ms_max or None,
        clocks=clocks, gpu_launches=int(launches),
    )
    if tensor_core:
        line["roofline"] = dict(
            bound="tensor", achieved=achieved, peak=peaks["bf16_tflops"], unit="TFLOP/s",
            frac=achieved / peaks["bf16_tflops"],
            traffic=(NCU_TRAFFIC_PER_UNIT[args.config] * b_local * h_local
                     if args.config in NCU_TRAFFIC_PER_UNIT and not spatial else None),
            kernel="fna_fwd_kernel", kernel_ms=kernel_ms_max,
            peak_source=peaks["source"] + " burst (kernel timed alone)",
            frac_of_sustained=achieved / peaks["bf16_tflops_sustained"])
        if args.config == "c3":
            # 84 FLOP/B: below the ridge, so the bound that applies is HBM, on the kernel's minimum
            # traffic (Q, K, V read once, O and LSE written once)
            es = 2
            alg = (4 * math.prod(shape) * D * es + math.prod(shape) * 4) * b_local * h_local
            gbs = alg / kernel_ms_max / 1e6
            line["roofline"].update(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                                    frac=gbs / peaks["hbm_gbs"], tensor_tflops=achieved,
                                    peak_source=peaks["source"] + " copy bandwidth")
    else:
        line["roofline"] = dict(bound="latency", achieved=None, peak=None, unit="ms", frac=None,
                                traffic=None, kernel="na_simt_kernel", kernel_ms=ms_step,
                                note="config 1 is 26 MFLOP on 2 MB: a latency figure")
    if args.config in PUBLISHED:
        pms, ptf, src = PUBLISHED[args.config]
        line["published"] = dict(ms=pms, eff_tflops=ptf, source=src,
                                 hardware="B200 (the reference authors' machine)",
                                 kernel_ms_here=kernel_ms_max, ratio_time=pms / kernel_ms_max)
    if checked is not None:
        line["checked"] = checked
    if kernels is not None:
        line["kernels"] = kernels
    if spatial_rec is not None:
        line["spatial"] = spatial_rec
    if e2e_ms_max > 0:
        line["e2e"] = dict(value=flops_all / (e2e_ms_max * 1e-3) / 1e12, unit="TFLOP/s",
                           ms_per_step=e2e_ms_max, h2d_bytes_per_step=int(h2d),
                           d2h_bytes_per_step=int(d2h))
    if world == 1 and not args.no_cpu_baseline:
        info, _, _ = cpu_baseline(cfg)
        line["cpu_baseline"] = info
    print(json.dumps(line), flush=True)
    if check_failed:
        raise SystemExit(f"output check failed: max|out| {worst_o:.3e}, max|lse| {worst_l:.3e}")


def graph_used(launches_per_step):
    return launches_per_step is not None


def run_backward(args, cfg, nb, L, q, k, v, ak, av, b_local, h_local, rank, world, barrier):
    """Times the backward (delta + dQ pass + dK/dV pass, or the CUDA-core kernels when the config
    has extra tokens) on device-resident operands and prints one JSON line of the same shape as
    the forward's, without the end-to-end and CPU legs."""
    import torch
    import torch.distributed as dist
    import natten_b200.functional as F
    from natten_b200 import ops
    op, dt, B, H, shape, D, ks, st, di, ca, n_extra, _ = cfg
    fn = getattr(nb, op)
    out, lse = fn(q, k, v, kernel_size=ks, stride=st, dilation=di, is_causal=ca,
                  additional_keys=ak, additional_values=av, return_lse=True)
    torch.manual_seed(77 + rank)
    d_out = torch.randn(out.shape, device=out.device).to(out.dtype)
    causal = [bool(c) for c in ca]
    q_tile, kv_tile = F.choose_backward_tile_shapes(shape, ks, st, di, ca)
    tensor_core = F.backward_layout_supported(q_tile, kv_tile, di)

    def step():
        if tensor_core:
            return ops.na_backward_direct(q, k, v, out, d_out, lse, ak, av, list(ks), list(st),
                                          list(di), causal, D ** -0.5, list(q_tile), list(kv_tile))
        return ops.na_backward_simt(q, k, v, out, d_out, lse, ak, av, list(ks), list(st), list(di),
                                    causal, D ** -0.5)

    for _ in range(max(1, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    L.launches = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    launches = L.launches
    clocks = sampler.stop() if rank == 0 else None
    status = L.device_status()
    t = torch.tensor([e0.elapsed_time(e1), float(status)], device=q.device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, status_max = (float(x) for x in t.tolist())
    if rank != 0:
        return
    if status_max != 0:
        raise SystemExit(f"device status word {int(status_max)}: a bounded wait expired in the kernel")
    peaks = read_peaks()
    flops = 2.5 * algorithmic_flops(cfg)       # 5 products in the backward for 2 in the forward
    ms_step = ms_total / args.steps
    value = flops / (ms_step * 1e-3) / 1e12
    print(json.dumps(dict(
        metric="FNA bwd effective TFLOPS (unmasked FLOPs, 2.5 x forward)", value=value,
        unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms_step,
        higher_is_better=True, scaling="strong", vs_baseline=None, dtype=dt, data="synthetic",
        config=dict(workload=WORKLOAD_TEXT[args.config] + " [backward pass]" + (
            f" [REDUCED to {args.units} (batch x head) units for profiling: not a benchmark value]"
            if args.units else ""),
                    partition="batch x heads, no collective", units_per_gpu=b_local * h_local,
                    launch="eager", l2="inputs larger than L2 (no flush needed)",
                    kernels=("delta_kernel + fna_bwd_kernel (dQ pass) + fna_bwd_kernel (dK/dV pass)"
                             if tensor_core else "CUDA-core gradient kernels"),
                    q_tile=list(q_tile), kv_tile=list(kv_tile)),
        clocks=clocks, gpu_launches=int(launches),
        roofline=dict(bound="tensor", achieved=value / world, peak=peaks["bf16_tflops"],
                      unit="TFLOP/s", frac=value / world / peaks["bf16_tflops"], traffic=None,
                      kernel="fna_bwd_kernel", kernel_ms=ms_step,
                      peak_source=peaks["source"] + " burst"))), flush=True)


if __name__ == "__main__":
    main()
