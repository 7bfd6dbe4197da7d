#!/usr/bin/env python
"""Benchmark of the sparse-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c5]

Headline workload (``config.workload``): the Infinity-2B 1024^2 last-scale block-sparse attention case -
B=2 (CFG pair), H=16, head dim 128, Lq=4096, Lkv=10521, bf16, 128x128 blocks with 17 of 83 KV blocks
active per query-block row (20 %): the KV blocks of scales <= 16x16, each query block's own position,
and the best remaining blocks by column-sum block score.  Q/K/V are seeded N(0,1) with a rank-8
component (scale 2.0) on K so the column sums are peaked.  Synthetic data of that shape stands in for
real Infinity activations.

One step = one block-sparse attention pass over the batch.  ``value`` is TFLOP/s on ACTIVE blocks
(4*D*rows*cols per active block pair, true extents) with inputs resident in HBM, timed with CUDA
events on the launching stream.  ``e2e`` is the same metric through ``sparse_attn_ops.block_sparse_attn``
starting from pinned HOST buffers (H2D of q/k/v/mask and D2H of the output inside the timed region).
With N > 1 every rank runs the same workload on its own GPU (the path shards by batch x head with no
data-path collective): weak scaling.  Before anything is timed, the mask is compared bit for bit and one
sampled head's output within tolerance with the CPU oracle (``config.parity_checked``).

``extra`` carries, untimed by the headline: the other kernels of the path (dense attention, column sums in
their three forms, column-sparse attention, CS4A layer steps, per-scale KV scoring), the HBM-bound index
kernels against the measured copy bandwidth, scheduling A/B runs, the sharded 2048px-style configuration with
its one all-gather, the reference's own Triton kernels on the same GPU (context only) and the full
generation loop in images/s.  ``--workload c5`` runs only the generation loop, longer.

``--impl reference`` times the CPU restatement of the reference's path (dense masked fp32 attention in
PyTorch on the host cores, ``oracle/``) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import contextlib
import gc
import io
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, H, D, LQ, LKV = 2, 16, 128, 4096, 10521
BLOCK = 128
K_TOTAL = 17          # round(0.2 * 83) active KV blocks per query-block row
SINK_TOKENS = 521     # scales <= 16x16
Q_OFFSET = 6425       # position of the last scale's first token on the KV axis
METRIC = "block_sparse_attn_tflops_active"
UNIT = "TFLOP/s"
WORKLOAD = ("infinity2b-1024px-last-scale block-sparse attention: B2 H16 D128 Lq4096 Lkv10521 bf16, "
            "128x128 blocks, 17/83 active per row (sink<=16x16 + local + top-k by colsum)")
PRE_ROLL = 8  # untimed steps queued between the synchronize and the start event of the timed region
# dram__bytes_read.sum + dram__bytes_write.sum of one attn_fwd_kernel<128, block-sparse> launch on this
# workload (one ncu capture of two full launches): 167.9 / 167.2 MB read + 27.0 / 21.8 MB written
TRAFFIC_BYTES_PER_LAUNCH = 192.0e6
C5_PROMPTS = 16       # prompts per generated batch of the full-loop configuration (x2 for guidance)


def make_inputs(seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, LQ, D, generator=g)
    k = torch.randn(B, H, LKV, D, generator=g)
    v = torch.randn(B, H, LKV, D, generator=g)
    k = k + 2.0 * (torch.randn(B, H, LKV, 8, generator=g) @ torch.randn(B, H, 8, D, generator=g))
    return q.bfloat16(), k.bfloat16(), v.bfloat16()


def cosine_variant(q, k):
    """The cosine-attention form of the same inputs (unit-norm q and k, q scaled by 4, softmax scale 1), as
    the model's self-attention produces them."""
    qn = (torch.nn.functional.normalize(q.float(), dim=-1) * 4.0).to(q.dtype)
    kn = torch.nn.functional.normalize(k.float(), dim=-1).to(k.dtype)
    return qn, kn


def recipe_mask(K, P, q, k, v, scale):
    """The benchmark's mask recipe on the GPU: fused attention + column sums -> block scores -> always-kept
    blocks (sink + own position) -> top-k to K_TOTAL per row.  Returns (mask, scores, always, cs, o, M, L)."""
    nq, nk = (LQ + BLOCK - 1) // BLOCK, (LKV + BLOCK - 1) // BLOCK
    o_dense, cs, M, L = K.dense_colsum_attn_fwd(q, k, v, scale, return_stats=True)
    scores = K.block_scores(cs, BLOCK)
    always = P.sink_local_blocks(nq, nk, BLOCK, SINK_TOKENS, Q_OFFSET, 0, LQ)
    mask = K.build_block_mask(scores, always.to(q.device), K_TOTAL)
    return mask, scores, always, cs, o_dense, M, L


def check_recipe_parity(K, q, k, v, scale, mask, scores, always, heads):
    """Mask bit for bit against the oracle's builder on the SAME scores; block-sparse output of the sampled
    (batch, head) pairs within max-abs 2e-2 / mean-abs 2e-3 of the oracle's dense masked fp32 attention."""
    from oracle import attention as oa
    from oracle import indexing as oi
    want = oi.build_block_mask(scores.cpu(), always, K_TOTAL)
    assert torch.equal(mask.cpu(), want), "block mask differs from the oracle's on identical scores"
    o = K.block_sparse_attn_fwd(q, k, v, mask, scale)
    worst = (0.0, 0.0)
    for b, h in heads:
        sl = (slice(b, b + 1), slice(h, h + 1))
        ref = oa.block_sparse_attn(q[sl].cpu(), k[sl].cpu(), v[sl].cpu(), mask[sl].cpu(), scale, block=BLOCK)
        d = (o[sl].float().cpu() - ref).abs()
        assert torch.isfinite(o[sl].float()).all()
        assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3, \
            f"block-sparse output of (b={b}, h={h}) off the oracle: max {d.max().item():.3e} mean {d.mean().item():.3e}"
        worst = (max(worst[0], d.max().item()), max(worst[1], d.mean().item()))
    return worst


def active_flops(mask: torch.Tensor) -> float:
    """4*D*rows*cols over the active (query block, KV block) pairs, true extents."""
    nq, nk = mask.shape[-2:]
    rows = torch.full((nq,), float(BLOCK))
    rows[-1] = LQ - (nq - 1) * BLOCK
    cols = torch.full((nk,), float(BLOCK))
    cols[-1] = LKV - (nk - 1) * BLOCK
    area = rows.view(-1, 1) * cols.view(1, -1)
    return float(4.0 * D * (mask.float().cpu() * area).sum())


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16": float(d["bf16_tflops"]), "bf16_sustained": float(d.get("bf16_tflops_sustained", 1400.0)),
                "hbm": float(d["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0,
            "source": "fallback (1.59 PFLOP/s, 6.65 TB/s: earlier measurement on this pool)"}


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_masked_attention_sample(q, k, v, mask, heads, threads):
    """Dense masked fp32 attention on the host for `heads` (batch, head) pairs -> seconds."""
    from oracle import attention as oa
    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    for i in range(heads):
        b, h = divmod(i, H)
        oa.block_sparse_attn(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1],
                             mask[b:b + 1, h:h + 1], 1.0 / math.sqrt(D), block=BLOCK)
    return time.perf_counter() - t0


def cpu_reference_mask(q, k, v):
    """CPU restatement of the mask recipe for the reference arm (column sums of 2 heads are enough to
    shape a representative mask; the remaining heads reuse them so the run stays bounded)."""
    from oracle import attention as oa
    from oracle import indexing as oi
    nq, nk = (LQ + BLOCK - 1) // BLOCK, (LKV + BLOCK - 1) // BLOCK
    always = oi.sink_local_blocks(nq, nk, BLOCK, SINK_TOKENS, Q_OFFSET, 0, LQ)
    _, cs = oa.dense_colsum_attn(q[:1, :2], k[:1, :2], v[:1, :2], 1.0 / math.sqrt(D), q_group_size=BLOCK)
    m = oi.build_block_mask(oi.block_scores(cs, BLOCK).float(), always, K_TOTAL)
    return m.repeat(B, H // 2, 1, 1)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cores = os.cpu_count() or 1
    q, k, v = make_inputs()
    mask = cpu_reference_mask(q, k, v)
    per_head = active_flops(mask[0, 0])
    heads_per_step = 1
    times = []
    for i in range(args.warmup + args.steps):
        dt = cpu_masked_attention_sample(q, k, v, mask, heads_per_step, cores)
        if i >= args.warmup:
            times.append(dt)
    t = sum(times) / len(times)
    val = per_head * heads_per_step / t / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"{heads_per_step} of {B * H} (batch, head) pairs per step"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"dense masked fp32 attention (oracle) on {heads_per_step} (batch, head) pair "
                                   f"per step, {args.steps} steps"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------------
# timing helpers
# ------------------------------------------------------------------------------------------------------
def ev():
    return torch.cuda.Event(enable_timing=True)


def timed(fn, iters, warm=3):
    """Mean milliseconds per call: CUDA events on the current stream, two untimed calls queued ahead of the
    start event so that the timed calls start on a busy GPU."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = ev(), ev()
    for _ in range(2):
        fn()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def timed_interleaved(fns, iters=4, rounds=7, warm=2, spread=False):
    """Median milliseconds per call of each function in `fns`, the functions taking turns in blocks of `iters`
    calls for `rounds` rounds: ratios between them are then taken at the same clocks and temperature.  With
    `spread`, (median, fastest round, slowest round) per function."""
    for fn in fns:
        for _ in range(warm):
            fn()
    torch.cuda.synchronize()
    marks = []
    for _ in range(rounds):
        for i, fn in enumerate(fns):
            a, b = ev(), ev()
            fn()  # untimed: the timed calls of this block start on a busy GPU
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            marks.append((i, a, b))
    torch.cuda.synchronize()
    out = []
    for i in range(len(fns)):
        ms = sorted(a.elapsed_time(b) / iters for j, a, b in marks if j == i)
        out.append(statistics.median(ms) if not spread else (statistics.median(ms), ms[0], ms[-1]))
    return out


def max_over_ranks(x: float, dev, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------------------------------------------
# extra legs
# ------------------------------------------------------------------------------------------------------
def leg_hbm_kernels(K, P, q, k, v, cs, scale, dev, hbm_gbs):
    """The index / glue kernels of the path against the measured copy bandwidth: algorithmic bytes (every input
    byte read once + every output byte written once) / CUDA-event time / hbm_gbs."""
    out = {}

    def rec(name, nbytes, fn, iters=20):
        ms = timed(fn, iters)
        out[name] = {"us": round(ms * 1e3, 2), "algorithmic_mb": round(nbytes / 1e6, 2),
                     "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm": round(nbytes / ms / 1e6 / hbm_gbs, 3)}

    nq, nk = (LQ + BLOCK - 1) // BLOCK, (LKV + BLOCK - 1) // BLOCK
    always = P.sink_local_blocks(nq, nk, BLOCK, SINK_TOKENS, Q_OFFSET, 0, LQ).to(dev)
    scores = K.block_scores(cs, BLOCK)
    rec("block_scores", cs.numel() * 4 + scores.numel() * 4, lambda: K.block_scores(cs, BLOCK))
    rec("build_block_mask", scores.numel() * 5 + always.numel(), lambda: K.build_block_mask(scores, always, K_TOTAL))
    rec("mask_from_colsums(block_scores+build_block_mask)", cs.numel() * 4 + scores.numel() * 9,
        lambda: K.build_block_mask(K.block_scores(cs, BLOCK), always, K_TOTAL))
    rec("block_mask_from_colsums(one pass)", cs.numel() * 4 + scores.numel(),
        lambda: K.block_mask_from_colsums(cs, always, K_TOTAL, BLOCK))
    # decision-step top-k: 16 groups of 256 rows per head, 2176 of 10521 keys, lists padded to Lkv columns
    cs256 = K.sum_tiles(cs, 2).contiguous()
    rows = cs256.numel() // LKV
    rec("topk_indices(512 rows x 10521, k=2176)", rows * (4 * LKV + 4 * LKV),
        lambda: K.topk_indices(cs256, 2176, out_cols=LKV, with_counts=True))
    cs_row = cs.sum(2, keepdim=True).contiguous()
    rec("topk_indices(32 rows x 10521, k=1052, ascending)", 32 * (4 * LKV + 4 * 1052),
        lambda: K.topk_indices(cs_row, 1052, ascending_index=True))
    # sparse-step lists at the last scale: 12 -> 16 groups, 896 remapped keys + a 768-key band
    inds, _ = K.topk_indices(K.sum_tiles(cs, 2)[:, :, :12].contiguous(), 896, out_cols=6425, with_counts=True)
    remap = P.group_remap_table(16, 12).to(device=dev, dtype=torch.int32)
    band = (torch.arange(16, device=dev).view(-1, 1) * 256 + Q_OFFSET + torch.arange(768, device=dev).view(1, -1)
            ).clamp_(max=LKV - 1).to(torch.int32)
    rec("sparse_step_lists(16 groups, 896 + 768 keys)", B * H * 16 * (LKV * 4 + 896 * 4) + band.numel() * 4,
        lambda: K.sparse_step_lists(inds, remap, band, 896, LKV, count_value=1664))
    # QKV prologue of the last scale: normalise, scale, RoPE, append to the cache
    qkv = torch.randn(B, LQ, 3, H, D, device=dev).bfloat16()
    kc = torch.empty(B, H, LKV, D, device=dev, dtype=torch.bfloat16)
    vc = torch.empty_like(kc)
    sm = torch.full((H,), 4.0, device=dev)
    cos = torch.rand(LKV, D // 2, device=dev)
    sin = torch.rand(LKV, D // 2, device=dev)
    rec("qkv_prologue(B2 L4096 H16 c128)", 2 * qkv.numel() * 2 + LQ * D * 4,
        lambda: K.qkv_prologue(qkv, sm, cos, sin, Q_OFFSET, kc, vc, Q_OFFSET))
    cache = torch.randn(B, H, 2304, D, device=dev).bfloat16()
    rec("upsample_ocache(48x48 -> 64x64)", cache.numel() * 2 + B * H * LQ * D * 2,
        lambda: K.upsample_ocache(cache, 2304, 4096))
    # ScaleKV compaction at the last scale: window scores, pooling, gather of the kept rows
    win = torch.arange(LKV - 16, LKV, device=dev, dtype=torch.int32)
    rec("scalekv_scores(16 window queries)", k.numel() * 2 + B * H * LKV * 4,
        lambda: K.scalekv_scores(q, k, win, Q_OFFSET))
    sc = K.scalekv_scores(q, k, win, Q_OFFSET)
    rec("scalekv_pool(k=5)", 2 * sc.numel() * 4, lambda: K.scalekv_pool(sc, win, 5, "maxpool"))
    keep = torch.arange(0, 6385, device=dev, dtype=torch.int32).expand(B, H, -1).contiguous()
    rec("gather_rows(6385 of 10521 keys)", 2 * B * H * 6385 * D * 2 + keep.numel() * 4, lambda: K.gather_rows(k, keep))
    return out


def leg_reference_triton(q, k, v, scale, csp_lists_192, csp_counts_192, o_in):
    """The reference's own Triton kernels (its 'triton' provider, the only kernels of the reference that run on
    this GPU) from baseline/_ref, timed with the reference's procedure (20 warm-up calls, 50 timed,
    kernels/sparse_attn/triton/attn_csp.py:511-555).  Context only: nothing of the product imports them."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "kernels" / "sparse_attn" / "sparse_attn_ops.py").exists():
        return {"unavailable": "baseline/_ref absent (python baseline/make_ref.py <reference checkout>)"}
    try:
        sys.path.insert(0, str(ref))
        import importlib
        rops = importlib.import_module("kernels.sparse_attn.sparse_attn_ops")
        rcfg = importlib.import_module("kernels.sparse_attn.sparse_attn_config")
        rcfg.GLOBAL_CONFIG["attn"]["provider"] = "triton"
        out = {"provider": "triton", "procedure": "20 warm-up + 50 timed calls, CUDA events"}
        for name, fn in (
                ("dense_attn_us", lambda: rops.dense_attn(q, k, v, scale)),
                ("dense_colsum_attn_us", lambda: rops.dense_colsum_attn_q(q, k, v, scale)),
                ("csp_attn_us", lambda: rops.csp_attn(q, k, v, scale, csp_lists_192, csp_counts_192, o_in, 1))):
            try:
                out[name] = round(1e3 * timed(fn, 50, warm=20), 1)
            except Exception as e:  # a JIT or launch failure of one kernel: quote it and go on
                out[name] = f"failed: {type(e).__name__}: {str(e)[:200]}"
        return out
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
    finally:
        if str(ref) in sys.path:
            sys.path.remove(str(ref))


def leg_c4_sharded(K, P, dev, world, rank):
    """The 2048px-style last scale (B2 H32 D128 Lq16384 Lkv24576, 10 % density) with its 64 (batch, head) units
    dealt round-robin to the ranks: per-rank attention + column sums -> block scores -> ONE all-gather of the
    block scores (the only collective of the path) -> the shared mask built redundantly -> block-sparse
    attention of the rank's units.  Strong scaling: the total work is fixed."""
    import torch.distributed as dist
    from lvar_b200 import partition as PT
    Bc, Hc, Lq, Lkv = 2, 32, 16384, 24576
    n_units = Bc * Hc
    mine = PT.unit_indices(n_units, world, rank)
    U = len(mine)
    g = torch.Generator(device=dev).manual_seed(100)
    # every rank draws the same stream and keeps its own units (no scatter needed for a benchmark)
    def draw(L, low_rank=False):
        parts = []
        for u in range(n_units):
            t = torch.randn(1, 1, L, D, generator=g, device=dev)
            if low_rank:
                t = t + 2.0 * (torch.randn(1, 1, L, 8, generator=g, device=dev) @ torch.randn(1, 1, 8, D, generator=g, device=dev))
            if u % world == rank:
                parts.append(t.bfloat16())
        return torch.cat(parts, 0)
    q, k, v = draw(Lq), draw(Lkv, True), draw(Lkv)
    scale = 1.0 / math.sqrt(D)
    nq, nk = Lq // 128, Lkv // 128
    always = P.sink_local_blocks(nq, nk, 128, 0, Lkv - Lq, 2, Lq).to(dev)

    def scoring():
        _, cs = K.dense_colsum_attn_fwd(q, k, v, scale)
        return K.block_scores(cs, 128).view(U, nq, nk)

    scores = scoring()
    gather_ms = timed(lambda: PT.all_gather_units(scores, n_units), 20)
    mask, _ = PT.shared_block_mask(scores, n_units, always, 19)
    torch.cuda.synchronize()
    assert int(mask.sum(-1).min()) == 19 == int(mask.sum(-1).max())
    if world > 1:  # every rank must hold the same mask
        ref = mask.to(torch.uint8)
        dist.broadcast(ref, 0)
        assert torch.equal(ref, mask.to(torch.uint8)), "ranks disagree on the shared block mask"

    def step():
        s = scoring()
        m, _ = PT.shared_block_mask(s, n_units, always, 19)
        return K.block_sparse_attn_fwd(q, k, v, m, scale)

    if world > 1:
        dist.barrier()
    step_ms = max_over_ranks(timed(step, 3, warm=1), dev, world)
    score_ms = max_over_ranks(timed(scoring, 3, warm=1), dev, world)
    attn_ms = max_over_ranks(timed(lambda: K.block_sparse_attn_fwd(q, k, v, mask, scale), 5, warm=1), dev, world)
    gather_ms = max_over_ranks(gather_ms, dev, world)
    flops_active = 4.0 * D * 128 * 128 * 19 * nq * n_units
    del q, k, v
    return {"workload": "B2 H32 D128 Lq16384 Lkv24576, window +-2 blocks + top-k to 19/192 blocks, one mask for all heads",
            "units_total": n_units, "units_per_rank": U, "scaling": "strong",
            "step_ms": round(step_ms, 3), "scoring_ms": round(score_ms, 3), "block_sparse_attn_ms": round(attn_ms, 3),
            "all_gather_us": round(gather_ms * 1e3, 1), "all_gather_bytes_per_rank": U * nq * nk * 4,
            "all_gather_share_of_step": round(gather_ms / step_ms, 5),
            "block_sparse_tflops_aggregate": round(flops_active / (attn_ms * 1e-3) / 1e12, 1)}


def leg_c5(dev, world, rank, variants, iters, eager_fallback=True):
    """The full generation loop (Infinity-2B architecture, random weights, 13 scales x 32 blocks, 16 prompts x 2
    for guidance, sharded by prompt over the ranks): images per second, whole job."""
    from lvar_b200 import infinity_loop as IL
    import torch.distributed as dist
    per_rank = C5_PROMPTS // world
    out = {"prompts": C5_PROMPTS, "prompts_per_rank": per_rank, "scaling": "strong",
           "model": "depth 32, width 2048, 16 heads x 128, FFN 8192, 64 text tokens, 13 scales to 64x64 (10521 tokens)"}
    text = torch.randn(per_rank, 64, 2048, generator=torch.Generator(device=dev).manual_seed(7 + rank), device=dev).bfloat16()
    for name in variants:
        loop = IL.InfinityLoop(IL.LoopConfig(attn_mode=name), batch=per_rank, device=dev, seed=0)
        mode = "cuda graph replay"
        try:
            loop.capture(text)
            run = loop.replay
        except Exception as e:
            if not eager_fallback:
                raise
            mode = f"eager ({type(e).__name__}: {str(e)[:120]})"
            run = lambda: loop.generate(text)  # noqa: E731
        if world > 1:
            dist.barrier()
        ms = max_over_ranks(timed(run, iters, warm=1), dev, world)
        out[name] = {"seconds_per_batch": round(ms / 1e3, 4), "images_per_s": round(C5_PROMPTS / (ms / 1e3), 3),
                     "mode": mode, "routes": dict(loop.routes)}
        fl = loop.flops_per_batch()
        out["pflop_linear_per_batch"] = round(world * fl["linear"] / 1e15, 3)
        out["pflop_dense_self_attention_per_batch"] = round(world * fl["self_attention_dense"] / 1e15, 3)
        del loop, run
        gc.collect()
        torch.cuda.empty_cache()
    if "sparse" in out and "dense" in out:
        out["speedup_sparse_over_dense_attention"] = round(out["dense"]["seconds_per_batch"] / out["sparse"]["seconds_per_batch"], 3)
    if "sparse" in out and "none" in out:
        out["self_attention_share_of_step"] = round(1.0 - out["none"]["seconds_per_batch"] / out["sparse"]["seconds_per_batch"], 3)
    return out


def c5_cpu_extrapolation(flops_lin, flops_attn, attn_tflops_cpu, cores):
    """images/s of the same loop on the host cores, extrapolated: fp32 GEMM rate of one FFN layer of one
    sequence at the last scale (4096 x 2048 @ 2048 x 8192) for the linear layers, the measured dense masked
    attention rate for self-attention."""
    torch.set_num_threads(cores)
    a = torch.randn(4096, 2048)
    w = torch.randn(2048, 8192)
    a @ w
    t0 = time.perf_counter()
    for _ in range(3):
        a @ w
    gemm_tflops = 3 * 2.0 * 4096 * 2048 * 8192 / (time.perf_counter() - t0) / 1e12
    sec = flops_lin / (gemm_tflops * 1e12) + flops_attn / (attn_tflops_cpu * 1e12)
    return {"images_per_s": C5_PROMPTS / sec, "seconds_per_batch": sec, "cores": cores, "kind": "port",
            "sample": f"extrapolated from fp32 GEMM 4096x2048x8192 ({gemm_tflops:.2f} TFLOP/s) for the linear layers and "
                      f"dense masked fp32 attention ({attn_tflops_cpu:.3f} TFLOP/s) for self-attention"}


# ------------------------------------------------------------------------------------------------------
# the repo's arm
# ------------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    from lvar_b200 import _lib
    from lvar_b200 import kernels as K
    from lvar_b200 import policy as P
    from lvar_b200 import sparse_attn_ops as ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()

    if args.workload == "c5":
        return run_c5_only(args, dev, world, rank, peaks)

    q_h, k_h, v_h = make_inputs()
    q_pin, k_pin, v_pin = (t.pin_memory() for t in (q_h, k_h, v_h))
    q, k, v = (t.to(dev) for t in (q_pin, k_pin, v_pin))
    scale = 1.0 / math.sqrt(D)
    nq, nk = (LQ + BLOCK - 1) // BLOCK, (LKV + BLOCK - 1) // BLOCK

    # ---- scoring + mask construction, and the parity gate of this very workload
    mask, scores, always_h, cs, o_dense, M, L = recipe_mask(K, P, q, k, v, scale)
    always = always_h.to(dev)
    torch.cuda.synchronize()
    assert int(mask.sum(-1).min()) == K_TOTAL and int(mask.sum(-1).max()) == K_TOTAL
    sample = [(rank % B, (5 + 3 * rank) % H)]
    parity_err = check_recipe_parity(K, q, k, v, scale, mask, scores, always_h, sample)
    flops = sum(active_flops(mask[b, h]) for b in range(B) for h in range(H))
    dense_flops = 4.0 * B * H * LQ * LKV * D
    extra = {}
    if not args.no_extra:
        # Absolute figures from short bursts of one kernel (as the headline is taken, and what the burst peak is the
        # denominator for) ...
        dense_ms = timed(lambda: K.dense_attn_fwd(q, k, v, scale), 10)
        fused_ms = timed(lambda: K.dense_colsum_attn_fwd(q, k, v, scale), 10)  # attention + column sums, one launch
        given_ms = timed(lambda: K.dense_colsum_attn_given_fwd(q, k, v, M, L, scale), 10)
        # ... and the overheads as ratios of medians with the three kernels taking turns, i.e. at the same clocks
        # (0.15 s of back-to-back heavy kernels: the part runs at its power-capped clock here)
        (dense_i, d_lo, d_hi), (fused_i, f_lo, f_hi), (given_i, g_lo, g_hi) = timed_interleaved([
            lambda: K.dense_attn_fwd(q, k, v, scale),
            lambda: K.dense_colsum_attn_fwd(q, k, v, scale),
            lambda: K.dense_colsum_attn_given_fwd(q, k, v, M, L, scale)], iters=6, rounds=9, spread=True)
        colsum_ms = timed(lambda: K.colsum_fwd(q, k, M, L, BLOCK, scale), 10)
        cs_only_ms = timed(lambda: K.colsum_tiles_fwd(q, k, scale), 10)
        cs_given_ms = timed(lambda: K.colsum_tiles_fwd(q, k, scale, stats=(M, L)), 10)
        mask_ms = timed(lambda: K.block_mask_from_colsums(cs, always, K_TOTAL, BLOCK), 10)
        extra.update({
            "dense_attn_ms": dense_ms, "dense_attn_tflops": dense_flops / dense_ms / 1e9,
            "dense_attn_frac_of_bf16_peak": dense_flops / dense_ms / 1e9 / peaks["bf16"],
            "colsum_sweep_us": colsum_ms * 1e3, "dense_colsum_fused_ms": fused_ms,
            "colsum_only_us": cs_only_ms * 1e3, "colsum_from_given_stats_us": cs_given_ms * 1e3,
            "colsum_over_dense_attn": (fused_i - dense_i) / dense_i,
            "colsum_over_dense_attn_separate_kernels": colsum_ms / dense_ms,
            "mask_build_us": mask_ms * 1e3, "density": K_TOTAL / nk})
        # the form the reference's CUDA operator has: row statistics supplied, ONE sweep, column sums of the same
        # probabilities that feed P V
        extra["dense_colsum_stats_given_ms"] = given_ms
        extra["colsum_over_dense_attn_stats_given"] = (given_i - dense_i) / dense_i
        extra["colsum_over_dense_attn_stats_given_bursts"] = (given_ms - dense_ms) / dense_ms
        # median, fastest and slowest of the nine interleaved rounds of each kernel
        extra["colsum_interleaved_ms"] = {"dense_attn": [round(dense_i, 4), round(d_lo, 4), round(d_hi, 4)],
                                          "dense_colsum_fused": [round(fused_i, 4), round(f_lo, 4), round(f_hi, 4)],
                                          "dense_colsum_stats_given": [round(given_i, 4), round(g_lo, 4), round(g_hi, 4)]}

        # ---- scheduling A/B on the headline kernel and on dense attention (same launch, different hand-out of
        # the last wave): pairs only / single tiles on one half of the CTA / single tiles split over both halves
        tags = (("pairs_only", _lib.SCHED_PAIRS_ONLY), ("single_tiles_one_half", _lib.SCHED_SINGLE_ONE_SLOT),
                ("single_tiles_split", 0))
        ms_b = timed_interleaved([(lambda f=f: K.block_sparse_attn_fwd(q, k, v, mask, scale, sched_flags=f))
                                  for _, f in tags], iters=10)
        ms_d = timed_interleaved([(lambda f=f: K.dense_attn_fwd(q, k, v, scale, sched_flags=f)) for _, f in tags])
        extra["schedule_ab"] = {tag: {"block_sparse_tflops": round(flops / ms_b[i] / 1e9, 1),
                                      "dense_tflops": round(dense_flops / ms_d[i] / 1e9, 1)}
                                for i, (tag, _) in enumerate(tags)}

        # ---- the column-sparse kernel on a list shaped like a last-scale sparse step: per 256-row query group
        # 1664 scattered keys (the decision scale's top-k) followed by a band of 512 consecutive keys
        csp_top, csp_band = 1664, 512

        def csp_lists(bm):
            n_groups = (LQ + bm - 1) // bm
            gen = torch.Generator(device=dev).manual_seed(1)
            top = torch.rand(B, H, n_groups, LKV, device=dev, generator=gen).argsort(-1)[..., :csp_top].to(torch.int32)
            start = torch.randint(0, LKV - csp_band, (B, H, n_groups, 1), device=dev, generator=gen)
            band = (start + torch.arange(csp_band, device=dev)).to(torch.int32)
            lists = torch.zeros(B, H, n_groups, LKV, dtype=torch.int32, device=dev)
            lists[..., :csp_top + csp_band] = torch.cat([top, band], dim=-1)
            return lists, torch.full((B, H, n_groups), csp_top + csp_band, dtype=torch.int32, device=dev)
        lists256, counts256 = csp_lists(256)
        csp_ms = timed(lambda: K.csp_attn_fwd(q, k, v, lists256, counts256, o_dense, 1, 256, scale), 10)
        csp_flops = 4.0 * B * H * LQ * (csp_top + csp_band) * D
        extra.update({"csp_attn_us": csp_ms * 1e3, "csp_attn_tflops": csp_flops / csp_ms / 1e9,
                      "csp_attn_workload": f"{csp_top} scattered + {csp_band} consecutive keys per 256-row group"})
        del lists256, counts256

        if world == 1 and not args.no_reference_kernels:
            lists192, counts192 = csp_lists(192)
            extra["reference_triton_us"] = leg_reference_triton(q, k, v, scale, lists192, counts192, o_dense)
            extra["reference_triton_us"]["ours_us"] = {
                "dense_attn_us": round(dense_ms * 1e3, 1), "dense_colsum_attn_us": round(fused_ms * 1e3, 1),
                "csp_attn_us": round(csp_ms * 1e3, 1)}
            del lists192, counts192

        extra["cs4a_layer_us"] = leg_cs4a_layer(K, P, k, v, scale, dev)
        extra["kv_scoring_colsum_topk_us"] = leg_kv_scoring(K, P, k, scale, dev)
        extra["hbm_kernels"] = leg_hbm_kernels(K, P, q, k, v, cs, scale, dev, peaks["hbm"])
        extra["hbm_kernels"]["peak_gbs"] = peaks["hbm"]

    # ---- timed region: K steps of block-sparse attention, inputs resident in HBM
    step = lambda: K.block_sparse_attn_fwd(q, k, v, mask, scale)  # noqa: E731
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local_rank) as clocks:
        a, b = ev(), ev()
        # The synchronize above leaves the GPU idle, and the first launches after an idle gap run slower (about
        # one step's time is lost, whatever K is).  PRE_ROLL more untimed steps are therefore queued directly
        # ahead of the start event: the K timed steps, taken with CUDA events on the launching stream, start on
        # a busy GPU, as the kernel does inside a generation loop.  Both synchronizes stay where they are.
        for _ in range(PRE_ROLL):
            step()
        a.record()
        for _ in range(args.steps):
            step()
        b.record()
        torch.cuda.synchronize()
    elapsed_ms = max_over_ranks(a.elapsed_time(b), dev, world)
    if world > 1:
        dist.barrier()
    ms_per_step = elapsed_ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    # ---- the same kernel over a region of at least a second: the part settles at its power-limited clock
    sustained = None
    if args.sustained_steps > 0:
        with ClockSampler(local_rank) as clocks_s:
            a, b = ev(), ev()
            for _ in range(PRE_ROLL):
                step()
            a.record()
            for _ in range(args.sustained_steps):
                step()
            b.record()
            torch.cuda.synchronize()
        s_ms = max_over_ranks(a.elapsed_time(b), dev, world) / args.sustained_steps
        sustained = {"steps": args.sustained_steps, "seconds": round(s_ms * args.sustained_steps / 1e3, 3),
                     "ms_per_step": s_ms, "tflops": flops / (s_ms * 1e-3) / 1e12, "clocks": clocks_s.summary()}

    # ---- end to end through the public operator, from pinned host memory
    mask_pin = mask.cpu().pin_memory()
    o_pin = torch.empty((B, H, LQ, D), dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (q_pin, k_pin, v_pin, mask_pin))
    d2h = o_pin.numel() * o_pin.element_size()

    # Three streams: step i's host->device copies, step i-1's kernel and step i-2's device->host copy run at
    # the same time (PCIe is full duplex and much slower than the kernel), every step still moves all of its
    # inputs from pinned host memory and its output back inside the timed region.
    s_in, s_run, s_out = (torch.cuda.Stream(dev) for _ in range(3))
    slots = [dict(q=torch.empty_like(q), k=torch.empty_like(k), v=torch.empty_like(v), m=torch.empty_like(mask),
                  o=None, loaded=torch.cuda.Event(), ran=torch.cuda.Event(), stored=torch.cuda.Event())
             for _ in range(2)]
    step_no = [0]

    def e2e_step(kv_resident=False):
        sl = slots[step_no[0] % 2]
        step_no[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(sl["ran"])      # the kernel that last read these device buffers has finished
            sl["q"].copy_(q_pin, non_blocking=True)
            if not kv_resident:
                sl["k"].copy_(k_pin, non_blocking=True)
                sl["v"].copy_(v_pin, non_blocking=True)
            sl["m"].copy_(mask_pin, non_blocking=True)
            sl["loaded"].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(sl["loaded"])
            s_run.wait_event(sl["stored"])  # the previous output of this slot has left the device
            sl["o"] = ops.block_sparse_attn(sl["q"], k if kv_resident else sl["k"], v if kv_resident else sl["v"],
                                            sl["m"], scale)
            sl["ran"].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(sl["ran"])
            o_pin.copy_(sl["o"], non_blocking=True)
            sl["stored"].record(s_out)

    def e2e_timed(iters, warm, **kw):
        for _ in range(warm):
            e2e_step(**kw)
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(iters):
            e2e_step(**kw)
        for st in (s_in, s_run, s_out):
            torch.cuda.current_stream().wait_stream(st)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters

    e2e_iters = max(3, min(args.steps, 20))
    if world > 1:
        dist.barrier()
    e2e_ms = max_over_ranks(e2e_timed(e2e_iters, 2), dev, world)
    e2e_val = world * flops / (e2e_ms * 1e-3) / 1e12
    if not args.no_extra:
        # the same call with K/V resident (they are the KV cache inside the generation loop): per step only q and
        # the mask go up and o comes back, so the curve over N shows the kernels rather than one host's PCIe root
        if world > 1:
            dist.barrier()
        eq_ms = max_over_ranks(e2e_timed(e2e_iters, 2, kv_resident=True), dev, world)
        extra["e2e_q_only"] = {"value": world * flops / (eq_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": eq_ms,
                               "h2d_bytes_per_step": q_pin.numel() * 2 + mask_pin.numel(), "d2h_bytes_per_step": d2h}
    del slots, mask_pin, o_pin

    # ---- the sharded configuration with the path's one collective, and the full generation loop
    if not args.no_extra:
        del o_dense, cs
        torch.cuda.empty_cache()
        try:
            extra["c4_sharded"] = leg_c4_sharded(K, P, dev, world, rank)
        except Exception as e:
            extra["c4_sharded"] = {"failed": f"{type(e).__name__}: {str(e)[:300]}"}
        torch.cuda.empty_cache()
        if not args.no_c5:
            del q, k, v
            torch.cuda.empty_cache()
            try:
                extra["c5_generation_loop"] = leg_c5(dev, world, rank, ("sparse", "dense", "none"), iters=2)
            except Exception as e:
                extra["c5_generation_loop"] = {"failed": f"{type(e).__name__}: {str(e)[:300]}"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    achieved = flops / (ms_per_step * 1e-3) / 1e12 if world == 1 else value / world
    roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16"], "unit": "TFLOP/s",
            "frac": achieved / peaks["bf16"], "traffic": TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peaks["source"],
            "kernel": "attn_fwd_kernel<128, block-sparse>"}
    if sustained is not None:
        roof.update({"achieved_sustained": sustained["tflops"], "peak_sustained": peaks["bf16_sustained"],
                     "frac_sustained": sustained["tflops"] / peaks["bf16_sustained"], "sustained_region": sustained})
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "units_per_gpu": B * H, "l2": "inputs (206 MB) larger than L2 (126 MB)",
                   "timing": f"CUDA events on the launching stream around exactly K steps; {PRE_ROLL} untimed steps "
                             "queued between the synchronize and the start event (no idle gap inside the region)",
                   "active_gflop_per_step": flops / 1e9, "dense_gflop": dense_flops / 1e9,
                   "parallelism": f"batch x head shards, {world} GPU(s), no data-path collective",
                   "parity_checked": True,
                   "parity": {"mask": "bit-exact vs oracle on identical scores", "sampled_heads": sample,
                              "o_max_abs": parity_err[0], "o_mean_abs": parity_err[1]}},
        "roofline": roof,
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms},
        "gpu_launches": args.steps,
        "clocks": clocks.summary(),
        "extra": extra,
    }
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        heads = 1
        t1 = cpu_masked_attention_sample(q_h, k_h, v_h, mask.cpu(), heads, cores)
        heads = int(max(1, min(B * H, 10.0 / max(t1, 1e-3))))
        t2 = cpu_masked_attention_sample(q_h, k_h, v_h, mask.cpu(), heads, cores)
        per_head = flops / (B * H)
        line["cpu_baseline"] = {"value": per_head * heads / t2 / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"dense masked fp32 attention (oracle) on {heads} of {B * H} "
                                          f"(batch, head) pairs, {t2:.1f} s"}
        c5 = extra.get("c5_generation_loop")
        if isinstance(c5, dict) and "pflop_linear_per_batch" in c5:
            # dense masked attention on the host costs the dense FLOPs whatever the mask keeps
            attn_cpu = (dense_flops / (B * H)) * heads / t2 / 1e12
            c5["cpu_baseline"] = c5_cpu_extrapolation(c5["pflop_linear_per_batch"] * 1e15,
                                                      c5["pflop_dense_self_attention_per_batch"] * 1e15, attn_cpu, cores)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def leg_cs4a_layer(K, P, k, v, scale, dev):
    """One CS4A layer of the last three scales through the policy class (decision step at 40x40: dense attention +
    column sums + top-k + O-cache; sparse steps at 48x48 and 64x64: list remap + band, O-cache resize inside the
    column-sparse launch), B2 H16 D128, keys = all tokens up to the scale; eager and as one CUDA-graph replay."""
    cum = P.cumulative_tokens(P.INFINITY_SCALES)
    layer = P.SparseDiffAttn(layer_num=0)
    us = {}
    gq = torch.Generator(device=dev).manual_seed(2)
    for si, full in ((10, True), (11, False), (12, False)):
        lq, lk = P.INFINITY_SCALES[si] ** 2, cum[si + 1]
        qs = torch.randn(B, H, lq, D, device=dev, generator=gq).bfloat16()
        ks, vs = k[:, :, :lk], v[:, :, :lk]
        # a sparse step rewrites the layer's stored lists, counts and O-cache: every timed call starts from
        # the state the preceding scale left, as it does inside one image generation
        st = layer.storage
        before = (st.indices, st.counts, st.count_value, st.out_cache)

        def one_call():
            st.indices, st.counts, st.count_value, st.out_cache = before
            return layer(qs, ks, vs, scale, do_full_step=full, scale_ind=si)
        us[f"scale{si}_{'decision' if full else 'sparse'}_q{lq}_k{lk}"] = 1e3 * timed(one_call, 10, warm=3)
    del layer, qs
    layer = P.SparseDiffAttn(layer_num=0)
    steps_in = [(si, full, torch.randn(B, H, P.INFINITY_SCALES[si] ** 2, D, device=dev, generator=gq).bfloat16())
                for si, full in ((10, True), (11, False), (12, False))]

    def three_steps():
        return [layer(qs_, k[:, :, :cum[si + 1]], v[:, :, :cum[si + 1]], scale, do_full_step=full, scale_ind=si)
                for si, full, qs_ in steps_in]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            three_steps()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        graph_out = three_steps()
    us["three_steps_eager_sum"] = sum(us.values())
    us["three_steps_one_graph_replay"] = 1e3 * timed(graph.replay, 10, warm=3)
    del graph, graph_out
    return us


def leg_kv_scoring(K, P, k, scale, dev):
    """Per-scale KV scoring of the 13-scale schedule: the column sums of each scale's queries over all keys so far,
    one score row per head (no attention output), then the ascending top-k that keeps 10 % of them."""
    cum = P.cumulative_tokens(P.INFINITY_SCALES)
    gq = torch.Generator(device=dev).manual_seed(3)
    us = {}
    q_sc = [torch.randn(B, H, s_ * s_, D, device=dev, generator=gq).bfloat16() for s_ in P.INFINITY_SCALES]

    def score(si):
        lk = cum[si + 1]
        keep = round(0.1 * lk)
        cs_row = K.colsum_tiles_fwd(q_sc[si], k[:, :, :lk], scale).sum(dim=2, keepdim=True)
        return K.topk_indices(cs_row, keep, ascending_index=True) if keep else cs_row
    for si, s_ in enumerate(P.INFINITY_SCALES):
        us[f"scale{si}_q{s_ * s_}_k{cum[si + 1]}_keep{round(0.1 * cum[si + 1])}"] = round(
            1e3 * timed(lambda: score(si), 10, warm=3), 1)
    us["total"] = round(sum(us.values()), 1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            [score(si) for si in range(len(P.INFINITY_SCALES))]
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        outs = [score(si) for si in range(len(P.INFINITY_SCALES))]
    us["total_one_graph_replay"] = round(1e3 * timed(graph.replay, 10, warm=3), 1)
    del graph, outs
    return us


def run_c5_only(args, dev, world, rank, peaks):
    """``--workload c5``: the generation loop alone, with the dense-attention and no-attention variants for the
    speed-up and the self-attention share, and the host extrapolation; prints one line in images/s."""
    import torch.distributed as dist
    steps = max(1, min(args.steps, 5))
    c5 = leg_c5(dev, world, rank, ("sparse", "dense", "none"), iters=steps)
    if rank == 0:
        line = {"metric": "images_per_s", "value": c5["sparse"]["images_per_s"], "unit": "images/s", "n_gpus": world,
                "steps": steps, "warmup": 1, "ms_per_step": c5["sparse"]["seconds_per_batch"] * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "infinity2b-architecture generation loop, random weights: " + c5["model"],
                           "prompts": C5_PROMPTS, "guidance_copies": 2, "parallelism": f"prompts sharded over {world} GPU(s)"},
                "extra": {"c5_generation_loop": c5}, "gpu_launches": steps}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["c2", "c5"], default="c2")
    ap.add_argument("--sustained-steps", type=int, default=7000,
                    help="steps of the second, >= 1 s timed region behind roofline.frac_sustained (0: skip)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the bounded CPU sample (profiling runs)")
    ap.add_argument("--no-extra", action="store_true", help="headline and e2e only (profiling runs)")
    ap.add_argument("--no-c5", action="store_true", help="skip the generation-loop leg")
    ap.add_argument("--no-reference-kernels", action="store_true", help="skip timing the reference's Triton kernels")
    args = ap.parse_args()
    # stdout carries the JSON line and nothing else: whatever libraries print at the C level while the bench
    # runs (NCCL's version banner, for one) goes to stderr, and the line is written to the real stdout
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        rc = run_reference(args) if args.impl == "reference" else run_ours(args)
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    os.close(real_stdout)
    sys.stdout.write(buf.getvalue())
    sys.stdout.flush()
    return rc


if __name__ == "__main__":
    sys.exit(main())
