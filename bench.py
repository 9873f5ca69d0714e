#!/usr/bin/env python3
"""Benchmark of the two attention hot paths on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload fa_c2|fa_c4]

Prints ONE JSON line.  The headline workload is BASELINE configuration 2 (FlashAttention forward,
BF16, causal, B=4 S=4096 H=32 D=128, N(0,1)*0.5, synthetic): metric = forward TFLOPS, a step = one
forward over one batch.  The same line carries the PagedAttention decode of configuration 3 (FP16,
batch 64, H=32 D=128, page 16, context ~ U[512, 8192]) under "paged_decode": HBM GB/s, tokens/s and
its own roofline / end-to-end / CPU-baseline figures, and under "paged_prefill" the headline
workload once more with K/V held in a paged pool (ahpc_paged_prefill reading the pages in place).

  value        kernel-only throughput, inputs resident in HBM, CUDA events, max over ranks
  e2e          the same metric through the C ABI with HOST (pinned) buffers: every step copies its
               inputs host->device and its result device->host inside the timed region
  roofline     algorithmic FLOPs (or bytes) per launch / average launch duration, against the
               measured peaks of MEASURED_PEAKS.json (fallback constants if the file is absent)
  cpu_baseline the CPU port of the reference algorithm (oracle/oracle.c, *_f32acc) on the host cores
               of this box, on a bounded sample of the same workload

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs its own batch of
the same shape - the (batch, head) partition of the work needs no collective - and the value is the
whole-job aggregate: scaling "weak".

--impl reference times the CPU port alone (the reference's own sources do not compile: its hot-path
files are truncated mid-statement), on rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (None where no capture exists for that workload).
# FA: 518.8 MB per launch of fa_fwd_tc2_kernel on configuration 2 in full (profiles/bench_launch_list_c2_c3.md), i.e.
# 4.05 MB per (batch, head) pair at S=4096 D=128; scaled by the pairs a launch processes.
# Decode: read+write = 1.0032 x the algorithmic bytes (same file).
# Prefill over pages: 519.0 MB per launch of fa_fwd_tc_kernel<MODE_PREFILL> on configuration 2 in full (same file).
NCU_TRAFFIC = {"fa_fwd_tc_kernel_bytes_per_bh_pair_s4096": 518.8e6 / 128, "paged_decode_kernel_ratio": 1.0032,
               "paged_prefill_bytes_per_bh_pair_s4096": 519.0e6 / 128}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a timed region runs."""

    def __init__(self, device_index: int, period_s: float = 0.01):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake_slowdown": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------ timing

def timed_steps(torch, dist, step, steps: int, warmup: int) -> float:
    """W warm-up steps, then exactly K steps between (barrier + synchronize) pairs; CUDA events on
    the launching stream; returns the max over ranks of the elapsed milliseconds."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


# ------------------------------------------------------------------------------------------ CPU baseline

def cpu_fa_baseline(cfg, budget_s: float, steps: int = 1, warmup: int = 0):
    """Times the float-accumulating CPU port on a bounded sample of `cfg`: the last `rows` query
    rows of `units` (batch, head) pairs, all host threads.  Returns (TFLOPS, description, seconds/step)."""
    from oracle import cpu_oracle as o
    threads = os.cpu_count() or 1
    S, D = cfg.seq, cfg.head_dim
    rng = np.random.default_rng(cfg.seed)
    units = max(1, min(threads, cfg.batch * cfg.heads))
    q, k, v = (rng.standard_normal((1, units, S, D)).astype(np.float32) * cfg.input_scale for _ in range(3))
    out = np.zeros_like(q)
    scale = 1.0 / math.sqrt(D)

    def flops(r0, r1):
        keys = sum(i + 1 for i in range(r0, r1)) if cfg.causal else (r1 - r0) * S
        return 4.0 * D * keys * units

    # calibrate on 32 rows per unit, then size the sample for the budget
    t0 = time.perf_counter()
    o.attention_fwd_f32acc(q, k, v, scale, cfg.causal, threads=threads, native=True, rows=(S - 32, S), out=out)
    cal = time.perf_counter() - t0
    t0 = time.perf_counter()
    o.attention_fwd_f32acc(q, k, v, scale, cfg.causal, threads=threads, native=True, rows=(S - 32, S), out=out)
    cal = min(cal, time.perf_counter() - t0)
    rate = flops(S - 32, S) / max(cal, 1e-6)
    per_step = budget_s / max(1, steps + warmup)
    rows = S
    while rows > 32 and flops(S - rows, S) / rate > per_step:
        rows //= 2
    r0 = S - rows
    for _ in range(warmup):
        o.attention_fwd_f32acc(q, k, v, scale, cfg.causal, threads=threads, native=True, rows=(r0, S), out=out)
    t0 = time.perf_counter()
    for _ in range(steps):
        o.attention_fwd_f32acc(q, k, v, scale, cfg.causal, threads=threads, native=True, rows=(r0, S), out=out)
    dt = (time.perf_counter() - t0) / steps
    sample = (f"CPU port (oracle_attention_fwd_f32acc, -O3 -march=native, OpenMP): last {rows} query rows of "
              f"{units} (batch, head) pairs of {cfg.name} per step ({flops(r0, S) / 1e9:.1f} GFLOP), scaled by FLOPs")
    return flops(r0, S) / dt / 1e12, sample, dt, threads


def cpu_decode_baseline(cfg, budget_s: float):
    """Times the float-accumulating CPU decode port on the first sequences of `cfg` (their pages dealt
    from the same seeded permutation), all host threads.  Returns (GB/s, tokens/s, description, threads)."""
    from attention_b200 import synth
    from oracle import cpu_oracle as o
    threads = os.cpu_count() or 1
    ctx = synth.context_lengths(cfg)
    n = min(len(ctx), 4)
    ctx = ctx[:n]
    ps, H, D = cfg.page_size, cfg.heads, cfg.head_dim
    pages = int(sum((int(c) + ps - 1) // ps for c in ctx))
    order = synth.page_permutation(pages, cfg.seed)
    table = np.full((n, int(max((ctx + ps - 1) // ps))), -1, np.int32)
    at = 0
    for i, c in enumerate(ctx):
        npg = (int(c) + ps - 1) // ps
        table[i, :npg] = order[at:at + npg]
        at += npg
    rng = np.random.default_rng(cfg.seed)
    kc = rng.standard_normal((pages, ps, H, D)).astype(np.float16)
    vc = rng.standard_normal((pages, ps, H, D)).astype(np.float16)
    q = rng.standard_normal((n, H, D)).astype(np.float32)
    scale = 1.0 / math.sqrt(D)
    best = None
    t_start = time.perf_counter()
    reps = 0
    while reps < 2 or (time.perf_counter() - t_start < budget_s and reps < 20):
        t0 = time.perf_counter()
        o.paged_decode_f32acc(q, kc.view(np.uint16), vc.view(np.uint16), "f16", table, ctx, scale, threads=threads, native=True)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        reps += 1
    kv_bytes = int(ctx.astype(np.int64).sum()) * synth.kv_bytes_per_token(cfg)
    sample = (f"CPU port (oracle_paged_decode_f32acc, -O3 -march=native, OpenMP): first {n} sequences of {cfg.name} "
              f"({kv_bytes / 1e6:.0f} MB of KV), best of {reps}")
    return kv_bytes / best / 1e9, n / best, sample, threads


# ------------------------------------------------------------------------------------------ workloads

def make_fa_inputs(torch, cfg, rank: int):
    g = torch.Generator(device="cuda").manual_seed(cfg.seed + 7919 * rank)
    shape = (cfg.batch, cfg.heads, cfg.seq, cfg.head_dim)       # [B,H,S,D]-contiguous memory
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[cfg.dtype]
    return [(torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * cfg.input_scale).to(dt) for _ in range(3)]


def bench_fa(torch, dist, cfg, args, rank: int, world: int, peaks, peak_kind):
    from attention_b200 import abi, ops
    q, k, v = make_fa_inputs(torch, cfg, rank)
    out = torch.empty_like(q)
    assert ops.select_kernel(q, k) == abi.KERNEL_TC, "the tensor-core kernel must be the one that runs"

    def step():
        ops.flash_attention_forward(q, k, v, causal=cfg.causal, out=out)

    with ClockSampler(torch.cuda.current_device()) as clk:
        ms = timed_steps(torch, dist, step, args.steps, args.warmup)
    ms_per_step = ms / args.steps
    flops = cfg.flops
    tflops_total = flops * world / (ms_per_step * 1e-3) / 1e12
    tflops_rank = flops / (ms_per_step * 1e-3) / 1e12

    if args.profile_small:
        return {"value": tflops_total, "ms_per_step": ms_per_step, "e2e": None, "clocks": clk.summary(), "gpu_launches": 2 * args.steps,
                "roofline": {"bound": "tensor", "achieved": tflops_rank, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                             "frac": tflops_rank / peaks["bf16_tflops"], "traffic": None, "flops_per_launch": flops}}
    # end to end: pinned host tensors through the C ABI; H2D + kernel + D2H inside every step
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    hout = torch.empty_like(hq).pin_memory()

    def step_e2e():
        ops.flash_attention_forward(hq, hk, hv, causal=cfg.causal, out=hout, device=torch.cuda.current_device())

    e2e_steps = max(2, min(args.steps, 20))
    ms_e2e = timed_steps(torch, dist, step_e2e, e2e_steps, min(args.warmup, 3)) / e2e_steps
    nbytes = q.numel() * q.element_size()
    peak = peaks["bf16_tflops"] if ms < 1000.0 else peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    res = {
        "value": tflops_total, "ms_per_step": ms_per_step,
        "e2e": {"value": flops * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOPS", "h2d_bytes_per_step": 3 * nbytes,
                "d2h_bytes_per_step": nbytes, "ms_per_step": ms_e2e},
        "roofline": {"bound": "tensor", "achieved": tflops_rank, "peak": peak, "unit": "TFLOP/s", "frac": tflops_rank / peak,
                     "traffic": (NCU_TRAFFIC["fa_fwd_tc_kernel_bytes_per_bh_pair_s4096"] * cfg.batch * cfg.heads if cfg.seq == 4096 else None),
                     "peak_source": peak_kind + (" burst" if ms < 1000.0 else " sustained"),
                     "frac_of_nominal_2250": tflops_rank / 2250.0, "kernel": "fa_fwd_tc2_kernel",
                     "note": "a step = fa_fwd_tc2_kernel + the second-pass launch of fa_fwd_tc_kernel, whose CTAs all return at "
                             "once when no tile was flagged: the figure is a lower bound for the first kernel alone",
                     "flops_per_launch": flops},
        "clocks": clk.summary(), "gpu_launches": 2 * args.steps,
    }
    del hq, hk, hv, hout
    return res


def bench_paged_prefill(torch, dist, cfg, args, rank: int, world: int, peaks, peak_kind):
    """The FlashAttention workload once more with K/V held in a paged pool (pages dealt from a seeded permutation):
    every sequence's tokens attend causally to the pages, read in place by ahpc_paged_prefill."""
    from attention_b200 import ops, synth
    q, k, v = make_fa_inputs(torch, cfg, rank)
    dense = ops.flash_attention_forward(q, k, v, causal=cfg.causal)
    ps = 16
    pages = cfg.batch * ((cfg.seq + ps - 1) // ps) + 8
    pool = ops.KVPool(num_pages=pages, heads=cfg.heads, head_dim=cfg.head_dim, dtype=q.dtype, page_size=ps, max_seqs=cfg.batch,
                      max_pages_per_seq=(cfg.seq + ps - 1) // ps, device=torch.cuda.current_device(),
                      free_order=synth.page_permutation(pages, cfg.seed + rank))
    seqs = [pool.seq_create() for _ in range(cfg.batch)]
    for b, s in enumerate(seqs):
        pool.append([s], [cfg.seq], k[b].permute(1, 0, 2).contiguous(), v[b].permute(1, 0, 2).contiguous())
    qt = q.permute(0, 2, 1, 3).reshape(cfg.batch * cfg.seq, cfg.heads, cfg.head_dim).contiguous()      # [tokens, H, D]
    out = torch.empty_like(qt)
    del k, v
    counts = [cfg.seq] * cfg.batch

    def step():
        pool.prefill(seqs, counts, qt, out, causal=cfg.causal)

    ms_per_step = timed_steps(torch, dist, step, args.steps, args.warmup) / args.steps
    diff = (out.reshape(cfg.batch, cfg.seq, cfg.heads, cfg.head_dim).permute(0, 2, 1, 3).float() - dense.float()).abs().max().item()
    tflops_rank = cfg.flops / (ms_per_step * 1e-3) / 1e12
    peak = peaks["bf16_tflops"]
    res = {"metric": "paged_prefill_tflops", "unit": "TFLOPS", "value": tflops_rank * world, "ms_per_step": ms_per_step, "dtype": cfg.dtype,
           "config": {"workload": f"{workload_name(cfg)}; K/V in a pool of {pages} pages of {ps} tokens, seeded page permutation"},
           "max_abs_diff_vs_dense_kernel": diff,
           "roofline": {"bound": "tensor", "achieved": tflops_rank, "peak": peak, "unit": "TFLOP/s", "frac": tflops_rank / peak,
                        "traffic": NCU_TRAFFIC["paged_prefill_bytes_per_bh_pair_s4096"] * cfg.batch * cfg.heads if cfg.seq == 4096 else None,
                        "peak_source": peak_kind + " burst", "kernel": "fa_fwd_tc_kernel<MODE_PREFILL>", "flops_per_launch": cfg.flops},
           "gpu_launches": args.steps}
    pool.close()
    return res


def build_decode_pool(torch, cfg, rank: int, q_heads: int | None = None):
    """Pool filled with the configuration's sequences: pages dealt from the seeded permutation, prefixes
    shared by fork when the configuration asks for sharing.  cfg.heads are the pool's (key/value) heads;
    q_heads (a multiple of them) the query's."""
    from attention_b200 import ops, synth
    plan = synth.sharing_plan(cfg)
    ps = cfg.page_size
    n = len(plan.ctx)
    q_heads = q_heads or cfg.heads
    pages_needed = int(sum((int(plan.ctx[i]) - int(plan.prefix_tokens[i]) + ps - 1) // ps for i in range(n))) + 16
    pool = ops.KVPool(num_pages=pages_needed, heads=cfg.heads, head_dim=cfg.head_dim, dtype=torch.float16, page_size=ps,
                      max_seqs=n, max_pages_per_seq=(cfg.ctx_hi + ps - 1) // ps, device=torch.cuda.current_device(),
                      free_order=synth.page_permutation(pages_needed, cfg.seed + rank))
    g = torch.Generator(device="cuda").manual_seed(cfg.seed + 104729 * rank)
    seqs = [-1] * n
    for i in range(n):
        leader, prefix = int(plan.group_leader[i]), int(plan.prefix_tokens[i])
        if prefix > 0:
            seqs[i] = pool.seq_fork(seqs[leader], prefix)
        else:
            seqs[i] = pool.seq_create()
        fresh = int(plan.ctx[i]) - prefix
        for at in range(0, fresh, 8192):                      # bounded temporaries
            m = min(8192, fresh - at)
            kv = torch.randn((2, m, cfg.heads, cfg.head_dim), generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
            pool.append([seqs[i]], [m], kv[0], kv[1])
    q = torch.randn((n, q_heads, cfg.head_dim), generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
    return pool, seqs, q, plan


def bench_decode(torch, dist, cfg, args, rank: int, world: int, peaks, peak_kind):
    from attention_b200 import synth
    q_heads = cfg.heads
    if args.decode_group > 1:
        # grouped-query attention: the configuration's heads are the query heads, 1/group of them the pool's
        import dataclasses
        assert cfg.heads % args.decode_group == 0, "--decode-group must divide the configuration's heads"
        cfg = dataclasses.replace(cfg, heads=cfg.heads // args.decode_group)
    pool, seqs, q, plan = build_decode_pool(torch, cfg, rank, q_heads)
    out = torch.empty_like(q)
    by = synth.decode_algorithmic_bytes(cfg, plan)
    by["total_unique"] += (q_heads - cfg.heads) * 2 * len(seqs) * cfg.head_dim * 2       # q and out of all query heads
    by["total_logical"] += (q_heads - cfg.heads) * 2 * len(seqs) * cfg.head_dim * 2

    def step():
        pool.decode(seqs, q, out)

    with ClockSampler(torch.cuda.current_device()) as clk:
        ms = timed_steps(torch, dist, step, args.steps, args.warmup)
    ms_per_step = ms / args.steps
    hq = q.cpu().pin_memory()
    hout = torch.empty_like(hq).pin_memory()

    def step_e2e():
        pool.decode(seqs, hq, hout)

    ms_e2e = ms_per_step if args.profile_small else timed_steps(torch, dist, step_e2e, args.steps, args.warmup) / args.steps
    sec = ms_per_step * 1e-3
    gbs_rank = by["total_unique"] / sec / 1e9
    res = {
        "metric": "paged_decode_hbm_gbs", "unit": "GB/s", "value": gbs_rank * world,
        "tokens_per_s": len(seqs) * world / sec, "effective_gbs_logical": by["total_logical"] * world / sec / 1e9,
        "ms_per_step": ms_per_step, "dtype": "f16",
        "config": {"workload": f"{cfg.name}: paged decode FP16 batch {cfg.batch} H{q_heads}{'' if q_heads == cfg.heads else '/' + str(cfg.heads) + ' key-value heads'} D{cfg.head_dim} page {cfg.page_size}, "
                               f"context {'logU' if cfg.log_uniform else 'U'}[{cfg.ctx_lo},{cfg.ctx_hi}], seeded page permutation",
                   "tokens_in_context": int(plan.ctx.astype(np.int64).sum()), "shared_page_fraction": plan.shared_fraction,
                   "l2": "KV read per step (GBs) far exceeds the 126 MB L2"},
        "e2e": {"value": by["total_unique"] * world / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "tokens_per_s": len(seqs) * world / (ms_e2e * 1e-3),
                "h2d_bytes_per_step": q.numel() * 2 + len(seqs) * 4, "d2h_bytes_per_step": q.numel() * 2, "ms_per_step": ms_e2e},
        "roofline": {"bound": "hbm", "achieved": gbs_rank, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs_rank / peaks["hbm_gbs"],
                     "traffic": NCU_TRAFFIC["paged_decode_kernel_ratio"] * by["total_unique"] if args.decode_group == 1 else None, "peak_source": peak_kind, "frac_of_nominal_8000": gbs_rank / 8000.0,
                     "kernel": ("paged_decode_kernel" if args.decode_group == 1 else "paged_decode_gqa_kernel" if args.decode_group == 2
                                else "paged_decode_tc_kernel" if args.decode_group <= 16 and cfg.head_dim == 128
                                else "fa_fwd_tc_kernel<MODE_DECODE>") + " (+ paged_combine_kernel in the same timed step)",
                     "bytes_per_launch": by["total_unique"]},
        "clocks": clk.summary(), "gpu_launches": 2 * args.steps,
    }
    pool.close()
    return res


# ------------------------------------------------------------------------------------------ main

def run_reference(args, cfg):
    """The CPU arm: the port of the reference algorithm on this box's host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tflops, sample, dt, threads = cpu_fa_baseline(cfg, budget_s=120.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": "flashattn_fwd_tflops", "value": tflops, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(cfg)},
        "cpu_baseline": {"value": tflops, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(cfg):
    return (f"{cfg.name}: FlashAttention forward {cfg.dtype.upper()} {'causal' if cfg.causal else 'non-causal'} "
            f"B={cfg.batch} S={cfg.seq} H={cfg.heads} D={cfg.head_dim}, memory [B,H,S,D]")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["fa_c2", "fa_c4"], default="fa_c2")
    ap.add_argument("--no-decode", action="store_true", help="skip the paged-decode section")
    ap.add_argument("--decode", choices=["c3", "c5"], default="c3",
                    help="paged-decode configuration: c3 (batch 64, U[512,8192]) or c5 (batch 256, logU[1024,32768], shared prefixes)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill-over-pages section")
    ap.add_argument("--decode-group", type=int, default=1,
                    help="grouped-query decode: the configuration's heads are the query heads, 1/GROUP of them key/value heads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--strong", action="store_true",
                    help="strong scaling: the heads of ONE configuration are split over the ranks (ahpc_shard_range) instead of "
                         "every rank running a full copy; heads must divide by the number of ranks")
    ap.add_argument("--profile-small", action="store_true",
                    help="reduced copies of the workloads for profiler captures: FA B=2 H=16 S=4096 D=128 causal BF16, "
                         "decode = the first 16 sequences of C3; no end-to-end or CPU legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from attention_b200 import synth
    cfg = synth.C2 if args.workload == "fa_c2" else synth.C4
    dec_cfg = synth.C3 if args.decode == "c3" else synth.C5
    scaling = "weak"
    if args.strong and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import dataclasses
        from attention_b200 import abi
        w, r = int(os.environ["WORLD_SIZE"]), int(os.environ.get("RANK", "0"))
        hb, he = abi.shard_range(cfg.heads, w, r)
        db, de = abi.shard_range(dec_cfg.heads, w, r)
        assert cfg.heads % w == 0 and dec_cfg.heads % w == 0, "--strong needs heads divisible by the number of ranks"
        cfg = dataclasses.replace(cfg, heads=he - hb)
        dec_cfg = dataclasses.replace(dec_cfg, heads=de - db)
        scaling = "strong"
    if args.profile_small:
        import dataclasses
        cfg = dataclasses.replace(synth.C2, name="C2-small", batch=2, heads=16)
        dec_cfg = dataclasses.replace(synth.C3, name="C3-small", batch=16)
        args.no_cpu_baseline = True
    if args.impl == "reference":
        run_reference(args, cfg)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the library has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    peaks, peak_kind = load_peaks()

    fa = bench_fa(torch, dist, cfg, args, rank, world, peaks, peak_kind)
    torch.cuda.empty_cache()
    pre = None
    if not args.no_prefill:
        pre = bench_paged_prefill(torch, dist, cfg, args, rank, world, peaks, peak_kind)
        torch.cuda.empty_cache()
    dec = None
    if not args.no_decode:
        dec = bench_decode(torch, dist, dec_cfg, args, rank, world, peaks, peak_kind)

    if rank == 0:
        line = {
            "metric": "flashattn_fwd_tflops", "value": fa["value"], "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": fa["ms_per_step"], "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic",
            "config": {"workload": workload_name(cfg), "per_gpu_batch": cfg.batch, "global_batch": cfg.batch * (1 if scaling == "strong" else world),
                       "per_gpu_heads": cfg.heads,
                       "partition": "(batch, head) ranges per GPU, no collective",
                       "l2": f"inputs + output of a step ({4 * cfg.batch * cfg.heads * cfg.seq * cfg.head_dim * 2 / 1e6:.0f} MB) "
                             "exceed the 126 MB L2; no explicit flush"},
            "e2e": fa["e2e"], "roofline": fa["roofline"], "clocks": fa["clocks"], "gpu_launches": fa["gpu_launches"],
        }
        if not args.no_cpu_baseline:
            tflops, sample, _, threads = cpu_fa_baseline(cfg, budget_s=15.0)
            line["cpu_baseline"] = {"value": tflops, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample}
        if pre is not None:
            line["paged_prefill"] = pre
            line["gpu_launches"] += pre["gpu_launches"]
        if dec is not None:
            if not args.no_cpu_baseline:
                gbs, tps, sample, threads = cpu_decode_baseline(dec_cfg, budget_s=10.0)
                dec["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "tokens_per_s": tps, "cores": threads, "kind": "port", "sample": sample}
            line["paged_decode"] = dec
            line["gpu_launches"] += dec["gpu_launches"]
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
