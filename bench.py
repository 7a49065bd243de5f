"""Benchmark of the TBE hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-others]

One step = one training pass of the table-wise-sharded TBE configuration over one synthetic
batch: pooled forward lookup over this rank's tables for the whole global batch, the exchange of
pooled rows (N > 1), the exchange of gradients back (N > 1) and the backward with fused exact
row-wise Adagrad. Tables are weak-scaled, 64 per GPU, because the literal 512-table configuration
(524 GB of fp16 rows) only fits at 4 and 8 GPUs. Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from torchlib_xpu_b200 import cabi, workloads  # noqa: E402

L2_FLUSH_BYTES = 512 << 20
TABLES_OVERRIDE = None   # --tables: fewer tables for --only runs (small profiler captures)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device_index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons = [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1]))
                out["sm_max_mhz"] = float(f[2])
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def zipf_indices_device(num_rows, alpha, n, gen):
    """Bounded Zipf row ids drawn on the device (inverse CDF), for inputs too large to draw on
    the host in reasonable time. Same distribution as workloads.bounded_zipf."""
    cdf = torch.cumsum(torch.arange(1, num_rows + 1, device="cuda", dtype=torch.float64) ** (-alpha), 0)
    cdf /= cdf[-1].clone()
    out = torch.empty(n, dtype=torch.int64, device="cuda")
    chunk = 1 << 24
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        u = torch.rand(b - a, device="cuda", dtype=torch.float64, generator=gen)
        out[a:b] = torch.searchsorted(cdf, u).clamp_(max=num_rows - 1)
    return out


def uniform_half_table(num_elems, lo, hi, gen):
    w = torch.empty(num_elems, dtype=torch.float16, device="cuda")
    chunk = 1 << 28
    for a in range(0, num_elems, chunk):
        b = min(num_elems, a + chunk)
        w[a:b] = (torch.rand(b - a, device="cuda", generator=gen) * (hi - lo) + lo).half()
    return w


def backward_launches(bits: int) -> int:
    passes = (bits + 9) // 10
    return 1 + passes * 5 + 3 + 3  # linearize, per pass hist+3 scan+scatter, segmentation, reduce


def time_launches(fn, iters, flush=None):
    """Median and mean device time (ms) of fn() over iters launches, one CUDA-event pair each, with an
    optional L2 flush between launches (outside the timed pairs), after 3 untimed launches."""
    times = []
    for _ in range(3):
        fn()
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return float(np.median(times)), float(np.mean(times))


# --------------------------------------------------------------------------------------------
# The sharded training configuration (the bench's step)
# --------------------------------------------------------------------------------------------
class ShardedTbeStep:
    def __init__(self, rank, world, cfg, small=False):
        self.rank, self.world = rank, world
        self.T = cfg["T_per_gpu"]
        self.E, self.D, self.B = cfg["E"], cfg["D"], cfg["B"]
        if small:
            self.T, self.E, self.B = 4, 100_000, 4096
        gen = torch.Generator(device="cuda").manual_seed(cfg["seed"] + 1000 * rank)
        T, E, D, B = self.T, self.E, self.D, self.B
        lengths = torch.randint(cfg["L_lo"], cfg["L_hi"] + 1, (T * B,), device="cuda", generator=gen)
        self.offsets = torch.zeros(T * B + 1, dtype=torch.int64, device="cuda")
        torch.cumsum(lengths, 0, out=self.offsets[1:])
        self.N = int(self.offsets[-1].item())
        self.indices = zipf_indices_device(E, cfg["alpha"], self.N, gen)
        self.weights = uniform_half_table(T * E * D, -0.01, 0.01, gen)
        self.momentum = torch.zeros(T * E, dtype=torch.float32, device="cuda")
        self.weights_offsets = torch.arange(T, device="cuda", dtype=torch.int64) * (E * D)
        self.D_offsets = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
        self.hash_size_cumsum = torch.arange(T + 1, device="cuda", dtype=torch.int64) * E
        self.momentum_offsets = self.hash_size_cumsum[:-1].clone()
        self.bits = max(1, (T * E - 1).bit_length())
        self.total_D = T * D
        # pooled rows and their gradients travel as fp16
        self.pooled = torch.empty((B, self.total_D), dtype=torch.float16, device="cuda")
        self.grad = (torch.randn((B, self.total_D), device="cuda", generator=gen)).half()
        need = cabi.backward_scratch_bytes(self.N, self.bits, D)
        self.scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        # distinct rows touched (for the compulsory-byte count)
        table_of = torch.repeat_interleave(
            torch.arange(T, device="cuda", dtype=torch.int64),
            self.offsets[B::B] - self.offsets[0:T * B:B])
        self.U = int(torch.unique(table_of * E + self.indices).numel())
        del table_of
        if world > 1:
            from torchlib_xpu_b200 import sharded
            self.exchange = sharded.PooledExchange(rank, world, B, self.total_D)
        else:
            self.exchange = None

    def forward(self):
        if self.exchange is None:
            cabi.forward(self.weights, self.weights_offsets, self.D_offsets, self.total_D, self.D,
                         self.indices, self.offsets, self.B, outputs=[self.pooled],
                         output_stride=self.total_D, rows_per_dest=self.B,
                         output_dtype=torch.float16)
        else:
            self.exchange.forward_lookup(self)

    def backward(self):
        grad, ready = (self.grad, None) if self.exchange is None else self.exchange.gather_gradients_async(self)
        cabi.backward(self.weights, self.weights_offsets, self.D_offsets, self.hash_size_cumsum,
                      self.bits, self.D, self.indices, self.offsets, self.B, grad,
                      cabi.OPT_ROWWISE_ADAGRAD, 0.01, 1e-8, self.momentum, self.momentum_offsets,
                      scratch=self.scratch, grad_ready_event=ready)

    def result(self):
        """Pooled rows this rank ends the forward with (its batch slice, all tables, when sharded)."""
        return self.pooled if self.exchange is None else self.exchange.recv

    def step(self):
        self.forward()
        self.backward()

    def launches_per_step(self):
        extra = 0 if self.exchange is None else self.exchange.launches_per_step()
        return 1 + backward_launches(self.bits) + extra

    def fwd_bytes(self):
        return workloads.forward_bytes(self.N, self.U, self.D * 2, self.T, self.B, self.D, 2)

    def bwd_bytes(self):
        return workloads.backward_bytes(self.N, self.U, self.D * 2, self.T, self.B, self.D, 2)


# --------------------------------------------------------------------------------------------
# CPU arm: FBGEMM-core forward + the C oracle's backward on a bounded sample of the same workload
# --------------------------------------------------------------------------------------------
def cpu_sample_rate(cfg, budget_s=12.0):
    import oracle
    T, E, D, B = 2, cfg["E"], cfg["D"], 8192
    inp = workloads.tbe_inputs(T, B, E, D, cfg["L_lo"], cfg["L_hi"], cfg["seed"], "zipf", cfg["alpha"])
    g = torch.Generator().manual_seed(7)
    W = ((torch.rand(T * E * D, generator=g) * 0.02) - 0.01).half().numpy()
    wo = np.arange(T, dtype=np.int64) * (E * D)
    Do = (np.arange(T + 1) * D).astype(np.int32)
    hs = np.arange(T + 1, dtype=np.int64) * E
    grad = torch.randn((B, T * D), generator=g).numpy()
    mom = np.zeros(T * E, dtype=np.float32)
    rows = [E] * T
    threads = oracle.num_threads()
    t0, reps = time.perf_counter(), 0
    while True:
        oracle.tbe_forward(W, oracle.FP16, wo, Do, B, inp.indices, inp.offsets, backend="ref",
                           rows_per_table=rows)
        oracle.tbe_backward(W, oracle.FP16, wo, Do, hs, B, inp.indices, inp.offsets, grad, mom, hs[:-1],
                            oracle.ROWWISE_ADAGRAD, 0.01, 1e-8)
        reps += 1
        if time.perf_counter() - t0 > budget_s or reps >= 200:
            break
    dt = time.perf_counter() - t0
    sample = ("%d reps of fwd (FBGEMM-core EmbeddingSpMDM, torch-bundled) + bwd/Adagrad (C oracle) on "
              "T=%d E=%d D=%d fp16 B=%d, %d lookups each, %.1f s" % (reps, T, E, D, B, inp.num_lookups, dt))
    return inp.num_lookups * reps / dt, threads, sample, dt / reps


def reference_arm(args, cfg, rank, json_out):
    if rank != 0:
        return
    steps, warm = args.steps, args.warmup
    per_step_budget = max(0.5, min(8.0, 100.0 / max(1, steps + warm)))
    rate, threads, sample, sec = cpu_sample_rate(cfg, budget_s=per_step_budget * (steps + warm))
    line = {
        "impl": "reference", "metric": "TBE pooled-row lookups/s (fwd + bwd with fused row-wise Adagrad)",
        "value": rate, "unit": "lookups/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16 rows, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "table-wise sharded TBE (config 5), CPU sample", "sample": sample},
        "cpu_baseline": {"value": rate, "unit": "lookups/s", "cores": threads, "kind": "reference",
                         "sample": sample},
        "e2e": {"value": rate, "unit": "lookups/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), file=json_out, flush=True)


# --------------------------------------------------------------------------------------------
# The other named configurations, single GPU, one kernel (or kernel group) each
# --------------------------------------------------------------------------------------------
def bench_others(peak_gbs, iters=20, only=None):
    """only: None (all), or one of 'jagged', 'fp32', 'train', 'nbit', 'nv12', 'permute'."""
    res = {}
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(99)

    def entry(name, bytes_, ms, lookups=None, extra=None):
        e = {"ms": ms, "algorithmic_GB": bytes_ / 1e9, "achieved_GBps": bytes_ / ms / 1e6,
             "frac_of_measured_hbm": bytes_ / ms / 1e6 / peak_gbs}
        if lookups:
            e["lookups_per_s"] = lookups / ms * 1e3
        if extra:
            e.update(extra)
        res[name] = e

    if only not in (None, "jagged"):
        return _others_tbe(res, entry, flush, gen, iters, only)
    # config 2: jagged ops
    c = workloads.CONFIGS["jagged"]
    j = workloads.jagged_inputs(c["B"], c["max_L"], c["D"], c["seed"])
    values = torch.randn((j.total_rows, j.D), device="cuda", generator=gen)
    y = torch.randn((j.B, j.max_L, j.D), device="cuda", generator=gen)
    off = torch.from_numpy(j.offsets).cuda()
    dense = cabi.jagged_to_padded_dense(values, [off], [j.max_L], 0.0)
    row = j.D * 4
    ms, _ = time_launches(lambda: cabi.jagged_to_padded_dense(values, [off], [j.max_L], 0.0), iters, flush)
    entry("jagged_to_padded_dense", j.total_rows * row + j.B * j.max_L * row + (j.B + 1) * 8, ms)
    ms, _ = time_launches(lambda: cabi.dense_to_jagged(dense, [off], j.total_rows), iters, flush)
    entry("dense_to_jagged", 2 * j.total_rows * row + (j.B + 1) * 8, ms)
    ms, _ = time_launches(lambda: cabi.jagged_dense_elementwise_add(values, [off], y), iters, flush)
    entry("jagged_dense_elementwise_add", j.total_rows * row + 2 * j.B * j.max_L * row + (j.B + 1) * 8, ms)
    del values, y, dense
    if only == "jagged":
        return res
    return _others_tbe(res, entry, flush, gen, iters, only)


def _others_tbe(res, entry, flush, gen, iters, only):
    if only in (None, "fp32"):
        _bench_fp32(entry, flush, gen, iters)
    if only in (None, "train"):
        _bench_train(entry, flush, gen, iters)
    if only in (None, "nbit"):
        _bench_nbit(entry, flush, gen, iters)
    if only in (None, "nv12"):
        _bench_nv12(entry, flush, gen, iters)
    if only in (None, "permute"):
        _bench_permute(entry, flush, gen, iters)
    return res


def _bench_fp32(entry, flush, gen, iters):
    # config 1: fp32 forward, uniform ids
    c = workloads.CONFIGS["tbe_fp32_fwd"]
    inp = workloads.tbe_inputs(c["T"], c["B"], c["E"], c["D"], c["L_lo"], c["L_hi"], c["seed"], c["dist"])
    T, E, D, B = c["T"], c["E"], c["D"], c["B"]
    W = torch.rand(T * E * D, device="cuda", generator=gen) * 0.02 - 0.01
    wo = torch.arange(T, device="cuda", dtype=torch.int64) * (E * D)
    Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
    idx, offs = torch.from_numpy(inp.indices).cuda(), torch.from_numpy(inp.offsets).cuda()
    out = torch.empty((B, T * D), device="cuda")
    fn = lambda: cabi.forward(W, wo, Do, T * D, D, idx, offs, B, outputs=[out], output_stride=T * D,
                              rows_per_dest=B)
    fn()
    ms, _ = time_launches(fn, iters, flush)
    entry("tbe_fp32_forward(config1)", workloads.forward_bytes(inp.num_lookups, inp.unique_rows(), D * 4, T, B, D, 4),
          ms, inp.num_lookups)


def _bench_train(entry, flush, gen, iters):
    # config 3: fp16 tables, forward and backward + Adagrad
    c = workloads.CONFIGS["tbe_fp16_train"]
    T, E, D, B = TABLES_OVERRIDE or c["T"], c["E"], c["D"], c["B"]
    inp = workloads.tbe_inputs(T, B, E, D, c["L_lo"], c["L_hi"], c["seed"], "zipf", c["alpha"], c["permute"])
    U = inp.unique_rows()
    W = uniform_half_table(T * E * D, -0.01, 0.01, gen)
    mom = torch.zeros(T * E, device="cuda")
    wo = torch.arange(T, device="cuda", dtype=torch.int64) * (E * D)
    Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
    hs = torch.arange(T + 1, device="cuda", dtype=torch.int64) * E
    idx, offs = torch.from_numpy(inp.indices).cuda(), torch.from_numpy(inp.offsets).cuda()
    out = torch.empty((B, T * D), device="cuda")
    grad = torch.randn((B, T * D), device="cuda", generator=gen)
    bits = (T * E - 1).bit_length()
    scratch = torch.empty(cabi.backward_scratch_bytes(inp.num_lookups, bits, D), dtype=torch.uint8, device="cuda")
    fwd = lambda: cabi.forward(W, wo, Do, T * D, D, idx, offs, B, outputs=[out], output_stride=T * D,
                               rows_per_dest=B)
    bwd = lambda: cabi.backward(W, wo, Do, hs, bits, D, idx, offs, B, grad, cabi.OPT_ROWWISE_ADAGRAD, 0.01,
                                1e-8, mom, hs[:-1], scratch=scratch)
    fwd(); bwd()
    ms, _ = time_launches(fwd, iters, flush)
    entry("tbe_fp16_forward(config3)", workloads.forward_bytes(inp.num_lookups, U, D * 2, T, B, D, 4), ms,
          inp.num_lookups, {"unique_rows": U})
    ms, _ = time_launches(bwd, iters, flush)
    entry("tbe_fp16_backward_adagrad(config3)", workloads.backward_bytes(inp.num_lookups, U, D * 2, T, B, D, 4),
          ms, inp.num_lookups, {"kernels_per_call": backward_launches(bits)})


def _bench_permute(entry, flush, gen, iters):
    # the regrouping step of the input distribution at the bench step's shape: what one rank of 8
    # receives, (source rank, local table, sample) -> (local table, global sample): 4.2 M bags,
    # about 107 M int64 ids; every id is read once and written once
    from torchlib_xpu_b200 import sharded
    world, T_local, B = 8, 64, 65536
    per = B // world
    lengths = torch.randint(1, 51, (world * T_local * per,), device="cuda", generator=gen)
    n = int(lengths.sum().item())
    ids = torch.randint(0, 4_000_000, (n,), device="cuda", generator=gen)
    perm = torch.arange(world * T_local * per, device="cuda").view(world, T_local, per).permute(1, 0, 2).reshape(-1)
    in_off = torch.zeros(lengths.numel() + 1, dtype=torch.int64, device="cuda")
    torch.cumsum(lengths, 0, out=in_off[1:])
    out_off = torch.zeros_like(in_off)
    torch.cumsum(lengths[perm], 0, out=out_off[1:])
    ms, _ = time_launches(lambda: cabi.permute_segments(ids, in_off, out_off, perm), max(3, iters // 2), flush)
    entry("permute_segments(config5 ids, 8 ranks)", 2 * n * 8 + 3 * lengths.numel() * 8, ms, n,
          {"segments": int(lengths.numel())})
    del ids, lengths, perm, in_off, out_off


def _bench_nv12(entry, flush, gen, iters):
    # the reference plugin's own kernel: one 3840 x 2160 NV12 frame to RGB24, and a batch of 32 such
    # frames back to back (a decoder's steady state); 1.5 bytes read + 3 written per pixel
    w, h = 3840, 2160
    frames = 32
    y = torch.randint(0, 256, (frames, h, w), dtype=torch.uint8, device="cuda", generator=gen)
    uv = torch.randint(0, 256, (frames, h // 2, w), dtype=torch.uint8, device="cuda", generator=gen)
    out = torch.empty((frames, h, w, 3), dtype=torch.uint8, device="cuda")
    bytes_frame = w * h * 3 // 2 + w * h * 3
    ms, _ = time_launches(lambda: cabi.nv12_to_rgb(y[0], uv[0], w, h, w, out=out[0]), iters, flush)
    entry("nv12_to_rgb(4K frame)", bytes_frame, ms, None, {"pixels_per_s": w * h / ms * 1e3})

    def batch():
        for f in range(frames):
            cabi.nv12_to_rgb(y[f], uv[f], w, h, w, out=out[f])
    ms, _ = time_launches(batch, max(3, iters // 4), flush)
    entry("nv12_to_rgb(32 x 4K frames)", bytes_frame * frames, ms, None,
          {"pixels_per_s": w * h * frames / ms * 1e3, "launches": frames})
    del y, uv, out


def _bench_nbit(entry, flush, gen, iters):
    # config 4: quantised inference forward, half INT8 / half INT4 tables
    c = workloads.CONFIGS["tbe_nbit_fwd"]
    T, E, D, B = TABLES_OVERRIDE or c["T"], c["E"], c["D"], c["B"]
    inp = workloads.tbe_inputs(T, B, E, D, c["L_lo"], c["L_hi"], c["seed"], "zipf", c["alpha"])
    U_by_table = []
    strides = [144 if t < T // 2 else 80 for t in range(T)]
    payload = [132 if t < T // 2 else 68 for t in range(T)]
    tl = inp.table_lookups()
    pos, row_bytes = 0, 0
    for t in range(T):
        u = int(np.unique(inp.indices[pos:pos + int(tl[t])]).size)
        U_by_table.append(u)
        row_bytes += u * payload[t]
        pos += int(tl[t])
    total = sum(E * s for s in strides)
    Wq = torch.randint(0, 256, (total,), dtype=torch.uint8, device="cuda", generator=gen)
    wo_np = np.zeros(T, dtype=np.int64)
    at = 0
    hdr = torch.tensor([2.0 / 255, -1.0], dtype=torch.float16).view(torch.uint8).cuda()
    for t in range(T):
        wo_np[t] = at
        Wq[at:at + E * strides[t]].view(E, strides[t])[:, :4] = hdr
        at += E * strides[t]
    tys = torch.tensor([cabi.INT8 if t < T // 2 else cabi.INT4 for t in range(T)], dtype=torch.uint8, device="cuda")
    wo = torch.from_numpy(wo_np).cuda()
    Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
    idx, offs = torch.from_numpy(inp.indices).cuda(), torch.from_numpy(inp.offsets).cuda()
    fn = lambda: cabi.nbit_forward(Wq, wo, tys, Do, T * D, D, idx, offs, B)
    fn()
    ms, _ = time_launches(fn, max(5, iters // 2), flush)
    bytes_ = row_bytes + inp.num_lookups * 8 + (T * B + 1) * 8 + B * T * D * 2
    entry("tbe_nbit_forward(config4)", bytes_, ms, inp.num_lookups, {"unique_rows": int(sum(U_by_table))})


def _claim_stdout():
    """Libraries (NCCL among them) print banners on stdout; the contract is ONE JSON line there. Point
    fd 1 at stderr for the run and hand back a file on the original stdout for the final line."""
    sys.stdout.flush()
    keep = os.dup(1)
    os.dup2(2, 1)
    return os.fdopen(keep, "w")


def main():
    json_out = _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-others", action="store_true", help="skip the single-kernel configurations")
    ap.add_argument("--small", action="store_true", help="tiny tables, for profiler captures and smoke runs")
    ap.add_argument("--only", default=None, choices=["jagged", "fp32", "train", "nbit", "nv12", "permute"],
                    help="run one single-GPU configuration alone (few launches; for profiler captures)")
    ap.add_argument("--iters", type=int, default=20, help="timed launches per single-GPU configuration")
    ap.add_argument("--tables", type=int, default=None,
                    help="with --only train|nbit: use this many tables (a small case for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.small else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = workloads.CONFIGS["tbe_sharded"]

    if args.impl == "reference":
        reference_arm(args, cfg, rank, json_out)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA kernels are the only implementation")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cabi.lib()
    peak_gbs, peak_kind = measured_peak_gbs()
    if args.only is not None:
        global TABLES_OVERRIDE
        TABLES_OVERRIDE = args.tables
        print(json.dumps({"only": args.only, "peak_gbs": peak_gbs,
                          "results": bench_others(peak_gbs, args.iters, args.only)}), file=json_out, flush=True)
        return

    step = ShardedTbeStep(rank, world, cfg, small=args.small)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step.step()
    barrier()

    # ---- device-resident timing: exactly K steps between barriers -------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    fwd_ms, bwd_ms = [], []
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        a.record()
        step.forward()
        b.record()
        step.backward()
        c.record()
        fwd_ms.append((a, b))
        bwd_ms.append((b, c))
    t_end.record()
    barrier()
    clocks = sampler.stop()
    total_ms = t_start.elapsed_time(t_end)
    fwd_avg = float(np.mean([a.elapsed_time(b) for a, b in fwd_ms]))
    bwd_avg = float(np.mean([a.elapsed_time(b) for a, b in bwd_ms]))
    if dist is not None:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        n_all = torch.tensor([step.N], device="cuda", dtype=torch.float64)
        dist.all_reduce(n_all)
        lookups_all = float(n_all.item())
    else:
        lookups_all = float(step.N)
    ms_per_step = total_ms / args.steps
    value = lookups_all / (ms_per_step / 1e3)

    # ---- end to end: host buffers in, pooled rows out, every step ---------------------------
    h_idx = step.indices.cpu().pin_memory()
    h_off = step.offsets.cpu().pin_memory()
    grad_in = step.grad if step.exchange is None else step.exchange.grad_slice
    h_grad = grad_in.cpu().pin_memory()
    h_out = torch.empty(step.result().shape, dtype=step.result().dtype).pin_memory()
    # whole-job bytes: every rank copies its own inputs and its own slice of the result
    h2d = (h_idx.numel() * 8 + h_off.numel() * 8 + h_grad.numel() * h_grad.element_size()) * world
    d2h = h_out.numel() * h_out.element_size() * world

    # The loop a trainer with host-side batches runs: the next step's ids are copied in while the
    # current step computes (two id buffers), the gradient copy overlaps the forward, the result
    # copy overlaps the backward. Every step's copies are inside the timed region.
    main = torch.cuda.current_stream()
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    idx_bufs = [step.indices, torch.empty_like(step.indices)]
    off_bufs = [step.offsets, torch.empty_like(step.offsets)]
    pipe = {"k": 0, "bwd_done": None, "out_done": None}

    def e2e_step():
        k = pipe["k"]
        pipe["k"] = k + 1
        idx, off = idx_bufs[k & 1], off_bufs[k & 1]
        in_ready, grad_ready = torch.cuda.Event(), torch.cuda.Event()
        fwd_done, out_done, bwd_done = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
        with torch.cuda.stream(copy_in):
            # this id buffer was last read by the backward two steps back, which the gradient
            # copy of the previous step already waited for
            idx.copy_(h_idx, non_blocking=True)
            off.copy_(h_off, non_blocking=True)
            in_ready.record(copy_in)
            if pipe["bwd_done"] is not None:
                copy_in.wait_event(pipe["bwd_done"])   # the previous backward reads the gradient buffer
            grad_in.copy_(h_grad, non_blocking=True)
            grad_ready.record(copy_in)
        step.indices, step.offsets = idx, off
        main.wait_event(in_ready)
        if world == 1 and pipe["out_done"] is not None:
            main.wait_event(pipe["out_done"])          # the result buffer is still being copied out
        step.forward()
        fwd_done.record(main)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(fwd_done)
            h_out.copy_(step.result(), non_blocking=True)
            out_done.record(copy_out)
        main.wait_event(grad_ready)
        if world > 1:
            # peers write the next forward's rows into this rank's result buffer: the copy-out has
            # to be over before the barrier inside the backward's gradient exchange
            main.wait_event(out_done)
        step.backward()
        bwd_done.record(main)
        pipe["bwd_done"], pipe["out_done"] = bwd_done, out_done

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(2, min(args.steps, 10))
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    main.wait_event(pipe["out_done"])   # the last result has to be on the host inside the timed region
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = lookups_all / (e2e_ms / e2e_steps / 1e3)
    step.indices, step.offsets = idx_bufs[0], off_bufs[0]
    del h_idx, h_off, h_grad, h_out, idx_bufs, off_bufs

    line = {
        "metric": "TBE pooled-row lookups/s (fwd + bwd with fused row-wise Adagrad)",
        "value": value, "unit": "lookups/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16 rows, fp32 accumulate", "data": "synthetic",
        "config": {
            "workload": "table-wise sharded TBE (config 5), weak-scaled: %d fp16 tables per GPU x %d rows x D=%d, "
                        "global B=%d, L~U{1..50}, Zipf(1.05) ids" % (step.T, step.E, step.D, step.B),
            "tables_per_gpu": step.T, "rows_per_table": step.E, "D": step.D, "global_batch": step.B,
            "lookups_per_rank": step.N, "unique_rows_per_rank": step.U,
            "l2": "inputs larger than L2 (%.1f GB of rows per rank)" % (step.weights.numel() * 2 / 1e9),
            "exchange": "none (1 GPU)" if world == 1 else step.exchange.describe(),
        },
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "lookups/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": step.launches_per_step() * args.steps,
        "phases_ms": {"forward": fwd_avg, "backward": bwd_avg},
    }
    # roofline of the dominant part of the step (the backward's kernel group) and of the forward
    # kernel; algorithmic bytes = compulsory traffic (distinct rows once)
    bwd_bytes, fwd_bytes = step.bwd_bytes(), step.fwd_bytes()
    line["roofline"] = {
        "bound": "hbm", "kernel": "b200tbe_backward (linearize + radix sort + segment + reduce/update)",
        "achieved": bwd_bytes / bwd_avg / 1e6, "peak": peak_gbs, "unit": "GB/s",
        "frac": bwd_bytes / bwd_avg / 1e6 / peak_gbs, "traffic": None, "peak_kind": "of " + peak_kind,
        "algorithmic_bytes": bwd_bytes,
    }
    line["roofline_forward"] = {
        "bound": "hbm", "kernel": "tbe_forward_bags_kernel", "achieved": fwd_bytes / fwd_avg / 1e6,
        "peak": peak_gbs, "unit": "GB/s", "frac": fwd_bytes / fwd_avg / 1e6 / peak_gbs,
        "traffic": None, "peak_kind": "of " + peak_kind, "algorithmic_bytes": fwd_bytes,
    }

    if rank == 0 and world == 1:
        del step
        torch.cuda.empty_cache()
        if not args.no_others and not args.small:
            line["others"] = bench_others(peak_gbs)
        torch.cuda.empty_cache()
        try:
            rate, threads, sample, _ = cpu_sample_rate(cfg)
            line["cpu_baseline"] = {"value": rate, "unit": "lookups/s", "cores": threads,
                                    "kind": "reference", "sample": sample}
        except Exception as exc:  # the CPU arm must not take the GPU numbers down with it
            line["cpu_baseline"] = {"value": None, "unit": "lookups/s", "cores": None, "kind": "reference",
                                    "sample": "failed: %r" % (exc,)}
    if rank == 0:
        print(json.dumps(line), file=json_out, flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
