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
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE table of the bench step -- 4 M fp16
# rows x D=128, B=65536, about 1.67 M lookups -- from the ncu capture summarised in
# profiles/tbe_step_one_table_traffic.md. Tables are processed one after another, each with its own
# rows, ids and gradient columns, so a step of T tables moves T times this.
FWD_TRAFFIC_PER_TABLE = 107.2e6   # lookup kernel: 101.9 MB read + 5.3 MB written
BWD_TRAFFIC_PER_TABLE = 254.9e6   # 20 kernels of one b200tbe_backward call: 213.4 MB read + 41.5 MB written
TRAFFIC_NOTE = ("one-table ncu capture x tables (profiles/tbe_step_one_table_traffic.md); bytes a kernel leaves "
                "dirty in L2 when it ends are not in its DRAM write counter")
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
    """nvidia-smi clock / throttle-reason samples taken while the GPU runs the step: the sampler is
    started well before the warm-up steps (nvidia-smi needs a few hundred milliseconds to answer for
    the first time), and the samples whose timestamps fall between the first warm-up step and the end
    of the timed region are the ones reported; `samples_in_timed_region` says how many of those fell
    into the timed steps themselves (the region is about a tenth of a second)."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.path = None
        self.t_load = self.t_timed = None
        self.nvml_thread = None

    def start(self):
        # NVML from a thread answers in well under a millisecond, nvidia-smi in a loop every ~100 ms:
        # the thread is the sampler, the nvidia-smi loop the fallback
        if self._start_nvml():
            return
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device_index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def _start_nvml(self):
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.device_index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            reasons_of = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self.nvml_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.nvml_rows = []          # (time, sm MHz, reasons bit mask)
            self.nvml_stop = threading.Event()

            def loop():
                while not self.nvml_stop.is_set():
                    try:
                        self.nvml_rows.append((time.time(),
                                               float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)),
                                               int(reasons_of(handle))))
                    except Exception:
                        pass
                    time.sleep(0.004)

            self.nvml_thread = threading.Thread(target=loop, daemon=True)
            self.nvml_thread.start()
            return True
        except Exception:
            self.nvml_thread = None
            return False

    def mark_load(self):
        """The GPU is busy with the step from now on (first warm-up step)."""
        self.t_load = time.time()

    def mark_timed(self):
        self.t_timed = time.time()

    @staticmethod
    def _when(stamp):
        import datetime
        return datetime.datetime.strptime(stamp, "%Y/%m/%d %H:%M:%S.%f").timestamp()

    def stop(self):
        t_end = time.time()
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "samples_in_timed_region": 0}
        if self.nvml_thread is not None:
            self.nvml_stop.set()
            self.nvml_thread.join(timeout=2)
            # NVML's bits: sw power cap 0x4, hw slowdown 0x8, sw thermal 0x20, hw thermal 0x40
            names = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"),
                     (0x4, "sw_power_cap"))
            rows = [r for r in self.nvml_rows if self.t_load is None or self.t_load <= r[0] <= t_end]
            if rows:
                out["sm_mhz"] = float(np.median([r[1] for r in rows]))
                out["sm_max_mhz"] = self.nvml_max
                out["samples"] = len(rows)
                out["samples_in_timed_region"] = sum(1 for r in rows if self.t_timed is not None and r[0] >= self.t_timed)
                mask = 0
                for r in rows:
                    mask |= r[2]
                out["reasons"] = sorted(n for b, n in names if mask & b)
            out["source"] = "NVML, sampled from a thread every 4 ms"
            return out
        if self.proc is None:
            return out
        time.sleep(0.05)
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
                try:
                    when = self._when(f[0])
                except Exception:
                    continue
                if self.t_load is not None and not (self.t_load <= when <= t_end + 0.02):
                    continue
                sm.append(float(f[1]))
                out["sm_max_mhz"] = float(f[2])
                if self.t_timed is not None and when >= self.t_timed:
                    out["samples_in_timed_region"] += 1
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


def backward_launches(row_bits: int) -> int:
    """Kernels one b200tbe_backward call launches for rows of at most 512 elements: two plan kernels,
    linearize, per sort pass (8 bits each) histogram + 3 scan kernels + scatter, sweep, finish."""
    passes = (row_bits + 7) // 8
    return 2 + 1 + passes * 5 + 2


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
        need = cabi.backward_scratch_bytes(self.N, self.bits, D, T)
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
                      scratch=self.scratch, grad_ready_event=ready, max_table_rows=self.E)

    def result(self):
        """Pooled rows this rank ends the forward with (its batch slice, all tables, when sharded)."""
        return self.pooled if self.exchange is None else self.exchange.recv

    def step(self):
        self.forward()
        self.backward()

    def launches_per_step(self):
        extra = 0 if self.exchange is None else self.exchange.launches_per_step()
        return 1 + backward_launches(max(1, (self.E - 1).bit_length())) + extra

    def fwd_bytes(self):
        return workloads.forward_bytes(self.N, self.U, self.D * 2, self.T, self.B, self.D, 2)

    def bwd_bytes(self):
        return workloads.backward_bytes(self.N, self.U, self.D * 2, self.T, self.B, self.D, 2)


# --------------------------------------------------------------------------------------------
# CPU arm: FBGEMM-core forward + the C oracle's backward on a bounded sample of the same workload
# --------------------------------------------------------------------------------------------
def cpu_sample_rate(cfg, limit_s=12.0):
    """One table of the bench step at the full batch (so that the share of repeated rows is the
    step's own), forward by FBGEMM-core + backward/Adagrad by the C oracle, on every core this
    process may run on -- set explicitly: launchers export OMP_NUM_THREADS=1."""
    import oracle
    T, E, D, B = 1, cfg["E"], cfg["D"], cfg["B"]
    threads = oracle.set_num_threads(len(os.sched_getaffinity(0)))
    inp = workloads.tbe_inputs(T, B, E, D, cfg["L_lo"], cfg["L_hi"], cfg["seed"], "zipf", cfg["alpha"])
    g = torch.Generator().manual_seed(7)
    W = ((torch.rand(T * E * D, generator=g) * 0.02) - 0.01).half().numpy()
    wo = np.arange(T, dtype=np.int64) * (E * D)
    Do = (np.arange(T + 1) * D).astype(np.int32)
    hs = np.arange(T + 1, dtype=np.int64) * E
    grad = torch.randn((B, T * D), generator=g).numpy()
    mom = np.zeros(T * E, dtype=np.float32)
    rows = [E] * T
    t0, reps = time.perf_counter(), 0
    while True:
        oracle.tbe_forward(W, oracle.FP16, wo, Do, B, inp.indices, inp.offsets, backend="ref",
                           rows_per_table=rows)
        oracle.tbe_backward(W, oracle.FP16, wo, Do, hs, B, inp.indices, inp.offsets, grad, mom, hs[:-1],
                            oracle.ROWWISE_ADAGRAD, 0.01, 1e-8)
        reps += 1
        if time.perf_counter() - t0 > limit_s or reps >= 400:
            break
    dt = time.perf_counter() - t0
    sample = ("%d reps of fwd (FBGEMM-core EmbeddingSpMDM, torch-bundled) + bwd/Adagrad (C oracle) on "
              "one table of the step: E=%d D=%d fp16, B=%d, %d lookups each, %d threads, %.1f s"
              % (reps, E, D, B, inp.num_lookups, threads, dt))
    return inp.num_lookups * reps / dt, threads, sample, dt / reps


def reference_arm(args, cfg, rank, json_out):
    if rank != 0:
        return
    steps, warm = args.steps, args.warmup
    per_step_limit = max(0.5, min(8.0, 100.0 / max(1, steps + warm)))
    rate, threads, sample, sec = cpu_sample_rate(cfg, limit_s=per_step_limit * (steps + warm))
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
    """only: None (all), or one of 'jagged', 'fp32', 'train', 'uniform', 'nbit', 'quantize', 'nv12', 'permute'."""
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
    if only in (None, "uniform"):
        _bench_uniform(entry, flush, gen, iters)
    if only in (None, "nbit"):
        _bench_nbit(entry, flush, gen, iters)
    if only in (None, "quantize"):
        _bench_quantize(entry, flush, gen, iters)
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
    scratch = torch.empty(cabi.backward_scratch_bytes(inp.num_lookups, bits, D, T), dtype=torch.uint8, device="cuda")
    fwd = lambda: cabi.forward(W, wo, Do, T * D, D, idx, offs, B, outputs=[out], output_stride=T * D,
                               rows_per_dest=B)
    bwd = lambda: cabi.backward(W, wo, Do, hs, bits, D, idx, offs, B, grad, cabi.OPT_ROWWISE_ADAGRAD, 0.01,
                                1e-8, mom, hs[:-1], scratch=scratch, max_table_rows=E)
    fwd(); bwd()
    ms, _ = time_launches(fwd, iters, flush)
    entry("tbe_fp16_forward(config3)", workloads.forward_bytes(inp.num_lookups, U, D * 2, T, B, D, 4), ms,
          inp.num_lookups, {"unique_rows": U})
    ms, _ = time_launches(bwd, iters, flush)
    entry("tbe_fp16_backward_adagrad(config3)", workloads.backward_bytes(inp.num_lookups, U, D * 2, T, B, D, 4),
          ms, inp.num_lookups, {"kernels_per_call": backward_launches((E - 1).bit_length())})


def _bench_uniform(entry, flush, gen, iters):
    # The training kernels where no lookup repeats a row: 4 fp16 tables x 16 M rows x D=128 (16.4 GB),
    # B=65536, every bag 32 uniform ids. Every row is a first touch, so the compulsory bytes ARE the
    # traffic and the fraction of the HBM copy rate says how well the kernels gather from DRAM; the
    # Zipf configurations above re-read most rows out of L2 and are bound by its row rate instead.
    T, E, D, B, L = 4, 16_000_000, 128, 65536, 32
    idx = torch.randint(0, E, (T * B * L,), device="cuda", generator=gen)
    offs = torch.arange(T * B + 1, device="cuda", dtype=torch.int64) * L
    U = sum(int(torch.unique(idx[t * B * L:(t + 1) * B * L]).numel()) for t in range(T))
    n = T * B * L
    W = uniform_half_table(T * E * D, -0.01, 0.01, gen)
    mom = torch.zeros(T * E, device="cuda")
    wo = torch.arange(T, device="cuda", dtype=torch.int64) * (E * D)
    Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
    hs = torch.arange(T + 1, device="cuda", dtype=torch.int64) * E
    out = torch.empty((B, T * D), device="cuda", dtype=torch.float16)
    grad = (torch.randn((B, T * D), device="cuda", generator=gen) * 0.1).half()
    bits = (T * E - 1).bit_length()
    scratch = torch.empty(cabi.backward_scratch_bytes(n, bits, D, T), dtype=torch.uint8, device="cuda")
    fwd = lambda: cabi.forward(W, wo, Do, T * D, D, idx, offs, B, outputs=[out], output_stride=T * D,
                               rows_per_dest=B, output_dtype=torch.float16)
    bwd = lambda: cabi.backward(W, wo, Do, hs, bits, D, idx, offs, B, grad, cabi.OPT_ROWWISE_ADAGRAD, 0.01,
                                1e-8, mom, hs[:-1], scratch=scratch, max_table_rows=E)
    fwd(); bwd()
    ms, _ = time_launches(fwd, max(5, iters // 2), flush)
    entry("tbe_fp16_forward(uniform ids, 16 GB of rows)", workloads.forward_bytes(n, U, D * 2, T, B, D, 2), ms, n,
          {"unique_rows": U})
    ms, _ = time_launches(bwd, max(5, iters // 2), flush)
    entry("tbe_fp16_backward_adagrad(uniform ids, 16 GB of rows)", workloads.backward_bytes(n, U, D * 2, T, B, D, 2),
          ms, n, {"unique_rows": U, "kernels_per_call": backward_launches((E - 1).bit_length())})
    del W, mom, idx, grad, scratch, out
    # the same lookup on rows of 128 and 64 bytes (D = 64, 32): random rows this short are no longer bound
    # by bytes but by how many rows a second HBM serves, which is what the quantised tables' rows meet
    for D in (64, 32):
        E = 16_000_000 * 128 // D
        idx = torch.randint(0, E, (T * B * L,), device="cuda", generator=gen)
        U = sum(int(torch.unique(idx[t * B * L:(t + 1) * B * L]).numel()) for t in range(T))
        W = uniform_half_table(T * E * D, -0.01, 0.01, gen)
        wo = torch.arange(T, device="cuda", dtype=torch.int64) * (E * D)
        Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
        out = torch.empty((B, T * D), device="cuda", dtype=torch.float16)
        fwd = lambda: cabi.forward(W, wo, Do, T * D, D, idx, offs, B, outputs=[out], output_stride=T * D,
                                   rows_per_dest=B, output_dtype=torch.float16)
        fwd()
        ms, _ = time_launches(fwd, max(5, iters // 2), flush)
        entry("tbe_fp16_forward(uniform ids, 16 GB of %d-byte rows)" % (D * 2),
              workloads.forward_bytes(n, U, D * 2, T, B, D, 2), ms, n, {"unique_rows": U})
        del W, idx, out


def _bench_quantize(entry, flush, gen, iters):
    # the step before the quantised lookup: 2 M fp32 rows of D=128 (1 GB) to INT8 / INT4 rows in the table
    # layout (fp16 scale and bias in front, rows padded to 16 bytes), and INT8 rows back to fp32
    rows, D = 2_000_000, 128
    src = torch.rand((rows, D), device="cuda", generator=gen) * 2 - 1
    for name, ty in (("INT8", cabi.INT8), ("INT4", cabi.INT4)):
        out = cabi.quantize_rows(src, ty, 16, True)
        ms, _ = time_launches(lambda: cabi.quantize_rows(src, ty, 16, True, out=out), max(5, iters // 2), flush)
        entry("quantize_rows(fp32 -> %s, 2 M rows x 128)" % name, src.numel() * 4 + out.numel(), ms, None,
              {"rows_per_s": rows / ms * 1e3})
        if ty == cabi.INT8:
            back = torch.empty_like(src)
            ms, _ = time_launches(lambda: cabi.dequantize_rows(out, D, ty, 16, True, out=back), max(5, iters // 2), flush)
            entry("dequantize_rows(INT8 -> fp32, 2 M rows x 128)", out.numel() + back.numel() * 4, ms, None,
                  {"rows_per_s": rows / ms * 1e3})
            del back
        del out
    del src


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
    fn = lambda: cabi.nbit_forward(Wq, wo, tys, Do, T * D, D, idx, offs, B, table_types=(cabi.INT8, cabi.INT4))
    fn()
    ms, _ = time_launches(fn, max(5, iters // 2), flush)
    bytes_ = row_bytes + inp.num_lookups * 8 + (T * B + 1) * 8 + B * T * D * 2
    entry("tbe_nbit_forward(config4)", bytes_, ms, inp.num_lookups, {"unique_rows": int(sum(U_by_table))})


# --------------------------------------------------------------------------------------------
# Parity of the bench step itself (sampled, against the CPU oracle) and of the exchange (bitwise,
# against NCCL's all-to-all). Runs once before the timed region; a mismatch ends the run.
# --------------------------------------------------------------------------------------------
def parity_checks(step, dist):
    import oracle
    from tests import sampled_parity

    T, E, D, B = step.T, step.E, step.D, step.B
    tables = sorted({0, T // 3, (2 * T) // 3, T - 1})
    checks = {}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rows = torch.full((T,), E, dtype=torch.int64, device="cuda")
    # the lookup of this rank's tables for the whole batch, as a local matrix
    pooled = cabi.forward(step.weights, step.weights_offsets, step.D_offsets, step.total_D, D, step.indices,
                          step.offsets, B, output_dtype=torch.float16, rows_per_table=rows, status=status)
    n_bags = 0
    for t in tables:
        g = torch.Generator().manual_seed(900 + t)
        bags = torch.sort(torch.randperm(B, generator=g)[:64]).values
        # fp16 pooled rows: the north-star tolerance plus the rounding of the stored value
        n_bags += sampled_parity.forward_sample_check(step.weights, D, t * E * D, t * D, D, oracle.FP16,
                                                      step.indices, step.offsets, B, t, pooled, bags, 2e-3, 1e-3)
    checks["forward_vs_oracle"] = "ok: %d sampled bags of tables %s" % (n_bags, tables)
    if step.exchange is not None:
        from torchlib_xpu_b200 import sharded
        step.forward()                                   # the fused lookup + peer stores + barrier
        ref = sharded.reference_exchange(pooled)         # NCCL all_to_all_single of the local matrix
        torch.cuda.synchronize()
        if not torch.equal(ref, step.exchange.recv):
            raise SystemExit("parity: the fused exchange differs from the all-to-all of the local lookups")
        checks["exchange_vs_all_to_all"] = "ok: bitwise, %d x %d" % tuple(ref.shape)
        del ref
    del pooled
    samples = [sampled_parity.BackwardSample(step.weights, t * E * D, D, oracle.FP16, step.momentum, t * E,
                                             step.indices, step.offsets, B, t, hot=16, extra=240, seed=t)
               for t in tables]
    if step.exchange is not None:
        from torchlib_xpu_b200 import sharded
        want = sharded.reference_gradient_exchange(step.exchange.grad_slice)
    step.backward()
    torch.cuda.synchronize()
    grad = step.grad if step.exchange is None else step.exchange.grad_local
    if step.exchange is not None:
        if not torch.equal(want, grad):
            raise SystemExit("parity: the gradient push differs from the all-to-all of the gradient slices")
        checks["gradient_push_vs_all_to_all"] = "ok: bitwise, %d x %d" % tuple(want.shape)
        del want
    n_rows = 0
    for t, smp in zip(tables, samples):
        n_rows += smp.check(step.weights, step.momentum, grad, t * D, oracle.ROWWISE_ADAGRAD, 0.01, 1e-8)
    checks["backward_vs_oracle"] = ("ok: %d sampled rows (16 hottest + 240 touched per table), longest run %d "
                                    "lookups" % (n_rows, max(smp.max_run for smp in samples)))
    if int(status.item()) != 0:
        raise SystemExit("parity: device status %d" % int(status.item()))
    if dist is not None:
        flag = torch.ones(1, device="cuda")
        dist.all_reduce(flag)                            # every rank got here
        checks["ranks_checked"] = int(flag.item())
    return checks


# --------------------------------------------------------------------------------------------
# End to end: the loop a trainer with host-side batches runs. Ids, offsets and gradients come from
# pinned host memory every step and the pooled rows go back to the host every step; the copies run
# on side streams (the next step's ids while this step computes, the gradients under the forward,
# the result under the backward) and every one of them is inside the timed region.
# One GPU: through the operator library, torch.ops.fbgemm.split_embedding_codegen_lookup_rowwise_
# adagrad_function and autograd's backward (the plugin call a user makes). Sharded: the lookup that
# scatters into the peers' buffers has no fbgemm operator, so the step stays on the C ABI.
# --------------------------------------------------------------------------------------------
def end_to_end(step, dist, world, args, lookups_all, idx_dtype, barrier):
    T, E, D, B = step.T, step.E, step.D, step.B
    h_idx = step.indices.to(idx_dtype).cpu().pin_memory()
    h_off = step.offsets.to(idx_dtype).cpu().pin_memory()
    grad_in = step.grad if step.exchange is None else step.exchange.grad_slice
    h_grad = grad_in.cpu().pin_memory()
    h_out = torch.empty(step.result().shape, dtype=step.result().dtype).pin_memory()
    # whole-job bytes: every rank copies its own inputs and its own slice of the result
    h2d = (h_idx.numel() * h_idx.element_size() + h_off.numel() * h_off.element_size() +
           h_grad.numel() * h_grad.element_size()) * world
    d2h = h_out.numel() * h_out.element_size() * world
    main = torch.cuda.current_stream()
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    idx_bufs = [torch.empty(step.N, dtype=idx_dtype, device="cuda") for _ in range(2)]
    off_bufs = [torch.empty(T * B + 1, dtype=idx_dtype, device="cuda") for _ in range(2)]
    keep = (step.indices, step.offsets)
    pipe = {"k": 0, "bwd_done": None, "out_done": None}
    module = None
    if step.exchange is None:
        from torchlib_xpu_b200 import tbe_modules as tm
        module = tm.SplitTableBatchedEmbeddingBagsCodegen(
            [(E, D)] * T, tm.OptimType.EXACT_ROWWISE_ADAGRAD, 0.01, 1e-8, tm.PoolingMode.SUM,
            tm.SparseType.FP16, tm.SparseType.FP16, weights_dev=step.weights, momentum1_dev=step.momentum)

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
        main.wait_event(in_ready)
        if module is not None:
            pooled = module(idx, off)                  # torch.ops.fbgemm.* forward: allocates its result
            fwd_done.record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(fwd_done)
                h_out.copy_(pooled, non_blocking=True)
                out_done.record(copy_out)
            pooled.record_stream(copy_out)
            main.wait_event(grad_ready)
            pooled.backward(grad_in)                   # the fused backward + Adagrad, through autograd
        else:
            step.indices, step.offsets = idx, off
            step.forward()
            fwd_done.record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(fwd_done)
                h_out.copy_(step.result(), non_blocking=True)
                out_done.record(copy_out)
            main.wait_event(grad_ready)
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
    step.indices, step.offsets = keep
    return {"value": lookups_all / (e2e_ms / e2e_steps / 1e3), "unit": "lookups/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps,
            "steps": e2e_steps, "ids": str(idx_dtype).replace("torch.", ""),
            "through": ("torch.ops.fbgemm.split_embedding_codegen_lookup_rowwise_adagrad_function + autograd "
                        "(libb200tbe_torch_ops.so)" if module is not None else
                        "b200tbe_forward / b200tbe_exchange_push / b200tbe_backward (C ABI; the sharded lookup "
                        "has no fbgemm operator)")}


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
    ap.add_argument("--only", default=None, choices=["jagged", "fp32", "train", "uniform", "nbit", "quantize", "nv12", "permute", "step"],
                    help="run one single-GPU configuration alone (few launches; for profiler captures); "
                         "'step' is the bench step itself cut to --tables tables (default 2)")
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
    if args.only == "step":
        # the bench step on a few tables: --iters backwards, then --iters forwards (same kernels, same
        # per-table sizes as the full step; small enough for full-metric profiler captures)
        small_cfg = dict(cfg, T_per_gpu=args.tables or 2)
        st = ShardedTbeStep(0, 1, small_cfg)
        bwd_ms, _ = time_launches(st.backward, args.iters)
        fwd_ms, _ = time_launches(st.forward, args.iters)
        print(json.dumps({"only": "step", "tables": st.T, "lookups": st.N, "unique_rows": st.U,
                          "backward_ms": bwd_ms, "forward_ms": fwd_ms}), file=json_out, flush=True)
        return
    if args.only is not None:
        global TABLES_OVERRIDE
        TABLES_OVERRIDE = args.tables
        print(json.dumps({"only": args.only, "peak_gbs": peak_gbs,
                          "results": bench_others(peak_gbs, args.iters, args.only)}), file=json_out, flush=True)
        return

    step = ShardedTbeStep(rank, world, cfg, small=args.small)
    if args.tables is not None:
        raise SystemExit("--tables goes with --only")

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- parity of this very workload, before anything is timed -----------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    checks = parity_checks(step, dist)
    barrier()

    sampler.mark_load()
    for _ in range(args.warmup):
        step.step()
    barrier()

    # ---- device-resident timing: exactly K steps between barriers -------------------------
    fwd_ms, bwd_ms = [], []
    barrier()
    sampler.mark_timed()
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

    # ---- the gradient push alone (N > 1): bytes that cross NVLink / device time ---------------
    nvlink = None
    if step.exchange is not None:
        ex = step.exchange
        times = []
        for _ in range(5):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            ex.push_gradients()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
            ex.barrier()
        push_ms = float(np.median(times))
        t = torch.tensor([push_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        push_ms = float(t.item())
        out_bytes = ex.grad_slice.numel() * ex.grad_slice.element_size() * (world - 1) // world
        nvlink = {"bound": "nvlink", "kernel": "exchange_push_kernel (gradient blocks to their owners)",
                  "bytes_out_per_rank": out_bytes, "ms": push_ms, "achieved": out_bytes / push_ms / 1e6,
                  "peak": 770.0, "unit": "GB/s", "frac": out_bytes / push_ms / 1e6 / 770.0,
                  "peak_kind": "of the peer-copy bandwidth measured on this pool (770 GB/s per direction; "
                               "900 nominal)",
                  "forward_note": "the pooled rows cross NVLink inside the lookup kernel (same bytes the "
                                  "other way); phases_ms.forward includes them"}

    # ---- end to end: host buffers in, pooled rows out, every step ---------------------------
    e2e = {}
    for label, idx_dtype in (("int64_ids", torch.int64), ("int32_ids", torch.int32)):
        e2e[label] = end_to_end(step, dist, world, args, lookups_all, idx_dtype, barrier)
    torch.cuda.empty_cache()

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
        "e2e": e2e["int64_ids"],
        "e2e_int32_ids": e2e["int32_ids"],
        "checks": checks,
        "gpu_launches": step.launches_per_step() * args.steps,
        "phases_ms": {"forward": fwd_avg, "backward": bwd_avg},
    }
    # roofline of the dominant part of the step (the backward's kernel group) and of the forward
    # kernel; algorithmic bytes = compulsory traffic (distinct rows once)
    bwd_bytes, fwd_bytes = step.bwd_bytes(), step.fwd_bytes()
    line["roofline"] = {
        "bound": "hbm", "kernel": "b200tbe_backward (linearize + radix sort + segment + reduce/update)",
        "achieved": bwd_bytes / bwd_avg / 1e6, "peak": peak_gbs, "unit": "GB/s",
        "frac": bwd_bytes / bwd_avg / 1e6 / peak_gbs,
        "traffic": None if BWD_TRAFFIC_PER_TABLE is None else BWD_TRAFFIC_PER_TABLE * step.T,
        "traffic_note": TRAFFIC_NOTE, "peak_kind": "of " + peak_kind, "algorithmic_bytes": bwd_bytes,
    }
    line["roofline_forward"] = {
        "bound": "hbm", "kernel": "tbe_forward_bag_groups_kernel", "achieved": fwd_bytes / fwd_avg / 1e6,
        "peak": peak_gbs, "unit": "GB/s", "frac": fwd_bytes / fwd_avg / 1e6 / peak_gbs,
        "traffic": None if FWD_TRAFFIC_PER_TABLE is None else FWD_TRAFFIC_PER_TABLE * step.T,
        "traffic_note": TRAFFIC_NOTE, "peak_kind": "of " + peak_kind, "algorithmic_bytes": fwd_bytes,
    }
    if nvlink is not None:
        line["roofline_nvlink"] = nvlink

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
