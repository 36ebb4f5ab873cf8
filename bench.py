"""Benchmark of the block-scaled quantized products on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline workload (BASELINE.json configs[4] at M = 1): the Q4_0 gemv of a 28672 x 8192 weight matrix (18-byte blocks)
against x f32[8192], the matrix sharded by output rows over the N ranks (strong scaling: the work is one matrix whatever
N is) and every rank ending up with the whole y f32[28672].  At N = 1 that is the plain gemv; at N > 1 each rank's
kernel stores its slice into every peer's copy of y (peer-mapped memory over NVLink) and a bounded wait on the peers'
flags follows it (qb200_shard_gemv / qb200_shard_wait).  The metric is algorithmic bytes per second of the whole
product: (weight blocks + x + y) bytes x launches / time, max over ranks.

A launch sequence = one pass over LAYERS distinct seeded weight matrices (LAYERS x shard > 2 x L2, so every launch reads
its weights from HBM), captured once as a CUDA graph.  One STEP = REPLAYS replays of that graph, timed with its own pair
of CUDA events on the launching stream; the timed region is exactly --steps steps and the line also carries the median,
fastest and slowest step.

Beside the headline the JSON line carries: `local` (the same sharded product without the exchange) and, at N > 1,
`with_allgather` (slices joined by NCCL instead); `c2` (BASELINE configs[1], Q4_0 8192 x 8192, every rank its own
matrices: calls independent of one another and calls chained through y); `configs` (the other gemv configurations, N = 1);
`abt` (the Q8_0 x Q8_0 A.B^T of configs[2] and the Q4_0-weight product of configs[4], N = 1); `abt_sharded` (N > 1: the
configs[4] A.B^T with B's rows over the ranks: column blocks alone, with the exchange inside the product kernel, with an NCCL
all-gather); `e2e` (the headline product
through the host-buffer C-ABI call: pinned host operands, H2D + kernel + D2H every call); `roofline`; `cpu_baseline` (the C
restatement of the reference's CPU gemv on this machine's host cores).  `--impl reference` times only that CPU
restatement (the reference itself is C#/.NET and cannot run here).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from qiyas_b200 import blocks as B  # noqa: E402

FMT_A, FMT_X = B.Q4_0, B.F32
N5, K5 = 28672, 8192                                      # configs[4]: the 70B-class FFN up-projection
WEIGHT5 = N5 * (K5 // 32) * 18
ALGO5 = WEIGHT5 + K5 * 4 + N5 * 4                         # weights once, x, y
REPLAYS = 100                                             # graph replays a step
L2_BYTES = 126e6
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the gemv on the headline matrix (ncu, profiles/): 132 225 536
# bytes read, nothing written that the kernel caused (y stays in L2), against 132 268 032 algorithmic; a rank's shard at
# N > 1 is taken at the same ratio (the kernel reads every byte of its rows once; 8192 x 8192: 37 852 928 against 37 814 272)
TRAFFIC_RATIO = 132225536 / 132268032
MMA_OPS = 2 * 128 * 128 * 32                              # int8 operations of one tcgen05.mma of the product's shape


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons of one GPU, read through NVML every millisecond or so while the timed region runs
    (reading only; `nvidia-smi -lms` as a fallback when the NVML binding is missing)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.sm, self.mx, self.reasons, self.rows = [], [], set(), []
        self.proc, self.nvml, self.running = None, None, True
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible:                     # NVML counts the machine's GPUs, CUDA the visible ones
                entry = visible.split(",")[index].strip()
                handle = pynvml.nvmlDeviceGetHandleByUUID(entry) if entry.startswith("GPU-") else pynvml.nvmlDeviceGetHandleByIndex(int(entry))
            else:
                handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nvml, self.handle = pynvml, handle
            self.mx.append(float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        masks = [(n.nvmlClocksThrottleReasonHwSlowdown, "hw_slowdown"), (n.nvmlClocksThrottleReasonHwThermalSlowdown, "hw_thermal_slowdown"),
                 (n.nvmlClocksThrottleReasonSwThermalSlowdown, "sw_thermal_slowdown"), (n.nvmlClocksThrottleReasonSwPowerCap, "sw_power_cap")]
        while self.running:
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for mask, name in masks:
                    if bits & mask:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.001)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nvml is not None:
            self.running = False
            self.thread.join(timeout=1)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": max(self.mx) if self.mx else None,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "via": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, r[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "via": "nvidia-smi"}


WORKLOAD = f"Q4_0 gemv {N5}x{K5} (BASELINE configs[4], M 1), x f32 -> Q8_0, sharded by output rows over the ranks, whole y on every rank"


def layers_for(shard_bytes):
    """Distinct weight matrices a pass rotates over: more than twice L2 in all."""
    return int(max(2, min(40, -(-2.2 * L2_BYTES // max(1, shard_bytes)))))


# ---------------------------------------------------------------------------------------------------------- the CPU arm

def cpu_gemv(seconds, layers):
    """The reference's CPU block gemv (src/BlockProducts.cs:17-71) as restated in oracle/, on all host threads, over the
    same rotation of `layers` matrices as the GPU arm; both integer-dot lanes, the faster one reported."""
    from oracle import qiyas_oracle as O
    ws = [B.make_weights(FMT_A, N5, K5, 1000 + i) for i in range(layers)]
    x = B.make_activations(K5, 2000)
    out = {}
    for variant, name in ((0, "plain integer loop (the reference's 's32 blocks' lane)"), (1, "AVX2 multiply-adds + F16C (standing in for its 's8dp blocks' lane)")):
        if not O.set_dot_variant(variant):
            continue
        for w in ws:
            O.time_gemv_blocks(FMT_A, FMT_X, w, x, N5, K5, 1)               # warm the team and the pages
        one = O.time_gemv_blocks(FMT_A, FMT_X, ws[0], x, N5, K5, 1)
        passes = max(1, min(200, int(seconds / 2 / max(one * layers, 1e-6))))
        t0 = time.perf_counter()
        for _ in range(passes):
            for w in ws:
                O.time_gemv_blocks(FMT_A, FMT_X, w, x, N5, K5, 1)
        per_call = (time.perf_counter() - t0) / (passes * layers)
        out[variant] = {"GBs": ALGO5 / per_call / 1e9, "ms_per_call": per_call * 1e3, "calls": passes * layers, "lane": name}
    O.set_dot_variant(0)
    best = max(out, key=lambda v: out[v]["GBs"])
    base = {"value": out[best]["GBs"], "unit": "GB/s", "cores": O.threads(), "kind": "port",
            "sample": f"{out[best]['calls']} calls of the {N5}x{K5} Q4_0 gemv (x f32 -> Q8_0) over {layers} matrices in rotation, "
                      f"{out[best]['ms_per_call']:.3f} ms each; C restatement of Kernels.GemvBlocks on the thread team, {out[best]['lane']}",
            "variants": {str(v): out[v] for v in out}}
    return base, out[best]["ms_per_call"] * 1e-3


def run_reference(args, rank):
    if rank != 0:
        return
    t0 = time.time()
    layers = layers_for(WEIGHT5)
    base, per_call = cpu_gemv(max(4.0, min(24.0, 1.2 * (args.steps + args.warmup))), layers)
    line = {"impl": "reference", "metric": "quant gemv HBM GB/s", "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_call * 1e3 * layers * REPLAYS, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "s8 dot / f32 scale", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers_per_pass": layers, "cpu": "one matrix a call on all host threads; a step is a bounded sample of the GPU arm's step"},
            "cpu_baseline": base, "gpu_launches": 0,
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.time() - t0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------- GPU helpers

class Timer:
    """Steps of REPLAYS graph replays on a side stream, each step between its own pair of events."""

    def __init__(self, torch, dist, world, dev, stream):
        self.torch, self.dist, self.world, self.dev, self.stream = torch, dist, world, dev, stream

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def run(self, replay, steps, warmup, replays=REPLAYS):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                for _ in range(replays):
                    replay()
        self.barrier()
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        self.barrier()
        with torch.cuda.stream(self.stream):
            for e0, e1 in events:
                e0.record()
                for _ in range(replays):
                    replay()
                e1.record()
        self.barrier()
        per_step = [e0.elapsed_time(e1) for e0, e1 in events]
        total = events[0][0].elapsed_time(events[-1][1])           # exactly `steps` steps, first start to last end
        t = torch.tensor([total] + per_step, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        t = t.cpu().numpy()
        return float(t[0]), [float(v) for v in t[1:]]


def capture(torch, stream, launch):
    with torch.cuda.stream(stream):
        launch(stream)                                  # once outside the capture: first-use set-up must not be captured
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            launch(stream)
    return graph


def stats(total_ms, per_step, launches_per_step, bytes_per_launch, peak):
    per_launch = total_ms * 1e-3 / (len(per_step) * launches_per_step)
    med = float(np.median(per_step)) * 1e-3 / launches_per_step
    return {"us_per_launch": per_launch * 1e6, "GBs": bytes_per_launch / per_launch / 1e9, "pct_of_measured_hbm": 100 * bytes_per_launch / per_launch / 1e9 / peak,
            "median_step_us_per_launch": med * 1e6, "fastest_step_us_per_launch": min(per_step) * 1e3 / launches_per_step,
            "slowest_step_us_per_launch": max(per_step) * 1e3 / launches_per_step}


def gemv_record(ops, torch, timer, fmt, rows, cols, steps, warmup, peak, chained=False, seed=100):
    """One gemv configuration on this rank's GPU: `layers` matrices in rotation, calls independent of one another or (square
    matrices) chained, each call's y the next call's x."""
    bytes_w = B.nbytes(fmt, rows * cols)
    layers = layers_for(bytes_w)
    ws = [torch.from_numpy(B.make_weights(fmt, rows, cols, seed + i)).to(timer.dev) for i in range(layers)]
    x = torch.from_numpy(B.make_activations(cols, seed + 50)).to(timer.dev)
    ys = [torch.empty(rows, dtype=torch.float32, device=timer.dev) for _ in range(layers)]

    def launch(stream):
        for i, w in enumerate(ws):
            src = ys[i - 1] if (chained and i) else (ys[-1] if chained else x)
            ops.GemvBlocks(fmt, w, src, ys[i], rows, cols, fmt_x=B.F32, stream=stream)

    if chained:
        ys[-1].copy_(x)                                  # the chain needs a finite start; values decay or grow, the time does not care
    graph = capture(torch, timer.stream, launch)
    total, per_step = timer.run(graph.replay, steps, warmup, replays=max(10, REPLAYS * 3 // layers))
    algo = bytes_w + cols * 4 + rows * 4
    out = stats(total, per_step, layers * max(10, REPLAYS * 3 // layers), algo, peak)
    out.update({"shape": f"{B.NAMES[fmt]} {rows}x{cols}", "layers": layers, "calls": "chained through y" if chained else "independent"})
    return out


def tensor_peak(ops, clock_mhz):
    """Dense int8 peak from the measured rate of the product's own tensor instruction (qb200_tensor_rate), at the max SM clock."""
    cycles = C.c_double(0.0)
    ops.gpu.check(ops.lib.qb200_tensor_rate(C.byref(cycles)), "tensor_rate")
    if cycles.value <= 0:
        return None, None
    return MMA_OPS / cycles.value * ops.gpu.caps.sm_count * clock_mhz * 1e6 / 1e12, cycles.value


def abt_record(ops, torch, timer, fmt_b, m, n, k, peak_measured):
    """A.B^T with Q8_0 activations: operands re-laid on every call, and weights prepacked once."""
    dev = timer.dev
    a = torch.from_numpy(B.make_weights(B.Q8_0, m, k, 5000)).to(dev)
    b = torch.from_numpy(B.make_weights(fmt_b, n, k, 5001)).to(dev)
    c = torch.empty(m * n, dtype=torch.float32, device=dev)
    need = ops.workspace_bytes(B.Q8_0, m, n, k, fmt_b=fmt_b)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    packed = ops.Prepack(fmt_b, b, n, k)
    need_a = int(ops.lib.qb200_matmul_prepacked_workspace_bytes(B.Q8_0, fmt_b, m, k))
    ws_a = torch.empty(need_a, dtype=torch.uint8, device=dev)

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / reps

    every = timed(lambda: ops.MatMulBlocks(B.Q8_0, a, b, c, m, n, k, fmt_b=fmt_b, workspace=ws, workspace_bytes=need))
    pre = timed(lambda: ops.MatMulBlocksPrepacked(B.Q8_0, a, packed, c, m, n, k, fmt_b=fmt_b, workspace=ws_a, workspace_bytes=need_a))
    ops_count = 2.0 * m * n * k
    return {"shape": f"Q8_0 x {B.NAMES[fmt_b]}  M {m} N {n} K {k}", "us_packed_every_call": every * 1e6, "us_weights_prepacked": pre * 1e6,
            "int8_TOPS": ops_count / pre / 1e12, "int8_TOPS_packed_every_call": ops_count / every / 1e12,
            "frac_of_nominal_4500": ops_count / pre / 1e12 / 4500.0,
            "frac_of_measured_mma_rate": ops_count / pre / 1e12 / peak_measured if peak_measured else None}


def abt_sharded_record(ops, torch, dist, timer, plan, rank, world, dev, shard, m):
    """The sharded A.B^T of the headline matrix at N > 1: rank r's rows of B give its column block of C.  Timed three ways
    (CUDA events around the calls, barrier on both sides, max over ranks; the first two as replayed CUDA graphs): the column block alone; with the exchange
    inside the product kernel (every rank ends with the whole C); and joined by an NCCL all-gather instead."""
    from qiyas_b200.shard import PeerExchange, ShardedMatMul, all_gather_columns
    n_local = plan.count(rank)
    a = torch.from_numpy(B.make_weights(B.Q8_0, m, K5, 4100 + m)).to(dev)
    mm = ShardedMatMul(ops, plan, rank, FMT_A, K5, shard)
    packed = ops.Prepack(FMT_A, shard, n_local, K5)
    c_slice = torch.empty(m * max(n_local, 1), dtype=torch.float32, device=dev)
    ex, exg = PeerExchange(ops, m * N5, rank, world), PeerExchange(ops, m * N5, rank, world)
    try:
        def local():
            ops.MatMulBlocksPrepacked(B.Q8_0, a, packed, c_slice, m, n_local, K5, fmt_b=FMT_A)

        def fused():
            return mm.exchange(B.Q8_0, a, m, ex, b_packed=packed)

        def fused_counted(stream):
            # epochs counted on the device (0): the form a captured graph can replay
            rc = ops.lib.qb200_shard_matmul(B.Q8_0, FMT_A, a.data_ptr(), None, packed.data_ptr(), m, N5, K5, C.byref(exg.peers), 0, None, 0,
                                            stream.cuda_stream)
            ops.gpu.check(rc, "shard_matmul")
            ops.gpu.check(ops.lib.qb200_shard_wait(C.byref(exg.peers), 0, 0, stream.cuda_stream), "shard_wait")

        def gathered():
            local()
            return all_gather_columns(plan, rank, c_slice, m)
        whole = fused()
        joined = gathered()
        torch.cuda.synchronize()
        if ops.gpu.status() != 0 or not torch.equal(whole.view(torch.int32), joined.view(torch.int32)):
            raise SystemExit(f"sharded A.B^T check failed on rank {rank}: C after the exchange differs from the gathered column blocks")
        rec = {"shape": f"Q8_0 x {B.NAMES[FMT_A]}  M {m} N {N5} K {K5}, B's rows over {world} ranks (weights prepacked)"}
        # each form as a CUDA graph of one product where it can be captured (small products are otherwise timed at the rate
        # the host can launch them), replayed on the side stream; the all-gather form is host-launched.  The captured
        # exchange counts its epochs on the device, so it has an exchange of its own (the two numberings do not mix).
        side = timer.stream
        graphs = {}
        try:
            graphs["local"] = capture(torch, side, lambda st: ops.MatMulBlocksPrepacked(B.Q8_0, a, packed, c_slice, m, n_local, K5, fmt_b=FMT_A, stream=st))
            graphs["with_exchange"] = capture(torch, side, fused_counted)
        except Exception as e:                     # noqa: BLE001 (a failed capture leaves the host-launched loop)
            graphs = {}
            rec["capture"] = f"not captured: {type(e).__name__}"
        torch.cuda.synchronize()
        dist.barrier()
        rec["launch"] = {k: ("one CUDA graph of a product, replayed" if k in graphs else "host-launched") for k in ("local", "with_exchange", "with_allgather")}
        for name, fn, reps in (("local", local, 20), ("with_exchange", fused, 20), ("with_allgather", gathered, 10)):
            graph = graphs.get(name)
            stream = side if graph is not None else torch.cuda.current_stream()
            if graph is not None:
                fn, reps = graph.replay, 40
            with torch.cuda.stream(stream):
                for _ in range(3):
                    fn()
            timer.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                e0.record()
                for _ in range(reps):
                    fn()
                e1.record()
            timer.barrier()
            t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item()) * 1e3 / reps
            rec[name] = {"us": us, "int8_TOPS": 2.0 * m * N5 * K5 / us / 1e6}
        if graphs:
            torch.cuda.synchronize()
            if not torch.equal(exg.y()[:m * N5].view(torch.int32), joined.reshape(-1).view(torch.int32)):
                raise SystemExit(f"sharded A.B^T check failed on rank {rank}: C after the replayed exchange differs from the gathered column blocks")
        if ops.gpu.status() != 0:
            raise SystemExit("a kernel gave up on a bounded wait: the timing is void")
        rec["exchange"] = "peer stores from the product kernel's epilogue + flags + bounded wait"
        rec["c_bytes_stored_to_each_peer"] = m * n_local * 4
        return rec
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        ex.close()
        exg.close()


def abt_cpu_baseline(seconds=8.0):
    """The reference's CPU tile product (src/MatMulBlocks.cs:28-36, 84-169) as restated in oracle/, on a reduced configs[2]."""
    from oracle import qiyas_oracle as O
    m, n, k = 512, 2048, 4096
    a = B.make_weights(B.Q8_0, m, k, 5000)
    b = B.make_weights(B.Q8_0, n, k, 5001)
    O.matmul_blocks(B.Q8_0, B.Q8_0, a, b, m, n, k, order=0)
    t0, calls = time.perf_counter(), 0
    while time.perf_counter() - t0 < seconds and calls < 50:
        O.matmul_blocks(B.Q8_0, B.Q8_0, a, b, m, n, k, order=0)
        calls += 1
    s = (time.perf_counter() - t0) / calls
    return {"value": 2.0 * m * n * k / s / 1e12, "unit": "int8 TOP/s", "cores": O.threads(), "kind": "port",
            "sample": f"{calls} calls of Q8_0 x Q8_0 M {m} N {n} K {k} (configs[2] with N reduced from 11008), {s * 1e3:.1f} ms each; "
                      "C restatement of Kernels.MatMulBlocks (unpack both operands, 4 x 2 tile, scalar integer dots) on the thread team"}


# ---------------------------------------------------------------------------------------------------------- main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-extra", action="store_true", help="only the headline (profiling runs)")
    ap.add_argument("--leg", default=None, choices=["c2", "c2-chained", "abt", "abt-few"],
                    help="run one small leg alone and print its record (profiling runs): the Q4_0 8192 x 8192 gemv with calls chained "
                         "through y, or the Q8_0 x Q8_0 A.B^T of configs[2] at M 512")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from qiyas_b200.ops import GpuOps
    from qiyas_b200.shard import PeerExchange, ShardedGemv, ShardPlan, all_gather_rows

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    ops = GpuOps(device=local)
    dev = f"cuda:{local}"
    side = torch.cuda.Stream(device=dev)
    timer = Timer(torch, dist, world, dev, side)
    peak, peak_kind = measured_peaks()
    if args.leg:
        if args.leg in ("c2", "c2-chained"):
            rec = gemv_record(ops, torch, timer, B.Q4_0, 8192, 8192, 3, 3, peak, chained=args.leg == "c2-chained")
        else:
            rec = abt_record(ops, torch, timer, B.Q8_0, 512 if args.leg == "abt" else 16, 11008, 4096, tensor_peak(ops, 1965.0)[0])
        if rank == 0:
            print(json.dumps({"leg": args.leg, "record": rec}), flush=True)
        return

    # ---- the rank's shard of every layer's matrix, x, and its copy of y
    plan = ShardPlan(N5, world)
    rows = plan.count(rank)
    shard_bytes = rows * (K5 // 32) * 18
    layers = layers_for(shard_bytes)
    host_shards = [B.make_weights(FMT_A, rows, K5, 1000 + 131 * rank + i) for i in range(layers)]
    host_x = B.make_activations(K5, 2000)
    shards = [torch.from_numpy(w).to(dev) for w in host_shards]
    x = torch.from_numpy(host_x).to(dev)
    exchange = PeerExchange(ops, N5, rank, world)
    y_full = exchange.y()
    first = plan.range(rank)[0]
    y_slice = y_full[first:first + rows]
    gemvs = [ShardedGemv(ops, plan, rank, FMT_A, K5, w) for w in shards]
    # without the exchange every layer writes a slice of its own (the calls are then independent of one another, as the
    # layers of a model are); with it all layers publish into the one whole y every rank holds
    y_locals = [y_slice] + [torch.empty(max(rows, 1), dtype=torch.float32, device=dev)[:rows] for _ in range(layers - 1)]

    def launch_local(stream):
        for g, y in zip(gemvs, y_locals):
            g.local(x, y, fmt_x=FMT_X, stream=stream)

    def launch_exchange(stream):
        for g in gemvs:
            rc = ops.lib.qb200_shard_gemv(g.fmt, FMT_X, g.w.data_ptr(), x.data_ptr(), N5, K5, C.byref(exchange.peers), 0, stream.cuda_stream)
            ops.gpu.check(rc, "shard_gemv")
            ops.gpu.check(ops.lib.qb200_shard_wait(C.byref(exchange.peers), 0, 0, stream.cuda_stream), "shard_wait")

    # ---- one pass checked before anything is timed: the rank's own rows against the oracle, and (N > 1) the whole y on
    # every rank against the slices the ranks computed
    from oracle import qiyas_oracle as O
    with torch.cuda.stream(side):
        (launch_exchange if world > 1 else launch_local)(side)
        side.synchronize()
    if ops.gpu.status() != 0:
        raise SystemExit("a kernel gave up on a bounded wait during the check pass")
    pick = np.unique(np.concatenate([[0, rows - 1], np.random.default_rng(rank).integers(0, rows, 6)])) if rows else np.array([], np.int64)
    xq = O.decode(B.Q8_0, O.encode(B.Q8_0, host_x), K5)
    rb = B.row_bytes(FMT_A, K5)
    got = y_full.cpu().numpy()
    for r in pick:
        want = float(O.gemv_f64(FMT_A, host_shards[-1 if world > 1 else 0].reshape(rows, rb)[r], xq, 1, K5)[0])
        if abs(float(got[first + r]) - want) > 1e-4 * max(1.0, abs(want)):
            raise SystemExit(f"bench output check failed on rank {rank}: row {first + r} = {got[first + r]}, float64 says {want}")
    if world > 1:
        joined = all_gather_rows(plan, rank, y_slice.clone())
        if not torch.equal(joined.view(torch.int32), y_full.view(torch.int32)):
            raise SystemExit(f"bench exchange check failed on rank {rank}: y after the exchange differs from the ranks' own slices")

    # ---- the headline: the sharded product with the exchange (N = 1: the plain product)
    graph_local = capture(torch, side, launch_local)
    graph_head = capture(torch, side, launch_exchange) if world > 1 else graph_local
    launches_per_step = layers * REPLAYS
    sampler = ClockSampler(local)
    total_ms, per_step = timer.run(graph_head.replay, args.steps, args.warmup)
    clocks = sampler.stop()
    if ops.gpu.status() != 0:
        raise SystemExit("a kernel gave up on a bounded wait: the timing is void")
    head = stats(total_ms, per_step, launches_per_step, ALGO5, peak)
    value = ALGO5 * args.steps * launches_per_step / (total_ms * 1e-3) / 1e9
    rank_algo = shard_bytes + K5 * 4 + rows * 4                       # what one rank's launch reads and writes
    per_launch_s = total_ms * 1e-3 / (args.steps * launches_per_step)

    extra_steps = max(3, min(args.steps, 7))
    local_rec = None
    if world > 1 and not args.no_extra:
        t, ps = timer.run(graph_local.replay, extra_steps, 3)
        local_rec = stats(t, ps, launches_per_step, ALGO5, peak)
        local_rec["note"] = "every rank its slice only, no exchange"

    gather_rec = None
    if world > 1 and not args.no_extra:
        y_tmp = torch.empty(N5, dtype=torch.float32, device=dev)
        reps = 40

        def gather_pass():
            for g in gemvs:
                g.local(x, y_slice, fmt_x=FMT_X)
                all_gather_rows(plan, rank, y_slice, out=y_tmp)
        for _ in range(2):
            gather_pass()
        timer.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            gather_pass()
        e1.record()
        timer.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        s = float(t.item()) * 1e-3 / (reps * layers)
        gather_rec = {"us_per_launch": s * 1e6, "GBs": ALGO5 / s / 1e9, "note": "slices joined by ncclAllGather, host-launched (not graph-replayed)"}

    # ---- end to end: the host-buffer call (pinned operands up, kernel, y down) on the rank's shard, every call
    e2e = None
    if not args.no_e2e and rows:
        pinned_w = [torch.from_numpy(w).pin_memory() for w in host_shards[:2]]
        pinned_x = torch.from_numpy(host_x).pin_memory()
        pinned_y = torch.empty(rows, dtype=torch.float32).pin_memory()
        wn, xn, yn = [p.numpy() for p in pinned_w], pinned_x.numpy(), pinned_y.numpy()
        calls = max(4, min(4 * args.steps, 24))
        for i in range(2):
            ops.GemvBlocksHost(FMT_A, wn[i % 2], xn, yn, rows, K5, fmt_x=FMT_X)
        timer.barrier()
        t0 = time.perf_counter()
        for i in range(calls):
            ops.GemvBlocksHost(FMT_A, wn[i % 2], xn, yn, rows, K5, fmt_x=FMT_X)
        torch.cuda.synchronize()
        e_s = time.perf_counter() - t0
        et = torch.tensor([e_s], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(et, op=dist.ReduceOp.MAX)
        e_s = float(et.item())
        dst = torch.empty(shard_bytes, dtype=torch.uint8, device=dev)
        dst.copy_(pinned_w[0], non_blocking=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(4):
            dst.copy_(pinned_w[i % 2], non_blocking=True)
        torch.cuda.synchronize()
        h2d_gbs = 4 * shard_bytes / (time.perf_counter() - t0) / 1e9
        # a step of this leg = `launches_per_step` host-buffer calls; the figure is per call, the bytes per step follow
        e2e = {"value": ALGO5 * calls / e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": launches_per_step * (shard_bytes + K5 * 4),
               "d2h_bytes_per_step": launches_per_step * rows * 4, "calls_timed": calls, "ms_per_call": e_s * 1e3 / calls,
               "pinned_h2d_copy_GBs": h2d_gbs, "note": "each rank uploads its shard and x, runs the gemv, downloads its slice; slices are not exchanged in this leg"}

    # ---- the other configurations (rank-local; N = 1 for the long lists)
    c2 = None
    configs = None
    abt = None
    if not args.no_extra:
        c2 = {"independent": gemv_record(ops, torch, timer, B.Q4_0, 8192, 8192, extra_steps, 3, peak),
              "chained": gemv_record(ops, torch, timer, B.Q4_0, 8192, 8192, extra_steps, 3, peak, chained=True),
              "workload": "BASELINE configs[1]: every rank its own matrices"}
        if world == 1:
            configs = [gemv_record(ops, torch, timer, f, r, c, 3, 3, peak) for f, r, c in
                       [(B.Q8_0, 4096, 4096), (B.Q8_0, 4093, 4064), (B.Q4_0, 8191, 8160), (B.Q4_K, 4096, 4096), (B.Q4_K, 11008, 4096),
                        (B.Q4_K, 4096, 11008), (B.Q6_K, 4096, 4096), (B.Q6_K, 11008, 4096), (B.Q6_K, 4096, 11008), (B.Q4_0, 28669, 8160)]]
            configs.append(gemv_record(ops, torch, timer, B.Q8_0, 4096, 4096, 3, 3, peak, chained=True))
            clock = clocks.get("sm_max_mhz") or 1965.0
            peak_mma, mma_cycles = tensor_peak(ops, clock)
            abt = {"configs2": [abt_record(ops, torch, timer, B.Q8_0, m, 11008, 4096, peak_mma) for m in (512, 2048, 128, 16)],
                   "configs4": [abt_record(ops, torch, timer, B.Q4_0, m, N5, K5, peak_mma) for m in (8, 64, 512)],
                   "roofline": {"bound": "tensor", "unit": "TOP/s", "peak_nominal": 4500.0, "peak_measured": peak_mma,
                                "cycles_per_mma_128x128x32": mma_cycles,
                                "peak_kind": "nominal dense int8; peak_measured = the rate of the product's tcgen05.mma measured in this run "
                                             "(qb200_tensor_rate) x SMs x the max SM clock"}}
            if not args.no_cpu:
                abt["cpu_baseline"] = abt_cpu_baseline()

    abt_sharded = None
    if world > 1 and not args.no_extra:
        abt_sharded = [abt_sharded_record(ops, torch, dist, timer, plan, rank, world, dev, shards[0], m) for m in (8, 64, 512, 2048)]

    if rank != 0:
        exchange.close()
        if world > 1:
            dist.destroy_process_group()
        return

    achieved = rank_algo / per_launch_s / 1e9
    kernels_per_call = 2 if world > 1 else 1
    line = {"metric": "quant gemv HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "s8 dot / f32 scale", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers_per_pass": layers, "graph_replays_per_step": REPLAYS, "launches_per_step": launches_per_step,
                       "launch": "one CUDA graph of a pass's kernels, replayed", "l2": f"inputs larger than L2: {layers} distinct shards of {shard_bytes / 1e6:.1f} MB a rank",
                       "exchange": "peer stores from the gemv kernel + flags + bounded wait" if world > 1 else "none (one rank holds all rows)",
                       "pct_of_8TBs_per_gpu": 100.0 * value / world / 8000.0, "median_step_ms": float(np.median(per_step)),
                       "fastest_step_ms": min(per_step), "slowest_step_ms": max(per_step)},
            "with_exchange": head,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": int(rank_algo * TRAFFIC_RATIO), "peak_kind": f"of {peak_kind}", "kernel": "gemv_kernel<Q4_0>",
                         "launch_us": per_launch_s * 1e6, "kernels_per_call": kernels_per_call, "algorithmic_bytes_per_launch": rank_algo,
                         "note": "per rank: its shard + x + its slice over the time of a launch, the exchange's wait included at N > 1"},
            "clocks": clocks, "gpu_launches": args.steps * launches_per_step * kernels_per_call}
    if local_rec is not None:
        line["local"] = local_rec
    if gather_rec is not None:
        line["with_allgather"] = gather_rec
    if e2e is not None:
        line["e2e"] = e2e
    if c2 is not None:
        line["c2"] = c2
    if configs is not None:
        line["configs"] = configs
    if abt is not None:
        line["abt"] = abt
    if abt_sharded is not None:
        line["abt_sharded"] = abt_sharded
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"], _ = cpu_gemv(10.0, layers)
    print(json.dumps(line), flush=True)
    exchange.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
