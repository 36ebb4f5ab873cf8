"""Benchmark of the block-scaled quantized gemv (the memory-bound decode path) on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (BASELINE.json configs[1]): Q4_0 gemv, weight 8192 x 8192 in 18-byte blocks, x f32[8192] ~ N(0,1),
y f32[8192].  One step = one pass of the gemv over LAYERS distinct seeded weight matrices (a stack of
layers, 8 x 37.7 MB = 302 MB > 2 x L2), so every launch reads its weights from HBM, not from L2.
The metric is algorithmic bytes per second: (weight blocks + x + y) bytes / time.

The JSON line carries the device-timed `value`, the end-to-end `e2e` through the host-buffer C-ABI
call (pinned host operands, H2D + kernel + D2H every launch), the `roofline` of the gemv kernel against
the measured HBM copy bandwidth, and `cpu_baseline`: the C restatement of the reference's CPU gemv
(thread team + integer block dots) timed on this machine's host cores.  `--impl reference` times only
that CPU restatement (the reference itself is C#/.NET and cannot run here).
"""
import argparse
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

ROWS, COLS, FMT_A, FMT_X = 8192, 8192, B.Q4_0, B.F32
LAYERS = 8
WEIGHT_BYTES = ROWS * (COLS // 32) * 18
ALGO_BYTES = WEIGHT_BYTES + COLS * 4 + ROWS * 4          # per launch: weights once, x, y
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload's kernel (ncu; profiles/), or None
TRAFFIC_BYTES = 37852160              # dram__bytes_read + write of one launch, from the ncu capture in profiles/


def measured_peak():
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


def cpu_baseline(seconds=12.0):
    """The reference's CPU block gemv (src/BlockProducts.cs:17-71) as restated in oracle/, on all host threads."""
    from oracle import qiyas_oracle as O
    weights = B.make_weights(FMT_A, ROWS, COLS, 1000)
    x = B.make_activations(COLS, 2000)
    O.time_gemv_blocks(FMT_A, FMT_X, weights, x, ROWS, COLS, 1)               # warm the team and the pages
    one = O.time_gemv_blocks(FMT_A, FMT_X, weights, x, ROWS, COLS, 2)
    reps = max(3, min(2000, int(seconds / max(one, 1e-6))))
    per_call = O.time_gemv_blocks(FMT_A, FMT_X, weights, x, ROWS, COLS, reps)
    return {"value": ALGO_BYTES / per_call / 1e9, "unit": "GB/s", "cores": O.threads(), "kind": "port",
            "sample": f"{reps} calls of the {ROWS}x{COLS} Q4_0 gemv (x f32 -> Q8_0), {per_call * 1e3:.3f} ms each, "
                      f"C restatement of Kernels.GemvBlocks on the thread team"}, per_call


def run_reference(args, rank, world):
    if rank != 0:
        return
    t0 = time.time()
    base, per_call = cpu_baseline(seconds=max(2.0, min(20.0, 1.5 * (args.steps + args.warmup))))
    line = {"impl": "reference", "metric": "quant gemv HBM GB/s", "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_call * 1e3 * LAYERS, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "s8 dot / f32 scale", "data": "synthetic",
            "config": {"workload": f"Q4_0 gemv {ROWS}x{COLS}, x f32, {LAYERS} weight matrices per step (CPU: one matrix repeated)"},
            "cpu_baseline": base, "gpu_launches": 0,
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.time() - t0}
    print(json.dumps(line), flush=True)


def sharded_gemv_leg(ops, torch, dist, rank, world, dev):
    """BASELINE configs[4] at M = 1: Q4_0 28672 x 8192 sharded by output rows over the ranks (strong scaling of one matrix),
    timed without and with the all-gather of the f32 slices.  Each rank rotates over copies of its shard larger than L2."""
    from qiyas_b200.shard import ShardPlan, all_gather_rows
    n, k = 28672, 8192
    plan = ShardPlan(n, world)
    rows = plan.count(rank)
    shard = plan.slice_weights(rank, FMT_A, k, B.make_weights(FMT_A, n, k, 4000))
    copies = max(2, min(24, int(300e6 // max(1, shard.size)) + 1))
    ws = [torch.from_numpy(shard).to(dev).clone() for _ in range(copies)]
    x = torch.from_numpy(B.make_activations(k, 4001)).to(dev)
    y = torch.empty(max(rows, 1), dtype=torch.float32, device=dev)
    y_full = torch.empty(n, dtype=torch.float32, device=dev)
    reps = 5

    def timed(gather):
        for w in ws[:2]:
            ops.GemvBlocks(FMT_A, w, x, y, rows, k, fmt_x=FMT_X)
            if gather:
                all_gather_rows(plan, rank, y, out=y_full)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for w in ws:
                ops.GemvBlocks(FMT_A, w, x, y, rows, k, fmt_x=FMT_X)
                if gather:
                    all_gather_rows(plan, rank, y, out=y_full)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / (reps * copies)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e-3

    local_s, full_s = timed(False), timed(True)
    algo = n * (k // 32) * 18 + k * 4 + n * 4
    return {"workload": f"Q4_0 gemv {n}x{k} sharded by output rows over {world} GPU(s), x f32 replicated", "scaling": "strong",
            "local_us": local_s * 1e6, "local_GBs": algo / local_s / 1e9,
            "with_allgather_us": full_s * 1e6, "with_allgather_GBs": algo / full_s / 1e9,
            "launch": "host-launched (not graph-replayed); max over ranks"}


def abt_leg(ops, torch, dev):
    """BASELINE configs[2]: Q8_0 x Q8_0 A.B^T, M 512, N 11008, K 4096 through qb200_matmul_blocks (repack + tcgen05 product)."""
    m, n, k = 512, 11008, 4096
    a = torch.from_numpy(B.make_weights(B.Q8_0, m, k, 5000)).to(dev)
    b = torch.from_numpy(B.make_weights(B.Q8_0, n, k, 5001)).to(dev)
    c = torch.empty(m * n, dtype=torch.float32, device=dev)
    need = ops.workspace_bytes(B.Q8_0, m, n, k)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    for _ in range(3):
        ops.MatMulBlocks(B.Q8_0, a, b, c, m, n, k, workspace=ws, workspace_bytes=need)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 20
    e0.record()
    for _ in range(reps):
        ops.MatMulBlocks(B.Q8_0, a, b, c, m, n, k, workspace=ws, workspace_bytes=need)
    e1.record()
    torch.cuda.synchronize()
    s = e0.elapsed_time(e1) * 1e-3 / reps
    tops = 2.0 * m * n * k / s / 1e12
    return {"workload": f"Q8_0 x Q8_0 A.B^T M {m} N {n} K {k} (BASELINE configs[2]), operands repacked every call",
            "us_per_call": s * 1e6, "int8_TOPS": tops,
            "roofline": {"bound": "tensor", "achieved": tops, "peak": 4500.0, "unit": "TOP/s", "frac": tops / 4500.0,
                         "peak_kind": "nominal dense int8 (no measured int8 figure exists)"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-extra", action="store_true", help="skip the sharded-gemv and A.B^T legs (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from qiyas_b200.ops import GpuOps

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    ops = GpuOps(device=local)

    # ---- inputs resident in HBM: LAYERS weight matrices, x, y (each rank its own stack: rows shard with no exchange)
    dev = f"cuda:{local}"
    host_w = [B.make_weights(FMT_A, ROWS, COLS, 1000 + 97 * rank + i) for i in range(LAYERS)]
    host_x = B.make_activations(COLS, 2000 + rank)
    weights = [torch.from_numpy(w).to(dev) for w in host_w]
    x = torch.from_numpy(host_x).to(dev)
    ys = [torch.empty(ROWS, dtype=torch.float32, device=dev) for _ in range(LAYERS)]

    # the step's launches are captured once in a CUDA graph on a side stream and replayed: at 6 us a kernel the
    # host's launch rate, not the GPU, would otherwise set the pace
    side = torch.cuda.Stream(device=dev)

    def launch_all(stream):
        for w, y in zip(weights, ys):
            ops.GemvBlocks(FMT_A, w, x, y, ROWS, COLS, fmt_x=FMT_X, stream=stream)

    with torch.cuda.stream(side):
        launch_all(side)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            launch_all(side)

    def step():
        graph.replay()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(side):
        for _ in range(args.warmup):
            step()
    barrier()
    # a first check that the timed thing computes the product: one row against the decoded dot (float64 on the host)
    sampler = ClockSampler(local)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with torch.cuda.stream(side):
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
    barrier()
    clocks = sampler.stop()
    ms = start.elapsed_time(stop)
    if ops.gpu.status() != 0:
        raise SystemExit("a kernel gave up on a bounded wait: the timing is void")
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    launches = args.steps * LAYERS
    per_launch_s = ms * 1e-3 / launches
    value = world * launches * ALGO_BYTES / (ms * 1e-3) / 1e9

    # ---- end to end: the host-buffer call (pinned operands up, kernel, y down) every launch
    e2e = None
    if not args.no_e2e:
        pinned_w = [torch.from_numpy(w).pin_memory() for w in host_w[:2]]
        pinned_x = torch.from_numpy(host_x).pin_memory()
        pinned_y = torch.empty(ROWS, dtype=torch.float32).pin_memory()
        wn, xn, yn = [p.numpy() for p in pinned_w], pinned_x.numpy(), pinned_y.numpy()
        e_steps = max(2, min(args.steps, 6))
        for i in range(2):
            ops.GemvBlocksHost(FMT_A, wn[i % 2], xn, yn, ROWS, COLS, fmt_x=FMT_X)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            for i in range(LAYERS):
                ops.GemvBlocksHost(FMT_A, wn[i % 2], xn, yn, ROWS, COLS, fmt_x=FMT_X)
        torch.cuda.synchronize()
        e_s = time.perf_counter() - t0
        et = torch.tensor([e_s], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(et, op=dist.ReduceOp.MAX)
        e_s = float(et.item())
        # the bound of this leg: a plain copy of one matrix from the same pinned buffer, timed the same way
        dst = torch.empty(WEIGHT_BYTES, dtype=torch.uint8, device=dev)
        dst.copy_(pinned_w[0], non_blocking=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(4):
            dst.copy_(pinned_w[i % 2], non_blocking=True)
        torch.cuda.synchronize()
        h2d_gbs = 4 * WEIGHT_BYTES / (time.perf_counter() - t0) / 1e9
        e2e = {"value": world * e_steps * LAYERS * ALGO_BYTES / e_s / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": LAYERS * (WEIGHT_BYTES + COLS * 4), "d2h_bytes_per_step": LAYERS * ROWS * 4,
               "steps": e_steps, "ms_per_step": e_s * 1e3 / e_steps, "pinned_h2d_copy_GBs": h2d_gbs}

    sharded = None if args.no_extra else sharded_gemv_leg(ops, torch, dist, rank, world, dev)
    abt = abt_leg(ops, torch, dev) if (world == 1 and not args.no_extra) else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # one output row checked on the host against float64 of the decoded stored values
    from oracle import qiyas_oracle as O
    r = 4321
    row = host_w[LAYERS - 1].reshape(ROWS, -1)[r]
    xq = O.decode(B.Q8_0, O.encode(B.Q8_0, host_x), COLS)
    want = float(O.gemv_f64(FMT_A, row, xq, 1, COLS)[0])
    got = float(ys[LAYERS - 1][r].item())
    if abs(got - want) > 1e-4 * max(1.0, abs(want)):
        raise SystemExit(f"bench output check failed: row {r} = {got}, float64 says {want}")

    peak, peak_kind = measured_peak()
    achieved = ALGO_BYTES / per_launch_s / 1e9
    line = {"metric": "quant gemv HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8 dot / f32 scale", "data": "synthetic",
            "config": {"workload": f"Q4_0 gemv {ROWS}x{COLS} (BASELINE configs[1]), x f32 -> Q8_0 in-kernel",
                       "layers_per_step": LAYERS, "launch": "one CUDA graph of the step's kernels, replayed", "l2": f"inputs larger than L2: {LAYERS} distinct weight matrices, "
                       f"{LAYERS * WEIGHT_BYTES / 1e6:.0f} MB per step", "pct_of_8TBs": 100.0 * value / world / 8000.0},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES, "peak_kind": f"of {peak_kind}", "kernel": "gemv_kernel<Q4_0>",
                         "launch_us": per_launch_s * 1e6, "kernels_per_call": 1, "algorithmic_bytes_per_launch": ALGO_BYTES},
            "clocks": clocks, "gpu_launches": launches}      # one kernel a call: x is encoded inside the gemv kernel
    if e2e is not None:
        line["e2e"] = e2e
    if sharded is not None:
        line["sharded"] = sharded
    if abt is not None:
        line["abt"] = abt
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"], _ = cpu_baseline()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
