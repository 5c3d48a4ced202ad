#!/usr/bin/env python
"""Benchmark of the W8A8 linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

One "step" is one pass of the column-sharded (tensor-parallel) W8A8 linear layer over one batch
of synthetic input:

    X bf16 [8192, 7168] -> per_token_quant_int8 -> w8a8_gemm with W int8 [28672 / G, 7168]
      -> bf16 [8192, 28672], complete and row-major on every rank

With G = 1 rank this is the largest single-GPU case of the benchmark configurations; with
G > 1 (one process per GPU, torchrun) the weight is split on N, every rank quantises X itself,
and the slabs are exchanged over NVLink inside the timed region: by the GEMM kernel's own
epilogue (tile stores into every rank's output through peer memory; the headline) and, for
comparison, by an NCCL all-gather.  The total work is fixed, so scaling is "strong".  Rank 0
prints ONE JSON line.

  value      whole-job int8 tera-ops per second (2*M*N*K per step), inputs resident in HBM,
             CUDA events, max over ranks; the K timed steps are repeated R times and the
             median repeat is reported (min and max beside it)
  e2e        the same step through the operator module with HOST buffers: pinned host ->
             device copy of X, the operators, device -> host copy of this rank's slab of the
             result, all inside the timed region
  roofline   the GEMM kernel against the measured tensor peak
  parity_ok  after the timed loop: sampled rows x column blocks that straddle the slab
             boundaries against an independent fp32 formula on the integer product, and (G > 1)
             the fused result against the NCCL result, bit for bit, on every rank
  cpu_baseline  the CPU oracle (a C port of the reference arithmetic; the reference has no
             CPU implementation and cannot be built here) on a fixed sample of rows
  extra      the other benchmark configurations: per-kernel times, GB/s, TOPS and roofline
             fractions, the dense chain, the MoE chain (expert-parallel at G > 1)

`--impl reference` times the CPU oracle on the host cores for the same configuration.
"""
import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

TP_M, K_DIM, TP_N = 8192, 7168, 28672
M_ROWS = 2048              # default rows of `--kernel` runs
CPU_ROWS = 128             # fixed row sample of the CPU legs (all N columns)
L2_BYTES = 126 * 1024 * 1024
METRIC = "W8A8 quant+GEMM TOPS"


def workload_config(world: int):
    """The `config` object; identical in both arms."""
    return {
        "workload": f"column-sharded W8A8 linear: per_token_quant_int8 -> w8a8_gemm -> all-gather; X bf16 "
                    f"[{TP_M},{K_DIM}] replicated, W int8 [{TP_N},{K_DIM}] split on N over the ranks, bf16 "
                    f"[{TP_M},{TP_N}] complete on every rank",
        "M": TP_M, "K": K_DIM, "N": TP_N, "ranks": world, "parallelism": f"tp{world}",
        "l2": "one step touches X (117 MB), its codes (59 MB), the weight slab (205 MB / ranks) and the full output "
              "(470 MB): far beyond the 126 MB L2; X alternates between two buffers",
    }


# ------------------------------------------------------------------------------------------
# peaks
# ------------------------------------------------------------------------------------------
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while running.  Every sample
    carries its host time, so that a summary can be restricted to a timed region."""

    REASONS = {
        0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
        0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
        0x100: "display_clock_setting",
    }

    def __init__(self, device_index: int, period_s: float = 0.002):
        self.samples, self.max_mhz = [], None     # (host time, MHz, reason bits)
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        self._handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = device_index
            if visible:
                try:
                    idx = int(visible.split(",")[device_index])
                except (ValueError, IndexError):
                    idx = device_index
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: clocks are reported as unknown
            self._handle = None

    def _run(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)
                bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                self.samples.append((time.perf_counter(), mhz, bits))
            except Exception:
                break
            time.sleep(self._period)

    def __enter__(self):
        if self._handle is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, t0=None, t1=None):
        """Median clock and the throttle reasons seen between host times t0 and t1 (everything if None)."""
        sel = [s for s in self.samples if (t0 is None or s[0] >= t0) and (t1 is None or s[0] <= t1)]
        if not sel:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        bits = 0
        for s in sel:
            bits |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if bits & bit]
        mhz = [s[1] for s in sel]
        return {"sm_mhz": statistics.median(mhz), "sm_min_mhz": min(mhz), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(sel),
                "window": "samples taken inside the timed region" if t0 is not None else "whole run"}


# ------------------------------------------------------------------------------------------
# timing helpers
# ------------------------------------------------------------------------------------------
def time_launches(fn, iters: int, warmup: int = 3) -> float:
    """Average milliseconds per call of fn(i), CUDA events on the current stream."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(iters):
        fn(i)
    end.record()
    end.synchronize()
    return start.elapsed_time(end) / iters


def time_launches_graph(fn, launches_per_graph: int = 20, replays: int = 10) -> float:
    """Median milliseconds per call of fn(i) with the calls captured in a CUDA graph and the graph
    replayed: the device time of short kernels without the host's per-call launch cost (the
    serving engine this path plugs into replays it from CUDA graphs as well)."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches_per_graph):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end) / launches_per_graph)
    return statistics.median(times)


def rotation_count(bytes_per_set: int) -> int:
    """How many buffer sets to rotate through so that the footprint is well beyond L2."""
    return max(2, min(64, (3 * L2_BYTES + bytes_per_set - 1) // bytes_per_set))


class BlockTimer:
    """R repeats of [barrier, K calls of fn bracketed by CUDA events, barrier]; each repeat's time is
    the maximum over the ranks.  Reports the median repeat with the spread beside it."""

    def __init__(self, world, dev):
        self.world, self.dev = world, dev

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def run(self, fn, steps, repeats, warmup=0):
        for i in range(warmup):
            fn(i)
        per_repeat = []
        t_host0 = None
        for _ in range(repeats):
            self.barrier()
            if t_host0 is None:
                t_host0 = time.perf_counter()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(steps):
                fn(i)
            end.record()
            end.synchronize()
            self.barrier()
            per_repeat.append(start.elapsed_time(end))
        t_host1 = time.perf_counter()
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor(per_repeat, device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            per_repeat = [float(v) for v in t.tolist()]
        per_step = sorted(v / steps for v in per_repeat)
        return {"ms_per_step": statistics.median(per_step), "ms_per_step_min": per_step[0],
                "ms_per_step_max": per_step[-1], "repeats": repeats, "steps": steps,
                "host_window": (t_host0, t_host1)}


def _public(t):
    return {k: v for k, v in t.items() if k != "host_window"}


# ------------------------------------------------------------------------------------------
# CPU oracle legs
# ------------------------------------------------------------------------------------------
def oracle_use_all_cores() -> int:
    """The CPU legs use every host thread, whatever OMP_NUM_THREADS the launcher exported."""
    from oracle import cpu as oracle
    return oracle.set_num_threads(os.cpu_count() or 1)


class OracleStep:
    """The CPU oracle on the first CPU_ROWS rows of the workload against all N columns:
    per_token_quant_int8 -> w8a8_gemm.  The weight (205 MB) is generated once."""

    def __init__(self):
        from tests import workloads as wl
        inp = wl.tp_linear_inputs(0, 1, m=CPU_ROWS, k=K_DIM, n=TP_N, device="cpu", seed=0)
        self.x, self.w, self.w_scale = inp.x, inp.w, inp.w_scale
        self.ops = 2.0 * CPU_ROWS * TP_N * K_DIM
        self.sample = (f"the first {CPU_ROWS} of {TP_M} rows against all {TP_N} columns per step (per_token_quant_int8 "
                       f"-> w8a8_gemm, K={K_DIM}); C oracle port of the reference arithmetic, OpenMP on all host threads")

    def __call__(self) -> float:
        from oracle import cpu as oracle
        t0 = time.perf_counter()
        q, s = oracle.per_token_quant_int8(self.x)
        oracle.w8a8_gemm(q, self.w, s.view(-1), self.w_scale)
        return time.perf_counter() - t0


def cpu_config1_leg():
    """The CPU-timed configuration: per_token_quant_int8 on X bf16 [64, 7168], seed 0, 1 % outliers."""
    from oracle import cpu as oracle
    from tests import workloads as wl
    x = wl.activations_with_outliers(64, K_DIM, device="cpu", seed=0)
    times = []
    for _ in range(50):
        t0 = time.perf_counter()
        oracle.per_token_quant_int8(x)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    nbytes = 3 * 64 * K_DIM + 4 * 64
    return {"workload": "per_token_quant_int8 X bf16 [64,7168], seed 0, N(0,1) with 1 % of entries x20",
            "us": med * 1e6, "GBps": nbytes / med / 1e9, "bytes": nbytes, "passes": len(times), "statistic": "median"}


def cpu_baseline_leg(target_s: float = 12.0):
    """The oracle on the fixed row sample, repeated for about target_s seconds; the median pass is reported."""
    cores = oracle_use_all_cores()
    step = OracleStep()
    step()  # first touch of the weight
    times, spent = [], 0.0
    while len(times) < 3 or (spent < target_s and len(times) < 100):
        dt = step()
        times.append(dt)
        spent += dt
    med = statistics.median(times)
    return {"value": step.ops / med / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
            "sample": f"{step.sample}; median of {len(times)} passes ({med:.3f} s each, min {min(times):.3f}, max "
                      f"{max(times):.3f}; {spent:.1f} s of CPU work)",
            "config1_per_token_quant_int8": cpu_config1_leg()}


def run_reference_arm(args):
    """The reference's arithmetic on the host cores (C oracle port; the reference is HIP-only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    cores = oracle_use_all_cores()
    step = OracleStep()
    for _ in range(max(args.warmup, 1)):
        step()
    times = [step() for _ in range(args.steps)]
    dt = sum(times) / max(len(times), 1)
    value = step.ops / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "ms_per_step_min": min(times) * 1e3, "ms_per_step_max": max(times) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(world),
        "reference_arm": "CPU oracle on a fixed row sample of the same workload; the reference has no CPU path and its "
                         "HIP sources cannot be built on this box",
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": cores, "kind": "port", "sample": step.sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def quant_bytes_add_rmsnorm(m, k):
    return m * (7 * k + 4) + 2 * k      # read res,x (4k) + write res (2k) + write q (k) + scale, gamma once


def gemm_bytes(m, n, k):
    return m * k + n * k + 2 * m * n + 4 * (m + n)


def regenerate_weight_rows(wl, lo, hi, device, seed=0, slab=512):
    """Rows [lo, hi) of the full [N, K] benchmark weight and their scales (seeded per 512-row slab,
    so any rank can rebuild any part of it)."""
    assert lo % slab == 0 and hi % slab == 0
    ws, ss = [], []
    for sid in range(lo // slab, hi // slab):
        ws.append(wl.int8_weights((slab, K_DIM), device, seed + 10 + 2 * sid))
        ss.append(wl.channel_scales((slab,), device, seed + 11 + 2 * sid))
    return torch.cat(ws), torch.cat(ss)


def parity_check(ext, wl, out, x, world, dev):
    """Sampled rows x column blocks of `out` (the layer's bf16 [M, N] result for x) against
    bf16((float(acc) * s_tok) * s_ch) computed by torch from the library integer product of the same
    codes.  The column blocks are the 512-column slabs either side of every boundary between two
    ranks' slabs (first and last slab on one rank); the rows are the first and last 64 and 128
    seeded random ones.  Bit for bit."""
    q, s = ext.per_token_quant_int8(x)
    gen = torch.Generator(device="cpu").manual_seed(1234)
    rows = torch.cat([torch.arange(0, 64), torch.arange(TP_M - 64, TP_M),
                      torch.randperm(TP_M - 128, generator=gen)[:128] + 64])
    rows = rows.sort().values.to(dev)
    n_local = TP_N // world
    if world == 1:
        blocks = [(0, 512), (TP_N - 512, TP_N)]
    else:
        blocks = [(b * n_local - 512, b * n_local + 512) for b in range(1, world)]
    qr, sr = q[rows].contiguous(), s[rows].contiguous()
    ok, checked = True, 0
    for lo, hi in blocks:
        w_blk, ws_blk = regenerate_weight_rows(wl, lo, hi, dev)
        acc = torch._int_mm(qr, w_blk.t())
        ref = ((acc.to(torch.float32) * sr) * ws_blk.unsqueeze(0)).to(torch.bfloat16)
        got = out[rows][:, lo:hi]
        ok = ok and bool(torch.equal(got.contiguous().view(torch.int16), ref.view(torch.int16)))
        checked += ref.numel()
    return ok, checked


def peer_copy_rates(dev, rank, world, fused):
    """NVLink rates measured in this run with plain tensor copies (no kernel of this package):
    one_peer: this rank copies 256 MB into rank+1's symmetric buffer while every rank does the same;
    all_peers: 64 MB to each of the other ranks at once, the traffic pattern of the all-gather."""
    import torch.distributed as dist
    out = {}
    try:
        handle = fused.handles[0]
        src = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        assert fused.outs[0].numel() * 2 >= src.numel()

        def peer_view(r, nbytes):
            return handle.get_buffer(r, (nbytes,), torch.uint8)

        def timed(fn, reps=5):
            ts = []
            for _ in range(reps):
                dist.barrier()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                b.synchronize()
                ts.append(a.elapsed_time(b))
            t = torch.tensor([statistics.median(ts)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        nxt = peer_view((rank + 1) % world, src.numel())
        ms = timed(lambda: nxt.copy_(src))
        out["one_peer_GBps"] = round(src.numel() / (ms * 1e-3) / 1e9, 1)
        per = 64 << 20
        views = [peer_view((rank + 1 + d) % world, per) for d in range(world - 1)]
        streams = [torch.cuda.Stream() for _ in views]

        def push_all():
            cur = torch.cuda.current_stream()
            for v, st in zip(views, streams):
                st.wait_stream(cur)
                with torch.cuda.stream(st):
                    v.copy_(src[:per])
            for st in streams:
                cur.wait_stream(st)

        ms = timed(push_all)
        out["all_peers_GBps_sent_per_rank"] = round(per * (world - 1) / (ms * 1e-3) / 1e9, 1)
        out["how"] = ("device-to-device tensor copies into the peers' symmetric memory, every rank sending at the same "
                      "time, median of 5, max over ranks")
        dist.barrier()
        torch.cuda.synchronize()
    except Exception as exc:  # pragma: no cover
        out["error"] = f"{type(exc).__name__}: {exc}"
    return out


def run_ours(args):
    import torch.distributed as dist

    import bw1000_dsv4_kernels_b200 as pkg
    from bw1000_dsv4_kernels_b200 import tp_linear
    from tests import workloads as wl

    ext = pkg.dsv4_native_ext
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"   # the version banner goes to stdout, which carries the JSON line
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    timer = BlockTimer(world, dev)
    steps, warmup = args.steps, max(args.warmup, 3)

    # ---- inputs ------------------------------------------------------------------------
    inp = wl.tp_linear_inputs(rank, world, m=TP_M, k=K_DIM, n=TP_N, device=dev, seed=0)
    xs = [inp.x, wl.randn_bf16((TP_M, K_DIM), device=dev, seed=7)]
    n_local = TP_N // world
    nccl_layer = tp_linear.ColumnParallelW8A8Linear(inp.w, inp.w_scale, rank, world)
    fused, fused_error = None, None
    if world > 1:
        try:
            fused = tp_linear.FusedColumnParallelW8A8Linear(inp.w, inp.w_scale, rank, world, m_max=TP_M, device=dev)
        except Exception as exc:  # symmetric memory unavailable: the NCCL path carries the headline, and says so
            fused_error = f"{type(exc).__name__}: {exc}"
        flag = torch.tensor([1 if fused is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            fused = None

    if world == 1:
        path = "per_token_quant_int8 + gemm_i8_pair_kernel (one rank: no exchange)"
        head_fn = lambda i: nccl_layer.forward_slabs(xs[i & 1])
    elif fused is not None:
        path = ("per_token_quant_int8 + gemm_i8_pair_kernel with the fused all-gather epilogue (TMA tile stores into every "
                "rank's output over NVLink) + one symmetric-memory barrier")
        head_fn = lambda i: fused.forward(xs[i & 1])
    else:
        path = ("per_token_quant_int8 + gemm_i8_pair_kernel + NCCL all_gather_into_tensor (fused path unavailable: "
                + str(fused_error) + ")")
        head_fn = lambda i: nccl_layer.forward_slabs(xs[i & 1])

    ops_step = 2.0 * TP_M * TP_N * K_DIM
    sampler = ClockSampler(local_rank)
    with sampler:
        # ---- headline: W warm-up steps, then R x K timed steps ---------------------------
        for i in range(warmup):
            head_fn(i)
        torch.cuda.synchronize()
        est = time_launches(head_fn, 3, warmup=0)
        if world > 1:
            t = torch.tensor([est], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            est = float(t.item())
        repeats = int(max(15, min(60, math.ceil(250.0 / max(est * steps, 1e-3)))))
        head = timer.run(head_fn, steps, repeats)
        ms_step = head["ms_per_step"]
        clocks = sampler.summary(*head["host_window"])

        if args.chain_only:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "value": ops_step / (ms_step * 1e-3) / 1e12, "unit": "TOPS",
                                  "ms_per_step": ms_step, "steps": steps, "n_gpus": world,
                                  "note": "--chain-only: the timed steps alone (for profiler launch lists)"}), flush=True)
            if world > 1:
                dist.destroy_process_group()
            return

        # ---- the same launches on their own ----------------------------------------------
        q0, s0 = ext.per_token_quant_int8(xs[0])
        slabs = nccl_layer._slabs(TP_M, dev)
        short = max(5, repeats // 3)
        t_gemm = timer.run(lambda i: ext.w8a8_gemm_into(q0, inp.w, s0, inp.w_scale, slabs[rank], 0), steps, short, warmup=2)
        t_quant = timer.run(lambda i: ext.per_token_quant_int8(xs[i & 1]), steps, short, warmup=2)
        t_local = timer.run(lambda i: nccl_layer.local_gemm(xs[i & 1], out=slabs[rank]), steps, short, warmup=2)
        variants = {}
        nvlink = {}
        if world > 1:
            t_nccl = timer.run(lambda i: nccl_layer.forward_slabs(xs[i & 1]), steps, short, warmup=2)
            variants["nccl_all_gather"] = _public(t_nccl)
            variants["nccl_all_gather"]["layout"] = ("slab-major [G, M, N/G] (what ncclAllGather produces); row-major needs "
                                                     "one more strided copy")
            if fused is not None:
                variants["fused_epilogue"] = _public(head)
                try:
                    single = tp_linear.FusedColumnParallelW8A8Linear(inp.w, inp.w_scale, rank, world, m_max=TP_M, device=dev,
                                                                     buffers=1, rotate_peers=False)
                    t_single = timer.run(lambda i: single.forward(xs[i & 1]), steps, short, warmup=2)
                    variants["fused_epilogue_one_buffer_two_barriers_peers_in_rank_order"] = _public(t_single)
                    del single
                except Exception as exc:  # pragma: no cover
                    variants["fused_epilogue_one_buffer_error"] = f"{type(exc).__name__}: {exc}"
                nvlink = peer_copy_rates(dev, rank, world, fused)
            sent = (world - 1) * TP_M * n_local * 2
            nvlink["bytes_sent_per_rank_per_step"] = sent
            nvlink["headline_GBps_sent_per_rank"] = round(sent / (ms_step * 1e-3) / 1e9, 1)
            exch_ms = max(ms_step - t_quant["ms_per_step"], 1e-6)
            nvlink["headline_GBps_sent_per_rank_excluding_quantiser"] = round(sent / (exch_ms * 1e-3) / 1e9, 1)
            ref_rate = nvlink.get("all_peers_GBps_sent_per_rank") or nvlink.get("one_peer_GBps")
            if ref_rate:
                nvlink["frac_of_measured_copy_rate"] = round(
                    nvlink["headline_GBps_sent_per_rank_excluding_quantiser"] / ref_rate, 4)

        # ---- parity, after the timed loops -------------------------------------------------
        parity = {}
        out_head = head_fn(0)
        torch.cuda.synchronize()
        if world == 1:
            out_rm = out_head[0]
        elif fused is None:
            out_rm = out_head.permute(1, 0, 2).reshape(TP_M, TP_N)
        else:
            out_rm = out_head
        ok_formula, n_checked = parity_check(ext, wl, out_rm, xs[0], world, dev)
        parity["sampled_blocks_vs_fp32_formula_on_library_int_mm"] = ok_formula
        parity["elements_checked"] = n_checked
        ok_all = ok_formula
        if world > 1 and fused is not None:
            ref_slabs = nccl_layer.forward_slabs(xs[0])
            same = bool(torch.equal(out_rm.view(TP_M, world, n_local).permute(1, 0, 2).contiguous().view(torch.int16),
                                    ref_slabs.view(torch.int16)))
            parity["fused_equals_nccl_all_elements"] = same
            ok_all = ok_all and same
            del ref_slabs
        status = int(ext.device_status())
        parity["device_status"] = status
        ok_all = ok_all and status == 0
        if world > 1:
            f = torch.tensor([1 if ok_all else 0], device=dev)
            dist.all_reduce(f, op=dist.ReduceOp.MIN)
            ok_all = bool(int(f.item()))
        parity["ranks_checked"] = world

        # ---- end to end through the operator module with host buffers --------------------
        # Every step copies X from pinned host memory, runs the layer and copies this rank's column
        # slab of the result back (the ranks' slabs together are the whole output).  Three streams
        # and two sets of buffers let step i+1's upload and step i-1's download overlap step i's
        # kernels; the timed region still contains every copy of every step.
        e2e_steps = max(4, min(steps, 10))
        hx = xs[0].cpu().pin_memory()
        houts = [torch.empty((TP_M, n_local), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        dxs = [torch.empty_like(xs[0]) for _ in range(2)]
        stage = [torch.empty((TP_M, n_local), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        s_in, s_comp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_comp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def e2e_run(n_steps):
            for i in range(n_steps):
                b = i & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_comp[b])         # buffer b's previous kernels have read it
                    dxs[b].copy_(hx, non_blocking=True)
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_comp):
                    s_comp.wait_event(ev_in[b])
                    s_comp.wait_event(ev_out[b])        # stage b's previous download has finished
                    if fused is not None:
                        full = fused.forward(dxs[b])
                        stage[b].copy_(full[:, rank * n_local:(rank + 1) * n_local])
                    else:
                        stage[b].copy_(nccl_layer.forward_slabs(dxs[b])[rank])
                    ev_comp[b].record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[b])
                    houts[b].copy_(stage[b], non_blocking=True)
                    ev_out[b].record(s_out)

        cur = torch.cuda.current_stream()
        e2e_run(2)
        torch.cuda.synchronize()
        timer.barrier()
        e2e_start, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_start.record(cur)
        for st_ in (s_in, s_comp, s_out):
            st_.wait_event(e2e_start)
        e2e_run(e2e_steps)
        for st_ in (s_in, s_comp, s_out):
            cur.wait_stream(st_)
        e2e_end.record(cur)
        e2e_end.synchronize()
        timer.barrier()
        ms_e2e = e2e_start.elapsed_time(e2e_end) / e2e_steps
        if world > 1:
            t = torch.tensor([ms_e2e], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())
        del houts, dxs, stage, hx

        extra = {}
        if not args.no_extras:
            del fused, nccl_layer, slabs, out_head, out_rm, q0, s0, inp, xs
            head_fn = None
            torch.cuda.empty_cache()
            try:
                import bench_extras
                extra = bench_extras.run(ext, dev, rank, world, peaks, time_launches, rotation_count, time_launches_graph, timer)
            except Exception as exc:  # extras never take the headline down
                extra = {"error": f"{type(exc).__name__}: {exc}"}

    value = ops_step / (ms_step * 1e-3) / 1e12
    e2e_value = ops_step / (ms_e2e * 1e-3) / 1e12
    ops_rank = ops_step / world
    gemm_tops = ops_rank / (t_gemm["ms_per_step"] * 1e-3) / 1e12
    peak_sustained = 2.0 * peaks["bf16_tflops_sustained"]
    peak_burst = 2.0 * peaks["bf16_tflops"]
    quant_gbs = (3 * TP_M * K_DIM + 4 * TP_M) / (t_quant["ms_per_step"] * 1e-3) / 1e9
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the GEMM at the one-rank shape, from the
    # profiler capture summarised under profiles/ (null at other shapes)
    traffic = GEMM_TP_TRAFFIC_BYTES if world == 1 else None

    line = {
        "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_step, "ms_per_step_min": head["ms_per_step_min"],
        "ms_per_step_max": head["ms_per_step_max"], "repeats": head["repeats"],
        "timing": f"the {steps} timed steps are repeated {head['repeats']} times, each repeat between a barrier + "
                  f"synchronise on both sides with CUDA events on the launching stream, max over ranks per repeat; "
                  f"ms_per_step is the median repeat",
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(world),
        "path": path,
        "parity_ok": ok_all, "parity": parity,
        "roofline": {
            "kernel": "gemm_i8_pair_kernel (tcgen05.mma.cta_group::2.kind::i8, 256x256 tile per CTA pair), this rank's "
                      f"[{TP_M} x {n_local} x {K_DIM}] launch timed on its own",
            "bound": "tensor", "achieved": gemm_tops, "peak": peak_sustained, "unit": "TFLOP/s",
            "frac": gemm_tops / peak_sustained,
            "frac_of_burst_peak": gemm_tops / peak_burst, "frac_of_nominal_4500": gemm_tops / 4500.0,
            "peak_source": f"int8 tera-ops; 2 x cuBLAS bf16 sustained ({peaks['bf16_tflops_sustained']} TF/s, "
                           f"{peaks['source']}): the launch is timed back to back inside loops of {steps} launches "
                           f"under the power cap; burst would be 2 x {peaks['bf16_tflops']}; nominal dense int8 4500",
            "traffic": traffic, "algorithmic_bytes": gemm_bytes(TP_M, n_local, K_DIM),
            "launch_us": t_gemm["ms_per_step"] * 1e3, "launch_us_min": t_gemm["ms_per_step_min"] * 1e3,
            "launch_us_max": t_gemm["ms_per_step_max"] * 1e3,
        },
        "kernels": {
            "per_token_quant_int8": {"bound": "hbm", "achieved": quant_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                     "frac": quant_gbs / peaks["hbm_gbs"], "launch_us": t_quant["ms_per_step"] * 1e3,
                                     "bytes": 3 * TP_M * K_DIM + 4 * TP_M},
            "quant_plus_gemm_no_exchange": {**_public(t_local),
                                            "TOPS_whole_job": ops_step / (t_local["ms_per_step"] * 1e-3) / 1e12},
        },
        "variants": variants,
        "nvlink": nvlink,
        "e2e": {"value": e2e_value, "unit": "TOPS", "ms_per_step": ms_e2e, "steps": e2e_steps,
                "how": "pinned host -> device copy of X, per_token_quant_int8, w8a8_gemm (+ exchange), device -> host copy "
                       "of this rank's column slab of the result, every step; upload / kernels / download of neighbouring "
                       "steps overlap on three streams; the copies run over PCIe and bound this number",
                "h2d_bytes_per_step": TP_M * K_DIM * 2, "d2h_bytes_per_step": TP_M * n_local * 2},
        "gpu_launches": 2 * steps * head["repeats"],
        "gpu_launches_note": "per step and rank: per_token_quant_int8 and the GEMM (the exchange is the GEMM's epilogue); "
                             "the symmetric-memory barrier is a library kernel and is not counted",
        "clocks": clocks,
        "extra": extra,
    }
    if world > 1:
        # lower bound of one step: the slower of the tensor work and the bytes that must leave over NVLink
        t_tensor = ops_rank / (peak_sustained * 1e12) * 1e3
        link = nvlink.get("all_peers_GBps_sent_per_rank") or nvlink.get("one_peer_GBps") or 770.0
        t_link = nvlink["bytes_sent_per_rank_per_step"] / (link * 1e9) * 1e3
        line["roofline_fused"] = {"target_ms": max(t_tensor, t_link), "tensor_ms": t_tensor, "nvlink_ms": t_link,
                                  "nvlink_GBps_used": link, "achieved_ms": ms_step,
                                  "frac": max(t_tensor, t_link) / ms_step,
                                  "note": "target = max(ops / measured tensor peak, bytes sent / copy rate measured in "
                                          "this run); the quantiser and the barrier are inside achieved_ms"}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_leg()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of gemm_i8_pair_kernel at M=8192 N=28672 K=7168
# (profiles/gemm_i8_pair_kernel_M8192_N28672_K7168.md)
GEMM_TP_TRAFFIC_BYTES = 513608704 + 448874752


def run_single_kernel(args):
    """`--kernel NAME [--m M]`: launches one kernel of the path `--steps` times on rotating
    inputs and prints its time.  Small, self-terminating: the case profilers capture."""
    import bw1000_dsv4_kernels_b200 as pkg
    from tests import workloads as wl

    ext = pkg.dsv4_native_ext
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    m = args.m
    K, N, I = wl.HIDDEN, wl.DENSE_N, wl.DENSE_INTER
    nsets = 4
    if args.kernel == "gemm":
        A = [wl.int8_weights((m, K), device=dev, seed=i) for i in range(nsets)]
        W = [wl.int8_weights((N, K), device=dev, seed=10 + i) for i in range(nsets)]
        sa = wl.channel_scales((m,), device=dev, seed=1)
        sb = wl.channel_scales((N,), device=dev, seed=2)
        fn = lambda i: ext.w8a8_scaled_gemm(A[i % nsets], W[i % nsets], sa, sb)
        work = {"ops": 2.0 * m * N * K, "bytes": gemm_bytes(m, N, K)}
    elif args.kernel == "gemm_tp":
        # the one-rank GEMM of the headline: M=8192 (or --m), N=28672, K=7168, output written in place
        m = TP_M if args.m == M_ROWS else args.m
        A = [wl.int8_weights((m, K), device=dev, seed=i) for i in range(2)]
        W = wl.int8_weights((TP_N, K), device=dev, seed=10)
        sa = wl.channel_scales((m,), device=dev, seed=1)
        sb = wl.channel_scales((TP_N,), device=dev, seed=2)
        outb = torch.empty((m, TP_N), dtype=torch.bfloat16, device=dev)
        fn = lambda i: ext.w8a8_gemm_into(A[i % 2], W, sa, sb, outb, 0)
        work = {"ops": 2.0 * m * TP_N * K, "bytes": gemm_bytes(m, TP_N, K)}
    elif args.kernel == "gemm_down":
        A = [wl.int8_weights((m, I), device=dev, seed=i) for i in range(2)]
        W = [wl.int8_weights((K, I), device=dev, seed=10 + i) for i in range(2)]
        sa = wl.channel_scales((m,), device=dev, seed=1)
        sb = wl.channel_scales((K,), device=dev, seed=2)
        fn = lambda i: ext.w8a8_scaled_gemm(A[i % 2], W[i % 2], sa, sb)
        work = {"ops": 2.0 * m * K * I, "bytes": gemm_bytes(m, K, I)}
    elif args.kernel == "add_rmsnorm_quant":
        xs = [wl.randn_bf16((m, K), device=dev, seed=i) for i in range(nsets)]
        rs = [wl.randn_bf16((m, K), device=dev, seed=10 + i) for i in range(nsets)]
        g = wl.gamma_bf16(K, device=dev)
        fn = lambda i: ext.add_rmsnorm_quant(rs[i % nsets], xs[i % nsets], g, 1e-6)
        work = {"bytes": quant_bytes_add_rmsnorm(m, K)}
    elif args.kernel == "silu_mul_quant":
        gus = [wl.randn_bf16((m, 2 * I), device=dev, seed=i) for i in range(nsets)]
        fn = lambda i: ext.silu_mul_quant(gus[i % nsets][:, :I], gus[i % nsets][:, I:])
        work = {"bytes": m * (5 * I + 4)}
    elif args.kernel == "ptq":
        xs = [wl.activations_with_outliers(m, K, device=dev, seed=i) for i in range(nsets)]
        fn = lambda i: ext.per_token_quant_int8(xs[i % nsets])
        work = {"bytes": 3 * m * K + 4 * m}
    elif args.kernel in ("grouped", "grouped_gs"):
        # 16 experts x `m` rows each (default 128), gate/up shape: N=4096, K=7168
        rows = 128 if m == M_ROWS else m
        E, N2 = 16, 2 * wl.MOE_INTER
        off = torch.arange(0, (E + 1) * rows, rows, dtype=torch.int32, device=dev)
        A = wl.int8_weights((E * rows, K), device=dev, seed=1)
        W = [wl.int8_weights((E, N2, K), device=dev, seed=10 + i) for i in range(2)]
        sw = wl.channel_scales((E, N2), device=dev, seed=3)
        if args.kernel == "grouped_gs":
            sa = wl.channel_scales((E * rows, K // 128), device=dev, seed=2)
        else:
            sa = wl.channel_scales((E * rows,), device=dev, seed=2)
        fn = lambda i: ext.grouped_gemm(A, W[i % 2], sa, sw, off)
        work = {"ops": 2.0 * E * rows * N2 * K, "bytes": E * N2 * K + E * rows * (K + 2 * N2)}
    elif args.kernel == "grouped_scatter":
        # the down projection that delivers its rows itself: 16 experts x `m` rows (default 128), N=7168, K=2048,
        # every result row stored at its own address (here: the rows of one local buffer in reverse order)
        rows = 128 if m == M_ROWS else m
        E, N2, K2 = 16, K, wl.MOE_INTER
        off = torch.arange(0, (E + 1) * rows, rows, dtype=torch.int32, device=dev)
        A = wl.int8_weights((E * rows, K2), device=dev, seed=1)
        W = [wl.int8_weights((E, N2, K2), device=dev, seed=10 + i) for i in range(4)]
        sw = wl.channel_scales((E, N2), device=dev, seed=3)
        sa = wl.channel_scales((E * rows,), device=dev, seed=2)
        inbox = torch.empty((E * rows, N2), dtype=torch.bfloat16, device=dev)
        row_ptr = (inbox.data_ptr() + torch.arange(E * rows - 1, -1, -1, dtype=torch.int64, device=dev) * (N2 * 2)).contiguous()
        fn = lambda i: ext.grouped_gemm_scatter(A, W[i % 4], sa, sw, off, row_ptr)
        work = {"ops": 2.0 * E * rows * N2 * K2, "bytes": E * N2 * K2 + E * rows * (K2 + 2 * N2)}
    elif args.kernel == "ptgq":
        xs = [wl.randn_bf16((m, K), device=dev, seed=i) for i in range(nsets)]
        fn = lambda i: ext.per_token_group_quant_int8(xs[i % nsets], 128)
        work = {"bytes": 3 * m * K + 4 * m * (K // 128)}
    elif args.kernel == "rmsnorm":
        xs = [wl.randn_bf16((m, K), device=dev, seed=i) for i in range(nsets)]
        fn = lambda i: ext.rmsnorm(xs[i % nsets], 1e-6)
        work = {"bytes": 4 * m * K}
    elif args.kernel == "silu_and_mul":
        gus = [wl.randn_bf16((m, 2 * I), device=dev, seed=i) for i in range(nsets)]
        fn = lambda i: ext.silu_and_mul(gus[i % nsets][:, :I], gus[i % nsets][:, I:])
        work = {"bytes": 6 * m * I}
    elif args.kernel in ("moe_topk", "moe_segments", "gather_rows", "moe_combine", "moe_combine_exchange"):
        # the MoE front and back end at the configuration's sizes: T tokens, 256 experts, top-8
        T, E, topk, H = wl.MOE_TOKENS, wl.MOE_EXPERTS, wl.MOE_TOPK, K
        gen = torch.Generator(device=dev).manual_seed(0)
        logits = torch.randn((T, E), device=dev, generator=gen)
        ids, w = ext.moe_topk(logits, topk)
        off, src_row, dst_slot = ext.moe_segments(ids, E, 0)
        if args.kernel == "moe_topk":
            fn = lambda i: ext.moe_topk(logits, topk)
            work = {"bytes": 4 * T * E + 8 * T * topk}
        elif args.kernel == "moe_segments":
            fn = lambda i: ext.moe_segments(ids, E, 0)
            work = {"bytes": 4 * T * topk * 4}
        elif args.kernel == "gather_rows":
            q = wl.int8_weights((T, H), device=dev, seed=1)
            sg = wl.channel_scales((T, H // 128), device=dev, seed=2)
            fn = lambda i: ext.gather_rows(q, src_row, sg, None)
            work = {"bytes": T * topk * (2 * H + 8 * (H // 128))}
        else:
            zs = [wl.randn_bf16((T * topk, H), device=dev, seed=i) for i in range(2)]
            if args.kernel == "moe_combine":
                fn = lambda i: ext.moe_combine(zs[i % 2], dst_slot, w, False)
            else:
                # one rank's call of the fused combine + exchange with every pointer local: all tokens,
                # one output buffer (the kernel only sees pointers)
                outb = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
                fn = lambda i: ext.moe_combine_exchange([zs[i % 2].data_ptr()], [dst_slot.data_ptr()], ids, w,
                                                        [outb.data_ptr()], E, 0, T, H)
            work = {"bytes": 2 * T * topk * H + 2 * T * H}
    elif args.kernel in ("moe_ffn", "moe_ffn_per_token"):
        # the whole MoE FFN of the configuration on one GPU (256 experts, 4096 tokens, top-8): nine launches per call
        from bw1000_dsv4_kernels_b200 import moe
        inp = wl.moe_inputs(device=dev, seed=0)
        layer = moe.W8A8MoE(inp.w13, inp.w13_scale, inp.w2, inp.w2_scale, wl.MOE_EXPERTS,
                            group_scaled=(args.kernel == "moe_ffn"))
        fn = lambda i: layer.forward(inp.x, inp.topk_ids, inp.topk_w)
        rows = wl.MOE_TOKENS * wl.MOE_TOPK
        work = {"ops": 2.0 * rows * 3 * wl.MOE_INTER * K, "bytes": wl.MOE_EXPERTS * 3 * wl.MOE_INTER * K}
    elif args.kernel == "gemm_allgather":
        # the CTA-pair GEMM with the fused all-gather epilogue (TMA tile stores), two local buffers
        # standing in for this rank's and one peer's output
        A = [wl.int8_weights((m, K), device=dev, seed=i) for i in range(nsets)]
        W = [wl.int8_weights((N, K), device=dev, seed=10 + i) for i in range(nsets)]
        sa = wl.channel_scales((m,), device=dev, seed=1)
        sb = wl.channel_scales((N,), device=dev, seed=2)
        out0 = torch.empty((m, 2 * N), dtype=torch.bfloat16, device=dev)
        out1 = torch.empty((m, 2 * N), dtype=torch.bfloat16, device=dev)
        fn = lambda i: ext.w8a8_gemm_allgather(A[i % nsets], W[i % nsets], sa, sb, out0, N, [out1.data_ptr()])
        work = {"ops": 2.0 * m * N * K, "bytes": gemm_bytes(m, N, K) + 2 * m * N}
    else:
        raise SystemExit(f"unknown --kernel {args.kernel}")
    # the last few results stay alive, so that outputs rotate through several buffers like the inputs
    # (a freed output would be handed out again at once and stay in L2)
    inner, kept = fn, [None] * nsets

    def fn(i):
        kept[i % nsets] = inner(i)

    ms = time_launches(fn, args.steps, warmup=max(1, args.warmup))
    out = {"kernel": args.kernel, "m": m, "us": ms * 1e3, **work}
    if args.graph:
        out["us_graph"] = time_launches_graph(fn) * 1e3
    if "bytes" in work:
        out["GBps"] = work["bytes"] / (ms * 1e-3) / 1e9
    if "ops" in work:
        out["TOPS"] = work["ops"] / (ms * 1e-3) / 1e12
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default=None,
                    help="run one kernel only: gemm, gemm_tp, gemm_down, gemm_allgather, grouped, grouped_gs, grouped_scatter, "
                         "add_rmsnorm_quant, silu_mul_quant, ptq, ptgq, rmsnorm, silu_and_mul, moe_topk, moe_segments, "
                         "gather_rows, moe_combine, moe_combine_exchange, moe_ffn (group scales), moe_ffn_per_token")
    ap.add_argument("--m", type=int, default=M_ROWS, help="rows for --kernel")
    ap.add_argument("--graph", action="store_true", help="with --kernel: also time CUDA-graph replays")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-configuration extras")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--chain-only", action="store_true",
                    help="run the warm-up and the timed steps only (short launch list for a profiler)")
    args = ap.parse_args()
    if args.kernel is not None:
        run_single_kernel(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
