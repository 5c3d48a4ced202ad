#!/usr/bin/env python
"""Benchmark of the W8A8 linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

One "step" is one pass of the hot path over one batch of synthetic input:
    add_rmsnorm_quant(res, x, gamma) -> w8a8_scaled_gemm(q, W, s_tok, s_ch) -> bf16 [M, N]
with M=2048 tokens, K=7168, N=4096 per rank (the largest case of the dense-projection
configuration).  Rows are independent, so N GPUs run N independent batches (weak scaling,
no data-path collective).  Rank 0 prints ONE JSON line.

  value      whole-job int8 tera-ops per second of the chain (2*M*N*K per rank and step),
             inputs resident in HBM, timed with CUDA events, max over ranks
  e2e        the same chain through the operator module with HOST buffers: pinned host ->
             device copies of x and res, the two operators, device -> host copy of the
             output and of the updated residual, all inside the timed region
  roofline   the dominant kernel (the GEMM) against the measured tensor peak; the quant
             kernel against measured HBM bandwidth is under "kernels"
  cpu_baseline  the CPU oracle (a C port of the reference arithmetic; the reference has no
             CPU implementation and cannot be built here) on a bounded sample of rows
  extra      the other benchmark configurations: per-kernel times, GB/s, TOPS and roofline
             fractions, the MoE chain, and the sharded configurations at N > 1

`--impl reference` times the CPU oracle on the host cores for the same configuration.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

M_ROWS, K_DIM, N_DIM = 2048, 7168, 4096
L2_BYTES = 126 * 1024 * 1024


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
    """Samples SM clock and throttle reasons of one GPU through NVML while running."""

    REASONS = {
        0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
        0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
        0x100: "display_clock_setting",
    }

    def __init__(self, device_index: int, period_s: float = 0.002):
        self.samples, self.reason_bits, self.max_mhz = [], 0, None
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
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
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

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        reasons = [name for bit, name in self.REASONS.items() if self.reason_bits & bit]
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.samples)}


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
    """Average milliseconds per call of fn(i) with the calls captured in a CUDA graph and the
    graph replayed: the device time of short kernels without the host's per-call launch cost
    (the serving engine this path plugs into replays it from CUDA graphs as well)."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches_per_graph):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    end.record()
    end.synchronize()
    return start.elapsed_time(end) / (replays * launches_per_graph)


def rotation_count(bytes_per_set: int) -> int:
    """How many buffer sets to rotate through so that the footprint is well beyond L2."""
    return max(2, min(64, (3 * L2_BYTES + bytes_per_set - 1) // bytes_per_set))


# ------------------------------------------------------------------------------------------
# CPU oracle legs
# ------------------------------------------------------------------------------------------
def oracle_chain_rate(rows: int, seed: int = 0, repeats: int = 1):
    """Seconds for the oracle's add_rmsnorm_quant -> w8a8_gemm on `rows` rows of the workload."""
    from bw1000_dsv4_kernels_b200 import workloads as wl
    from oracle import cpu as oracle

    inp = wl.norm_gemm_inputs(rows, seed=seed)
    best = None
    for _ in range(repeats):
        res = inp.res.clone()
        t0 = time.perf_counter()
        q, s = oracle.add_rmsnorm_quant(res, inp.x, inp.gamma, inp.eps)
        oracle.w8a8_gemm(q, inp.w, s.view(-1), inp.w_scale)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def oracle_use_all_cores() -> int:
    """The CPU legs use every host thread, whatever OMP_NUM_THREADS the launcher exported."""
    from oracle import cpu as oracle
    return oracle.set_num_threads(os.cpu_count() or 1)


def calibrate_oracle_rows(target_s: float) -> int:
    oracle_use_all_cores()
    probe_rows = 4
    dt = oracle_chain_rate(probe_rows)
    rows = int(max(1, min(M_ROWS, probe_rows * target_s / max(dt, 1e-6))))
    return rows


def cpu_baseline_leg(target_s: float = 12.0):
    """The oracle on a bounded sample: as many rows as fit about target_s / 4 seconds, repeated until
    about target_s seconds of CPU work have been spent; the best pass is reported."""
    rows = calibrate_oracle_rows(target_s / 4.0)
    best, spent, passes = None, 0.0, 0
    while passes < 2 or (spent < target_s and passes < 8):
        dt = oracle_chain_rate(rows)
        best = dt if best is None else min(best, dt)
        spent += dt
        passes += 1
    ops = 2.0 * rows * N_DIM * K_DIM
    return {"value": ops / best / 1e12, "unit": "TOPS", "cores": oracle_use_all_cores(), "kind": "port",
            "sample": f"{rows} of {M_ROWS} rows of the same workload (add_rmsnorm_quant -> w8a8_gemm, "
                      f"K={K_DIM}, N={N_DIM}), C oracle with OpenMP on all host threads, best of {passes} passes "
                      f"({best:.2f} s; {spent:.1f} s of CPU work in total)"}


def run_reference_arm(args):
    """The reference's arithmetic on the host cores (C oracle port; the reference is HIP-only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    total_steps = args.steps + args.warmup
    per_step = max(0.05, min(2.0, 100.0 / max(total_steps, 1)))
    rows = calibrate_oracle_rows(per_step)
    for _ in range(args.warmup):
        oracle_chain_rate(rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle_chain_rate(rows)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    ops = 2.0 * rows * N_DIM * K_DIM
    value = ops / dt / 1e12
    sample = (f"{rows} of {M_ROWS} rows per step of add_rmsnorm_quant -> w8a8_gemm (K={K_DIM}, N={N_DIM}); "
              f"C oracle port of the reference arithmetic, OpenMP on all host threads")
    line = {
        "impl": "reference", "metric": "W8A8 quant+GEMM TOPS", "value": value, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": f"add_rmsnorm_quant->w8a8_gemm M={M_ROWS} K={K_DIM} N={N_DIM} per rank",
                   "reference_arm": "CPU oracle on a bounded row sample; the reference has no CPU path and its HIP "
                                    "sources cannot be built on this box"},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": oracle_use_all_cores(), "kind": "port", "sample": sample},
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


def run_ours(args):
    import torch.distributed as dist

    import bw1000_dsv4_kernels_b200 as pkg
    from bw1000_dsv4_kernels_b200 import workloads as wl

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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- inputs: rotating sets, generated on the device --------------------------------
    set_bytes = 2 * M_ROWS * K_DIM * 2 + N_DIM * K_DIM
    nsets = rotation_count(set_bytes)
    sets = []
    for i in range(nsets):
        inp = wl.norm_gemm_inputs(M_ROWS, device=dev, seed=100 * rank + 10 * i)
        sets.append(inp)
    gamma = sets[0].gamma

    def step(i):
        s_ = sets[i % nsets]
        q, sc = ext.add_rmsnorm_quant(s_.res, s_.x, gamma, 1e-6)
        return ext.w8a8_scaled_gemm(q, s_.w, sc, s_.w_scale)

    # The K timed steps are replayed from CUDA graphs of up to 25 steps each (the serving engine
    # this path plugs into replays it from CUDA graphs too); a remainder is launched directly.
    per_graph = min(args.steps, 25)
    n_replays, remainder = args.steps // per_graph, args.steps % per_graph
    sampler = ClockSampler(local_rank)
    with sampler:
        for i in range(max(args.warmup, 3)):
            step(i)
        torch.cuda.synchronize()

        def capture(overlap: bool):
            """A CUDA graph of per_graph steps.  overlap=False: one stream, strictly serial.
            overlap=True: the quantiser of step i+1 (HBM-bound) runs on a second stream beside the GEMM
            of step i (tensor-bound); each GEMM still waits for its own step's quantiser."""
            g = torch.cuda.CUDAGraph()
            alive = []  # keep every intermediate until the capture ends: no block is recycled across streams
            with torch.cuda.graph(g):
                if not overlap:
                    for i in range(per_graph):
                        alive.append(step(i))
                else:
                    main = torch.cuda.current_stream()
                    sq, sg = torch.cuda.Stream(), torch.cuda.Stream()
                    sq.wait_stream(main)
                    sg.wait_stream(main)
                    for i in range(per_graph):
                        s_ = sets[i % nsets]
                        with torch.cuda.stream(sq):
                            q, sc = ext.add_rmsnorm_quant(s_.res, s_.x, gamma, 1e-6)
                            ev = torch.cuda.Event()
                            ev.record(sq)
                        with torch.cuda.stream(sg):
                            sg.wait_event(ev)
                            alive.append((q, sc, ext.w8a8_scaled_gemm(q, s_.w, sc, s_.w_scale)))
                    main.wait_stream(sq)
                    main.wait_stream(sg)
            g.replay()  # one untimed replay: first-use costs of the graph itself
            torch.cuda.synchronize()
            return g, alive

        def time_graph(g):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(n_replays):
                g.replay()
            t1.record()
            t1.synchronize()
            return t0.elapsed_time(t1) / (n_replays * per_graph)

        graph_serial, alive_serial = capture(False)
        ms_serial = time_graph(graph_serial)
        del graph_serial, alive_serial
        # the same serial chain with the GEMM allowed to start (set-up, weight loads) while the
        # quantiser before it is still running (programmatic dependent launch)
        ext.set_overlap_previous_kernel(True)
        try:
            graph_pdl, alive_pdl = capture(False)
            ms_serial_pdl = time_graph(graph_pdl)
            del graph_pdl, alive_pdl
        finally:
            ext.set_overlap_previous_kernel(False)
        graph, alive = capture(True)
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(n_replays):
            graph.replay()
        for i in range(remainder):
            step(i)
        end.record()
        end.synchronize()
        barrier()
        ms_total = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms_total], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_total = float(t.item())
        ms_step = ms_total / args.steps

        if args.chain_only:
            ops_step = 2.0 * M_ROWS * N_DIM * K_DIM
            if rank == 0:
                print(json.dumps({"metric": "W8A8 quant+GEMM TOPS", "value": ops_step * world / (ms_step * 1e-3) / 1e12,
                                  "unit": "TOPS", "ms_per_step": ms_step, "steps": args.steps, "n_gpus": world,
                                  "note": "--chain-only: the timed chain alone (for profiler launch lists)"}), flush=True)
            if world > 1:
                dist.destroy_process_group()
            return

        # ---- per-kernel durations of the same launches (their own timed loops) -----------
        qs = [ext.add_rmsnorm_quant(s_.res, s_.x, gamma, 1e-6) for s_ in sets]
        iters = max(20, min(args.steps, 200))
        ms_quant = time_launches_graph(lambda i: ext.add_rmsnorm_quant(sets[i % nsets].res, sets[i % nsets].x, gamma, 1e-6))
        ms_gemm = time_launches_graph(lambda i: ext.w8a8_scaled_gemm(qs[i % nsets][0], sets[i % nsets].w, qs[i % nsets][1],
                                                                    sets[i % nsets].w_scale))

        # ---- end to end through the operator module with host buffers --------------------
        # Every step copies its x and res from pinned host memory, runs the two operators and copies
        # the output and the updated residual back.  Three streams and two sets of device buffers
        # let step i+1's upload and step i-1's download overlap step i's kernels (PCIe is full
        # duplex); the timed region still contains every copy of every step.
        e2e_steps = max(4, min(args.steps, 40))
        hx = sets[0].x.cpu().pin_memory()
        hres = sets[0].res.cpu().pin_memory()
        houts = [torch.empty((M_ROWS, N_DIM), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        hres_outs = [torch.empty((M_ROWS, K_DIM), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        dxs = [torch.empty_like(sets[0].x) for _ in range(2)]
        dress = [torch.empty_like(sets[0].res) for _ in range(2)]
        s_in, s_comp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_comp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        keep = [None, None]

        def e2e_run(n_steps):
            for i in range(n_steps):
                b = i & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_out[b])          # buffer b's previous download has finished
                    dxs[b].copy_(hx, non_blocking=True)
                    dress[b].copy_(hres, non_blocking=True)
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_comp):
                    s_comp.wait_event(ev_in[b])
                    q, sc = ext.add_rmsnorm_quant(dress[b], dxs[b], gamma, 1e-6)
                    out = ext.w8a8_scaled_gemm(q, sets[i % nsets].w, sc, sets[i % nsets].w_scale)
                    keep[b] = (q, sc, out)
                    ev_comp[b].record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[b])
                    houts[b].copy_(out, non_blocking=True)
                    hres_outs[b].copy_(dress[b], non_blocking=True)
                    ev_out[b].record(s_out)

        cur = torch.cuda.current_stream()
        e2e_run(4)
        torch.cuda.synchronize()
        barrier()
        e2e_start, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_start.record(cur)
        for st_ in (s_in, s_comp, s_out):
            st_.wait_event(e2e_start)
        e2e_run(e2e_steps)
        for st_ in (s_in, s_comp, s_out):
            cur.wait_stream(st_)
        e2e_end.record(cur)
        e2e_end.synchronize()
        ms_e2e = e2e_start.elapsed_time(e2e_end) / e2e_steps
        if world > 1:
            t = torch.tensor([ms_e2e], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())

        extra = {}
        if not args.no_extras:
            try:
                from bw1000_dsv4_kernels_b200 import bench_extras
                extra = bench_extras.run(ext, dev, rank, world, peaks, time_launches, rotation_count, time_launches_graph)
            except Exception as exc:  # extras never take the headline down
                extra = {"error": f"{type(exc).__name__}: {exc}"}

    ops_step = 2.0 * M_ROWS * N_DIM * K_DIM
    value = ops_step * world / (ms_step * 1e-3) / 1e12
    e2e_value = ops_step * world / (ms_e2e * 1e-3) / 1e12
    int8_peak = 2.0 * peaks["bf16_tflops"]
    gemm_tops = ops_step / (ms_gemm * 1e-3) / 1e12
    quant_gbs = quant_bytes_add_rmsnorm(M_ROWS, K_DIM) / (ms_quant * 1e-3) / 1e9

    line = {
        "metric": "W8A8 quant+GEMM TOPS", "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {
            "workload": f"add_rmsnorm_quant->w8a8_gemm M={M_ROWS} K={K_DIM} N={N_DIM} per rank "
                        f"(rows data-parallel across ranks, no collective)",
            "l2": f"inputs and weights rotate through {nsets} buffer sets ({nsets * set_bytes / 1e6:.0f} MB) "
                  f"> 126 MB L2",
            "eps": 1e-6,
            "launch": f"timed steps replayed from CUDA graphs of {per_graph} steps; inside a graph the quantiser of "
                      f"step i+1 runs on a second stream beside the GEMM of step i (independent batches)",
        },
        "roofline": {
            "kernel": "gemm_i8_pair_kernel (tcgen05.mma.cta_group::2.kind::i8, 256x256 tile per CTA pair)", "bound": "tensor", "achieved": gemm_tops,
            "peak": int8_peak, "unit": "TFLOP/s", "frac": gemm_tops / int8_peak,
            "peak_source": f"2 x cuBLAS bf16 burst ({peaks['bf16_tflops']} TF/s, {peaks['source']}); int8 ops; "
                           f"nominal dense int8 4500",
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this shape, from an
            # ncu capture (A and B are read exactly once; most of C is still in L2 when the kernel ends)
            "traffic": 44098560 + 2173440, "algorithmic_bytes": gemm_bytes(M_ROWS, N_DIM, K_DIM),
            "launch_us": ms_gemm * 1e3,
        },
        "kernels": {
            "add_rmsnorm_quant": {"bound": "hbm", "achieved": quant_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": quant_gbs / peaks["hbm_gbs"], "launch_us": ms_quant * 1e3,
                                  "bytes": quant_bytes_add_rmsnorm(M_ROWS, K_DIM),
                                  # from an ncu capture of this launch (the writes are still in L2)
                                  "traffic": 58750208 + 2085376},
        },
        "serial_overlap_option": {"ms_per_step": ms_serial_pdl, "value": ops_step * world / (ms_serial_pdl * 1e-3) / 1e12,
                                  "unit": "TOPS", "note": "one stream; set_overlap_previous_kernel(True): each GEMM starts its "
                                  "set-up and weight loads while the quantiser before it is still running"},
        "serial": {"ms_per_step": ms_serial, "value": ops_step * world / (ms_serial * 1e-3) / 1e12, "unit": "TOPS",
                   "note": "the same chain with every kernel on one stream (no overlap between steps), rank 0's time"},
        "e2e": {"value": e2e_value, "unit": "TOPS", "ms_per_step": ms_e2e, "steps": e2e_steps,
                "how": "pinned host -> device copies of x and res, add_rmsnorm_quant, w8a8_scaled_gemm, device -> host "
                       "copies of the output and the updated residual, every step; upload / kernels / download of "
                       "neighbouring steps overlap on three streams",
                "h2d_bytes_per_step": 2 * M_ROWS * K_DIM * 2, "d2h_bytes_per_step": M_ROWS * N_DIM * 2 + M_ROWS * K_DIM * 2},
        "gpu_launches": 2 * args.steps,
        "clocks": sampler.summary(),
        "extra": extra,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_leg()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_single_kernel(args):
    """`--kernel NAME [--m M]`: launches one kernel of the path `--steps` times on rotating
    inputs and prints its time.  Small, self-terminating: the case profilers capture."""
    import bw1000_dsv4_kernels_b200 as pkg
    from bw1000_dsv4_kernels_b200 import workloads as wl

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
                    help="run one kernel only: gemm, gemm_down, gemm_allgather, grouped, grouped_gs, "
                         "add_rmsnorm_quant, silu_mul_quant, ptq, ptgq, rmsnorm, silu_and_mul, moe_topk, moe_segments, "
                         "gather_rows, moe_combine, moe_combine_exchange")
    ap.add_argument("--m", type=int, default=M_ROWS, help="rows for --kernel")
    ap.add_argument("--graph", action="store_true", help="with --kernel: also time CUDA-graph replays")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-configuration extras")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--chain-only", action="store_true",
                    help="run the warm-up and the timed chain only (short launch list for a profiler)")
    args = ap.parse_args()
    if args.kernel is not None:
        run_single_kernel(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
