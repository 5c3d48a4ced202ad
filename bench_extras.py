"""Per-configuration measurements that accompany the headline benchmark line: every kernel
of the W8A8 path at the benchmark shapes, with its algorithmic bytes or ops, its CUDA-event
time and its fraction of the measured roofline.  Called by bench.py; returns a dict.

Inputs are generated on the device and rotated through enough buffer sets to exceed L2
wherever one set is smaller than L2, so HBM-bound numbers are not L2 numbers.
"""
import torch

from tests import workloads as wl

HBM = "hbm"
TENSOR = "tensor"


def _entry(us, peaks, bytes_=None, ops=None, us_host_loop=None):
    """`us` is the device time per launch (CUDA-graph replay where given); `us_host_loop` the
    time per call when every call is launched from Python (adds the host's per-call cost)."""
    out = {"us": round(us, 3)}
    if us_host_loop is not None:
        out["us_host_loop"] = round(us_host_loop, 3)
    if bytes_ is not None:
        gbs = bytes_ / (us * 1e-6) / 1e9
        out.update({"bytes": int(bytes_), "GBps": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 4)})
    if ops is not None:
        tops = ops / (us * 1e-6) / 1e12
        out.update({"ops": float(ops), "TOPS": round(tops, 1), "tensor_frac": round(tops / (2.0 * peaks["bf16_tflops"]), 4)})
    return out


def _hold(fn, n):
    """fn with its last n results kept alive, so that the outputs rotate through as many buffers as
    the inputs do (a freed output would be handed out again at once and stay in L2)."""
    keep = [None] * max(1, n)

    def call(i):
        keep[i % len(keep)] = fn(i)

    return call


def _iters(us_guess):
    return int(max(10, min(200, 20000 / max(us_guess, 1.0))))


def run(ext, dev, rank, world, peaks, time_launches, rotation_count, time_launches_graph, timer=None):
    res = {"timing": "us = per-launch device time from CUDA-graph replays of 20 launches over rotating buffers; "
                     "us_host_loop = per-call time when launched one by one from Python"}

    def both(fn, iters=100):
        loop_us = 1e3 * time_launches(fn, iters)
        graph_us = 1e3 * time_launches_graph(fn)
        return graph_us, loop_us

    K, N1, I, H = wl.HIDDEN, wl.DENSE_N, wl.DENSE_INTER, wl.HIDDEN

    def copy_same_bytes(entry):
        """Context for an HBM-bound entry: a library elementwise kernel (torch.neg on int32) that moves the same
        total bytes (half read, half written), over rotating buffers and timed the same way.  How far below
        the peak a plain pass of this size sits is what launch, ramp and tail cost at this size.  (A
        device-to-device copy_ is not used: inside a graph it may run on a copy engine.)"""
        half = max(1 << 20, entry["bytes"] // 2) // 16 * 16
        n = max(2, rotation_count(2 * half))
        src = [torch.empty(half // 4, dtype=torch.int32, device=dev).random_(0, 255) for _ in range(n)]
        dst = [torch.empty(half // 4, dtype=torch.int32, device=dev) for _ in range(n)]
        us = 1e3 * time_launches_graph(lambda i: torch.neg(src[i % n], out=dst[i % n]))
        entry["copy_same_bytes_us"] = round(us, 3)
        entry["frac_of_copy_same_bytes"] = round(us / entry["us"], 4)
        return entry

    # ---- per_token_quant_int8 ------------------------------------------------------------
    sec = {}
    for m in (64, 2048, 8192):
        nb = m * K * 2
        n = rotation_count(nb * 3 // 2)
        xs = [wl.activations_with_outliers(m, K, device=dev, seed=i) for i in range(n)]
        us, lp = both(_hold(lambda i: ext.per_token_quant_int8(xs[i % n]), n))
        sec[f"M={m}"] = _entry(us, peaks, bytes_=3 * m * K + 4 * m, us_host_loop=lp)
        del xs
        if m >= 2048:
            copy_same_bytes(sec[f"M={m}"])
    res["per_token_quant_int8 K=7168"] = sec

    # ---- per_token_group_quant_int8 ------------------------------------------------------
    sec = {}
    for m in (4096,):
        n = rotation_count(m * K * 3)
        xs = [wl.randn_bf16((m, K), device=dev, seed=i) for i in range(n)]
        us, lp = both(_hold(lambda i: ext.per_token_group_quant_int8(xs[i % n], 128), n))
        sec[f"M={m}"] = _entry(us, peaks, bytes_=3 * m * K + 4 * m * (K // 128), us_host_loop=lp)
        del xs
        copy_same_bytes(sec[f"M={m}"])
    res["per_token_group_quant_int8 K=7168 gs=128"] = sec

    # ---- add_rmsnorm_quant -> w8a8_gemm --------------------------------------------------
    NW = 8   # 8 x 29 MB of weights: far beyond the 126 MB L2
    w_sets = [wl.int8_weights((N1, K), device=dev, seed=50 + i) for i in range(NW)]
    w_scale = wl.channel_scales((N1,), device=dev, seed=60)
    gamma = wl.gamma_bf16(K, device=dev, seed=2)
    quant_sec, gemm_sec = {}, {}
    for m in (1, 16, 64, 256, 2048):
        nb = 2 * m * K * 2 + m * K
        n = rotation_count(nb)
        n = min(n, 48)
        xs = [wl.randn_bf16((m, K), device=dev, seed=i) for i in range(n)]
        rs = [wl.randn_bf16((m, K), device=dev, seed=100 + i) for i in range(n)]
        us, lp = both(_hold(lambda i: ext.add_rmsnorm_quant(rs[i % n], xs[i % n], gamma, 1e-6), n))
        quant_sec[f"M={m}"] = _entry(us, peaks, bytes_=m * (7 * K + 4) + 2 * K, us_host_loop=lp)
        if m >= 2048:
            copy_same_bytes(quant_sec[f"M={m}"])
        qs = [ext.add_rmsnorm_quant(rs[i], xs[i], gamma, 1e-6) for i in range(min(n, 5))]
        nq = len(qs)
        us, lp = both(lambda i: ext.w8a8_scaled_gemm(qs[i % nq][0], w_sets[i % NW], qs[i % nq][1], w_scale))
        gemm_sec[f"M={m}"] = _entry(us, peaks, bytes_=m * K + N1 * K + 2 * m * N1 + 4 * (m + N1), ops=2.0 * m * N1 * K,
                                    us_host_loop=lp)
        del xs, rs, qs
    res["add_rmsnorm_quant K=7168"] = quant_sec
    res["w8a8_gemm N=4096 K=7168"] = gemm_sec
    # the dependent chain at decode sizes, strictly serialised and with the GEMM allowed to overlap
    # the quantiser before it (set-up and weight loads start early; see set_overlap_previous_kernel)
    chain_sec = {}
    for m in (1, 16, 64, 256, 2048):
        n = 6
        xs = [wl.randn_bf16((m, K), device=dev, seed=i) for i in range(n)]
        rs = [wl.randn_bf16((m, K), device=dev, seed=100 + i) for i in range(n)]

        def step(i):
            q, s = ext.add_rmsnorm_quant(rs[i % n], xs[i % n], gamma, 1e-6)
            return ext.w8a8_scaled_gemm(q, w_sets[i % NW], s, w_scale)

        def lone(i):
            return ext.w8a8_scaled_gemm(qs1[0], w_sets[i % NW], qs1[1], w_scale)

        qs1 = ext.add_rmsnorm_quant(rs[0].clone(), xs[0], gamma, 1e-6)
        us_serial = 1e3 * time_launches_graph(step)
        try:
            ext.set_overlap_previous_kernel(True)
            us_overlap = 1e3 * time_launches_graph(step)
            us_gemm_overlap = 1e3 * time_launches_graph(lone)
        finally:
            ext.set_overlap_previous_kernel(False)
        chain_sec[f"M={m}"] = {"us_per_step": round(us_serial, 3), "us_per_step_overlap": round(us_overlap, 3),
                               "us_gemm_back_to_back_overlap": round(us_gemm_overlap, 3)}
        del xs, rs, qs1
    res["chain add_rmsnorm_quant->w8a8_gemm N=4096 K=7168 (decode sizes)"] = chain_sec
    # cuBLASLt through torch._int_mm on the same operands, int32 output, no scale epilogue: a
    # library reference point only, not part of the product path
    try:
        a = wl.int8_weights((2048, K), device=dev, seed=7)
        us = 1e3 * time_launches(lambda i: torch._int_mm(a, w_sets[i % NW].t()), 50)
        res["library torch._int_mm M=2048 N=4096 K=7168 (int32 out, no epilogue)"] = _entry(us, peaks, ops=2.0 * 2048 * N1 * K)
        del a
    except Exception as exc:  # pragma: no cover
        res["library torch._int_mm"] = {"error": str(exc)}
    del w_sets

    # ---- silu_mul_quant -> down projection -----------------------------------------------
    wd_sets = [wl.int8_weights((H, I), device=dev, seed=70 + i) for i in range(2)]
    wd_scale = wl.channel_scales((H,), device=dev, seed=80)
    silu_sec, down_sec = {}, {}
    for m in (64, 2048, 8192):
        nb = m * 2 * I * 2
        n = max(2, min(rotation_count(nb), 24)) if m < 8192 else 2
        gus = [wl.randn_bf16((m, 2 * I), device=dev, seed=i) for i in range(n)]
        us, lp = both(_hold(lambda i: ext.silu_mul_quant(gus[i % n][:, :I], gus[i % n][:, I:]), n), _iters(100 if m > 64 else 5))
        silu_sec[f"M={m}"] = _entry(us, peaks, bytes_=m * (5 * I + 4), us_host_loop=lp)
        q, s = ext.silu_mul_quant(gus[0][:, :I], gus[0][:, I:])
        del gus
        if m == 2048:
            copy_same_bytes(silu_sec[f"M={m}"])
        us, lp = both(lambda i: ext.w8a8_scaled_gemm(q, wd_sets[i % 2], s, wd_scale), _iters(150 if m > 64 else 30))
        down_sec[f"M={m}"] = _entry(us, peaks, bytes_=m * I + H * I + 2 * m * H + 4 * (m + H), ops=2.0 * m * H * I,
                                    us_host_loop=lp)
        del q, s
    res["silu_mul_quant N=18432"] = silu_sec
    res["w8a8_gemm N=7168 K=18432"] = down_sec
    del wd_sets
    torch.cuda.empty_cache()

    try:
        res["moe_ffn T=4096 E=256 I=2048 top8"] = _moe_section(ext, dev, rank, world, peaks, timer, time_launches_graph)
    except Exception as exc:  # pragma: no cover
        res["moe_ffn"] = {"error": f"{type(exc).__name__}: {exc}"}
    torch.cuda.empty_cache()
    return res


def _moe_reference_rows(ext, tokens, x, topk_ids, topk_w, dev, group_scaled):
    """The single-GPU chain for a few tokens, recomputed on this device with one launch per routed
    (token, expert) pair: the expert's weights are regenerated from their seed, the token goes
    through quantiser -> gate/up GEMM -> silu_mul_quant -> down GEMM as a one-row batch, and the
    token's rows are summed by moe_combine in slot order.  Different launch shapes from the layer
    (one row, one expert), same arithmetic: the result must equal the layer's rows bit for bit."""
    H, I, topk = wl.HIDDEN, wl.MOE_INTER, wl.MOE_TOPK
    rows = []
    off = torch.tensor([0, 1], dtype=torch.int32, device=dev)
    for t in tokens:
        xt = x[t:t + 1].contiguous()
        if group_scaled:
            q, s = ext.per_token_group_quant_int8(xt, 128)
        else:
            q, s = ext.per_token_quant_int8(xt)
        zs = []
        for j in range(topk):
            e = int(topk_ids[t, j])
            base = 1000 + 4 * e
            w13 = wl.int8_weights((2 * I, H), dev, base).unsqueeze(0)      # the seeds moe_inputs gives expert e
            w2 = wl.int8_weights((H, I), dev, base + 1).unsqueeze(0)
            s13 = wl.channel_scales((2 * I,), dev, base + 2).unsqueeze(0)
            s2 = wl.channel_scales((H,), dev, base + 3).unsqueeze(0)
            y = ext.grouped_gemm(q, w13, s, s13, off)
            hq, hs = ext.silu_mul_quant(y[:, :I], y[:, I:])
            zs.append(ext.grouped_gemm(hq, w2, hs, s2, off))
        z = torch.cat(zs)
        slot = torch.arange(topk, dtype=torch.int32, device=dev).view(1, topk)
        rows.append(ext.moe_combine(z, slot.contiguous(), topk_w[t:t + 1].contiguous(), False))
    return torch.cat(rows)


def _moe_section(ext, dev, rank, world, peaks, timer, time_launches_graph):
    """MoE FFN, experts sharded over the ranks (expert parallel), tokens and routing replicated.
    Weight-bandwidth-bound: ~128 routed rows per expert against 44 MB of int8 weights per expert.
    Times are medians over repeats of 10 forward calls, max over ranks per repeat."""
    from bw1000_dsv4_kernels_b200 import moe
    T, H, E, I, topk = wl.MOE_TOKENS, wl.HIDDEN, wl.MOE_EXPERTS, wl.MOE_INTER, wl.MOE_TOPK
    lo, hi = moe.expert_range(rank, world, E)
    inp = wl.moe_inputs(T, H, E, I, topk, device=dev, seed=0, expert_lo=lo, expert_hi=hi)
    out = {}
    K_CALLS, REPEATS = 10, 7

    def med(fn):
        t = timer.run(fn, K_CALLS, REPEATS, warmup=2)
        return {"ms": round(t["ms_per_step"], 4), "ms_min": round(t["ms_per_step_min"], 4), "ms_max": round(t["ms_per_step_max"], 4)}

    for name, gs in (("group_scaled", True), ("per_token", False)):
        layer = moe.W8A8MoE(inp.w13, inp.w13_scale, inp.w2, inp.w2_scale, E, expert_lo=lo, group_scaled=gs)
        part = lambda i: layer.local_partial(inp.x, inp.topk_ids, inp.topk_w, out_f32=(world > 1))
        t_local = med(part)
        rows_total = T * topk
        ops = 2.0 * rows_total * (2 * I * H + H * I)
        w_bytes = (hi - lo) * (2 * I * H + H * I)
        sec = {
            "local_experts": t_local,
            # the same chain replayed from a CUDA graph: device time without the host's launch cost (nine
            # launches and two dozen tensor-map encodes per forward)
            "local_experts_graph_replay_ms": round(time_launches_graph(part, 4, 9), 4),
            "weight_GBps_per_rank": None, "weight_hbm_frac": None,
            "experts_per_rank": hi - lo, "ranks": world,
        }
        g_ms = sec["local_experts_graph_replay_ms"]
        sec["weight_GBps_per_rank"] = round(w_bytes / (g_ms * 1e-3) / 1e9, 1)
        sec["weight_hbm_frac"] = round(w_bytes / (g_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        if world == 1:
            sec["TOPS_whole_job"] = round(ops / (g_ms * 1e-3) / 1e12, 1)
            y = layer.forward(inp.x, inp.topk_ids, inp.topk_w)
        else:
            t_ar = med(lambda i: layer.forward(inp.x, inp.topk_ids, inp.topk_w))
            sec["with_nccl_allreduce"] = t_ar
            y = None
            try:
                # combine fused with the exchange over peer memory instead of fp32 partials + all-reduce
                ex = moe.ExchangeW8A8MoE(inp.w13, inp.w13_scale, inp.w2, inp.w2_scale, E, rank, world, t_max=T,
                                         topk=topk, device=dev, group_scaled=gs)
                t_ex = med(lambda i: ex.forward(inp.x, inp.topk_ids, inp.topk_w))
                sec["with_fused_exchange"] = t_ex
                sec["TOPS_whole_job"] = round(ops / (t_ex["ms"] * 1e-3) / 1e12, 1)
                y = ex.forward(inp.x, inp.topk_ids, inp.topk_w).clone()
                del ex
                # the down GEMM stores every row into the inbox of the token's owner; the combine reads local memory
                push = moe.PushExchangeW8A8MoE(inp.w13, inp.w13_scale, inp.w2, inp.w2_scale, E, rank, world, t_max=T,
                                               topk=topk, device=dev, group_scaled=gs)
                t_push = med(lambda i: push.forward(inp.x, inp.topk_ids, inp.topk_w))
                sec["with_rows_pushed_by_down_gemm"] = t_push
                y_push = push.forward(inp.x, inp.topk_ids, inp.topk_w).clone()
                torch.cuda.synchronize()
                sec["pushed_rows_equal_fused_exchange"] = bool(torch.equal(y_push.view(torch.int16), y.view(torch.int16)))
                if t_push["ms"] < t_ex["ms"]:
                    sec["TOPS_whole_job"] = round(ops / (t_push["ms"] * 1e-3) / 1e12, 1)
                del push
            except Exception as exc:  # pragma: no cover
                sec["fused_exchange_error"] = f"{type(exc).__name__}: {exc}"
                sec.setdefault("TOPS_whole_job", round(ops / (t_ar["ms"] * 1e-3) / 1e12, 1))
        if y is not None:
            # parity inside the run: a few of this rank's tokens against the one-GPU chain recomputed here
            t0, t1 = moe.token_range(rank, world, T)
            tokens = [t0, (t0 + t1) // 2, t1 - 1]
            ref = _moe_reference_rows(ext, tokens, inp.x, inp.topk_ids, inp.topk_w, dev, gs)
            torch.cuda.synchronize()
            ok = bool(torch.equal(y[tokens].contiguous().view(torch.int16), ref.view(torch.int16)))
            if world > 1:
                import torch.distributed as dist
                f = torch.tensor([1 if ok else 0], device=dev)
                dist.all_reduce(f, op=dist.ReduceOp.MIN)
                ok = bool(int(f.item()))
            sec["parity_ok"] = ok
            sec["parity"] = "3 tokens per rank recomputed with one-row launches from regenerated expert weights, bit for bit"
        out[name] = sec
        del layer
    # stage breakdown of the group-scaled chain on this rank
    layer = moe.W8A8MoE(inp.w13, inp.w13_scale, inp.w2, inp.w2_scale, E, expert_lo=lo, group_scaled=True)
    layer.local_partial(inp.x, inp.topk_ids, inp.topk_w, out_f32=False, keep_trace=True)
    tr = layer.last_trace
    q, sg = ext.per_token_group_quant_int8(inp.x, 128)
    valid = tr.offsets[hi - lo:]
    logits = torch.randn((T, E), device=dev, generator=torch.Generator(device=dev).manual_seed(0))
    stages = {
        "moe_topk": lambda i: ext.moe_topk(logits, topk),
        "per_token_group_quant_int8": lambda i: ext.per_token_group_quant_int8(inp.x, 128),
        "moe_segments": lambda i: ext.moe_segments(inp.topk_ids, hi - lo, lo),
        "gather_rows": lambda i: ext.gather_rows(q, tr.src_row, sg, valid),
        "grouped_gemm gate_up": lambda i: ext.grouped_gemm(tr.a_q, inp.w13, tr.a_s, inp.w13_scale, tr.offsets),
        "silu_mul_quant": lambda i: ext.silu_mul_quant_rows(tr.y[:, :I], tr.y[:, I:], valid),
        "grouped_gemm down": lambda i: ext.grouped_gemm(tr.h_q, inp.w2, tr.h_s, inp.w2_scale, tr.offsets),
        "moe_combine": lambda i: ext.moe_combine(tr.z, tr.dst_slot, inp.topk_w, False),
    }
    out["stages_us_rank0"] = {k: round(1e3 * time_launches_graph(f, 10, 7), 1) for k, f in stages.items()}
    return out
