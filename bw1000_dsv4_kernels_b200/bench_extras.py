"""Per-configuration measurements that accompany the headline benchmark line: every kernel
of the W8A8 path at the benchmark shapes, with its algorithmic bytes or ops, its CUDA-event
time and its fraction of the measured roofline.  Called by bench.py; returns a dict.

Inputs are generated on the device and rotated through enough buffer sets to exceed L2
wherever one set is smaller than L2, so HBM-bound numbers are not L2 numbers.
"""
import torch

from . import workloads as wl

HBM = "hbm"
TENSOR = "tensor"


def _entry(us, peaks, bytes_=None, ops=None):
    out = {"us": round(us, 3)}
    if bytes_ is not None:
        gbs = bytes_ / (us * 1e-6) / 1e9
        out.update({"bytes": int(bytes_), "GBps": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 4)})
    if ops is not None:
        tops = ops / (us * 1e-6) / 1e12
        out.update({"ops": float(ops), "TOPS": round(tops, 1), "tensor_frac": round(tops / (2.0 * peaks["bf16_tflops"]), 4)})
    return out


def _iters(us_guess):
    return int(max(10, min(200, 20000 / max(us_guess, 1.0))))


def run(ext, dev, rank, world, peaks, time_launches, rotation_count):
    res = {}
    K, N1, I, H = wl.HIDDEN, wl.DENSE_N, wl.DENSE_INTER, wl.HIDDEN

    # ---- per_token_quant_int8 ------------------------------------------------------------
    sec = {}
    for m in (64, 2048, 8192):
        nb = m * K * 2
        n = rotation_count(nb * 3 // 2)
        xs = [wl.activations_with_outliers(m, K, device=dev, seed=i) for i in range(n)]
        us = 1e3 * time_launches(lambda i: ext.per_token_quant_int8(xs[i % n]), 100)
        sec[f"M={m}"] = _entry(us, peaks, bytes_=3 * m * K + 4 * m)
        del xs
    res["per_token_quant_int8 K=7168"] = sec

    # ---- per_token_group_quant_int8 ------------------------------------------------------
    sec = {}
    for m in (4096,):
        n = rotation_count(m * K * 3)
        xs = [wl.randn_bf16((m, K), device=dev, seed=i) for i in range(n)]
        us = 1e3 * time_launches(lambda i: ext.per_token_group_quant_int8(xs[i % n], 128), 100)
        sec[f"M={m}"] = _entry(us, peaks, bytes_=3 * m * K + 4 * m * (K // 128))
        del xs
    res["per_token_group_quant_int8 K=7168 gs=128"] = sec

    # ---- add_rmsnorm_quant -> w8a8_gemm --------------------------------------------------
    w_sets = [wl.int8_weights((N1, K), device=dev, seed=50 + i) for i in range(5)]
    w_scale = wl.channel_scales((N1,), device=dev, seed=60)
    gamma = wl.gamma_bf16(K, device=dev, seed=2)
    quant_sec, gemm_sec = {}, {}
    for m in (1, 16, 64, 256, 2048):
        nb = 2 * m * K * 2 + m * K
        n = rotation_count(nb)
        n = min(n, 48)
        xs = [wl.randn_bf16((m, K), device=dev, seed=i) for i in range(n)]
        rs = [wl.randn_bf16((m, K), device=dev, seed=100 + i) for i in range(n)]
        us = 1e3 * time_launches(lambda i: ext.add_rmsnorm_quant(rs[i % n], xs[i % n], gamma, 1e-6), 100)
        quant_sec[f"M={m}"] = _entry(us, peaks, bytes_=m * (7 * K + 4) + 2 * K)
        qs = [ext.add_rmsnorm_quant(rs[i], xs[i], gamma, 1e-6) for i in range(min(n, 5))]
        nq = len(qs)
        us = 1e3 * time_launches(lambda i: ext.w8a8_scaled_gemm(qs[i % nq][0], w_sets[i % 5], qs[i % nq][1], w_scale), 100)
        gemm_sec[f"M={m}"] = _entry(us, peaks, bytes_=m * K + N1 * K + 2 * m * N1 + 4 * (m + N1), ops=2.0 * m * N1 * K)
        del xs, rs, qs
    res["add_rmsnorm_quant K=7168"] = quant_sec
    res["w8a8_gemm N=4096 K=7168"] = gemm_sec
    # cuBLASLt through torch._int_mm on the same operands, int32 output, no scale epilogue: a
    # library reference point only, not part of the product path
    try:
        a = wl.int8_weights((2048, K), device=dev, seed=7)
        us = 1e3 * time_launches(lambda i: torch._int_mm(a, w_sets[i % 5].t()), 50)
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
        us = 1e3 * time_launches(lambda i: ext.silu_mul_quant(gus[i % n][:, :I], gus[i % n][:, I:]), _iters(100 if m > 64 else 5))
        silu_sec[f"M={m}"] = _entry(us, peaks, bytes_=m * (5 * I + 4))
        q, s = ext.silu_mul_quant(gus[0][:, :I], gus[0][:, I:])
        del gus
        us = 1e3 * time_launches(lambda i: ext.w8a8_scaled_gemm(q, wd_sets[i % 2], s, wd_scale), _iters(150 if m > 64 else 30))
        down_sec[f"M={m}"] = _entry(us, peaks, bytes_=m * I + H * I + 2 * m * H + 4 * (m + H), ops=2.0 * m * H * I)
        del q, s
    res["silu_mul_quant N=18432"] = silu_sec
    res["w8a8_gemm N=7168 K=18432"] = down_sec
    del wd_sets
    torch.cuda.empty_cache()
    return res
