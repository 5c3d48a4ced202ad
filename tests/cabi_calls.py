"""Calls into the C-ABI library (include/dsv4_w8a8.h) through ctypes, with torch CUDA
tensors as the device buffers.  The parity tests go through here so that what they
exercise is the boundary a non-Python host would bind."""
import ctypes

import torch

import bw1000_dsv4_kernels_b200 as pkg

_lib = None


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(pkg.LIB_PATH)
        L.dsv4_last_error.restype = ctypes.c_char_p
        _lib = L
    return _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc):
    if rc != 0:
        raise RuntimeError(f"C-ABI status {rc}: {lib().dsv4_last_error().decode()}")


def last_error():
    return lib().dsv4_last_error().decode()


def ptq(x):
    m, n = x.numel() // x.shape[-1], x.shape[-1]
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(m, dtype=torch.float32, device=x.device)
    _check(lib().launch_ptq(_p(x), _p(q), _p(s), m, n, _stream()))
    return q, s.unsqueeze(-1)


def ptq_strided(x):
    """x: 2-D view with unit inner stride"""
    m, n = x.shape
    q = torch.empty((m, n), dtype=torch.int8, device=x.device)
    s = torch.empty(m, dtype=torch.float32, device=x.device)
    _check(lib().launch_ptq_strided(_p(x), ctypes.c_int64(x.stride(0)), _p(q), _p(s), m, n, _stream()))
    return q, s.unsqueeze(-1)


def ptgq(x, gs):
    m, n = x.numel() // x.shape[-1], x.shape[-1]
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    s = torch.empty((m, (n + gs - 1) // gs), dtype=torch.float32, device=x.device)
    _check(lib().launch_ptgq(_p(x), _p(q), _p(s), m, n, gs, _stream()))
    return q, s


def add_rmsnorm_quant(res, x, w, eps):
    m, n = x.shape
    q = torch.empty((m, n), dtype=torch.int8, device=x.device)
    s = torch.empty(m, dtype=torch.float32, device=x.device)
    _check(lib().launch_add_rmsnorm_quant(_p(res), _p(x), _p(w), _p(q), _p(s), m, n, ctypes.c_float(eps), _stream()))
    return q, s.unsqueeze(-1)


def rmsnorm(x, eps):
    m, n = x.shape
    _check(lib().launch_rmsnorm(_p(x), m, n, ctypes.c_float(eps), _stream()))
    return x


def silu_mul(g, u):
    m, n = g.shape
    out = torch.empty((m, n), dtype=torch.bfloat16, device=g.device)
    _check(lib().launch_silu_mul(_p(g), _p(u), _p(out), m, n, _stream()))
    return out


def silu_mul_quant(g, u, mask=None, valid_rows=None):
    m, n = g.shape
    q = torch.zeros((m, n), dtype=torch.int8, device=g.device)
    s = torch.zeros(m, dtype=torch.float32, device=g.device)
    _check(lib().launch_silu_mul_quant_strided(_p(g), ctypes.c_int64(g.stride(0)), _p(u), ctypes.c_int64(u.stride(0)),
                                               _p(mask), _p(valid_rows), _p(q), _p(s), m, n, _stream()))
    return q, s.unsqueeze(-1)


def w8a8_gemm(A, B, sa, sb):
    m, k = A.shape
    n = B.shape[0]
    C = torch.empty((m, n), dtype=torch.bfloat16, device=A.device)
    _check(lib().launch_w8a8_gemm(_p(A), _p(B), _p(sa), _p(sb), _p(C), m, n, k, _stream()))
    return C


def w8a8_gemm_i32(A, B):
    m, k = A.shape
    n = B.shape[0]
    C = torch.empty((m, n), dtype=torch.int32, device=A.device)
    _check(lib().launch_w8a8_gemm_i32(_p(A), _p(B), _p(C), m, n, k, _stream()))
    return C


def scale_convert(acc, sa, sb):
    m, n = acc.shape
    out = torch.empty((m, n), dtype=torch.bfloat16, device=acc.device)
    _check(lib().launch_scale_convert(_p(acc), _p(sa), _p(sb), _p(out), m, n, _stream()))
    return out


def grouped_gemm(A, W, sa, sw, off):
    r, k = A.shape
    e, n, _ = W.shape
    groups = 1 if sa.numel() == r else sa.shape[-1]
    C = torch.zeros((r, n), dtype=torch.bfloat16, device=A.device)
    _check(lib().launch_grouped_gemm(_p(A), _p(W), _p(sa), _p(sw), _p(off), _p(C), r, e, n, k, groups, _stream()))
    return C


def moe_segments(ids, num_experts, expert_lo=0):
    t, topk = ids.shape
    off = torch.empty(num_experts + 1, dtype=torch.int32, device=ids.device)
    src = torch.full((t * topk,), -1, dtype=torch.int32, device=ids.device)
    dst = torch.empty(t * topk, dtype=torch.int32, device=ids.device)
    _check(lib().launch_moe_segments(_p(ids), t, topk, num_experts, expert_lo, _p(off), _p(src), _p(dst), _stream()))
    return off, src, dst


def moe_topk(logits, k):
    t, e = logits.shape
    ids = torch.empty((t, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((t, k), dtype=torch.float32, device=logits.device)
    _check(lib().launch_moe_topk(_p(logits), t, e, k, _p(ids), _p(w), _stream()))
    return ids, w


def moe_combine(z, dst_slot, topk_w, out_f32=False):
    t, topk = topk_w.shape
    out = torch.empty((t, z.shape[1]), dtype=torch.float32 if out_f32 else torch.bfloat16, device=z.device)
    _check(lib().launch_moe_combine(_p(z), _p(dst_slot), _p(topk_w), _p(out), t, topk, z.shape[1], int(out_f32),
                                    _stream()))
    return out


def w8a8_gemm_ld(A, B, sa, sb, out, col0):
    m, k = A.shape
    n = B.shape[0]
    base = ctypes.c_void_p(out.data_ptr() + 2 * col0)
    _check(lib().launch_w8a8_gemm_ld(_p(A), _p(B), _p(sa), _p(sb), base, ctypes.c_int64(out.stride(0)), m, n, k,
                                     _stream()))
    return out


def gather_rows(src, src_row, scales=None, valid_rows=None):
    r = src_row.numel()
    dst = torch.empty((r, src.shape[1]), dtype=src.dtype, device=src.device)
    ds = None
    spr = 0
    if scales is not None:
        spr = scales.shape[1]
        ds = torch.empty((r, spr), dtype=torch.float32, device=src.device)
    _check(lib().launch_gather_rows(_p(src), _p(src_row), _p(dst), r, src.shape[1] * src.element_size(), _p(scales),
                                    _p(ds), spr, _p(valid_rows), _stream()))
    return dst, ds


def device_status():
    v = ctypes.c_int(0)
    _check(lib().dsv4_device_status(_stream(), ctypes.byref(v)))
    return v.value
