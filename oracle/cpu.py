"""ctypes front end of the C oracle (oracle/w8a8_oracle.c).  Test infrastructure only.

All functions take and return CPU torch tensors (bf16 / int8 / float32 / int32) so that
a test can feed the same seeded tensors to the oracle and, after .cuda(), to the kernels.
"""
import ctypes
import functools

import torch

from . import build_oracle

_c_i8p = ctypes.c_void_p


@functools.lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    path = build_oracle.build()
    L = ctypes.CDLL(path)
    L.oracle_exp.restype = ctypes.c_float
    L.oracle_exp.argtypes = [ctypes.c_float]
    return L


def set_num_threads(n: int) -> int:
    """OpenMP threads the oracle uses (0 = leave unchanged); returns the count in effect."""
    return int(lib().oracle_set_num_threads(ctypes.c_int(n)))


def _p(t: torch.Tensor) -> ctypes.c_void_p:
    assert t.device.type == "cpu" and t.is_contiguous(), "oracle takes contiguous CPU tensors"
    return ctypes.c_void_p(t.data_ptr())


def _rows(x: torch.Tensor):
    n = x.shape[-1]
    return (x.numel() // n if n else 0), n


def per_token_quant_int8(x: torch.Tensor, divide_form: bool = False):
    """-> (q int8 like x, s float32 [M,1]).  divide_form=True uses round(x/s) clamped to +-127."""
    assert x.dtype == torch.bfloat16
    x = x.contiguous()
    m, n = _rows(x)
    q = torch.empty(x.shape, dtype=torch.int8)
    s = torch.empty(m, dtype=torch.float32)
    fn = lib().oracle_ptq_divide_form if divide_form else lib().oracle_ptq
    fn(_p(x), ctypes.c_int64(n), _p(q), _p(s), ctypes.c_int(m), ctypes.c_int(n))
    return q, s.unsqueeze(-1)


def per_token_group_quant_int8(x: torch.Tensor, group_size: int):
    """-> (q int8 like x, s float32 [M, ceil(N/group_size)])."""
    assert x.dtype == torch.bfloat16
    x = x.contiguous()
    m, n = _rows(x)
    g = (n + group_size - 1) // group_size
    q = torch.empty(x.shape, dtype=torch.int8)
    s = torch.empty((m, g), dtype=torch.float32)
    lib().oracle_ptgq(_p(x), _p(q), _p(s), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(group_size))
    return q, s


def add_rmsnorm_quant(res: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float):
    """Mutates res (res <- res + x) like the operator; -> (q, s [M,1])."""
    assert res.dtype == x.dtype == w.dtype == torch.bfloat16 and res.is_contiguous()
    x = x.contiguous()
    w = w.contiguous()
    m, n = _rows(x)
    q = torch.empty(x.shape, dtype=torch.int8)
    s = torch.empty(m, dtype=torch.float32)
    lib().oracle_add_rmsnorm_quant(_p(res), _p(x), _p(w), _p(q), _p(s), ctypes.c_int(m), ctypes.c_int(n),
                                   ctypes.c_float(eps))
    return q, s.unsqueeze(-1)


def rmsnorm(x: torch.Tensor, eps: float):
    """In place, no gamma; returns x."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    m, n = _rows(x)
    lib().oracle_rmsnorm(_p(x), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_float(eps))
    return x


def _gate_up(gate, up):
    assert gate.dtype == up.dtype == torch.bfloat16 and gate.dim() == 2 and gate.shape == up.shape
    assert gate.stride(1) == 1 and up.stride(1) == 1
    return gate.shape[0], gate.shape[1], gate.stride(0), up.stride(0)


def silu_and_mul(gate: torch.Tensor, up: torch.Tensor):
    m, n, ldg, ldu = _gate_up(gate, up)
    out = torch.empty((m, n), dtype=torch.bfloat16)
    lib().oracle_silu_mul(ctypes.c_void_p(gate.data_ptr()), ctypes.c_int64(ldg), ctypes.c_void_p(up.data_ptr()),
                          ctypes.c_int64(ldu), _p(out), ctypes.c_int(m), ctypes.c_int(n))
    return out


def silu_mul_quant(gate: torch.Tensor, up: torch.Tensor, mask: torch.Tensor = None, q=None, s=None):
    """gate/up may be row-strided halves of a packed [M,2N] tensor.  -> (q, s [M,1])."""
    m, n, ldg, ldu = _gate_up(gate, up)
    if q is None:
        q = torch.zeros((m, n), dtype=torch.int8)
    if s is None:
        s = torch.zeros(m, dtype=torch.float32)
    s_flat = s.view(-1)
    mp = ctypes.c_void_p(0) if mask is None else _p(mask.to(torch.int32).contiguous())
    lib().oracle_silu_mul_quant(ctypes.c_void_p(gate.data_ptr()), ctypes.c_int64(ldg),
                                ctypes.c_void_p(up.data_ptr()), ctypes.c_int64(ldu), mp, _p(q), _p(s_flat),
                                ctypes.c_int(m), ctypes.c_int(n))
    return q, s_flat.unsqueeze(-1)


def gemm_i32(A: torch.Tensor, B: torch.Tensor):
    assert A.dtype == B.dtype == torch.int8
    A, B = A.contiguous(), B.contiguous()
    m, k = A.shape
    n = B.shape[0]
    C = torch.empty((m, n), dtype=torch.int32)
    lib().oracle_gemm_i32(_p(A), _p(B), _p(C), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k))
    return C


def scale_convert(acc: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor):
    m, n = acc.shape
    out = torch.empty((m, n), dtype=torch.bfloat16)
    lib().oracle_scale_convert(_p(acc.contiguous()), _p(sa.contiguous().view(-1).float()),
                               _p(sb.contiguous().view(-1).float()), _p(out), ctypes.c_int(m), ctypes.c_int(n))
    return out


def w8a8_gemm(A, B, sa, sb):
    A, B = A.contiguous(), B.contiguous()
    m, k = A.shape
    n = B.shape[0]
    out = torch.empty((m, n), dtype=torch.bfloat16)
    lib().oracle_w8a8_gemm(_p(A), _p(B), _p(sa.contiguous().view(-1)), _p(sb.contiguous().view(-1)), _p(out),
                           ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k))
    return out


def grouped_gemm(A, W, sa, sw, expert_offsets):
    """A int8 [R,K] sorted by expert, W int8 [E,N,K], sa [R] / [R,1] or [R,K/128], sw [E,N]."""
    A, W = A.contiguous(), W.contiguous()
    r, k = A.shape
    e, n, _ = W.shape
    sa = sa.contiguous().float()
    groups = 1 if sa.numel() == r else sa.shape[-1]
    out = torch.zeros((r, n), dtype=torch.bfloat16)
    lib().oracle_grouped_gemm(_p(A), _p(W), _p(sa), _p(sw.contiguous()), _p(expert_offsets.to(torch.int32).contiguous()),
                              _p(out), ctypes.c_int(r), ctypes.c_int(e), ctypes.c_int(n), ctypes.c_int(k),
                              ctypes.c_int(groups))
    return out


def masked_row_flags(masked_m: torch.Tensor, max_m: int):
    """Per-row flags [E * max_m] of the masked expert layout: row i of block e is valid iff i < masked_m[e]."""
    m = masked_m.to(torch.int64).clamp(0, max_m).view(-1, 1)
    return (torch.arange(max_m).view(1, -1) < m).to(torch.int32).reshape(-1)


def silu_and_mul_masked_post_quant(gate: torch.Tensor, up: torch.Tensor, masked_m: torch.Tensor):
    """Masked expert layout (the engine op of DSV4_OPERATOR_ANALYSIS.md:45): gate, up [E, max_m, N],
    masked_m [E].  The reference kernel takes per-row flags (dsv4_all_hip_kernels.hip:172-196); the flags
    here are i < masked_m[e].  -> (q [E, max_m, N], s [E, max_m, 1]), zero in the skipped rows."""
    e, max_m, n = gate.shape
    flags = masked_row_flags(masked_m, max_m)
    q, s = silu_mul_quant(gate.reshape(e * max_m, n), up.reshape(e * max_m, n), flags)
    return q.view(e, max_m, n), s.view(e, max_m, 1)


def grouped_gemm_masked(A, W, sa, sw, masked_m, out=None):
    """Masked expert layout (the engine op of DSV4_OPERATOR_ANALYSIS.md:43; no source in the reference):
    A int8 [E, max_m, K], W int8 [E, N, K], sa [E, max_m] or [E, max_m, K/128], sw [E, N], masked_m [E].
    Expert e multiplies its first masked_m[e] rows (arithmetic of grouped_gemm); other rows of `out`
    (zero if not given) are left as they are."""
    e, max_m, k = A.shape
    n = W.shape[1]
    if out is None:
        out = torch.zeros((e, max_m, n), dtype=torch.bfloat16)
    sa = sa.contiguous().float().view(e, max_m, -1)
    for i in range(e):
        m = int(min(max(int(masked_m[i]), 0), max_m))
        if m == 0:
            continue
        s_i = sa[i, :m]
        s_i = s_i.reshape(-1) if s_i.shape[-1] == 1 else s_i
        out[i, :m] = grouped_gemm(A[i, :m], W[i:i + 1], s_i, sw[i:i + 1], torch.tensor([0, m], dtype=torch.int32))
    return out


def moe_segments(topk_ids: torch.Tensor, num_experts: int, expert_lo: int = 0):
    """-> (offsets [E+1], src_row [T*topk] (valid below offsets[-1]), dst_slot [T*topk] with -1 for
    pairs routed outside [expert_lo, expert_lo + num_experts))."""
    ids = topk_ids.to(torch.int32).contiguous()
    t, topk = ids.shape
    off = torch.empty(num_experts + 1, dtype=torch.int32)
    src = torch.full((t * topk,), -1, dtype=torch.int32)
    dst = torch.empty(t * topk, dtype=torch.int32)
    lib().oracle_moe_segments(_p(ids), ctypes.c_int(t), ctypes.c_int(topk), ctypes.c_int(num_experts),
                              ctypes.c_int(expert_lo), _p(off), _p(src), _p(dst))
    return off, src, dst


def moe_combine(z: torch.Tensor, dst_slot: torch.Tensor, topk_w: torch.Tensor, out_f32: bool = False):
    z = z.contiguous()
    t, topk = topk_w.shape
    h = z.shape[1]
    out = torch.empty((t, h), dtype=torch.float32 if out_f32 else torch.bfloat16)
    null = ctypes.c_void_p(0)
    lib().oracle_moe_combine(_p(z), _p(dst_slot.to(torch.int32).contiguous()), _p(topk_w.contiguous().float()),
                             null if out_f32 else _p(out), _p(out) if out_f32 else null, ctypes.c_int(t),
                             ctypes.c_int(topk), ctypes.c_int(h))
    return out


def moe_combine_exchange(z_ranks, slot_ranks, topk_ids, topk_w, out, experts_per_rank: int, t0: int, t1: int):
    """Rows t0..t1 of `out` (bf16 [T,H], updated in place) from the per-rank expert outputs and slot maps."""
    g = len(z_ranks)
    zs = [z.contiguous() for z in z_ranks]
    ss = [s.to(torch.int32).contiguous() for s in slot_ranks]
    zp = (ctypes.c_void_p * g)(*[z.data_ptr() for z in zs])
    sp = (ctypes.c_void_p * g)(*[s.data_ptr() for s in ss])
    ids = topk_ids.to(torch.int32).contiguous()
    w = topk_w.contiguous().float()
    assert out.is_contiguous() and out.dtype == torch.bfloat16
    lib().oracle_moe_combine_exchange(zp, sp, _p(ids), _p(w), _p(out), ctypes.c_int(g), ctypes.c_int(experts_per_rank),
                                      ctypes.c_int(t0), ctypes.c_int(t1), ctypes.c_int(ids.shape[1]),
                                      ctypes.c_int(out.shape[1]))
    return out


def moe_topk(logits: torch.Tensor, k: int):
    """-> (ids int32 [T,k] descending, ties to the lower index; weights fp32 [T,k] softmax over the selection)."""
    logits = logits.contiguous().float()
    t, e = logits.shape
    ids = torch.empty((t, k), dtype=torch.int32)
    w = torch.empty((t, k), dtype=torch.float32)
    lib().oracle_moe_topk(_p(logits), ctypes.c_int(t), ctypes.c_int(e), ctypes.c_int(k), _p(ids), _p(w))
    return ids, w


def exp_fixed(x: float) -> float:
    return float(lib().oracle_exp(ctypes.c_float(x)))
