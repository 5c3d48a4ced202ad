"""Independent numpy / torch formulas the C oracle is checked against.  Test infrastructure.

Where the arithmetic is order-independent or a plain sequence of IEEE binary32 operations
(numpy float32 arithmetic is IEEE), the formula must agree with the C oracle bit for bit.
Where a fused multiply-add is involved (the exp polynomial) numpy cannot reproduce the
rounding, so the formula is evaluated in float64 and compared with a stated tolerance.
"""
import numpy as np
import torch


def bf16_to_f32_np(x: torch.Tensor) -> np.ndarray:
    return x.float().numpy()


def f32_to_bf16_bits_np(a: np.ndarray) -> np.ndarray:
    """round-to-nearest-even truncation of float32 to the upper 16 bits"""
    u = a.astype(np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def per_token_quant_int8(x: torch.Tensor):
    xf = x.float()
    am = xf.abs().amax(-1, keepdim=True).clamp_min(1e-10)
    scale = am / 127.0
    inv = torch.full_like(am, 127.0) / am          # true division (127/am in torch is a reciprocal-multiply)
    q = torch.round(xf * inv).clamp(-128, 127).to(torch.int8)
    return q, scale.reshape(-1, 1)


def per_token_group_quant_int8(x: torch.Tensor, gs: int):
    m, n = x.shape
    assert n % gs == 0
    xf = x.float().view(m, n // gs, gs)
    scale = xf.abs().amax(-1, keepdim=True).clamp_min(1e-10) / 127.0
    q = torch.trunc((xf / scale).clamp(-128, 127)).to(torch.int8)
    return q.view(m, n), scale.view(m, n // gs)


def sum_squares_fixed_order_np(a: np.ndarray) -> np.float32:
    """256 lanes, vector v -> lane v mod 256, sequential inside a lane, xor butterfly inside
    groups of 32, the 8 group sums left to right; all in float32."""
    n = a.shape[0]
    sq = (a.astype(np.float32) * a.astype(np.float32)).astype(np.float32)
    nvec = (n + 7) // 8
    pad = np.zeros(nvec * 8, dtype=np.float32)
    pad[:n] = sq
    vec = pad.reshape(nvec, 8)
    lanes = np.zeros(256, dtype=np.float32)
    for v in range(nvec):
        acc = lanes[v & 255]
        cnt = min(8, n - v * 8)
        for e in range(cnt):
            acc = np.float32(acc + vec[v, e])
        lanes[v & 255] = acc
    idx = np.arange(256)
    for o in (16, 8, 4, 2, 1):
        lanes = (lanes + lanes[idx ^ o]).astype(np.float32)
    total = lanes[0]
    for w in range(1, 8):
        total = np.float32(total + lanes[32 * w])
    return np.float32(total)


def add_rmsnorm_quant_np(res: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float):
    """Bit-exact numpy restatement -> (res_out bf16 bits uint16, q int8, s float32 [M])."""
    r, xx, ww = bf16_to_f32_np(res), bf16_to_f32_np(x), bf16_to_f32_np(w)
    m, n = r.shape
    a = (r + xx).astype(np.float32)
    res_bits = f32_to_bf16_bits_np(a)
    q = np.empty((m, n), dtype=np.int8)
    s = np.empty(m, dtype=np.float32)
    for i in range(m):
        total = sum_squares_fixed_order_np(a[i])
        mean = np.float32(total / np.float32(n))
        rrms = np.float32(np.float32(1.0) / np.sqrt(np.float32(mean + np.float32(eps))))
        y = ((a[i] * rrms).astype(np.float32) * ww).astype(np.float32)
        am = np.float32(max(np.abs(y).max(), np.float32(1e-10)))
        s[i] = np.float32(am / np.float32(127.0))
        inv = np.float32(np.float32(127.0) / am)
        q[i] = np.clip(np.rint((y * inv).astype(np.float32)), -128, 127).astype(np.int8)
    return res_bits, q, s


def add_rmsnorm_quant_f64(res, x, w, eps):
    """Plain double-precision formula (no fixed order): codes may differ by one."""
    a = res.float() + x.float()
    ad = a.double()
    rrms = torch.rsqrt((ad * ad).mean(-1, keepdim=True) + eps)
    y = ad * rrms * w.double()
    am = y.abs().amax(-1, keepdim=True).clamp_min(1e-10)
    q = torch.round(y * (127.0 / am)).clamp(-128, 127).to(torch.int8)
    return a.bfloat16(), q, (am / 127.0).float()


def silu_mul_f64(g, u):
    gd, ud = g.double(), u.double()
    return torch.sigmoid(gd) * gd * ud


def silu_mul_quant_f64(g, u):
    h = silu_mul_f64(g, u)
    am = h.abs().amax(-1, keepdim=True).clamp_min(1e-10)
    q = torch.round(h * (127.0 / am)).clamp(-128, 127).to(torch.int8)
    return q, (am / 127.0).float()


def gemm_i32(A: torch.Tensor, B: torch.Tensor):
    """exact: |sum| <= 128*128*K < 2^53 for any practical K"""
    return (A.double() @ B.double().t()).to(torch.int64).to(torch.int32)


def scale_convert(acc: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor):
    return ((acc.float() * sa.view(-1, 1)) * sb.view(1, -1)).bfloat16()
