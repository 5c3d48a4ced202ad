"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations of the W8A8 linear path.  No dataset is involved: the reference's own
measurements used random tensors.

Every generator takes a torch device.  Parity tests generate on the CPU and copy, so
that the CPU oracle and the GPU kernels see the same bits; the benchmark generates the
large weight tensors directly on the GPU.
"""
from dataclasses import dataclass

import torch

HIDDEN = 7168          # model width (K of the first projections)
DENSE_N = 4096         # output width of the dense projection in the add_rmsnorm_quant chain
DENSE_INTER = 18432    # intermediate width of the dense FFN (K of the down projection)
MOE_EXPERTS = 256
MOE_INTER = 2048
MOE_TOPK = 8
MOE_TOKENS = 4096
TP_M = 8192
TP_N = 28672


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def randn_bf16(shape, device="cpu", seed=0):
    return torch.randn(shape, generator=_gen(device, seed), device=device, dtype=torch.float32).to(torch.bfloat16)


def int8_weights(shape, device="cpu", seed=0):
    """U{-127..127}"""
    return torch.randint(-127, 128, shape, generator=_gen(device, seed), device=device, dtype=torch.int8)


def channel_scales(shape, device="cpu", seed=0):
    """fp32 U(1e-3, 1e-2)"""
    u = torch.rand(shape, generator=_gen(device, seed), device=device, dtype=torch.float32)
    return u * (1e-2 - 1e-3) + 1e-3


def activations_with_outliers(m=64, k=HIDDEN, device="cpu", seed=0):
    """per_token_quant_int8 input: N(0,1) with 1 % of the entries scaled x20."""
    g = _gen(device, seed)
    x = torch.randn((m, k), generator=g, device=device, dtype=torch.float32)
    outlier = torch.rand((m, k), generator=g, device=device) < 0.01
    x = torch.where(outlier, x * 20.0, x)
    return x.to(torch.bfloat16)


def gamma_bf16(k=HIDDEN, device="cpu", seed=0):
    """RMSNorm weight, bf16 U(0.5, 1.5)"""
    u = torch.rand((k,), generator=_gen(device, seed), device=device, dtype=torch.float32)
    return (u + 0.5).to(torch.bfloat16)


@dataclass
class NormGemmInputs:
    x: torch.Tensor        # bf16 [M, K]
    res: torch.Tensor      # bf16 [M, K]
    gamma: torch.Tensor    # bf16 [K]
    w: torch.Tensor        # int8 [N, K]
    w_scale: torch.Tensor  # fp32 [N]
    eps: float = 1e-6


def norm_gemm_inputs(m, k=HIDDEN, n=DENSE_N, device="cpu", seed=0) -> NormGemmInputs:
    """add_rmsnorm_quant -> w8a8_gemm"""
    return NormGemmInputs(
        x=randn_bf16((m, k), device, seed),
        res=randn_bf16((m, k), device, seed + 1),
        gamma=gamma_bf16(k, device, seed + 2),
        w=int8_weights((n, k), device, seed + 3),
        w_scale=channel_scales((n,), device, seed + 4),
    )


@dataclass
class SiluDownInputs:
    gate_up: torch.Tensor  # bf16 [M, 2*I]  (gate = [:, :I], up = [:, I:])
    w: torch.Tensor        # int8 [N, I]
    w_scale: torch.Tensor  # fp32 [N]


def silu_down_inputs(m, inter=DENSE_INTER, n=HIDDEN, device="cpu", seed=0) -> SiluDownInputs:
    """silu_mul_quant -> down-projection w8a8_gemm"""
    return SiluDownInputs(
        gate_up=randn_bf16((m, 2 * inter), device, seed),
        w=int8_weights((n, inter), device, seed + 1),
        w_scale=channel_scales((n,), device, seed + 2),
    )


@dataclass
class MoeInputs:
    x: torch.Tensor          # bf16 [T, H]
    topk_ids: torch.Tensor   # int32 [T, topk]
    topk_w: torch.Tensor     # fp32 [T, topk]  softmax of the selected logits
    w13: torch.Tensor        # int8 [E, 2*I, H]   gate rows first, then up rows
    w13_scale: torch.Tensor  # fp32 [E, 2*I]
    w2: torch.Tensor         # int8 [E, H, I]
    w2_scale: torch.Tensor   # fp32 [E, H]


def moe_routing(tokens, experts, topk, device="cpu", seed=0):
    """top-k of seeded N(0,1) router logits -> (ids int32 [T,topk], weights fp32 [T,topk])."""
    logits = torch.randn((tokens, experts), generator=_gen(device, seed), device=device, dtype=torch.float32)
    vals, ids = torch.topk(logits, topk, dim=-1)
    return ids.to(torch.int32), torch.softmax(vals, dim=-1)


def moe_inputs(tokens=MOE_TOKENS, hidden=HIDDEN, experts=MOE_EXPERTS, inter=MOE_INTER, topk=MOE_TOPK,
               device="cpu", seed=0, expert_lo=0, expert_hi=None) -> MoeInputs:
    """MoE FFN inputs.  expert_lo/hi restrict the generated WEIGHTS to a slice of experts
    (expert parallelism); each expert's weights depend only on (seed, expert index) so that
    any sharding sees the same values."""
    expert_hi = experts if expert_hi is None else expert_hi
    ids, tw = moe_routing(tokens, experts, topk, device, seed)
    n_local = expert_hi - expert_lo
    w13 = torch.empty((n_local, 2 * inter, hidden), dtype=torch.int8, device=device)
    w2 = torch.empty((n_local, hidden, inter), dtype=torch.int8, device=device)
    w13_s = torch.empty((n_local, 2 * inter), dtype=torch.float32, device=device)
    w2_s = torch.empty((n_local, hidden), dtype=torch.float32, device=device)
    for i, e in enumerate(range(expert_lo, expert_hi)):
        base = seed + 1000 + 4 * e
        w13[i] = int8_weights((2 * inter, hidden), device, base)
        w2[i] = int8_weights((hidden, inter), device, base + 1)
        w13_s[i] = channel_scales((2 * inter,), device, base + 2)
        w2_s[i] = channel_scales((hidden,), device, base + 3)
    return MoeInputs(x=randn_bf16((tokens, hidden), device, seed + 1), topk_ids=ids, topk_w=tw,
                     w13=w13, w13_scale=w13_s, w2=w2, w2_scale=w2_s)


@dataclass
class TpLinearInputs:
    x: torch.Tensor        # bf16 [M, K] (replicated)
    w: torch.Tensor        # int8 [N_local, K] (this rank's rows of the [N, K] weight)
    w_scale: torch.Tensor  # fp32 [N_local]


def tp_linear_inputs(rank=0, world=1, m=TP_M, k=HIDDEN, n=TP_N, device="cpu", seed=0, slab=512) -> TpLinearInputs:
    """Column-sharded linear: rank r owns output columns [r*N/world, (r+1)*N/world).
    The weight is generated in slabs of `slab` rows seeded by the slab index, so every
    sharding produces the same full matrix."""
    assert n % world == 0 and (n // world) % slab == 0
    n_local = n // world
    lo = rank * n_local
    w = torch.empty((n_local, k), dtype=torch.int8, device=device)
    ws = torch.empty((n_local,), dtype=torch.float32, device=device)
    for i in range(n_local // slab):
        sid = (lo // slab) + i
        w[i * slab:(i + 1) * slab] = int8_weights((slab, k), device, seed + 10 + 2 * sid)
        ws[i * slab:(i + 1) * slab] = channel_scales((slab,), device, seed + 11 + 2 * sid)
    return TpLinearInputs(x=randn_bf16((m, k), device, seed), w=w, w_scale=ws)
