"""W8A8 MoE feed-forward on top of the operator module: the chain the reference describes
around its grouped GEMM (DSV4_OPERATOR_ANALYSIS.md:38-48) -- quantise, gate/up grouped GEMM,
silu_mul_quant, down grouped GEMM, weighted sum -- with expert parallelism across ranks.

    routing          : moe_topk(router_logits, k)                     ids int32 [T,k], weights fp32 [T,k]
    group quantiser  : per_token_group_quant_int8(x, 128)            [T,H] -> int8, fp32 [T,H/128]
    segments         : moe_segments(topk_ids, E_local, expert_lo)     expert offsets on the device
    permute          : gather_rows(q, src_row, scales)                rows in expert order
    gate/up GEMM     : grouped_gemm(Aq, W13, As[R,H/128], s13, off)   bf16 [R, 2I]
    activation       : silu_mul_quant(Y[:, :I], Y[:, I:])             int8 [R,I], fp32 [R,1]
    down GEMM        : grouped_gemm(Hq, W2, Hs, s2, off)              bf16 [R, H]
    combine          : moe_combine(Z, dst_slot, topk_w)               [T,H]

Every step is a kernel of this package; torch only allocates.  Nothing synchronises the host:
the number of routed rows of a rank stays on the device (expert_offsets[-1]) and the kernels
that walk rows take it from there.

Expert parallelism: rank r owns experts [r*E/G, (r+1)*E/G).  Tokens and routing are replicated
(every rank computes the same top-k from the same logits), each rank runs the chain for its own
experts and produces an fp32 partial [T,H]; one NCCL all-reduce sums the partials.  The sum over
ranks associates differently from the single-GPU sum, so the bf16 result agrees to rounding, not
bit for bit; integer codes, scales and accumulators per expert are identical.
"""
from dataclasses import dataclass
from typing import Optional

import torch

GROUP = 128


def _ext():
    import bw1000_dsv4_kernels_b200 as pkg
    return pkg.dsv4_native_ext


@dataclass
class MoeTrace:
    """Intermediates of one forward call (kept only when asked, for the parity tests)."""
    offsets: torch.Tensor
    src_row: torch.Tensor
    dst_slot: torch.Tensor
    a_q: torch.Tensor
    a_s: torch.Tensor
    y: torch.Tensor
    h_q: torch.Tensor
    h_s: torch.Tensor
    z: torch.Tensor


class W8A8MoE:
    """Expert weights of one rank and the forward chain.

    w13 int8 [E_local, 2I, H] (gate rows then up rows), w13_scale fp32 [E_local, 2I],
    w2 int8 [E_local, H, I], w2_scale fp32 [E_local, H].
    """

    def __init__(self, w13, w13_scale, w2, w2_scale, num_experts: int, expert_lo: int = 0,
                 group_scaled: bool = True, process_group=None):
        self.w13, self.w13_scale, self.w2, self.w2_scale = w13, w13_scale, w2, w2_scale
        self.e_local = w13.shape[0]
        self.inter = w2.shape[2]
        self.hidden = w2.shape[1]
        assert w13.shape[1] == 2 * self.inter and w13.shape[2] == self.hidden
        self.num_experts, self.expert_lo = num_experts, expert_lo
        self.group_scaled = group_scaled
        self.pg = process_group
        self.last_trace: Optional[MoeTrace] = None

    def local_partial(self, x, topk_ids, topk_w, out_f32: bool, keep_trace: bool = False):
        """This rank's experts only -> [T,H] (bf16, or fp32 when out_f32)."""
        ext = _ext()
        inter = self.inter
        if self.group_scaled:
            q, s = ext.per_token_group_quant_int8(x, GROUP)
        else:
            q, s = ext.per_token_quant_int8(x)
        off, src_row, dst_slot = ext.moe_segments(topk_ids, self.e_local, self.expert_lo)
        valid = off[self.e_local:]
        a_q, a_s = ext.gather_rows(q, src_row, s, valid)
        y = ext.grouped_gemm(a_q, self.w13, a_s, self.w13_scale, off)
        h_q, h_s = ext.silu_mul_quant_rows(y[:, :inter], y[:, inter:], valid)
        z = ext.grouped_gemm(h_q, self.w2, h_s, self.w2_scale, off)
        out = ext.moe_combine(z, dst_slot, topk_w, out_f32)
        if keep_trace:
            self.last_trace = MoeTrace(off, src_row, dst_slot, a_q, a_s, y, h_q, h_s, z)
        return out

    def forward(self, x, topk_ids, topk_w, keep_trace: bool = False):
        """x bf16 [T,H], topk_ids int32 [T,topk], topk_w fp32 [T,topk] -> bf16 [T,H]."""
        single = self.pg is None and self.e_local == self.num_experts
        if single:
            return self.local_partial(x, topk_ids, topk_w, out_f32=False, keep_trace=keep_trace)
        import torch.distributed as dist
        part = self.local_partial(x, topk_ids, topk_w, out_f32=True, keep_trace=keep_trace)
        if self.pg is not None or dist.is_initialized():
            dist.all_reduce(part, group=self.pg)
        return part.to(torch.bfloat16)


def route(router_logits: torch.Tensor, topk: int):
    """Router top-k on the device: fp32 logits [T,E] -> (ids int32 [T,topk], weights fp32 [T,topk] =
    softmax over the selected logits).  Ties go to the lower expert index."""
    ids, w = _ext().moe_topk(router_logits, topk)
    return ids, w


def expert_range(rank: int, world: int, num_experts: int):
    """Experts [lo, hi) owned by `rank` (contiguous blocks)."""
    assert num_experts % world == 0, "experts must divide evenly over the ranks"
    per = num_experts // world
    return rank * per, (rank + 1) * per
