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
(every rank computes the same top-k from the same logits) and each rank runs the chain for its own
experts.  Two ways to put the rows together:
  * W8A8MoE: every rank produces an fp32 partial [T,H]; one NCCL all-reduce sums the partials.  The
    sum over ranks associates differently from the single-GPU sum, so the bf16 result agrees to
    rounding, not bit for bit; integer codes, scales and accumulators per expert are identical.
  * ExchangeW8A8MoE: the combine pulls the expert rows from peer memory and pushes the finished bf16
    rows to every rank in one kernel; the result is bit-identical to the single-GPU forward.
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
        if self.pg is None and not dist.is_initialized():
            raise RuntimeError("W8A8MoE.forward: this rank holds an expert shard but there is no process group to sum the "
                               "ranks' partial results over; call local_partial() if the partial sum is what you want")
        part = self.local_partial(x, topk_ids, topk_w, out_f32=True, keep_trace=keep_trace)
        dist.all_reduce(part, group=self.pg)
        return part.to(torch.bfloat16)


def token_range(rank: int, world: int, tokens: int):
    """Tokens [t0, t1) whose output rows `rank` produces in the fused combine (contiguous blocks)."""
    per = (tokens + world - 1) // world
    return min(tokens, rank * per), min(tokens, (rank + 1) * per)


class ExchangeW8A8MoE(W8A8MoE):
    """Expert-parallel forward whose combine is fused with the exchange (`moe_combine_exchange`).

    The down GEMM writes this rank's expert outputs z and `moe_segments` its slot map into symmetric
    memory (every rank's buffers are mapped into every other rank's address space).  After a barrier
    on the stream, the rank that owns a token pulls the token's top-k rows from the ranks that hold
    them over NVLink, sums them in slot order -- the single-GPU arithmetic, so the bf16 result is
    bit-identical to the one-GPU forward whatever the number of ranks -- and pushes the row into every
    rank's output buffer.  A second barrier makes the rows visible.  No NCCL call on the data path and
    no fp32 [T,H] partials: per rank about T/G*topk rows come in and T/G*(G-1) rows go out.
    """

    def __init__(self, w13, w13_scale, w2, w2_scale, num_experts: int, rank: int, world: int, t_max: int, topk: int,
                 device, group_scaled: bool = True, process_group=None):
        per = num_experts // world
        assert per * world == num_experts and w13.shape[0] == per
        super().__init__(w13, w13_scale, w2, w2_scale, num_experts, rank * per, group_scaled, process_group)
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.world, self.t_max, self.topk = rank, world, t_max, topk
        group = process_group if process_group is not None else dist.group.WORLD
        self.z = symm_mem.empty((t_max * topk, self.hidden), dtype=torch.bfloat16, device=device)
        self.slots = symm_mem.empty((t_max * topk,), dtype=torch.int32, device=device)
        self.out = symm_mem.empty((t_max, self.hidden), dtype=torch.bfloat16, device=device)
        self.handle = symm_mem.rendezvous(self.z, group=group)
        self.z_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.slot_ptrs = [int(p) for p in symm_mem.rendezvous(self.slots, group=group).buffer_ptrs]
        self.out_ptrs = [int(p) for p in symm_mem.rendezvous(self.out, group=group).buffer_ptrs]

    def local_rows(self, x, topk_ids):
        """This rank's experts up to the down GEMM: z and the slot map land in symmetric memory."""
        ext = _ext()
        inter = self.inter
        if self.group_scaled:
            q, s = ext.per_token_group_quant_int8(x, GROUP)
        else:
            q, s = ext.per_token_quant_int8(x)
        off, src_row, _ = ext.moe_segments_into(topk_ids, self.e_local, self.expert_lo, self.slots)
        valid = off[self.e_local:]
        a_q, a_s = ext.gather_rows(q, src_row, s, valid)
        y = ext.grouped_gemm(a_q, self.w13, a_s, self.w13_scale, off)
        h_q, h_s = ext.silu_mul_quant_rows(y[:, :inter], y[:, inter:], valid)
        ext.grouped_gemm_into(h_q, self.w2, h_s, self.w2_scale, off, self.z)

    def forward(self, x, topk_ids, topk_w, keep_trace: bool = False):
        t = x.shape[0]
        assert t <= self.t_max and topk_ids.shape[1] == self.topk, "batch larger than the symmetric buffers"
        self.local_rows(x, topk_ids)
        t0, t1 = token_range(self.rank, self.world, t)
        self.handle.barrier(channel=0)      # every rank's z and slots are complete
        _ext().moe_combine_exchange(self.z_ptrs, self.slot_ptrs, topk_ids, topk_w, self.out_ptrs,
                                    self.num_experts // self.world, t0, t1, self.hidden)
        self.handle.barrier(channel=1)      # every rank's rows have landed everywhere
        return self.out[:t]


class PushExchangeW8A8MoE(W8A8MoE):
    """Expert-parallel forward whose down GEMM delivers its rows itself.

    `ExchangeW8A8MoE` lets the rank that owns a token PULL the token's expert rows from the other ranks
    after a barrier: loads over NVLink, on the critical path.  Here every rank knows where each of its
    expert output rows is needed (`moe_push_rows`: the inbox of the token's owner, at row
    (token - t0) * topk + slot) and the down GEMM stores each result row straight there
    (`grouped_gemm_scatter`), as posted peer stores, while it is still streaming weights.  After the barrier
    the owner's combine reads its own memory only, sums in slot order -- the single-GPU arithmetic and bits
    -- and pushes the finished row into every rank's output as before.  No NCCL on the data path.
    """

    def __init__(self, w13, w13_scale, w2, w2_scale, num_experts: int, rank: int, world: int, t_max: int, topk: int,
                 device, group_scaled: bool = True, process_group=None):
        per = num_experts // world
        assert per * world == num_experts and w13.shape[0] == per
        super().__init__(w13, w13_scale, w2, w2_scale, num_experts, rank * per, group_scaled, process_group)
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.world, self.t_max, self.topk = rank, world, t_max, topk
        group = process_group if process_group is not None else dist.group.WORLD
        rows = -(-t_max // world) * topk
        self.inbox = symm_mem.empty((rows, self.hidden), dtype=torch.bfloat16, device=device)
        self.out = symm_mem.empty((t_max, self.hidden), dtype=torch.bfloat16, device=device)
        self.handle = symm_mem.rendezvous(self.inbox, group=group)
        self.inbox_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.out_ptrs = [int(p) for p in symm_mem.rendezvous(self.out, group=group).buffer_ptrs]
        self.row_ptr = torch.zeros(t_max * topk, dtype=torch.int64, device=device)
        self.pair_index = torch.arange(t_max * topk, dtype=torch.int32, device=device)
        self._slot_for = {}

    def _local_slots(self, t: int, t0: int):
        """slot table for the combine: pair (token, j) of an own token sits at inbox row (token - t0) * topk + j"""
        key = (t, t0)
        if key not in self._slot_for:
            self._slot_for[key] = (self.pair_index[: t * self.topk] - t0 * self.topk).contiguous()
        return self._slot_for[key]

    def forward(self, x, topk_ids, topk_w, keep_trace: bool = False):
        t = x.shape[0]
        assert t <= self.t_max and topk_ids.shape[1] == self.topk, "batch larger than the symmetric buffers"
        ext = _ext()
        inter = self.inter
        t0, t1 = token_range(self.rank, self.world, t)
        per = -(-t // self.world)
        if self.group_scaled:
            q, s = ext.per_token_group_quant_int8(x, GROUP)
        else:
            q, s = ext.per_token_quant_int8(x)
        off, src_row, dst_slot = ext.moe_segments(topk_ids, self.e_local, self.expert_lo)
        ext.moe_push_rows(dst_slot, self.topk, per, self.inbox_ptrs, self.hidden, self.row_ptr)
        valid = off[self.e_local:]
        a_q, a_s = ext.gather_rows(q, src_row, s, valid)
        y = ext.grouped_gemm(a_q, self.w13, a_s, self.w13_scale, off)
        h_q, h_s = ext.silu_mul_quant_rows(y[:, :inter], y[:, inter:], valid)
        ext.grouped_gemm_scatter(h_q, self.w2, h_s, self.w2_scale, off, self.row_ptr)
        self.handle.barrier(channel=0)      # every rank's rows have been delivered
        inbox = [self.inbox_ptrs[self.rank]] * self.world
        slots = [self._local_slots(t, t0).data_ptr()] * self.world
        ext.moe_combine_exchange(inbox, slots, topk_ids, topk_w, self.out_ptrs, self.num_experts // self.world,
                                 t0, t1, self.hidden)
        self.handle.barrier(channel=1)      # every rank's output rows have landed everywhere, inboxes are free again
        return self.out[:t]


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
