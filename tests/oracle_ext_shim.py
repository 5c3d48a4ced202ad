"""A stand-in for the operator module backed by the CPU oracle, so that the multi-rank host
logic (sharding, all-gather layout, all-reduce of partials) can run as gloo ranks on CPU.
Test infrastructure only: the product path never sees it."""
import torch

from oracle import cpu as oracle


class OracleExt:
    @staticmethod
    def per_token_quant_int8(x):
        return oracle.per_token_quant_int8(x)

    @staticmethod
    def per_token_group_quant_int8(x, gs=128):
        return oracle.per_token_group_quant_int8(x, gs)

    @staticmethod
    def w8a8_scaled_gemm(a, b, sa, sb):
        return oracle.w8a8_gemm(a, b, sa.reshape(-1), sb)

    @staticmethod
    def w8a8_gemm_into(a, b, sa, sb, out, col0):
        out[:, col0:col0 + b.shape[0]] = oracle.w8a8_gemm(a, b, sa.reshape(-1), sb)

    @staticmethod
    def moe_segments(ids, num_experts, expert_lo=0):
        return oracle.moe_segments(ids, num_experts, expert_lo)

    @staticmethod
    def gather_rows(src, src_row, scales=None, valid_rows=None):
        r = src_row.numel() if valid_rows is None else int(valid_rows[0])
        idx = src_row[:r].long()
        dst = torch.zeros((src_row.numel(), src.shape[1]), dtype=src.dtype)
        dst[:r] = src[idx]
        if scales is None:
            return [dst]
        ds = torch.zeros((src_row.numel(), scales.shape[1]), dtype=scales.dtype)
        ds[:r] = scales[idx]
        return [dst, ds]

    @staticmethod
    def grouped_gemm(a, w, sa, sw, off):
        return oracle.grouped_gemm(a, w, sa, sw, off)

    @staticmethod
    def silu_mul_quant_rows(g, u, valid_rows):
        r = int(valid_rows[0])
        q = torch.zeros(g.shape, dtype=torch.int8)
        s = torch.zeros((g.shape[0], 1), dtype=torch.float32)
        if r:
            q[:r], s[:r] = oracle.silu_mul_quant(g[:r], u[:r])
        return q, s

    @staticmethod
    def moe_combine(z, dst_slot, topk_w, out_f32=False):
        return oracle.moe_combine(z, dst_slot, topk_w, out_f32)
