"""The two sharded configurations on real GPUs (needs at least two; skipped otherwise): one
process per GPU over NCCL, results compared with a single-GPU run of the same seeded problem."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import workloads as wl

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                 reason="needs two GPUs")]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from bw1000_dsv4_kernels_b200 import moe, tp_linear

        # ---- column-parallel linear: NCCL all-gather and fused peer stores ----
        m, k, n = 1024, 1024, 4096
        inp = wl.tp_linear_inputs(rank, world, m=m, k=k, n=n, device=dev, seed=2, slab=256)
        full = wl.tp_linear_inputs(0, 1, m=m, k=k, n=n, device=dev, seed=2, slab=256)
        ref = tp_linear.ColumnParallelW8A8Linear(full.w, full.w_scale).forward(full.x)
        out = tp_linear.ColumnParallelW8A8Linear(inp.w, inp.w_scale, rank, world).forward(inp.x)
        assert torch.equal(out.contiguous().view(torch.int16), ref.view(torch.int16)), "NCCL all-gather result"
        # fused epilogue: two alternating output buffers (no barrier in front) and one buffer (barrier on
        # both sides); three calls in a row with changing inputs, each compared with the one-GPU layer
        x_alt = wl.randn_bf16((m, k), device=dev, seed=9)
        ref_alt = tp_linear.ColumnParallelW8A8Linear(full.w, full.w_scale).forward(x_alt)
        for buffers in (2, 1):
            fused = tp_linear.FusedColumnParallelW8A8Linear(inp.w, inp.w_scale, rank, world, m_max=m, device=dev,
                                                            buffers=buffers)
            for call in range(3):
                xin, want = (inp.x, ref) if call != 1 else (x_alt, ref_alt)
                out2 = fused.forward(xin)
                torch.cuda.synchronize()
                assert torch.equal(out2.view(torch.int16), want.view(torch.int16)), f"fused all-gather, {buffers} buffer(s), call {call}"
            del fused

        # ---- expert-parallel MoE ----
        t, h, e, inter, topk = 256, 1024, 16, 512, 4
        lo, hi = moe.expert_range(rank, world, e)
        part = wl.moe_inputs(t, h, e, inter, topk, device=dev, seed=4, expert_lo=lo, expert_hi=hi)
        whole = wl.moe_inputs(t, h, e, inter, topk, device=dev, seed=4)
        ref_m = moe.W8A8MoE(whole.w13, whole.w13_scale, whole.w2, whole.w2_scale, e).forward(whole.x, whole.topk_ids, whole.topk_w)
        out_m = moe.W8A8MoE(part.w13, part.w13_scale, part.w2, part.w2_scale, e, expert_lo=lo).forward(part.x, part.topk_ids, part.topk_w)
        err = (out_m.float() - ref_m.float()).abs().max().item()
        assert err <= 1e-2 * ref_m.float().abs().max().item(), f"EP MoE off by {err}"
        # fused combine + exchange over peer memory: the single-GPU bits on every rank, twice in a row
        ex = moe.ExchangeW8A8MoE(part.w13, part.w13_scale, part.w2, part.w2_scale, e, rank, world, t_max=t, topk=topk,
                                 device=dev)
        for _ in range(2):
            out_x = ex.forward(part.x, part.topk_ids, part.topk_w)
            torch.cuda.synchronize()
            assert torch.equal(out_x.view(torch.int16), ref_m.view(torch.int16)), "fused EP combine"
        # the push form: the down GEMM stores every row into the inbox of the token's owner
        push = moe.PushExchangeW8A8MoE(part.w13, part.w13_scale, part.w2, part.w2_scale, e, rank, world, t_max=t,
                                       topk=topk, device=dev)
        for _ in range(3):
            out_p = push.forward(part.x, part.topk_ids, part.topk_w)
            torch.cuda.synchronize()
            assert torch.equal(out_p.view(torch.int16), ref_m.view(torch.int16)), "EP forward with pushed rows"
        ret[rank] = "ok"
    except Exception as exc:  # pragma: no cover
        import traceback
        ret[rank] = f"{type(exc).__name__}: {exc}\n{traceback.format_exc()[-1500:]}"
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_sharded_configurations_on_two_gpus():
    world = 2
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {r: "ok" for r in range(world)}, dict(ret)
