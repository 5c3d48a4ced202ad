"""Host logic of the two sharded configurations as world_size-2 gloo ranks on CPU.

The kernels are replaced by the oracle-backed shim (tests/oracle_ext_shim.py); what is under
test is the sharding arithmetic, the all-gather layout of the column-parallel linear and the
all-reduce of the expert-parallel partial sums, each against the single-rank result.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import workloads as wl


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _patch(module):
    from tests.oracle_ext_shim import OracleExt
    module._ext = lambda: OracleExt


def _tp_worker(rank, world, port, ret):
    try:
        _init(rank, world, port)
        from bw1000_dsv4_kernels_b200 import tp_linear
        _patch(tp_linear)
        m, k, n = 24, 256, 1024
        inp = wl.tp_linear_inputs(rank, world, m=m, k=k, n=n, slab=128, seed=3)
        layer = tp_linear.ColumnParallelW8A8Linear(inp.w, inp.w_scale, rank, world)
        out = layer.forward(inp.x)
        full = wl.tp_linear_inputs(0, 1, m=m, k=k, n=n, slab=128, seed=3)
        ref = tp_linear.ColumnParallelW8A8Linear(full.w, full.w_scale).forward(full.x)
        lo, hi = tp_linear.column_range(rank, world, n)
        assert torch.equal(inp.w, full.w[lo:hi]) and torch.equal(inp.x, full.x)
        assert out.shape == (m, n)
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), "gathered output differs from 1-rank result"
        ret[rank] = "ok"
    except Exception as exc:  # pragma: no cover
        ret[rank] = f"{type(exc).__name__}: {exc}"
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _ep_worker(rank, world, port, ret):
    try:
        _init(rank, world, port)
        from bw1000_dsv4_kernels_b200 import moe
        _patch(moe)
        t, h, e, inter, topk = 40, 256, 8, 128, 2
        lo, hi = moe.expert_range(rank, world, e)
        inp = wl.moe_inputs(t, h, e, inter, topk, seed=5, expert_lo=lo, expert_hi=hi)
        layer = moe.W8A8MoE(inp.w13, inp.w13_scale, inp.w2, inp.w2_scale, e, expert_lo=lo)
        out = layer.forward(inp.x, inp.topk_ids, inp.topk_w)
        full = wl.moe_inputs(t, h, e, inter, topk, seed=5)
        assert torch.equal(inp.w13, full.w13[lo:hi]) and torch.equal(inp.topk_ids, full.topk_ids)
        ref = moe.W8A8MoE(full.w13, full.w13_scale, full.w2, full.w2_scale, e).forward(full.x, full.topk_ids, full.topk_w)
        err = (out.float() - ref.float()).abs().max().item()
        absmax = ref.float().abs().max().item()
        assert err <= 1e-2 * absmax, f"EP result off by {err} (absmax {absmax})"
        ret[rank] = "ok"
    except Exception as exc:  # pragma: no cover
        ret[rank] = f"{type(exc).__name__}: {exc}"
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run(worker, world=2):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {r: "ok" for r in range(world)}, dict(ret)


def test_column_parallel_linear_two_ranks_gloo():
    _run(_tp_worker)


def test_expert_parallel_moe_two_ranks_gloo():
    _run(_ep_worker)


def test_shard_ranges_and_seeded_shards_are_consistent():
    from bw1000_dsv4_kernels_b200 import moe, tp_linear
    assert [tp_linear.column_range(r, 4, 28672) for r in range(4)] == [(0, 7168), (7168, 14336), (14336, 21504), (21504, 28672)]
    assert [moe.expert_range(r, 8, 256) for r in range(8)][-1] == (224, 256)
    with pytest.raises(AssertionError):
        tp_linear.column_range(0, 3, 28672 + 1)
    # token ownership of the fused combine: contiguous blocks that cover every token exactly once
    for tokens, world in ((4096, 8), (4099, 8), (7, 8), (1, 2), (0, 4)):
        ranges = [moe.token_range(r, world, tokens) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == tokens
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:])) and all(lo <= hi for lo, hi in ranges)
    full = wl.tp_linear_inputs(0, 1, m=4, k=64, n=512, slab=64, seed=1)
    parts = [wl.tp_linear_inputs(r, 4, m=4, k=64, n=512, slab=64, seed=1) for r in range(4)]
    assert torch.equal(torch.cat([p.w for p in parts]), full.w)
    assert torch.equal(torch.cat([p.w_scale for p in parts]), full.w_scale)
