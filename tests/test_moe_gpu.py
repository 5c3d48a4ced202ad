"""GPU parity of the MoE segment builder and the row gather."""
import pytest
import torch

from bw1000_dsv4_kernels_b200 import workloads as wl
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,e,topk", [(4096, 256, 8), (1, 256, 8), (77, 16, 2), (1000, 5, 1), (300, 64, 6)])
def test_moe_segments_match_oracle(cabi, ext, t, e, topk):
    ids, _ = wl.moe_routing(t, e, topk, seed=t + e)
    off_ref, src_ref, dst_ref = oracle.moe_segments(ids, e)
    off, src, dst = cabi.moe_segments(ids.cuda(), e)
    assert torch.equal(off.cpu(), off_ref)
    assert torch.equal(src.cpu(), src_ref)
    assert torch.equal(dst.cpu(), dst_ref)
    off2, src2, dst2 = ext.moe_segments(ids.cuda(), e)
    assert torch.equal(off2.cpu(), off_ref) and torch.equal(src2.cpu(), src_ref) and torch.equal(dst2.cpu(), dst_ref)
    # a permutation: every routed row is produced exactly once
    assert int(off_ref[-1]) == t * topk
    assert torch.equal(torch.sort(dst.cpu()).values, torch.arange(t * topk, dtype=torch.int32))


def test_gather_rows(cabi, ext):
    t, k = 50, 7168
    q = wl.int8_weights((t, k), seed=1)
    s = wl.channel_scales((t, 56), seed=2)
    idx = torch.randint(0, t, (333,), dtype=torch.int32, generator=torch.Generator().manual_seed(0))
    dq, ds = cabi.gather_rows(q.cuda(), idx.cuda(), s.cuda())
    assert torch.equal(dq.cpu(), q[idx.long()]) and torch.equal(ds.cpu(), s[idx.long()])
    out = ext.gather_rows(q.cuda(), idx.cuda(), s.cuda())
    assert torch.equal(out[0].cpu(), q[idx.long()]) and torch.equal(out[1].cpu(), s[idx.long()])
    xb = wl.randn_bf16((t, 512), seed=3)
    out = ext.gather_rows(xb.cuda(), idx.cuda())
    assert torch.equal(out[0].cpu().view(torch.int16), xb[idx.long()].view(torch.int16))
