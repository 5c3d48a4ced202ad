"""GPU parity of the MoE segment builder and the row gather."""
import pytest
import torch

from tests import workloads as wl
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,e,topk", [(4096, 256, 8), (1, 256, 8), (77, 16, 2), (1000, 5, 1), (300, 64, 6),
                                      (700, 384, 8), (1500, 1000, 3), (4099, 32, 8), (9000, 257, 5)])
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


@pytest.mark.parametrize("t,e,topk,lo,n_local", [(300, 64, 6, 16, 16), (77, 16, 2, 8, 8), (64, 8, 2, 0, 4),
                                                 (4096, 256, 8, 96, 32), (2000, 640, 4, 320, 320)])
def test_moe_segments_expert_slice(cabi, ext, t, e, topk, lo, n_local):
    ids, _ = wl.moe_routing(t, e, topk, seed=t)
    off_ref, src_ref, dst_ref = oracle.moe_segments(ids, n_local, lo)
    off, src, dst = cabi.moe_segments(ids.cuda(), n_local, lo)
    r = int(off_ref[-1])
    assert torch.equal(off.cpu(), off_ref) and torch.equal(dst.cpu(), dst_ref)
    assert torch.equal(src.cpu()[:r], src_ref[:r])
    off2, src2, dst2 = ext.moe_segments(ids.cuda(), n_local, lo)
    assert torch.equal(off2.cpu(), off_ref) and torch.equal(dst2.cpu(), dst_ref) and torch.equal(src2.cpu()[:r], src_ref[:r])
    inside = (ids >= lo) & (ids < lo + n_local)
    assert torch.equal(dst_ref.view(t, topk) >= 0, inside)


def test_gather_rows_and_silu_respect_device_row_count(cabi, ext):
    t, k = 40, 1024
    q = wl.int8_weights((t, k), seed=1)
    idx = torch.randint(0, t, (100,), dtype=torch.int32, generator=torch.Generator().manual_seed(0))
    valid = torch.tensor([37], dtype=torch.int32).cuda()
    dq, _ = cabi.gather_rows(q.cuda(), idx.cuda(), None, valid)
    assert torch.equal(dq.cpu()[:37], q[idx[:37].long()])
    gu = wl.randn_bf16((100, 512), seed=2)
    qh_ref, sh_ref = oracle.silu_mul_quant(gu[:37, :256], gu[:37, 256:])
    gud = gu.cuda()
    qh, sh = ext.silu_mul_quant_rows(gud[:, :256], gud[:, 256:], valid)
    assert torch.equal(qh.cpu()[:37], qh_ref) and torch.equal(sh.cpu()[:37], sh_ref)
    # rows past the count are not touched (the C-ABI helper hands in zero-filled outputs)
    q_c, s_c = cabi.silu_mul_quant(gud[:, :256], gud[:, 256:], None, valid)
    assert torch.equal(q_c.cpu()[:37], qh_ref) and torch.equal(s_c.cpu()[:37], sh_ref)
    assert q_c[37:].abs().sum().item() == 0 and s_c[37:].abs().sum().item() == 0


@pytest.mark.parametrize("out_f32", [False, True])
def test_moe_combine_matches_oracle(cabi, ext, out_f32):
    t, topk, h, e = 50, 4, 512, 8
    ids, w = wl.moe_routing(t, e, topk, seed=3)
    _, _, dst = oracle.moe_segments(ids, 4, 2)          # half of the experts: some slots are -1
    r = t * topk
    z = wl.randn_bf16((r, h), seed=4)
    ref = oracle.moe_combine(z, dst, w, out_f32)
    out = cabi.moe_combine(z.cuda(), dst.cuda(), w.cuda(), out_f32)
    out2 = ext.moe_combine(z.cuda(), dst.cuda(), w.cuda(), out_f32)
    if out_f32:
        assert torch.equal(out.cpu(), ref) and torch.equal(out2.cpu(), ref)
    else:
        assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))
        assert torch.equal(out2.cpu().view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("t,topk,h,e", [(33, 12, 2304, 16), (5, 1, 8, 4), (9, 17, 7168, 32)])
def test_moe_combine_many_slots_and_wide_rows(cabi, t, topk, h, e):
    # more than eight slots per token (two batches of row pointers) and rows wider than one pass
    ids, w = wl.moe_routing(t, e, topk, seed=t + topk)
    _, _, dst = oracle.moe_segments(ids, e - e // 4, 0)   # a quarter of the experts elsewhere: some slots are -1
    z = wl.randn_bf16((t * topk, h), seed=8)
    for out_f32 in (False, True):
        ref = oracle.moe_combine(z, dst, w, out_f32)
        out = cabi.moe_combine(z.cuda(), dst.cuda(), w.cuda(), out_f32).cpu()
        if out_f32:
            assert torch.equal(out, ref)
        else:
            assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


def _oracle_moe(inp, e, lo, hi, group_scaled, out_f32):
    """The MoE chain with every step taken from the oracle."""
    inter = inp.w2.shape[2]
    if group_scaled:
        q, s = oracle.per_token_group_quant_int8(inp.x, 128)
    else:
        q, s = oracle.per_token_quant_int8(inp.x)
    off, src, dst = oracle.moe_segments(inp.topk_ids, hi - lo, lo)
    r = int(off[-1])
    a_q, a_s = q[src[:r].long()], s[src[:r].long()]
    y = oracle.grouped_gemm(a_q, inp.w13, a_s, inp.w13_scale, off)
    h_q, h_s = oracle.silu_mul_quant(y[:, :inter], y[:, inter:])
    z = oracle.grouped_gemm(h_q, inp.w2, h_s.view(-1), inp.w2_scale, off)
    zz = torch.zeros((inp.topk_ids.numel(), z.shape[1]), dtype=torch.bfloat16)
    zz[:r] = z
    return oracle.moe_combine(zz, dst, inp.topk_w, out_f32), (off, a_q, a_s, y, h_q, h_s, z, r)


@pytest.mark.parametrize("group_scaled", [True, False])
def test_moe_chain_matches_oracle(group_scaled):
    from bw1000_dsv4_kernels_b200 import moe
    t, h, e, inter, topk = 96, 512, 8, 256, 2
    inp = wl.moe_inputs(t, h, e, inter, topk, seed=9)
    ref, (off, a_q, a_s, y, h_q, h_s, z, r) = _oracle_moe(inp, e, 0, e, group_scaled, False)
    layer = moe.W8A8MoE(inp.w13.cuda(), inp.w13_scale.cuda(), inp.w2.cuda(), inp.w2_scale.cuda(), e,
                        group_scaled=group_scaled)
    out = layer.forward(inp.x.cuda(), inp.topk_ids.cuda(), inp.topk_w.cuda(), keep_trace=True)
    tr = layer.last_trace
    assert torch.equal(tr.offsets.cpu(), off)
    assert torch.equal(tr.a_q.cpu()[:r], a_q) and torch.equal(tr.a_s.cpu()[:r], a_s)
    assert torch.equal(tr.y.cpu()[:r].view(torch.int16), y.view(torch.int16)), "gate/up grouped GEMM"
    assert torch.equal(tr.h_q.cpu()[:r], h_q) and torch.equal(tr.h_s.cpu()[:r], h_s), "silu_mul_quant"
    assert torch.equal(tr.z.cpu()[:r].view(torch.int16), z.view(torch.int16)), "down grouped GEMM"
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16)), "combined output"


def test_moe_expert_slice_partials_sum_to_full():
    # two expert slices on one GPU: their fp32 partials add up to the single-rank result (to rounding)
    from bw1000_dsv4_kernels_b200 import moe
    t, h, e, inter, topk = 64, 512, 8, 256, 2
    full = wl.moe_inputs(t, h, e, inter, topk, seed=11)
    ref, _ = _oracle_moe(full, e, 0, e, True, False)
    total = torch.zeros((t, h), dtype=torch.float32, device="cuda")
    for lo, hi in ((0, 4), (4, 8)):
        part_in = wl.moe_inputs(t, h, e, inter, topk, seed=11, expert_lo=lo, expert_hi=hi)
        layer = moe.W8A8MoE(part_in.w13.cuda(), part_in.w13_scale.cuda(), part_in.w2.cuda(), part_in.w2_scale.cuda(),
                            e, expert_lo=lo)
        part = layer.local_partial(part_in.x.cuda(), part_in.topk_ids.cuda(), part_in.topk_w.cuda(), out_f32=True)
        ref_part, _ = _oracle_moe(part_in, e, lo, hi, True, True)
        assert torch.equal(part.cpu(), ref_part), "fp32 partial of an expert slice"
        total += part
    err = (total.cpu() - ref.float()).abs().max().item()
    assert err <= 1e-2 * ref.float().abs().max().item()


@pytest.mark.parametrize("world,t,topk", [(2, 64, 2), (4, 131, 4), (8, 40, 8), (3, 7, 12)])
def test_moe_combine_exchange_on_one_gpu(ext, world, t, topk):
    # the fused combine + exchange only sees pointers: with every "rank's" buffers on one GPU, each
    # rank's call fills its token range of every output buffer, and the result must have the bits of
    # the single-rank forward (same fma order) and of the oracle
    from bw1000_dsv4_kernels_b200 import moe
    h, e, inter = 512, 24, 256
    full = wl.moe_inputs(t, h, e, inter, topk, seed=21)
    whole = moe.W8A8MoE(full.w13.cuda(), full.w13_scale.cuda(), full.w2.cuda(), full.w2_scale.cuda(), e)
    ref = whole.forward(full.x.cuda(), full.topk_ids.cuda(), full.topk_w.cuda())
    ids, w = full.topk_ids.cuda(), full.topk_w.cuda()
    zs, slots = [], []
    for r in range(world):
        lo, hi = moe.expert_range(r, world, e)
        part_in = wl.moe_inputs(t, h, e, inter, topk, seed=21, expert_lo=lo, expert_hi=hi)
        layer = moe.W8A8MoE(part_in.w13.cuda(), part_in.w13_scale.cuda(), part_in.w2.cuda(), part_in.w2_scale.cuda(),
                            e, expert_lo=lo)
        layer.local_partial(part_in.x.cuda(), ids, w, out_f32=True, keep_trace=True)
        zs.append(layer.last_trace.z)
        slots.append(layer.last_trace.dst_slot)
    outs = [torch.full((t, h), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for r in range(world):
        t0, t1 = moe.token_range(r, world, t)
        ext.moe_combine_exchange([z.data_ptr() for z in zs], [s.data_ptr() for s in slots], ids, w,
                                 [o.data_ptr() for o in outs], e // world, t0, t1, h)
    for r in range(world):
        assert torch.equal(outs[r].view(torch.int16), ref.view(torch.int16)), f"rank {r}'s output buffer"
    ref_o = torch.zeros((t, h), dtype=torch.bfloat16)
    oracle.moe_combine_exchange([z.cpu() for z in zs], [s.cpu() for s in slots], full.topk_ids, full.topk_w, ref_o,
                                e // world, 0, t)
    assert torch.equal(outs[0].cpu().view(torch.int16), ref_o.view(torch.int16)), "oracle"


@pytest.mark.parametrize("world,t,topk", [(2, 64, 2), (4, 131, 4), (8, 40, 8)])
def test_moe_down_gemm_pushes_rows_to_the_owners_on_one_gpu(ext, world, t, topk):
    # the push form of the expert-parallel forward, every "rank's" inbox on one GPU: each rank's down GEMM
    # stores its rows into the inbox of the token's owner (moe_push_rows + grouped_gemm_scatter); the owner's
    # combine then reads its own inbox only.  Same bits as the single-rank forward.
    from bw1000_dsv4_kernels_b200 import moe
    h, e, inter = 512, 24, 256
    if e % world:
        e = world * 3
    full = wl.moe_inputs(t, h, e, inter, topk, seed=33)
    whole = moe.W8A8MoE(full.w13.cuda(), full.w13_scale.cuda(), full.w2.cuda(), full.w2_scale.cuda(), e)
    ids, w = full.topk_ids.cuda(), full.topk_w.cuda()
    ref = whole.forward(full.x.cuda(), ids, w)
    per = -(-t // world)
    inboxes = [torch.full((per * topk, h), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for r in range(world):
        lo, hi = moe.expert_range(r, world, e)
        part_in = wl.moe_inputs(t, h, e, inter, topk, seed=33, expert_lo=lo, expert_hi=hi)
        layer = moe.W8A8MoE(part_in.w13.cuda(), part_in.w13_scale.cuda(), part_in.w2.cuda(), part_in.w2_scale.cuda(),
                            e, expert_lo=lo)
        layer.local_partial(part_in.x.cuda(), ids, w, out_f32=True, keep_trace=True)
        tr = layer.last_trace
        row_ptr = torch.zeros(t * topk, dtype=torch.int64, device="cuda")
        ext.moe_push_rows(tr.dst_slot, topk, per, [b.data_ptr() for b in inboxes], h, row_ptr)
        # the table against its definition
        slot = tr.dst_slot.cpu()
        want = torch.zeros(t * topk, dtype=torch.int64)
        for i in range(t * topk):
            if slot[i] >= 0:
                tok, j = divmod(i, topk)
                g = min(tok // per, world - 1)
                want[slot[i]] = inboxes[g].data_ptr() + ((tok - g * per) * topk + j) * h * 2
        rows = int(tr.offsets[-1])
        assert torch.equal(row_ptr.cpu()[:rows], want[:rows])
        ext.grouped_gemm_scatter(tr.h_q, layer.w2, tr.h_s, layer.w2_scale, tr.offsets, row_ptr)
    torch.cuda.synchronize()
    outs = [torch.full((t, h), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    pair = torch.arange(t * topk, dtype=torch.int32, device="cuda")
    for r in range(world):
        t0, t1 = moe.token_range(r, world, t)
        local = (pair - t0 * topk).contiguous()
        ext.moe_combine_exchange([inboxes[r].data_ptr()] * world, [local.data_ptr()] * world, ids, w,
                                 [o.data_ptr() for o in outs], e // world, t0, t1, h)
    for r in range(world):
        assert torch.equal(outs[r].view(torch.int16), ref.view(torch.int16)), f"rank {r}'s output buffer"


def test_grouped_gemm_scatter_rejects_group_scales_and_null(cabi):
    import ctypes
    a = torch.zeros((16, 128), dtype=torch.int8, device="cuda")
    wgt = torch.zeros((1, 128, 128), dtype=torch.int8, device="cuda")
    sa = torch.ones(16, device="cuda")
    sw = torch.ones((1, 128), device="cuda")
    off = torch.tensor([0, 16], dtype=torch.int32, device="cuda")
    lib = cabi.lib()
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    rc = lib.launch_grouped_gemm_scatter(p(a), p(wgt), p(sa), p(sw), p(off), ctypes.c_void_p(0), 16, 1, 128, 128,
                                         ctypes.c_void_p(0))
    assert rc != 0 and "row_ptr" in cabi.last_error()


def test_moe_combine_exchange_rejects_bad_arguments(ext):
    ids = torch.zeros((4, 2), dtype=torch.int32, device="cuda")
    w = torch.zeros((4, 2), dtype=torch.float32, device="cuda")
    buf = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    slot = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError):
        ext.moe_combine_exchange([buf.data_ptr()] * 9, [slot.data_ptr()] * 9, ids, w, [buf.data_ptr()] * 9, 1, 0, 4, 64)
    with pytest.raises(RuntimeError):
        ext.moe_combine_exchange([buf.data_ptr()], [slot.data_ptr()], ids, w, [buf.data_ptr()], 1, 0, 5, 64)
    with pytest.raises(RuntimeError):
        ext.moe_combine_exchange([0], [slot.data_ptr()], ids, w, [buf.data_ptr()], 1, 0, 4, 64)


@pytest.mark.parametrize("t,e,k", [(4096, 256, 8), (33, 64, 6), (7, 384, 8), (5, 8, 8), (1, 256, 1)])
def test_moe_topk_matches_oracle(cabi, ext, t, e, k):
    logits = torch.randn((t, e), generator=torch.Generator().manual_seed(t + e))
    logits[0, : min(e, 5)] = 1.25              # ties: the lower expert index wins
    ids_ref, w_ref = oracle.moe_topk(logits, k)
    ids, w = cabi.moe_topk(logits.cuda(), k)
    assert torch.equal(ids.cpu(), ids_ref)
    # device expf and libm expf may differ in the last bit
    assert torch.allclose(w.cpu(), w_ref, rtol=2e-6, atol=1e-9)
    ids2, w2 = ext.moe_topk(logits.cuda(), k)
    assert torch.equal(ids2.cpu(), ids_ref) and torch.allclose(w2.cpu(), w_ref, rtol=2e-6, atol=1e-9)
    # same set (and order) as torch.topk where there are no ties
    tv, ti = torch.topk(logits[1:], k, dim=-1)
    assert torch.equal(ids_ref[1:].long(), ti)
    assert torch.allclose(w_ref[1:], torch.softmax(tv, dim=-1), rtol=1e-5, atol=1e-8)


def test_moe_full_size_sampled_experts_match_oracle():
    # the configuration's full size (4096 tokens, 256 experts of 4096 x 7168 + 7168 x 2048, top-8,
    # group-128 activation scales) on the device; the oracle re-derives every stage for a few
    # experts (their routed rows only) and the combined output for the tokens those experts serve
    from bw1000_dsv4_kernels_b200 import moe
    dev = torch.device("cuda")
    t, h, e, inter, topk = wl.MOE_TOKENS, wl.HIDDEN, wl.MOE_EXPERTS, wl.MOE_INTER, wl.MOE_TOPK
    inp = wl.moe_inputs(t, h, e, inter, topk, device=dev, seed=0)
    layer = moe.W8A8MoE(inp.w13, inp.w13_scale, inp.w2, inp.w2_scale, e, group_scaled=True)
    out = layer.forward(inp.x, inp.topk_ids, inp.topk_w, keep_trace=True)
    tr = layer.last_trace
    torch.cuda.synchronize()
    # front end against the oracle on the whole problem (cheap)
    q_ref, s_ref = oracle.per_token_group_quant_int8(inp.x.cpu(), 128)
    off_ref, src_ref, dst_ref = oracle.moe_segments(inp.topk_ids.cpu(), e)
    assert int(off_ref[-1]) == t * topk
    assert torch.equal(tr.offsets.cpu(), off_ref) and torch.equal(tr.dst_slot.cpu(), dst_ref)
    assert torch.equal(tr.src_row.cpu(), src_ref)
    assert torch.equal(tr.a_q.cpu(), q_ref[src_ref.long()]) and torch.equal(tr.a_s.cpu(), s_ref[src_ref.long()])
    rows = (off_ref[1:] - off_ref[:-1])
    picks = [int(rows.argmax()), int(rows.argmin()), 123]          # the fullest, the emptiest, one more
    z_dev = tr.z.cpu()
    for ex in picks:
        lo, hi = int(off_ref[ex]), int(off_ref[ex + 1])
        if hi == lo:
            continue
        one = torch.tensor([0, hi - lo], dtype=torch.int32)
        a_q, a_s = q_ref[src_ref[lo:hi].long()], s_ref[src_ref[lo:hi].long()]
        y = oracle.grouped_gemm(a_q, inp.w13[ex:ex + 1].cpu(), a_s, inp.w13_scale[ex:ex + 1].cpu(), one)
        assert torch.equal(tr.y[lo:hi].cpu().view(torch.int16), y.view(torch.int16)), f"gate/up GEMM, expert {ex}"
        h_q, h_s = oracle.silu_mul_quant(y[:, :inter], y[:, inter:])
        assert torch.equal(tr.h_q[lo:hi].cpu(), h_q) and torch.equal(tr.h_s[lo:hi].cpu(), h_s), f"silu, expert {ex}"
        z = oracle.grouped_gemm(h_q, inp.w2[ex:ex + 1].cpu(), h_s.view(-1), inp.w2_scale[ex:ex + 1].cpu(), one)
        assert torch.equal(z_dev[lo:hi].view(torch.int16), z.view(torch.int16)), f"down GEMM, expert {ex}"
    # combine: the oracle on the device's z (verified above for the sampled experts) for every token
    ref = oracle.moe_combine(z_dev, dst_ref, inp.topk_w.cpu())
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16)), "combined output"
