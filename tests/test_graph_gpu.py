"""The operators under CUDA-graph capture (how the serving engine runs them): capture the chain once,
refill the static inputs, replay, and compare with the oracle."""
import pytest
import torch

from tests import workloads as wl
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu


def test_chain_replays_from_a_cuda_graph(ext):
    m, k, n = 48, 2048, 512
    first = wl.norm_gemm_inputs(m, k=k, n=n, seed=1)
    x, res = first.x.cuda(), first.res.cuda()
    gamma, w, ws = first.gamma.cuda(), first.w.cuda(), first.w_scale.cuda()
    # warm up outside capture (first-use attribute set-up happens here)
    q, s = ext.add_rmsnorm_quant(res.clone(), x, gamma, 1e-6)
    ext.w8a8_scaled_gemm(q, w, s, ws)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        q, s = ext.add_rmsnorm_quant(res, x, gamma, 1e-6)
        y = ext.w8a8_scaled_gemm(q, w, s, ws)
    for seed in (7, 8):
        inp = wl.norm_gemm_inputs(m, k=k, n=n, seed=seed)
        x.copy_(inp.x)
        res.copy_(inp.res)
        graph.replay()
        torch.cuda.synchronize()
        res_ref = inp.res.clone()
        q_ref, s_ref = oracle.add_rmsnorm_quant(res_ref, inp.x, first.gamma, 1e-6)
        y_ref = oracle.w8a8_gemm(q_ref, first.w, s_ref.view(-1), first.w_scale)
        assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
        assert torch.equal(res.cpu().view(torch.int16), res_ref.view(torch.int16))
        assert torch.equal(y.cpu().view(torch.int16), y_ref.view(torch.int16))
    assert ext.device_status() == 0


def test_stream_variant_under_capture_matches_patch_wrapper(ext):
    from bw1000_dsv4_kernels_b200 import lmslim_patch
    wrapper = lmslim_patch.make_wrapper(ext, lambda: torch.cuda.current_stream().cuda_stream)
    x = wl.activations_with_outliers(32, 4096, seed=3).cuda()
    wrapper(x)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        q, s = wrapper(x, scale_dtype=None, cal_sum=False)
    x2 = wl.activations_with_outliers(32, 4096, seed=4)
    x.copy_(x2)
    graph.replay()
    torch.cuda.synchronize()
    q_ref, s_ref = oracle.per_token_quant_int8(x2)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)


@pytest.mark.parametrize("m", [1, 16, 64, 200, 256])
def test_overlap_with_previous_kernel_gives_the_same_bits(ext, m):
    # with the option on, the GEMM for M <= 256 starts (set-up, weight loads) while the quantiser
    # before it is still running and waits for it only before it touches activations or output:
    # a chain of dependent launches, eagerly and from a CUDA graph, must give the bits of the
    # fully serialised run, also when every step reuses the same buffers
    k, n = 2048, 1024
    steps = [wl.norm_gemm_inputs(m, k=k, n=n, seed=30 + i) for i in range(4)]
    gamma, w, ws = steps[0].gamma.cuda(), steps[0].w.cuda(), steps[0].w_scale.cuda()
    x, res = torch.empty_like(steps[0].x, device="cuda"), torch.empty_like(steps[0].res, device="cuda")
    keep = torch.empty((len(steps), m, n), dtype=torch.bfloat16, device="cuda")

    def run_eager():
        for i, st in enumerate(steps):
            x.copy_(st.x, non_blocking=True)
            res.copy_(st.res, non_blocking=True)
            q, s = ext.add_rmsnorm_quant(res, x, gamma, 1e-6)
            keep[i].copy_(ext.w8a8_scaled_gemm(q, w, s, ws))
        torch.cuda.synchronize()
        return keep.clone()

    assert not ext.get_overlap_previous_kernel()
    ref = run_eager()
    try:
        ext.set_overlap_previous_kernel(True)
        assert ext.get_overlap_previous_kernel()
        out = run_eager()
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), "eager launches"
        xs = torch.stack([st.x for st in steps]).cuda()
        rs = torch.stack([st.res for st in steps]).cuda()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(len(steps)):
                q, s = ext.add_rmsnorm_quant(rs[i], xs[i], gamma, 1e-6)
                y = ext.w8a8_scaled_gemm(q, w, s, ws)
                keep[i].copy_(y)
        for _ in range(2):
            rs.copy_(torch.stack([st.res for st in steps]))
            keep.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(keep.view(torch.int16), ref.view(torch.int16)), "graph replay"
    finally:
        ext.set_overlap_previous_kernel(False)
    assert ext.device_status() == 0


def test_overlap_option_on_the_cta_pair_gemm(ext):
    # M large enough for the CTA-pair kernel: the same contract (weight tiles before the dependency wait,
    # activation tiles and the epilogue after it), same bits as the serialised run
    m, k, n = 1024, 1024, 2304
    steps = [wl.norm_gemm_inputs(m, k=k, n=n, seed=50 + i) for i in range(3)]
    gamma, w, ws = steps[0].gamma.cuda(), steps[0].w.cuda(), steps[0].w_scale.cuda()
    xs = torch.stack([st.x for st in steps]).cuda()
    rs0 = torch.stack([st.res for st in steps]).cuda()

    def run():
        rs = rs0.clone()
        outs = []
        for i in range(len(steps)):
            q, s = ext.add_rmsnorm_quant(rs[i], xs[i], gamma, 1e-6)
            outs.append(ext.w8a8_scaled_gemm(q, w, s, ws))
        torch.cuda.synchronize()
        return torch.stack(outs)

    ref = run()
    try:
        ext.set_overlap_previous_kernel(True)
        out = run()
    finally:
        ext.set_overlap_previous_kernel(False)
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    assert ext.device_status() == 0
