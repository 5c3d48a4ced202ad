"""The operators under CUDA-graph capture (how the serving engine runs them): capture the chain once,
refill the static inputs, replay, and compare with the oracle."""
import pytest
import torch

from bw1000_dsv4_kernels_b200 import workloads as wl
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
