"""GPU parity of the int8 GEMM (dense and grouped) against the CPU oracle.
int32 accumulators bit-exact; bf16 outputs are compared bit-exact too (the epilogue is a
fixed sequence of rounded operations) and, as the stated bar, within 1e-2 of the output's
absolute maximum."""
import pytest
import torch

from tests import workloads as wl
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu

TOL_REL_TO_ABSMAX = 1e-2


def _operands(m, n, k, seed):
    A = wl.int8_weights((m, k), seed=seed)
    B = wl.int8_weights((n, k), seed=seed + 1)
    sa = wl.channel_scales((m,), seed=seed + 2) * 3.0
    sb = wl.channel_scales((n,), seed=seed + 3)
    return A, B, sa, sb


def _check_bf16(out, ref, what):
    out, ref = out.cpu(), ref.cpu()
    assert out.shape == ref.shape
    absmax = ref.float().abs().max().item()
    err = (out.float() - ref.float()).abs().max().item()
    assert err <= TOL_REL_TO_ABSMAX * max(absmax, 1e-30), f"{what}: max abs err {err} vs absmax {absmax}"
    bad = (out.view(torch.int16) != ref.view(torch.int16)).sum().item()
    assert bad == 0, f"{what}: {bad} of {out.numel()} bf16 outputs differ in bits"


SHAPES = [
    (128, 256, 128),     # one tile, one k-block
    (128, 256, 512),     # one tile, several k-blocks (ring wraps at 4 stages)
    (256, 512, 1024),    # several tiles per CTA? no: 4 tiles over 4 CTAs
    (1, 4096, 7168),     # decode row
    (16, 4096, 7168),
    (64, 4096, 7168),
    (256, 4096, 7168),
    (100, 200, 304),     # ragged M, N; K not a multiple of 128
    (130, 264, 2064),    # ragged last tiles in both dimensions
    (5, 72, 16),         # smallest K
    (300, 1000, 4096),
    (64, 7168, 18432),   # down projection, long K: |acc| exceeds 2^24
    (200, 1000, 1040),   # 129..256 tokens: weight streaming on CTA pairs, ragged N and K
    (129, 256, 16),      # the same with a single K block (no split)
    (256, 1160, 400),    # last pair tile half empty
]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_i32_bit_exact(cabi, m, n, k):
    A, B, _, _ = _operands(m, n, k, seed=m + n + k)
    ref = oracle.gemm_i32(A, B)
    out = cabi.w8a8_gemm_i32(A.cuda(), B.cuda())
    assert cabi.device_status() == 0
    bad = (out.cpu() != ref).sum().item()
    assert bad == 0, f"{bad} of {ref.numel()} int32 accumulators differ"


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_w8a8_gemm_matches_oracle(cabi, ext, m, n, k):
    A, B, sa, sb = _operands(m, n, k, seed=m + n + k)
    ref = oracle.w8a8_gemm(A, B, sa, sb)
    out = cabi.w8a8_gemm(A.cuda(), B.cuda(), sa.cuda(), sb.cuda())
    assert cabi.device_status() == 0
    _check_bf16(out, ref, "C-ABI")
    out2 = ext.w8a8_scaled_gemm(A.cuda(), B.cuda(), sa.cuda().unsqueeze(-1), sb.cuda())
    _check_bf16(out2, ref, "operator")
    out3 = ext.w8a8_gemm(A.cuda(), B.cuda(), sa.cuda(), sb.cuda())
    _check_bf16(out3, ref, "alias")


@pytest.mark.parametrize("m,n,k", [(1100, 2320, 272), (2048, 4096, 128), (1537, 4104, 400), (4096, 2560, 7168)])
def test_gemm_cta_pair_kernel(cabi, m, n, k):
    # large enough for the 256 x 256 CTA-pair kernel; ragged last tiles in M and N, short and long K
    A, B, sa, sb = _operands(m, n, k, seed=m + n + k)
    Ad, Bd = A.cuda(), B.cuda()
    acc = cabi.w8a8_gemm_i32(Ad, Bd)
    out = cabi.w8a8_gemm(Ad, Bd, sa.cuda(), sb.cuda())
    assert cabi.device_status() == 0
    if m * n * k <= 2e10:
        ref_acc = oracle.gemm_i32(A, B)
        assert (acc.cpu() != ref_acc).sum().item() == 0
        _check_bf16(out, oracle.w8a8_gemm(A, B, sa, sb), "pair kernel")
    else:
        rows = torch.arange(0, m, 37)
        ref_acc = oracle.gemm_i32(A[rows], B)
        assert (acc.cpu()[rows] != ref_acc).sum().item() == 0
        _check_bf16(out[rows.cuda()], oracle.scale_convert(ref_acc, sa[rows], sb), "pair kernel (sampled rows)")


def test_gemm_many_tiles_per_cta(cabi):
    # 2048 x 4096 -> 256 tiles of 128x256 on 148 CTAs: every CTA loops, both accumulators cycle
    m, n, k = 2048, 4096, 1024
    A, B, sa, sb = _operands(m, n, k, seed=1)
    ref = oracle.w8a8_gemm(A, B, sa, sb)
    out = cabi.w8a8_gemm(A.cuda(), B.cuda(), sa.cuda(), sb.cuda())
    assert cabi.device_status() == 0
    _check_bf16(out, ref, "2048x4096x1024")


def test_gemm_extreme_values_no_overflow_surprise(cabi):
    # all operands at +-127/-128: the largest magnitudes the accumulator can see
    m, n, k = 128, 256, 18432
    A = torch.full((m, k), 127, dtype=torch.int8)
    B = torch.full((n, k), 127, dtype=torch.int8)
    B[::2] = -128
    ref = oracle.gemm_i32(A, B)
    out = cabi.w8a8_gemm_i32(A.cuda(), B.cuda())
    assert (out.cpu() != ref).sum().item() == 0
    sa = torch.full((m,), 1e-3)
    sb = torch.full((n,), 1e-3)
    _check_bf16(cabi.w8a8_gemm(A.cuda(), B.cuda(), sa.cuda(), sb.cuda()), oracle.w8a8_gemm(A, B, sa, sb), "extremes")


def test_scale_convert_matches_oracle(cabi, ext):
    m, n = 37, 1000
    acc = torch.randint(-(2 ** 28), 2 ** 28, (m, n), dtype=torch.int32, generator=torch.Generator().manual_seed(3))
    sa = wl.channel_scales((m,), seed=1)
    sb = wl.channel_scales((n,), seed=2)
    ref = oracle.scale_convert(acc, sa, sb)
    _check_bf16(cabi.scale_convert(acc.cuda(), sa.cuda(), sb.cuda()), ref, "C-ABI")
    _check_bf16(ext.scale_convert(acc.cuda(), sa.cuda(), sb.cuda()), ref, "operator")


def test_linearity_at_full_size(cabi):
    # size-independent property at the benchmark's largest dense shape: the int32 product is
    # linear in A, so (A1 + A2) B^T == A1 B^T + A2 B^T exactly when A1 + A2 stays in int8
    m, n, k = 2048, 4096, 7168
    g = torch.Generator(device="cuda").manual_seed(0)
    A1 = torch.randint(-60, 61, (m, k), dtype=torch.int8, device="cuda", generator=g)
    A2 = torch.randint(-60, 61, (m, k), dtype=torch.int8, device="cuda", generator=g)
    B = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda", generator=g)
    c12 = cabi.w8a8_gemm_i32(A1 + A2, B)
    c1 = cabi.w8a8_gemm_i32(A1, B)
    c2 = cabi.w8a8_gemm_i32(A2, B)
    assert cabi.device_status() == 0
    assert torch.equal(c12, c1 + c2)
    # and a sampled block against the oracle
    ref = oracle.gemm_i32(A1[:64].cpu(), B[:512].cpu())
    assert torch.equal(c1[:64, :512].cpu(), ref)


def _boundary_indices(size, step=256, halo=2):
    """Indices either side of every multiple of `step` (tile boundaries), plus both ends."""
    idx = set(range(0, min(halo, size))) | set(range(max(0, size - halo), size))
    for b in range(step, size, step):
        idx |= set(range(b - halo, min(b + halo, size)))
    return torch.tensor(sorted(idx))


@pytest.mark.parametrize("m,n,k", [(2048, 4096, 7168), (2048, 7168, 18432)])
def test_dense_gemm_full_size_every_tile_boundary(cabi, m, n, k):
    # the two dense projections at M=2048, at full size.  (1) every int32 accumulator against the library
    # integer product (a second opinion on all M*N elements); (2) the bf16 result on the rows and columns either
    # side of EVERY 256-row / 256-column tile boundary of the CTA-pair tiling against the oracle, over the whole
    # K (first and last K block included)
    g = torch.Generator(device="cuda").manual_seed(m + n)
    A = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda", generator=g)
    B = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda", generator=g)
    sa = wl.channel_scales((m,), device="cuda", seed=1)
    sb = wl.channel_scales((n,), device="cuda", seed=2)
    acc = cabi.w8a8_gemm_i32(A, B)
    assert torch.equal(acc, torch._int_mm(A, B.t()))
    out = cabi.w8a8_gemm(A, B, sa, sb)
    assert cabi.device_status() == 0
    rows, cols = _boundary_indices(m), _boundary_indices(n)
    ref = oracle.w8a8_gemm(A[rows.cuda()].cpu(), B[cols.cuda()].cpu(), sa[rows.cuda()].cpu(), sb[cols.cuda()].cpu())
    got = out[rows.cuda()][:, cols.cuda()].cpu()
    assert torch.equal(got.contiguous().view(torch.int16), ref.view(torch.int16))
    # and the whole bf16 result against the formula on the (already checked) accumulators
    full = ((acc.to(torch.float32) * sa.view(-1, 1)) * sb.view(1, -1)).to(torch.bfloat16)
    assert torch.equal(out.view(torch.int16), full.view(torch.int16))


def test_gemm_argument_errors(cabi, ext):
    A = torch.zeros((4, 24), dtype=torch.int8, device="cuda")
    B = torch.zeros((8, 24), dtype=torch.int8, device="cuda")
    s = torch.ones(8, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ext.w8a8_scaled_gemm(A, B, s[:4], s)
    with pytest.raises(RuntimeError):
        ext.w8a8_scaled_gemm(A.cpu(), B.cpu(), s[:4].cpu(), s.cpu())
    with pytest.raises(RuntimeError):
        ext.w8a8_scaled_gemm(A.float(), B, s[:4], s)
    out = ext.w8a8_scaled_gemm(torch.zeros((0, 32), dtype=torch.int8, device="cuda"),
                               torch.zeros((8, 32), dtype=torch.int8, device="cuda"), s[:0], s)
    assert out.shape == (0, 8)


# ---- grouped GEMM ---------------------------------------------------------------------
def _grouped_case(seg_lens, n, k, seed):
    e = len(seg_lens)
    off = torch.zeros(e + 1, dtype=torch.int32)
    off[1:] = torch.cumsum(torch.tensor(seg_lens), 0)
    r = int(off[-1])
    A = wl.int8_weights((r, k), seed=seed)
    W = wl.int8_weights((e, n, k), seed=seed + 1)
    sa = wl.channel_scales((r,), seed=seed + 2) * 3.0
    sw = wl.channel_scales((e, n), seed=seed + 3)
    return A, W, sa, sw, off


@pytest.mark.parametrize("seg_lens,n,k", [
    ([128, 128], 256, 256),
    ([5, 0, 300, 128, 1, 0, 77], 512, 384),
    ([130] * 16, 1024, 512),
    ([0, 0, 9], 72, 64),
    ([64, 200, 17, 129, 255, 3, 0, 90], 4096, 7168),
])
def test_grouped_gemm_matches_oracle(cabi, ext, seg_lens, n, k):
    A, W, sa, sw, off = _grouped_case(seg_lens, n, k, seed=len(seg_lens) + n)
    ref = oracle.grouped_gemm(A, W, sa, sw, off)
    out = cabi.grouped_gemm(A.cuda(), W.cuda(), sa.cuda(), sw.cuda(), off.cuda())
    assert cabi.device_status() == 0
    _check_bf16(out, ref, "C-ABI")
    out2 = ext.grouped_gemm(A.cuda(), W.cuda(), sa.cuda().unsqueeze(-1), sw.cuda(), off.cuda())
    _check_bf16(out2, ref, "operator")


@pytest.mark.parametrize("seg_lens,n,k,shift", [
    ([5, 0, 300, 128, 1, 0, 77], 512, 384, 0),      # 16-byte aligned rows: 256-byte segments
    ([130] * 4, 1000, 512, 0),                       # N ends inside a 16-byte piece of the last tile
    ([64, 200, 17], 200, 7168, 1),                   # rows aligned to 2 bytes only: element stores
])
def test_grouped_gemm_with_row_destinations(cabi, ext, seg_lens, n, k, shift):
    # every result row is stored at its own address: here the rows of a wider buffer in reverse order
    A, W, sa, sw, off = _grouped_case(seg_lens, n, k, seed=len(seg_lens) + n + k)
    ref = oracle.grouped_gemm(A, W, sa, sw, off)
    r = A.shape[0]
    width = n + 24
    buf = torch.full((r, width), float("nan"), dtype=torch.bfloat16, device="cuda")
    rows = torch.arange(r - 1, -1, -1, dtype=torch.int64, device="cuda")
    row_ptr = (buf.data_ptr() + rows * (width * 2) + 2 * shift).contiguous()
    ext.grouped_gemm_scatter(A.cuda(), W.cuda(), sa.cuda(), sw.cuda(), off.cuda(), row_ptr)
    torch.cuda.synchronize()
    assert cabi.device_status() == 0
    got = buf.flip(0)[:, shift:shift + n].contiguous()
    _check_bf16(got, ref, "row destinations")
    untouched = torch.cat([buf[:, :shift], buf[:, shift + n:]], dim=1)
    assert bool(torch.isnan(untouched.float()).all()), "stores outside the rows' N elements"


@pytest.mark.parametrize("seg_lens,n,k", [
    ([128, 128], 256, 256),
    ([5, 0, 300, 128, 1, 0, 77], 520, 384),
    ([0, 0, 9], 72, 128),
    ([64, 200, 17, 129, 255, 3, 0, 90], 4096, 7168),
])
def test_group_scaled_grouped_gemm_matches_oracle(cabi, ext, seg_lens, n, k):
    # one activation scale per (row, 128 columns of K): y = fma(float(acc_g), s[r,g], y), then * sw
    A, W, _, sw, off = _grouped_case(seg_lens, n, k, seed=3 * len(seg_lens) + n)
    r = A.shape[0]
    sg = (wl.channel_scales((r, k // 128), seed=77) * 3.0).contiguous()
    ref = oracle.grouped_gemm(A, W, sg, sw, off)
    out = cabi.grouped_gemm(A.cuda(), W.cuda(), sg.cuda(), sw.cuda(), off.cuda())
    assert cabi.device_status() == 0
    _check_bf16(out, ref, "C-ABI")
    out2 = ext.grouped_gemm(A.cuda(), W.cuda(), sg.cuda(), sw.cuda(), off.cuda())
    _check_bf16(out2, ref, "operator")


def test_gemm_writes_into_column_slab(cabi, ext):
    # the column-sharded linear writes each rank's result into a slab of a wider buffer (ldc > N)
    m, n, k, width = 300, 256, 512, 1024
    A, B, sa, sb = _operands(m, n, k, seed=5)
    ref = oracle.w8a8_gemm(A, B, sa, sb)
    buf = torch.full((m, width), 7.0, dtype=torch.bfloat16, device="cuda")
    cabi.w8a8_gemm_ld(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), buf, 512)
    assert torch.equal(buf[:, 512:768].cpu().view(torch.int16), ref.view(torch.int16))
    assert (buf[:, :512] == 7.0).all() and (buf[:, 768:] == 7.0).all()
    buf2 = torch.zeros((m, width), dtype=torch.bfloat16, device="cuda")
    ext.w8a8_gemm_into(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), buf2, 256)
    assert torch.equal(buf2[:, 256:512].cpu().view(torch.int16), ref.view(torch.int16))
    # large enough for the CTA-pair kernel
    m, n, k = 2048, 2048, 256
    A, B, sa, sb = _operands(m, n, k, seed=6)
    buf3 = torch.zeros((m, 4096), dtype=torch.bfloat16, device="cuda")
    cabi.w8a8_gemm_ld(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), buf3, 2048)
    assert torch.equal(buf3[:, 2048:].cpu().view(torch.int16), oracle.w8a8_gemm(A, B, sa, sb).view(torch.int16))
    assert buf3[:, :2048].abs().sum().item() == 0


def test_gemm_fused_allgather_stores_to_every_buffer(cabi, ext):
    # the peer buffers of the fused all-gather, emulated on one GPU: three [M, 1024] buffers, the
    # GEMM must write the same slab into all of them and touch nothing else
    m, n, k, width, col0 = 2048, 512, 384, 1024, 256
    A, B, sa, sb = _operands(m, n, k, seed=9)
    ref = oracle.w8a8_gemm(A, B, sa, sb)
    bufs = [torch.full((m, width), 3.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    ext.w8a8_gemm_allgather(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), bufs[0], col0, [b.data_ptr() for b in bufs[1:]])
    assert cabi.device_status() == 0
    for b in bufs:
        assert torch.equal(b[:, col0:col0 + n].cpu().view(torch.int16), ref.view(torch.int16))
        assert (b[:, :col0] == 3.0).all() and (b[:, col0 + n:] == 3.0).all()
    # few rows: the one-CTA-per-tile kernel takes the peer path as well
    m2 = 100
    bufs = [torch.zeros((m2, width), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    ext.w8a8_gemm_allgather(A[:m2].cuda(), B.cuda(), sa[:m2].cuda(), sb.cuda(), bufs[0], 0, [bufs[1].data_ptr()])
    for b in bufs:
        assert torch.equal(b[:, :n].cpu().view(torch.int16), ref[:m2].view(torch.int16))


@pytest.mark.parametrize("m,n", [(2048, 2560), (1900, 2592), (4096, 3072)])
def test_gemm_fused_allgather_tile_store_path(cabi, ext, m, n):
    # enough tiles for the CTA-pair kernel, whose fused epilogue stages the tile in shared memory and
    # sends it with TMA tile stores; ragged M, and N that is a multiple of 32 but not of 64; the last
    # case gives every CTA pair three or four tiles, so the ring of staging slabs wraps several times
    k, width, col0 = 256, 4096, 1024
    A, B, sa, sb = _operands(m, n, k, seed=m + n)
    ref = oracle.w8a8_gemm(A, B, sa, sb)
    bufs = [torch.full((m, width), 5.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    ext.w8a8_gemm_allgather(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), bufs[0], col0, [b.data_ptr() for b in bufs[1:]])
    assert cabi.device_status() == 0
    for b in bufs:
        assert torch.equal(b[:, col0:col0 + n].cpu().view(torch.int16), ref.view(torch.int16))
        assert (b[:, :col0] == 5.0).all() and (b[:, col0 + n:] == 5.0).all()


def test_gemm_fused_allgather_eight_destinations(cabi, ext):
    # the widest case the entry point takes: this rank's buffer and seven peers (eight tensor maps of stores),
    # emulated with eight local buffers; the destinations are written in the order given
    m, n, k, width, col0 = 2048, 2560, 256, 3072, 512
    A, B, sa, sb = _operands(m, n, k, seed=77)
    ref = oracle.w8a8_gemm(A, B, sa, sb)
    bufs = [torch.full((m, width), 5.0, dtype=torch.bfloat16, device="cuda") for _ in range(8)]
    order = [3, 4, 5, 6, 7, 1, 2]      # a rotated peer order, as a rank in the middle would pass it
    ext.w8a8_gemm_allgather(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), bufs[0], col0, [bufs[i].data_ptr() for i in order])
    assert cabi.device_status() == 0
    for b in bufs:
        assert torch.equal(b[:, col0:col0 + n].cpu().view(torch.int16), ref.view(torch.int16))
        assert (b[:, :col0] == 5.0).all() and (b[:, col0 + n:] == 5.0).all()
    with pytest.raises(RuntimeError):   # an eighth peer is one too many
        ext.w8a8_gemm_allgather(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), bufs[0], col0, [b.data_ptr() for b in bufs])


def test_tp_linear_full_size_shards_equal_the_whole(ext):
    # the column-sharded configuration at its full size (M=8192, K=7168, N=28672) on one device: the
    # eight ranks' slabs, each from that rank's own seeded weight shard and written into its column
    # range, give the bits of the unsharded layer (columns are independent: a size-independent
    # property); a sampled block of rows and columns is also checked against the oracle
    from bw1000_dsv4_kernels_b200 import tp_linear
    dev = torch.device("cuda")
    m, k, n, world = wl.TP_M, wl.HIDDEN, wl.TP_N, 8
    full = wl.tp_linear_inputs(0, 1, m=m, k=k, n=n, device=dev, seed=0)
    whole = tp_linear.ColumnParallelW8A8Linear(full.w, full.w_scale).forward(full.x)
    q, s = ext.per_token_quant_int8(full.x)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    per = n // world
    for r in range(world):
        shard = wl.tp_linear_inputs(r, world, m=m, k=k, n=n, device=dev, seed=0)
        assert torch.equal(shard.w, full.w[r * per:(r + 1) * per])
        ext.w8a8_gemm_into(q, shard.w, s, shard.w_scale, out, r * per)
    assert torch.equal(out.view(torch.int16), whole.view(torch.int16))
    rows, cols = slice(4000, 4064), slice(per * 3 - 32, per * 3 + 32)    # straddles two ranks' slabs
    q_ref, s_ref = oracle.per_token_quant_int8(full.x[rows].cpu())
    ref = oracle.w8a8_gemm(q_ref, full.w[cols].cpu(), s_ref.view(-1), full.w_scale[cols].cpu())
    assert torch.equal(whole[rows, cols].cpu().contiguous().view(torch.int16), ref.view(torch.int16))


def test_down_projection_chain_full_size_sampled(ext):
    # silu_mul_quant -> down-projection GEMM at the configuration's largest size (M=8192, N=18432 ->
    # 7168): every row's codes and scale are checked against the oracle on sampled rows (rows are
    # independent), the GEMM on a sampled block of rows and columns
    dev = torch.device("cuda")
    m, inter, h = 8192, wl.DENSE_INTER, wl.HIDDEN
    gu = wl.randn_bf16((m, 2 * inter), device=dev, seed=3)
    w = wl.int8_weights((h, inter), device=dev, seed=4)
    ws = wl.channel_scales((h,), device=dev, seed=5)
    q, s = ext.silu_mul_quant(gu[:, :inter], gu[:, inter:])
    y = ext.w8a8_scaled_gemm(q, w, s, ws)
    q2, s2 = ext.silu_mul_quant(gu[:, :inter], gu[:, inter:])
    assert torch.equal(q, q2) and torch.equal(s, s2), "same input, same codes"
    rows = torch.tensor([0, 1, 777, 4095, 4096, 8190, 8191] + list(range(3000, 3057)))
    gu_s = gu[rows].cpu()
    q_ref, s_ref = oracle.silu_mul_quant(gu_s[:, :inter], gu_s[:, inter:])
    assert torch.equal(q[rows].cpu(), q_ref) and torch.equal(s[rows].cpu(), s_ref)
    cols = slice(7168 - 96, 7168)
    ref = oracle.w8a8_gemm(q_ref, w[cols].cpu(), s_ref.view(-1), ws[cols].cpu())
    assert torch.equal(y[rows][:, cols].cpu().contiguous().view(torch.int16), ref.view(torch.int16))
