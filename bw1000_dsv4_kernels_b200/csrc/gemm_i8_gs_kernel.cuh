// Private part of gemm_i8_sm100.cu (included by that translation unit only, hence the unnamed
// namespace): the group-scaled kernel (one activation scale per 128 of K).
#ifndef W8A8_GEMM_I8_GS_KERNEL_CUH
#define W8A8_GEMM_I8_GS_KERNEL_CUH

#include "gemm_i8_common.cuh"

namespace w8a8 {
namespace {

// ------------------------------------------------------------------------------------
// Group-scaled kernel (grouped or dense): the activation scale changes every 128 columns
// of K, so each 128-deep K block is its own int32 accumulator.  The MMA warp alternates
// between two 128-column accumulators in tensor memory; the drain warps fold block g into
// fp32 registers as y = fma(float(acc_g), sa[row, g], y) while the MMAs of block g+1 run,
// and apply the channel scale once at the end of the tile.  Tile = 128 x 128.
// ------------------------------------------------------------------------------------
constexpr int GSN = 256;               // tile width: the wider tile halves the re-reads of the A rows from L2
constexpr int kGsBufs = 2;             // 256-column accumulators in flight (all 512 TMEM columns)
constexpr int kGsDrainWarps = 16;      // four per TMEM lane quarter, 64 columns each
constexpr int kGsThreads = 64 + 32 * kGsDrainWarps;  // producer warp, MMA warp, drain warps

template <int STAGES>
__global__ void __launch_bounds__(kGsThreads, 1)
gemm_i8_gs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const Params p) {
    using L = Smem<GSN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* sb_tile = reinterpret_cast<float*>(smem + L::kSbOff);
    int* prefix = reinterpret_cast<int*>(smem + L::kPrefixOff);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ((L::kBarOff + 7) & ~7));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

    const uint32_t tiles_base = ptx::smem_u32(smem);
    const uint32_t bar_base = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto blk_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto blk_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + kGsBufs + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kTmemCols = kGsBufs * GSN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < kGsBufs; ++a) {
            ptx::mbar_init(blk_full_bar(a), 1);
            ptx::mbar_init(blk_empty_bar(a), kGsDrainWarps);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    if (p.offsets != nullptr && warp == 2) build_tile_prefix(p, prefix, lane);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const Scheduler sched(p, prefix, GSN);
    const int k_blocks = (p.K + BK - 1) / BK;

    if (warp == 0) {
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
                const TileCoord c = sched.at(t, GSN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u) || *abort_flag) {
                        report_wait_failure(kWaitEmptyStage);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = tiles_base + stage * L::kStageBytes;
                    ptx::mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
                    ptx::tma_load_2d(a_dst, &tmA, kb * BK, c.a_row0, full_bar(stage));
                    ptx::tma_load_2d(a_dst + L::kABytes, &tmB, kb * BK, c.b_row0, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(BM, GSN);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t blk = 0;  // running K-block counter: buffer = blk % kGsBufs, parity = (blk / kGsBufs) & 1
            bool ok = true;
            for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
                for (int kb = 0; kb < k_blocks; ++kb, ++blk) {
                    const int b = blk % kGsBufs;
                    if (!ptx::mbar_wait_bounded(blk_empty_bar(b), ((blk / kGsBufs) & 1u) ^ 1u) ||
                        !ptx::mbar_wait_bounded(full_bar(stage), phase) || *abort_flag) {
                        report_wait_failure(kWaitFullStage);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_src = tiles_base + stage * L::kStageBytes;
                    const uint64_t adesc = ptx::smem_desc_k_sw128(a_src);
                    const uint64_t bdesc = ptx::smem_desc_k_sw128(a_src + L::kABytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        ptx::mma_i8_ss(tmem_base + b * GSN, adesc + 2u * k, bdesc + 2u * k, idesc, k != 0 ? 1u : 0u);
                    ptx::tc_commit(empty_bar(stage));
                    ptx::tc_commit(blk_full_bar(b));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
        // Sixteen drain warps: warps w, w+4, w+8, w+12 share TMEM lane quarter w%4 and take 64 columns
        // each, 16 at a time (the fp32 accumulators of the 128 x 256 tile fill half the register file,
        // so the tensor-memory loads are kept narrow).
        constexpr int HC = GSN * 4 / kGsDrainWarps;   // columns per warp
        static_assert(HC == 64, "four 16-column tcgen05.ld per warp and K block");
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;             // which 64-column quarter of the tile
        float* sbs = sb_tile + quarter * GSN;         // each warp fills and reads its own 64 columns
        const bool vec_ok = c_vector_stores_ok(p);
        uint32_t blk = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
            const TileCoord c = sched.at(t, GSN);
            __syncwarp();
            {
                const float* sb_row = p.sb + (int64_t)c.expert * p.N;
                for (int j = lane; j < HC; j += 32) {
                    const int col = half * HC + j;
                    sbs[col] = (c.n0 + col < p.N) ? __ldg(sb_row + c.n0 + col) : 0.0f;
                }
            }
            __syncwarp();
            const int row = c.a_row0 + quarter * 32 + lane;
            const bool row_ok = row < c.row_end;
            // A warp whose 32 rows all lie past the end of the segment (the mostly empty last tile of
            // an expert) only keeps the buffer hand-over going: no tensor-memory loads, no arithmetic.
            const bool warp_has_rows = c.a_row0 + quarter * 32 < c.row_end;
            const float* sa_row = p.sa + (int64_t)(row_ok ? row : 0) * p.sa_groups;
            // y as float2 lanes: the fold below runs on packed f32x2 instructions.  float(acc) is
            // formed without a conversion instruction (those issue at a quarter of the FMA rate):
            // |acc| <= 128*128*128 < 2^22, so the bit pattern 0x4B400000 + acc is the float
            // 1.5*2^23 + acc exactly, and subtracting 1.5*2^23 leaves float(acc) exactly.
            float2 y2[HC / 2];
#pragma unroll
            for (int j = 0; j < HC / 2; ++j) y2[j] = make_float2(0.0f, 0.0f);
            // the row's group scales are fetched three K blocks ahead: a load issued in the block
            // that needs it would expose a full L2 round trip in every block
            float sg_a = (row_ok && 0 < k_blocks) ? __ldg(sa_row + 0) : 0.0f;
            float sg_b = (row_ok && 1 < k_blocks) ? __ldg(sa_row + 1) : 0.0f;
            float sg_c = (row_ok && 2 < k_blocks) ? __ldg(sa_row + 2) : 0.0f;
            for (int kb = 0; kb < k_blocks; ++kb, ++blk) {
                const int b = blk % kGsBufs;
                const float sg = sg_a;
                sg_a = sg_b;
                sg_b = sg_c;
                sg_c = (row_ok && kb + 3 < k_blocks) ? __ldg(sa_row + kb + 3) : 0.0f;
                if (!ptx::mbar_wait_bounded(blk_full_bar(b), (blk / kGsBufs) & 1u) || *abort_flag) {
                    report_wait_failure(kWaitAccFull);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                __syncwarp();  // tcgen05.ld is warp-collective
                if (!warp_has_rows) {
                    ptx::tc_fence_before_sync();
                    if (lane == 0) ptx::mbar_arrive(blk_empty_bar(b));
                    continue;
                }
                const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + b * GSN + half * HC;
                const float2 sg2 = splat2(sg), unbias = splat2(-12582912.0f);
                // eight columns per tcgen05.ld, two loads deep: the load of the next eight columns is in
                // flight while the current eight are folded into y
                uint32_t ra[8], rb[8];
                auto fold = [&](const uint32_t (&r)[8], int c8) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float2 f = make_float2(__int_as_float((int)r[2 * j] + 0x4B400000),
                                               __int_as_float((int)r[2 * j + 1] + 0x4B400000));
                        y2[c8 * 4 + j] = __ffma2_rn(__fadd2_rn(f, unbias), sg2, y2[c8 * 4 + j]);
                    }
                };
                ptx::tmem_ld_32x32b_x8(t_lane, ra);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int c8 = 0; c8 < HC / 8; c8 += 2) {
                    ptx::tmem_ld_32x32b_x8(t_lane + (c8 + 1) * 8, rb);
                    fold(ra, c8);
                    ptx::tmem_ld_wait();
                    if (c8 + 2 < HC / 8) {
                        ptx::tmem_ld_32x32b_x8(t_lane + (c8 + 2) * 8, ra);
                    } else {
                        // the last columns are in registers: the accumulator can be overwritten
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(blk_empty_bar(b));
                    }
                    fold(rb, c8 + 1);
                    if (c8 + 2 < HC / 8) ptx::tmem_ld_wait();
                }
            }
            if (!ok) break;
            if (row_ok) {
                const int nbase = c.n0 + half * HC;
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.C) + (int64_t)row * p.ldc + nbase;
                const float* sbh = sbs + half * HC;
#pragma unroll
                for (int j8 = 0; j8 < HC / 8; ++j8) {
                    const int n = nbase + j8 * 8;
                    if (n >= p.N) break;
                    const float4 s0 = *reinterpret_cast<const float4*>(sbh + j8 * 8);
                    const float4 s1 = *reinterpret_cast<const float4*>(sbh + j8 * 8 + 4);
                    uint4 o;
                    o.x = pack_bf16x2_rn(__fmul_rn(y2[j8 * 4 + 0].x, s0.x), __fmul_rn(y2[j8 * 4 + 0].y, s0.y));
                    o.y = pack_bf16x2_rn(__fmul_rn(y2[j8 * 4 + 1].x, s0.z), __fmul_rn(y2[j8 * 4 + 1].y, s0.w));
                    o.z = pack_bf16x2_rn(__fmul_rn(y2[j8 * 4 + 2].x, s1.x), __fmul_rn(y2[j8 * 4 + 2].y, s1.y));
                    o.w = pack_bf16x2_rn(__fmul_rn(y2[j8 * 4 + 3].x, s1.z), __fmul_rn(y2[j8 * 4 + 3].y, s1.w));
                    if (vec_ok && n + 8 <= p.N) {
                        *reinterpret_cast<uint4*>(out + j8 * 8) = o;
                    } else {
                        const uint32_t w4[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (n + j < p.N)
                                reinterpret_cast<uint16_t*>(out)[j8 * 8 + j] =
                                    (j & 1) ? (uint16_t)(w4[j >> 1] >> 16) : (uint16_t)(w4[j >> 1] & 0xffffu);
                    }
                }
            }
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace
}  // namespace w8a8

#endif  // W8A8_GEMM_I8_GS_KERNEL_CUH
