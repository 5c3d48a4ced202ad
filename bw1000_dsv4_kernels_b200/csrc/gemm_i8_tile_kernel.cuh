// Private part of gemm_i8_sm100.cu (included by that translation unit only, hence the unnamed
// namespace): the one-CTA-per-tile kernel (dense problems with few tiles, raw int32 output).
#ifndef W8A8_GEMM_I8_TILE_KERNEL_CUH
#define W8A8_GEMM_I8_TILE_KERNEL_CUH

#include "gemm_i8_common.cuh"

namespace w8a8 {
namespace {

// ------------------------------------------------------------------------------------
// Per-token-scaled (or raw int32) kernel: whole K accumulates in tensor memory.
// ------------------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const Params p) {
    using L = Smem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* sb_tile = reinterpret_cast<float*>(smem + L::kSbOff);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ((L::kBarOff + 7) & ~7));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

    const uint32_t tiles_base = ptx::smem_u32(smem);
    const uint32_t bar_base = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(acc_full_bar(a), 1);
            ptx::mbar_init(acc_empty_bar(a), kDrainThreads / 32);
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
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const Scheduler sched(p, BN);
    const int k_blocks = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (!p.withhold_loads && ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
                const TileCoord c = sched.at(t, BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, p.wait_limit_ns) || *abort_flag) {
                        report_wait_failure(kWaitEmptyStage);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = tiles_base + stage * L::kStageBytes;
                    const uint32_t b_dst = a_dst + L::kABytes;
                    ptx::mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
                    ptx::tma_load_2d(a_dst, &tmA, kb * BK, c.a_row0, full_bar(stage));
                    ptx::tma_load_2d(b_dst, &tmB, kb * BK, c.b_row0, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
                if (!ptx::mbar_wait_bounded(acc_empty_bar(acc), acc_phase ^ 1u, p.wait_limit_ns) || *abort_flag) {
                    report_wait_failure(kWaitAccEmpty);
                    *abort_flag = 1;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(full_bar(stage), phase, p.wait_limit_ns) || *abort_flag) {
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
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        ptx::mma_i8_ss(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc,
                                       (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(empty_bar(stage));  // stage reusable once these MMAs retire
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit(acc_full_bar(acc));
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- drain warps (2..5) ----------------
        const int quarter = warp & 3;  // TMEM lanes a warp may touch: 32*(warp%4)..+31
        float* sbs = sb_tile + (warp - 2) * BN;  // private to this warp: no block-level barrier
        int acc = 0;
        uint32_t acc_phase = 0;
        const bool vec_ok = c_vector_stores_ok(p);
        for (int t = blockIdx.x; t < sched.total; t += gridDim.x) {
            const TileCoord c = sched.at(t, BN);
            // column scales of this tile -> this warp's shared copy
            __syncwarp();
            if (!p.out_i32) {
                for (int j = lane; j < BN; j += 32)
                    sbs[j] = (c.n0 + j < p.N) ? __ldg(p.sb + c.n0 + j) : 0.0f;
            }
            __syncwarp();
            bool got = ptx::mbar_wait_bounded(acc_full_bar(acc), acc_phase, p.wait_limit_ns);
            if (!got || *abort_flag) {
                report_wait_failure(kWaitAccFull);
                *abort_flag = 1;
                break;
            }
            ptx::tc_fence_after_sync();
            const int row = c.a_row0 + quarter * 32 + lane;
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
            // a warp whose 32 rows all lie past the last row has nothing to load or store
            if (c.a_row0 + quarter * 32 < c.row_end)
                drain_accumulator<BN>(p, t_lane, sbs, row, row < c.row_end, c.n0, vec_ok);
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(acc_empty_bar(acc));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
    }

    // ---------------- teardown ----------------
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace
}  // namespace w8a8

#endif  // W8A8_GEMM_I8_TILE_KERNEL_CUH
