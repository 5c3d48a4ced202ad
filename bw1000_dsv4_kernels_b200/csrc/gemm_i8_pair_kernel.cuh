// Private part of gemm_i8_sm100.cu (included by that translation unit only, hence the unnamed
// namespace): the CTA-pair kernel for dense GEMMs and its fused all-gather epilogue.
#ifndef W8A8_GEMM_I8_PAIR_KERNEL_CUH
#define W8A8_GEMM_I8_PAIR_KERNEL_CUH

#include "gemm_i8_common.cuh"

namespace w8a8 {
namespace {

// ------------------------------------------------------------------------------------
// CTA-pair kernel (dense GEMM, M > 128): a cluster of two CTAs owns a 256 x 256 output
// tile.  CTA r of the pair loads rows [256*mt + 128*r, +128) of A and rows
// [256*nt + 128*r, +128) of B, so a 128-deep K block costs each SM 32 KB of L2 traffic
// instead of 48 KB for the same number of MMA cycles.  The even CTA issues
// tcgen05.mma.cta_group::2 (M256 x N256 x K32) for both; each CTA drains the accumulator of
// its own 128 rows from its own tensor memory.
//   full[s]      lives in the even CTA; both CTAs' tile loads complete on it
//   empty[s]     one in each CTA; the even CTA's commit arrives on both
//   acc_full[a]  one in each CTA; the even CTA's commit arrives on both
//   acc_empty[a] lives in the even CTA; the drain warps of both CTAs arrive on it
// ------------------------------------------------------------------------------------
template <int STAGES, bool TMA_STORE>
struct PairSmem {
    static constexpr int kABytes = BM * BK;        // this CTA's 128 rows of A
    static constexpr int kBBytes = 128 * BK;       // this CTA's 128 of the tile's 256 rows of B
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTilesBytes = STAGES * kStageBytes;
    // output staging for the TMA-store epilogue: a ring of kOutSlots slabs of [128 rows][64 bf16 = 128 B],
    // 128B-swizzled; a tile is four slabs, so the ring holds more than one tile's worth and the drain of
    // a slab only waits for the stores of the slab kOutSlots back
    static constexpr int kOutSlots = 5;
    static constexpr int kOutSlabBytes = 128 * 128;
    static constexpr int kOutOff = kTilesBytes;
    static constexpr int kOutBytes = TMA_STORE ? kOutSlots * kOutSlabBytes : 0;
    static constexpr int kSbOff = kOutOff + kOutBytes;          // 4 warps x 256 column scales
    static constexpr int kBarOff = kSbOff + 4 * 256 * 4;        // 8-byte aligned
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemSlotOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

// Tile order of the pair kernel.  The m-tiles are cut into groups of `gm`; inside a group the order is
// m fastest, then n.  The CTA pairs that run at the same time then share the group's rows of A (which
// stay in the L2 while the whole weight streams past once per group) and a few weight bands, instead
// of cycling through all of A for every few weight bands: with M = 8192, K = 7168 the 58.7 MB of A do
// not stay resident beside the output stream, half of them do.
struct PairTileOrder {
    int tiles_m, tiles_n, gm;
    __device__ __forceinline__ void at(int t, int& mt, int& nt) const {
        const int per_group = gm * tiles_n;
        int g = t / per_group;
        const int last = (tiles_m - 1) / gm;
        if (g > last) g = last;
        const int r = t - g * per_group;
        const int cnt = min(gm, tiles_m - g * gm);
        mt = g * gm + r % cnt;
        nt = r / cnt;
    }
};

// Tensor maps of the output slab in this rank's buffer (index 0) and in every peer's buffer.
struct StoreMaps {
    CUtensorMap m[8];
    int count;
};

template <int STAGES, bool TMA_STORE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_i8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const Params p, const __grid_constant__ StoreMaps smaps) {
    using L = PairSmem<STAGES, TMA_STORE>;
    constexpr int PBN = 256;  // tile width of the pair
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* sb_tile = reinterpret_cast<float*>(smem + L::kSbOff);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

    const uint32_t tiles_base = ptx::smem_u32(smem);
    const uint32_t bar_base = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

    ptx::grid_launch_dependents();  // a kernel launched to overlap this one may start its set-up and weight loads
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    constexpr uint32_t kTmemCols = 512;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(acc_full_bar(a), 1);
            ptx::mbar_init(acc_empty_bar(a), 2 * (kDrainThreads / 32));  // drain warps of both CTAs
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();  // the peer's barriers exist before anything arrives on them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m = (p.M + 255) / 256;
    const int tiles_n = (p.N + PBN - 1) / PBN;
    const int total = tiles_m * tiles_n;
    const PairTileOrder order{tiles_m, tiles_n, p.pair_group_m};
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int k_blocks = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (!p.withhold_loads && ptx::elect_one()) {
            // The first ring-full needs no free-stage wait; its B (weight) tiles are requested before the
            // dependency wait and its A tiles after it, so that a launch that overlaps the preceding
            // kernel (see set_overlap_previous_kernel) streams weights while that kernel still runs.
            // (t, kb) walks this pair's tiles and their K blocks.
            struct Cursor {
                int t, kb;
            };
            auto advance = [&](Cursor& c) {
                if (++c.kb == k_blocks) {
                    c.kb = 0;
                    c.t += npairs;
                }
            };
            Cursor c0{pair, 0};
            int first = 0;
            for (Cursor c = c0; first < STAGES && c.t < total; ++first, advance(c)) {
                int mt, nt;
                order.at(c.t, mt, nt);
                const int b_row0 = nt * PBN + (int)rank * 128;
                if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(first), 2 * L::kStageBytes);
                ptx::tma_load_2d_pair(tiles_base + first * L::kStageBytes + L::kABytes, &tmB, c.kb * BK, b_row0,
                                      ptx::map_to_cta(full_bar(first), 0));
            }
            ptx::grid_dependency_wait();
            Cursor c = c0;
            for (int i = 0; i < first; ++i, advance(c)) {
                int mt, nt;
                order.at(c.t, mt, nt);
                const int a_row0 = mt * 256 + (int)rank * 128;
                ptx::tma_load_2d_pair(tiles_base + i * L::kStageBytes, &tmA, c.kb * BK, a_row0,
                                      ptx::map_to_cta(full_bar(i), 0));
            }
            int stage = first == STAGES ? 0 : first;
            uint32_t phase = first == STAGES ? 1u : 0u;
            while (c.t < total) {
                int mt, nt;
                order.at(c.t, mt, nt);
                const int a_row0 = mt * 256 + (int)rank * 128;
                const int b_row0 = nt * PBN + (int)rank * 128;
                for (; c.kb < k_blocks; ++c.kb) {
                    if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, p.wait_limit_ns) || *abort_flag) {
                        report_wait_failure(kWaitEmptyStage);
                        *abort_flag = 1;
                        c.t = total;  // leave both loops
                        break;
                    }
                    const uint32_t a_dst = tiles_base + stage * L::kStageBytes;
                    const uint32_t b_dst = a_dst + L::kABytes;
                    const uint32_t leader_full = ptx::map_to_cta(full_bar(stage), 0);
                    if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
                    ptx::tma_load_2d_pair(a_dst, &tmA, c.kb * BK, a_row0, leader_full);
                    ptx::tma_load_2d_pair(b_dst, &tmB, c.kb * BK, b_row0, leader_full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (c.t < total) {
                    c.kb = 0;
                    c.t += npairs;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (even CTA only) ----------------
        if (rank == 0 && ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(256, PBN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += npairs) {
                if (!ptx::mbar_wait_bounded(acc_empty_bar(acc), acc_phase ^ 1u, p.wait_limit_ns) || *abort_flag) {
                    report_wait_failure(kWaitAccEmpty);
                    *abort_flag = 1;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * PBN;
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
                        ptx::mma_i8_ss_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit_pair(empty_bar(stage), 0x3);  // frees the stage in both CTAs
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit_pair(acc_full_bar(acc), 0x3);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- drain warps (both CTAs) ----------------
        ptx::grid_dependency_wait();  // before reading activation scales or writing C
        const int quarter = warp & 3;
        float* sbs = sb_tile + (warp - 2) * PBN;
        int acc = 0;
        uint32_t acc_phase = 0;
        int out_slot = 0;  // next slab of the output staging ring (fused all-gather epilogue)
        const bool vec_ok = c_vector_stores_ok(p);
        for (int t = pair; t < total; t += npairs) {
            int mt, nt;
            order.at(t, mt, nt);
            const int n0 = nt * PBN;
            __syncwarp();
            if (!p.out_i32) {
                for (int j = lane; j < PBN; j += 32) sbs[j] = (n0 + j < p.N) ? __ldg(p.sb + n0 + j) : 0.0f;
            }
            __syncwarp();
            bool go = ptx::mbar_wait_bounded(acc_full_bar(acc), acc_phase, p.wait_limit_ns) && !*abort_flag;
            // the epilogue below meets at named barriers, so its four warps leave together or not at all
            if constexpr (TMA_STORE) go = ptx::barrier_and<2, kDrainThreads>(go);
            if (!go) {
                report_wait_failure(kWaitAccFull);
                *abort_flag = 1;
                break;
            }
            ptx::tc_fence_after_sync();
            const int row = mt * 256 + (int)rank * 128 + quarter * 32 + lane;
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * PBN;
            if constexpr (!TMA_STORE) {
                drain_accumulator<PBN>(p, t_lane, sbs, row, row < p.M, n0, vec_ok);
            } else {
                // Fused all-gather epilogue: the bf16 tile goes through shared memory one 64-column slab
                // at a time (128-byte swizzle so that the 16-byte stores of a quarter-warp hit all banks)
                // and one thread sends each slab with TMA tile stores to this rank's buffer and to every
                // peer's: full 128-byte rows per request over NVLink, no store instruction per
                // destination.  The slabs rotate through a ring of kOutSlots buffers, one bulk group per
                // slab, so filling a slab waits only for the stores issued kOutSlots slabs earlier.
                const int r = quarter * 32 + lane;  // row inside this CTA's 128-row half tile
                const float sa = (row < p.M) ? __ldg(p.sa + row) : 0.0f;
                const bool issuer = (warp == 2 && lane == 0);
#pragma unroll 1
                for (int sl = 0; sl < 4; ++sl) {
                    const uint32_t slab = tiles_base + L::kOutOff + (uint32_t)out_slot * L::kOutSlabBytes;
                    if (issuer) ptx::bulk_wait_group_read<L::kOutSlots - 1>();  // this slot's last stores have read it
                    asm volatile("bar.sync 2, %0;" ::"n"(kDrainThreads) : "memory");
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int cc = 2 * sl + h;
                        uint32_t acc_r[32];
                        __syncwarp();
                        ptx::tmem_ld_32x32b_x32(t_lane + cc * 32, acc_r);
                        ptx::tmem_ld_wait();
                        const float4* sb4 = reinterpret_cast<const float4*>(sbs + cc * 32);
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 s4 = sb4[j];
                            const float v0 = __fmul_rn(__fmul_rn(__int2float_rn((int)acc_r[4 * j + 0]), sa), s4.x);
                            const float v1 = __fmul_rn(__fmul_rn(__int2float_rn((int)acc_r[4 * j + 1]), sa), s4.y);
                            const float v2 = __fmul_rn(__fmul_rn(__int2float_rn((int)acc_r[4 * j + 2]), sa), s4.z);
                            const float v3 = __fmul_rn(__fmul_rn(__int2float_rn((int)acc_r[4 * j + 3]), sa), s4.w);
                            packed[2 * j] = pack_bf16x2_rn(v0, v1);
                            packed[2 * j + 1] = pack_bf16x2_rn(v2, v3);
                        }
                        const uint32_t row_base = slab + (uint32_t)r * 128u;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t phys = ((uint32_t)h * 4u + j) ^ (uint32_t)(r & 7);
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + phys * 16u),
                                         "r"(packed[4 * j]), "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]),
                                         "r"(packed[4 * j + 3])
                                         : "memory");
                        }
                    }
                    ptx::fence_proxy_async_smem();  // the staged slab becomes visible to the TMA engine
                    asm volatile("bar.sync 2, %0;" ::"n"(kDrainThreads) : "memory");
                    if (issuer) {
                        const int y = mt * 256 + (int)rank * 128;
                        if (n0 + sl * 64 < p.N)
                            for (int d = 0; d < smaps.count; ++d) ptx::tma_store_2d(&smaps.m[d], n0 + sl * 64, y, slab);
                        ptx::bulk_commit_group();  // one group per slab, empty or not, keeps the ring count in step
                    }
                    if (++out_slot == L::kOutSlots) out_slot = 0;
                }
            }
            ptx::tc_fence_before_sync();  // the accumulator reads above are ordered before the release below
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(acc_empty_bar(acc), 0));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
    }

    // ---------------- teardown ----------------
    if (TMA_STORE && warp == 2 && lane == 0) ptx::bulk_wait_group0();  // this thread's tile stores are complete
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();  // neither CTA leaves while the other may still touch its memory
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

}  // namespace
}  // namespace w8a8

#endif  // W8A8_GEMM_I8_PAIR_KERNEL_CUH
