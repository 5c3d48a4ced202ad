// Private part of gemm_i8_sm100.cu (included by that translation unit only, hence the unnamed
// namespace): the weight-streaming split-K kernels for M <= 256.
#ifndef W8A8_GEMM_I8_STREAM_KERNELS_CUH
#define W8A8_GEMM_I8_STREAM_KERNELS_CUH

#include "gemm_i8_common.cuh"

namespace w8a8 {
namespace {

// Split-K epilogue of the weight-streaming kernels: sums the S partial tiles ([token][128 weight
// rows] int32, one in each peer CTA's shared memory, fixed order r = 0..S-1), applies the scales and
// stores.  Work item = (token column c, group of four weight rows): 16-byte loads through
// distributed shared memory, four outputs that are contiguous in C; consecutive threads take
// consecutive row groups of one column.  U items are in flight per thread (four with up to eight
// partials, eight with up to four), because one item at a time would cost a full remote-load latency
// per item; measured, a remote read costs about a microsecond and moves about 25 GB/s per SM, and a
// bulk reduce-add into the owner's shared memory (tried instead of these loads) is no faster.  The
// token and channel scales were put into shared memory (sa_s[token], sb_s[row in tile]) while the
// weight streamed, so that no global-memory latency follows the remote loads.
template <int MAXS, int U>
__device__ __forceinline__ void reduce_partials_and_store(const Params& p, const uint32_t (&peer_base)[MAXS], int S,
                                                          int cols_lo, int cols_hi, int n0, int tid, int nthreads,
                                                          const float* sa_s, const float* sb_s) {
    const bool vec_store = p.out_i32 ? ((p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0))
                                     : ((p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 7) == 0));
    const int items = (cols_hi - cols_lo) * 32;
    for (int it0 = tid; it0 < items; it0 += nthreads * U) {
        uint4 v[U][MAXS];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int it = it0 + u * nthreads;
            if (it < items) {
                const uint32_t off = (uint32_t)((cols_lo + (it >> 5)) * 128 + (it & 31) * 4) * 4u;
#pragma unroll
                for (int r = 0; r < MAXS; ++r)
                    if (r < S) v[u][r] = ptx::ld_shared_cluster_v4(peer_base[r] + off);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int it = it0 + u * nthreads;
            if (it >= items) break;
            const int c = cols_lo + (it >> 5), g = it & 31;
            int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
#pragma unroll
            for (int r = 0; r < MAXS; ++r) {
                if (r < S) {
                    a0 += (int)v[u][r].x; a1 += (int)v[u][r].y; a2 += (int)v[u][r].z; a3 += (int)v[u][r].w;
                }
            }
            const int n = n0 + g * 4;
            if (n >= p.N) continue;
            if (p.out_i32) {
                int* out = static_cast<int*>(p.C) + (int64_t)c * p.ldc + n;
                if (vec_store && n + 4 <= p.N) {
                    *reinterpret_cast<int4*>(out) = make_int4(a0, a1, a2, a3);
                } else {
                    const int v4[4] = {a0, a1, a2, a3};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (n + j < p.N) out[j] = v4[j];
                }
            } else {
                const float sa = sa_s[c];
                const float4 sb4 = *reinterpret_cast<const float4*>(sb_s + g * 4);
                const float sbv[4] = {sb4.x, sb4.y, sb4.z, sb4.w};
                const uint32_t lo = pack_bf16x2_rn(__fmul_rn(__fmul_rn(__int2float_rn(a0), sa), sbv[0]),
                                                   __fmul_rn(__fmul_rn(__int2float_rn(a1), sa), sbv[1]));
                const uint32_t hi = pack_bf16x2_rn(__fmul_rn(__fmul_rn(__int2float_rn(a2), sa), sbv[2]),
                                                   __fmul_rn(__fmul_rn(__int2float_rn(a3), sa), sbv[3]));
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.C) + (int64_t)c * p.ldc + n;
                if (vec_store && n + 4 <= p.N) {
                    *reinterpret_cast<uint2*>(out) = make_uint2(lo, hi);
                } else {
                    const uint16_t h4[4] = {(uint16_t)(lo & 0xffffu), (uint16_t)(lo >> 16), (uint16_t)(hi & 0xffffu),
                                            (uint16_t)(hi >> 16)};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (n + j < p.N) reinterpret_cast<uint16_t*>(out)[j] = h4[j];
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------
// Weight-streaming kernel for few tokens (M <= 256): HBM-bound on the weight read, so the
// operands are swapped and K is split.
//   * The 128 weight rows of a tile sit on the MMA's M axis (TMEM lanes), the tokens on its
//     N axis (NTOK columns, 16..256), so no tensor-core rows are spent on padding and the
//     whole weight is read exactly once whatever M is.
//   * A cluster of S CTAs shares one 128-row weight tile and splits K between its CTAs, so
//     that ~all SMs stream weights at once.  Each CTA parks its int32 partial [NTOK][128] in
//     its own shared memory (on top of the drained stage ring); after a cluster barrier CTA s
//     sums the S partials of its share of the token columns through distributed shared memory
//     (exact int32 adds, fixed order), applies the scales and stores.  No scratch in HBM.
// One tile per CTA: not persistent.
// ------------------------------------------------------------------------------------
template <int NTOK>
struct StreamSmem {
    static constexpr int kWBytes = 128 * BK;
    static constexpr int kXBytes = NTOK * BK;
    static constexpr int kStageBytes = kWBytes + kXBytes;
    static constexpr int kRingBytes = 196 * 1024;
    static constexpr int kStages = kRingBytes / kStageBytes;
    static constexpr int kTilesBytes = kStages * kStageBytes;
    static constexpr int kPartialBytes = NTOK * 128 * 4;
    static_assert(kPartialBytes <= kTilesBytes, "the partial tile reuses the stage ring");
    static constexpr int kScaleOff = kTilesBytes;             // token scales [256], then the tile's 128 channel scales
    static constexpr int kBarOff = kScaleOff + (256 + 128) * 4;
    static constexpr int kNumBars = 2 * kStages + 1;
    static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemSlotOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

// The drain warps (threads 64..191) have nothing to do while the weight streams: they fetch the scales the
// epilogue needs.  Activation scales may come from the kernel before this one, hence the dependency wait.
__device__ __forceinline__ void stage_scales(const Params& p, float* sa_s, float* sb_s, int ntok, int n0) {
    ptx::grid_dependency_wait();
    if (p.out_i32) return;
    const int t = threadIdx.x - 64;
    for (int i = t; i < ntok; i += kDrainThreads) sa_s[i] = i < p.M ? __ldg(p.sa + i) : 0.0f;
    for (int j = t; j < 128; j += kDrainThreads) sb_s[j] = n0 + j < p.N ? __ldg(p.sb + n0 + j) : 0.0f;
}

template <int NTOK>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_stream_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const Params p) {
    using L = StreamSmem<NTOK>;
    constexpr int STAGES = L::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
    int* partial = reinterpret_cast<int*>(smem);  // [NTOK][128] once the ring has drained
    float* sa_s = reinterpret_cast<float*>(smem + L::kScaleOff);
    float* sb_s = sa_s + 256;

    const uint32_t tiles_base = ptx::smem_u32(smem);
    const uint32_t bar_base = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * STAGES);

    ptx::grid_launch_dependents();  // a kernel launched to overlap this one may start its set-up and weight loads
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = (int)ptx::cluster_nctarank();
    const int split = (int)ptx::cluster_ctarank();
    const int nt = blockIdx.x / S;
    const int n0 = nt * 128;
    constexpr uint32_t kTmemCols = NTOK < 32 ? 32 : NTOK;

    // this CTA's share of the K blocks
    const int k_blocks = (p.K + BK - 1) / BK;
    const int kb0 = (int)((int64_t)k_blocks * split / S), kb1 = (int)((int64_t)k_blocks * (split + 1) / S);
    // the first ring-full of loads needs no wait on an empty stage: it is issued before the block-wide
    // set-up barrier, so the weight stream starts while tensor memory is still being allocated
    const int prologue = (kb1 - kb0) < STAGES ? (kb1 - kb0) : STAGES;
    bool ok = true;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(acc_full_bar, 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        // The weight does not depend on the kernel that runs before this one: its loads start at once.
        // The tokens do: their loads come after the dependency wait (which returns immediately unless
        // this kernel was launched to overlap its predecessor).
        for (int i = 0; i < prologue; ++i) {
            ptx::mbar_arrive_expect_tx(full_bar(i), L::kStageBytes);
            ptx::tma_load_2d(tiles_base + i * L::kStageBytes, &tmW, (kb0 + i) * BK, n0, full_bar(i));
        }
        ptx::grid_dependency_wait();
        for (int i = 0; i < prologue; ++i)
            ptx::tma_load_2d(tiles_base + i * L::kStageBytes + L::kWBytes, &tmX, (kb0 + i) * BK, 0, full_bar(i));
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (ptx::elect_one()) {
            int stage = prologue == STAGES ? 0 : prologue;
            uint32_t phase = prologue == STAGES ? 1u : 0u;
            for (int kb = kb0 + prologue; kb < kb1; ++kb) {
                if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u) || *abort_flag) {
                    report_wait_failure(kWaitEmptyStage);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t w_dst = tiles_base + stage * L::kStageBytes;
                ptx::mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
                ptx::tma_load_2d(w_dst, &tmW, kb * BK, n0, full_bar(stage));
                ptx::tma_load_2d(w_dst + L::kWBytes, &tmX, kb * BK, 0, full_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(128, NTOK);
            int stage = 0;
            uint32_t phase = 0;
            bool issued_all = true;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!ptx::mbar_wait_bounded(full_bar(stage), phase) || *abort_flag) {
                    report_wait_failure(kWaitFullStage);
                    *abort_flag = 1;
                    issued_all = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t w_src = tiles_base + stage * L::kStageBytes;
                const uint64_t adesc = ptx::smem_desc_k_sw128(w_src);
                const uint64_t bdesc = ptx::smem_desc_k_sw128(w_src + L::kWBytes);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    ptx::mma_i8_ss(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > kb0 || k != 0) ? 1u : 0u);
                ptx::tc_commit(empty_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (issued_all) ptx::tc_commit(acc_full_bar);
        }
    } else {
        // drain warps: the epilogue's scales first, then accumulator -> shared partial
        stage_scales(p, sa_s, sb_s, NTOK, n0);
        const int quarter = warp & 3;
        const int wrow = quarter * 32 + lane;  // weight row inside the tile = TMEM lane
        if (kb1 > kb0) {
            if (!ptx::mbar_wait_bounded(acc_full_bar, 0) || *abort_flag) {
                report_wait_failure(kWaitAccFull);
                *abort_flag = 1;
                ok = false;
            }
        }
        ptx::tc_fence_after_sync();
        __syncwarp();
        if (ok) {
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int cc = 0; cc < (NTOK + 31) / 32; ++cc) {
                uint32_t r[32];
                if (kb1 > kb0) {
                    if (NTOK >= 32) {
                        ptx::tmem_ld_32x32b_x32(t_lane + cc * 32, r);
                    } else {
                        uint32_t r16[16];
                        ptx::tmem_ld_32x32b_x16(t_lane, r16);
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = r16[j];
#pragma unroll
                        for (int j = 16; j < 32; ++j) r[j] = 0;
                    }
                    ptx::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0;  // a CTA without K blocks contributes zero
                }
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (cc * 32 + j < NTOK) partial[(cc * 32 + j) * 128 + wrow] = (int)r[j];
            }
        }
    }

    // every CTA's partial is complete and visible to the cluster
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    ptx::grid_dependency_wait();     // before this thread reads activation scales or writes C

    {
        // all six warps take part: the producer and MMA threads are done by now
        const int cols_lo = (int)((int64_t)NTOK * split / S);
        int cols_hi = (int)((int64_t)NTOK * (split + 1) / S);
        if (cols_hi > p.M) cols_hi = p.M;
        const uint32_t my_partial = ptx::smem_u32(partial);
        uint32_t peer_base[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) peer_base[r] = ptx::map_to_cta(my_partial, r < S ? r : 0);
        reduce_partials_and_store<8, 4>(p, peer_base, S, cols_lo, cols_hi, n0, threadIdx.x, kThreads, sa_s, sb_s);
    }

    // nobody leaves while a peer may still read its shared memory
    __syncthreads();
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------
// Weight-streaming kernel for 128 < M <= 256 tokens: the same swap-AB split-K scheme on CTA pairs.
// With 256 tokens on the MMA's N axis a single CTA re-reads the whole token block for every
// 128-row weight tile, and that L2 -> SM traffic (not HBM) sets the time.  Here a pair of CTAs
// owns 256 weight rows: each CTA loads its own 128 weight rows and only ITS HALF of the tokens
// (tcgen05.mma.cta_group::2, M256 x N256), so a 128-deep K block costs each SM 32 KB instead of
// 48 KB.  A cluster is S pairs that split K; CTA (split s, half h) has cluster rank 2s + h and
// sums, for its share of the token columns, the partials of the S CTAs with the same h.
// Barrier protocol of the pair as in gemm_i8_pair_kernel (full[] in the even CTA, commits arrive in
// both CTAs).
// ------------------------------------------------------------------------------------
struct StreamPairSmem {
    static constexpr int kWBytes = 128 * BK;
    static constexpr int kXBytes = 128 * BK;   // this CTA's half of the 256 token rows
    static constexpr int kStageBytes = kWBytes + kXBytes;
    static constexpr int kStages = 6;
    static constexpr int kTilesBytes = kStages * kStageBytes;
    static constexpr int kPartialBytes = 256 * 128 * 4;
    static_assert(kPartialBytes <= kTilesBytes, "the partial tile reuses the stage ring");
    static constexpr int kScaleOff = kTilesBytes;             // token scales [256], then the tile's 128 channel scales
    static constexpr int kBarOff = kScaleOff + (256 + 128) * 4;
    static constexpr int kNumBars = 2 * kStages + 1;
    static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemSlotOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_stream_pair_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                           const Params p) {
    using L = StreamPairSmem;
    constexpr int STAGES = L::kStages, NTOK = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
    int* partial = reinterpret_cast<int*>(smem);  // [NTOK][128] once the ring has drained
    float* sa_s = reinterpret_cast<float*>(smem + L::kScaleOff);
    float* sb_s = sa_s + 256;

    const uint32_t tiles_base = ptx::smem_u32(smem);
    const uint32_t bar_base = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * STAGES);

    ptx::grid_launch_dependents();  // a kernel launched to overlap this one may start its set-up and weight loads
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int csize = (int)ptx::cluster_nctarank();
    const int crank = (int)ptx::cluster_ctarank();
    const int S = csize >> 1, split = crank >> 1, half = crank & 1;
    const uint32_t leader = (uint32_t)(crank & ~1);
    const uint16_t pair_mask = (uint16_t)(0x3u << leader);
    const int nt = blockIdx.x / csize;
    const int n0 = nt * 256 + half * 128;         // this CTA's weight rows
    constexpr uint32_t kTmemCols = NTOK;

    const int k_blocks = (p.K + BK - 1) / BK;
    const int kb0 = (int)((int64_t)k_blocks * split / S), kb1 = (int)((int64_t)k_blocks * (split + 1) / S);
    bool ok = true;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(acc_full_bar, 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::prefetch_tensormap(&tmW);
        ptx::prefetch_tensormap(&tmX);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();  // the peers' barriers exist before anything arrives on them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (ptx::elect_one()) {
            // first ring-full: the stages are free; the weight loads go out before the dependency wait
            // (the weight does not depend on the preceding kernel), the token loads after it
            const int prologue = (kb1 - kb0) < STAGES ? (kb1 - kb0) : STAGES;
            for (int i = 0; i < prologue; ++i) {
                const uint32_t leader_full = ptx::map_to_cta(full_bar(i), leader);
                if (half == 0) ptx::mbar_arrive_expect_tx(full_bar(i), 2 * L::kStageBytes);
                ptx::tma_load_2d_pair(tiles_base + i * L::kStageBytes, &tmW, (kb0 + i) * BK, n0, leader_full);
            }
            ptx::grid_dependency_wait();
            for (int i = 0; i < prologue; ++i)
                ptx::tma_load_2d_pair(tiles_base + i * L::kStageBytes + L::kWBytes, &tmX, (kb0 + i) * BK, half * 128,
                                      ptx::map_to_cta(full_bar(i), leader));
            int stage = prologue == STAGES ? 0 : prologue;
            uint32_t phase = prologue == STAGES ? 1u : 0u;
            for (int kb = kb0 + prologue; kb < kb1; ++kb) {
                if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u) || *abort_flag) {
                    report_wait_failure(kWaitEmptyStage);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t w_dst = tiles_base + stage * L::kStageBytes;
                const uint32_t leader_full = ptx::map_to_cta(full_bar(stage), leader);
                if (half == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
                ptx::tma_load_2d_pair(w_dst, &tmW, kb * BK, n0, leader_full);
                ptx::tma_load_2d_pair(w_dst + L::kWBytes, &tmX, kb * BK, half * 128, leader_full);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (half == 0 && ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(256, NTOK);
            int stage = 0;
            uint32_t phase = 0;
            bool issued_all = true;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!ptx::mbar_wait_bounded(full_bar(stage), phase) || *abort_flag) {
                    report_wait_failure(kWaitFullStage);
                    *abort_flag = 1;
                    issued_all = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t w_src = tiles_base + stage * L::kStageBytes;
                const uint64_t adesc = ptx::smem_desc_k_sw128(w_src);
                const uint64_t bdesc = ptx::smem_desc_k_sw128(w_src + L::kWBytes);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    ptx::mma_i8_ss_pair(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > kb0 || k != 0) ? 1u : 0u);
                ptx::tc_commit_pair(empty_bar(stage), pair_mask);  // frees the stage in both CTAs
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (issued_all) ptx::tc_commit_pair(acc_full_bar, pair_mask);
        }
    } else {
        // drain warps of both CTAs: the epilogue's scales first, then the accumulator of this CTA's 128 weight
        // rows -> shared partial
        stage_scales(p, sa_s, sb_s, NTOK, n0);
        const int quarter = warp & 3;
        const int wrow = quarter * 32 + lane;
        if (kb1 > kb0) {
            if (!ptx::mbar_wait_bounded(acc_full_bar, 0) || *abort_flag) {
                report_wait_failure(kWaitAccFull);
                *abort_flag = 1;
                ok = false;
            }
        }
        ptx::tc_fence_after_sync();
        __syncwarp();
        if (ok) {
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int cc = 0; cc < NTOK / 32; ++cc) {
                uint32_t r[32];
                if (kb1 > kb0) {
                    ptx::tmem_ld_32x32b_x32(t_lane + cc * 32, r);
                    ptx::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0;  // a pair without K blocks contributes zero
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) partial[(cc * 32 + j) * 128 + wrow] = (int)r[j];
            }
        }
    }

    // every CTA's partial is complete and visible to the cluster
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    ptx::grid_dependency_wait();     // before this thread reads activation scales or writes C

    {
        const int cols_lo = (int)((int64_t)NTOK * split / S);
        int cols_hi = (int)((int64_t)NTOK * (split + 1) / S);
        if (cols_hi > p.M) cols_hi = p.M;
        const uint32_t my_partial = ptx::smem_u32(partial);
        uint32_t peer_base[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) peer_base[r] = ptx::map_to_cta(my_partial, (uint32_t)(2 * (r < S ? r : 0) + half));
        reduce_partials_and_store<4, 8>(p, peer_base, S, cols_lo, cols_hi, n0, threadIdx.x, kThreads, sa_s, sb_s);
    }

    // nobody leaves while a peer may still read its shared memory
    __syncthreads();
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

}  // namespace
}  // namespace w8a8

#endif  // W8A8_GEMM_I8_STREAM_KERNELS_CUH
