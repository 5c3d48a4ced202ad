// Private part of gemm_i8_sm100.cu (included by that translation unit only, hence the unnamed
// namespace): the grouped (MoE) kernel with the expert's weight rows on the tensor core's M axis.
#ifndef W8A8_GEMM_I8_WT_KERNEL_CUH
#define W8A8_GEMM_I8_WT_KERNEL_CUH

#include <type_traits>

#include "gemm_i8_common.cuh"

namespace w8a8 {
namespace {

// ------------------------------------------------------------------------------------
// Grouped GEMM for experts with few rows each (an MoE layer routes ~128 tokens to an expert,
// unevenly).  The problem is bound by the weight stream (44 MB of int8 per expert against
// ~128 rows), so the operands are swapped: 128 rows of the expert's weight sit on the MMA's M
// axis (TMEM lanes) and the expert's tokens on its N axis, N = the number of routed rows
// rounded up to 16 (at most 160 per work item).  An expert with 130 rows therefore costs ONE
// pass over its weights with N = 144, where 128-row token tiles would need two passes, the
// second one almost empty.
//
//   work item   (expert e, chunk of <= 160 of its rows, 128-row weight tile); items that share
//               their tokens are consecutive, so the CTAs that run at the same time read the
//               same token block (from L2) and different weight tiles (from HBM, once)
//   producer    TMA: weight tile [128 x 128 B] and token tile [N x 128 B] per 128-deep K block
//               (one tensor map per N = 16, 32, ..., 160, so that no bytes beyond N rows move)
//   MMA         tcgen05.mma.kind::i8, M128 x N x K32, instruction descriptor built per item
//   drain       per-token scales (GS = false): whole K accumulates in tensor memory, three
//               accumulators rotate between items; thread = weight row (output column),
//               columns = tokens: C[row0 + c, n] = bf16((float(acc) * sa[row0 + c]) * sw[e, n])
//               group scales (GS = true): every K block is its own accumulator, three rotate;
//               y[c] = fma(float(acc_g[c]), sa[row0 + c, g], y[c]) in registers, sixteen drain
//               warps (four per lane quarter, the columns dealt round robin eight at a time);
//               the token scales of each block come from a ring in shared memory that the
//               otherwise idle lanes of the producer warp fill four blocks at a time, so the
//               drain warps load nothing from global memory and never wait for one another
//
// The row segments come from expert_offsets (rows sorted by expert) or, for the masked layout
// [E, max_m, K], from masked_m: expert e owns rows [e * max_m, e * max_m + masked_m[e]).
// ------------------------------------------------------------------------------------
constexpr int kWtChunk = 160;                       // most tokens per work item (MMA N)
constexpr int kWtWarpCols = kWtChunk / 4;           // group scales: columns per drain warp of a lane quarter
constexpr int kWtPieces = kWtWarpCols / 8;          // ... in pieces of eight
constexpr int kWtMaps = kWtChunk / 16;              // token tensor maps: box rows 16, 32, ..., 160
constexpr int kWtWBytes = 128 * BK;
constexpr int kWtXBytes = kWtChunk * BK;
constexpr int kWtStageBytes = kWtWBytes + kWtXBytes;
constexpr int kWtAccs = 3;                          // accumulators in tensor memory (3 x 160 of its 512 columns)
constexpr int kWtAccCols = kWtChunk;                // column stride between them

struct WtMaps {
    CUtensorMap x[kWtMaps];
};

template <bool GS, bool STAGED = false>
struct WtSmem {
    // how far the weight stream runs ahead decides the HBM rate (four stages 395 us, five 345, six 328 on 64
    // experts of 136 rows); with group scales the scale ring takes the room of the sixth stage
    static constexpr int kStages = (GS || STAGED) ? 5 : 6;   // STAGED: the sixth stage's room holds the output tile
    static constexpr int kTilesBytes = kStages * kWtStageBytes;
    // token scales: [160] (per-token scales) or, for group scales, a ring of 32 K blocks x 160 tokens that the
    // producer warp fills (it runs at most kStages + 2 + 4 blocks ahead of the slowest reader)
    static constexpr int kScaleOff = kTilesBytes;
    static constexpr int kScaleBytes = (GS ? 32 : 1) * kWtChunk * 4;
    // STAGED: bf16 [160 tokens][128 weight rows], the item's result before it leaves in 256-byte row segments
    static constexpr int kOutOff = kScaleOff + kScaleBytes;
    static constexpr int kOutBytes = STAGED ? kWtChunk * 128 * 2 : 0;
    static constexpr int kPrefixOff = kOutOff + kOutBytes;
    static constexpr int kBarOff = (kPrefixOff + (kMaxExperts + 1) * 4 + 7) & ~7;
    static constexpr int kNumBars = 2 * kStages + 2 * kWtAccs;
    static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemSlotOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

__device__ __forceinline__ int wt_seg_start(const Params& p, int e) {
    return p.masked_m != nullptr ? e * p.max_m : p.offsets[e];
}
__device__ __forceinline__ int wt_seg_count(const Params& p, int e) {
    if (p.masked_m != nullptr) return max(0, min(p.masked_m[e], p.max_m));
    return max(0, min(p.offsets[e + 1], p.M) - p.offsets[e]);
}

// One warp: prefix[e] = number of token chunks of the experts before e, prefix[E] = all of them.
__device__ __forceinline__ void wt_build_prefix(const Params& p, int* prefix, int lane) {
    int carry = 0;
    for (int e0 = 0; e0 < p.E; e0 += 32) {
        const int e = e0 + lane;
        const int cnt = e < p.E ? (wt_seg_count(p, e) + kWtChunk - 1) / kWtChunk : 0;
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (e < p.E) prefix[e] = carry + incl - cnt;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) prefix[p.E] = carry;
}

struct WtItem {
    int expert;
    int row0;    // first token row (of A and of C)
    int cnt;     // valid tokens in this chunk (1..160)
    int nmma;    // cnt rounded up to 16
    int n0;      // first weight row of the tile inside the expert (= first output column)
    int w_row0;  // the same in the [E*N, K] weight tensor
};

__device__ __forceinline__ WtItem wt_item(const Params& p, const int* prefix, int tiles_w, int t) {
    const int idx = t / tiles_w, wt = t - idx * tiles_w;
    int lo = 0, hi = p.E;  // invariant: prefix[lo] <= idx < prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= idx) lo = mid; else hi = mid;
    }
    WtItem it;
    it.expert = lo;
    const int chunk = idx - prefix[lo];
    it.row0 = wt_seg_start(p, lo) + chunk * kWtChunk;
    it.cnt = min(kWtChunk, wt_seg_count(p, lo) - chunk * kWtChunk);
    it.nmma = (it.cnt + 15) & ~15;
    it.n0 = wt * 128;
    it.w_row0 = lo * p.N + it.n0;
    return it;
}

template <bool GS, bool STAGED = false>
__global__ void __launch_bounds__(GS ? 576 : 192, 1)
gemm_i8_wt_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ WtMaps xmaps, const Params p) {
    static_assert(!(GS && STAGED), "row destinations go with per-token scales");
    using L = WtSmem<GS, STAGED>;
    constexpr int STAGES = L::kStages;
    constexpr int kDrainWarps = GS ? 16 : 4;
    constexpr int kDrain = kDrainWarps * 32;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* tok_scale = reinterpret_cast<float*>(smem + L::kScaleOff);
    __nv_bfloat16* out_tile = reinterpret_cast<__nv_bfloat16*>(smem + L::kOutOff);   // STAGED only
    int* prefix = reinterpret_cast<int*>(smem + L::kPrefixOff);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

    const uint32_t tiles_base = ptx::smem_u32(smem);
    const uint32_t bar_base = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + kWtAccs + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kTmemCols = 512;
    static_assert(kWtAccs * kWtAccCols <= 512, "the accumulators fit tensor memory");

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < kWtAccs; ++a) {
            ptx::mbar_init(acc_full_bar(a), 1);
            ptx::mbar_init(acc_empty_bar(a), kDrainWarps);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::prefetch_tensormap(&tmW);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    if (warp == 2) wt_build_prefix(p, prefix, lane);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_w = (p.N + 127) / 128;
    const int total = prefix[p.E] * tiles_w;
    const int k_blocks = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ---------------- TMA producer (lane 0) and, for group scales, the scale ring (all lanes) ----------------
        if (!p.withhold_loads) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t gb = 0;   // K blocks issued before this item: block kb of the item uses ring slot (gb + kb) & 31
            bool ok = true;
            const bool vec4 = (p.sa_groups % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.sa) & 15) == 0);
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const WtItem it = wt_item(p, prefix, tiles_w, t);
                const CUtensorMap* xm = &xmaps.x[it.nmma / 16 - 1];
                const uint32_t bytes = kWtWBytes + (uint32_t)it.nmma * BK;
                // group scales: lane l keeps the scales of the item's tokens l, l + 32, ... for four K blocks at a
                // time (one 16-byte load per token when the scale rows allow it), requested four blocks before they
                // are written into the ring; the write precedes the arrive on the stage's barrier, which the MMA
                // thread waits for before the block's MMAs, whose completion the drain warps wait for
                float4 nxt[kWtChunk / 32];
                auto fetch_batch = [&](int g0) {
#pragma unroll
                    for (int j = 0; j < kWtChunk / 32; ++j) {
                        const int c = lane + 32 * j;
                        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        if (c < it.cnt && g0 < k_blocks) {
                            const float* base = p.sa + (int64_t)(it.row0 + c) * p.sa_groups + g0;
                            if (vec4) {
                                v = __ldg(reinterpret_cast<const float4*>(base));
                            } else {
                                v.x = __ldg(base);
                                if (g0 + 1 < k_blocks) v.y = __ldg(base + 1);
                                if (g0 + 2 < k_blocks) v.z = __ldg(base + 2);
                                if (g0 + 3 < k_blocks) v.w = __ldg(base + 3);
                            }
                        }
                        nxt[j] = v;
                    }
                };
                if constexpr (GS) fetch_batch(0);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if constexpr (GS) {
                        if ((kb & 3) == 0) {
#pragma unroll
                            for (int j = 0; j < kWtChunk / 32; ++j) {
                                const int c = lane + 32 * j;
                                tok_scale[((gb + kb + 0) & 31) * kWtChunk + c] = nxt[j].x;
                                tok_scale[((gb + kb + 1) & 31) * kWtChunk + c] = nxt[j].y;
                                tok_scale[((gb + kb + 2) & 31) * kWtChunk + c] = nxt[j].z;
                                tok_scale[((gb + kb + 3) & 31) * kWtChunk + c] = nxt[j].w;
                            }
                            fetch_batch(kb + 4);
                        }
                        __syncwarp();   // the ring writes of all lanes precede lane 0's arrive below
                    }
                    if (lane == 0) {
                        if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, p.wait_limit_ns) || *abort_flag) {
                            report_wait_failure(kWaitEmptyStage);
                            *abort_flag = 1;
                            ok = false;
                        } else {
                            const uint32_t w_dst = tiles_base + stage * kWtStageBytes;
                            ptx::mbar_arrive_expect_tx(full_bar(stage), bytes);
                            ptx::tma_load_2d(w_dst, &tmW, kb * BK, it.w_row0, full_bar(stage));
                            ptx::tma_load_2d(w_dst + kWtWBytes, xm, kb * BK, it.row0, full_bar(stage));
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                gb += (uint32_t)k_blocks;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t blk = 0;  // accumulator hand-overs so far: buffer = blk % kWtAccs, parity = (blk / kWtAccs) & 1
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const WtItem it = wt_item(p, prefix, tiles_w, t);
                const uint32_t idesc = ptx::idesc_i8(128, it.nmma);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    const bool new_acc = GS || kb == 0;
                    const uint32_t b = blk % kWtAccs;
                    if (new_acc && (!ptx::mbar_wait_bounded(acc_empty_bar(b), ((blk / kWtAccs) & 1u) ^ 1u, p.wait_limit_ns) ||
                                    *abort_flag)) {
                        report_wait_failure(kWaitAccEmpty);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    if (!ptx::mbar_wait_bounded(full_bar(stage), phase, p.wait_limit_ns) || *abort_flag) {
                        report_wait_failure(kWaitFullStage);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t w_src = tiles_base + stage * kWtStageBytes;
                    const uint64_t adesc = ptx::smem_desc_k_sw128(w_src);
                    const uint64_t bdesc = ptx::smem_desc_k_sw128(w_src + kWtWBytes);
                    const uint32_t d_tmem = tmem_base + b * kWtAccCols;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        ptx::mma_i8_ss(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc,
                                       (GS ? k != 0 : (kb | k) != 0) ? 1u : 0u);
                    ptx::tc_commit(empty_bar(stage));
                    if (GS || kb == k_blocks - 1) {
                        ptx::tc_commit(acc_full_bar(b));
                        ++blk;
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
        // ---------------- drain warps ----------------
        const int dtid = threadIdx.x - 64;               // 0 .. kDrain-1
        const int quarter = warp & 3;                    // TMEM lanes this warp may touch
        const int sub = (warp - 2) >> 2;                 // GS: this warp takes the 16-column groups sub, sub + 4, sub + 8
        const int wrow = quarter * 32 + lane;            // weight row inside the tile = TMEM lane
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        uint32_t blk = 0;
        uint32_t gb = 0;   // K blocks before this item (group scales: ring slot of block kb = (gb + kb) & 31)
        for (int t = blockIdx.x; t < total; t += gridDim.x) {
            const WtItem it = wt_item(p, prefix, tiles_w, t);
            const int n = it.n0 + wrow;
            const bool n_ok = n < p.N;
            const float sbn = n_ok ? __ldg(p.sb + (int64_t)it.expert * p.N + n) : 0.0f;
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.C) + (int64_t)it.row0 * p.ldc + n;
            if constexpr (!GS) {
                // token scales of the item -> shared memory (everybody reads all of them)
                asm volatile("bar.sync 1, %0;" ::"n"(kDrain) : "memory");   // the previous item's readers are done
                for (int i = dtid; i < kWtChunk; i += kDrain) tok_scale[i] = i < it.cnt ? __ldg(p.sa + it.row0 + i) : 0.0f;
                // STAGED: where this thread's rows go (rows dtid / 16, + 8, + 16, ...), asked for now so that the
                // loads are long done when the tile is written out
                constexpr int kRowsPerThread = STAGED ? kWtChunk / (kDrain / 16) : 1;
                __nv_bfloat16* dstp[kRowsPerThread];
                if constexpr (STAGED) {
#pragma unroll
                    for (int k = 0; k < kRowsPerThread; ++k) {
                        const int c = (dtid >> 4) + k * (kDrain / 16);
                        dstp[k] = nullptr;
                        if (c < it.cnt)
                            dstp[k] = p.row_ptr != nullptr
                                ? reinterpret_cast<__nv_bfloat16*>(__ldg(reinterpret_cast<const unsigned long long*>(p.row_ptr) + it.row0 + c))
                                : static_cast<__nv_bfloat16*>(p.C) + (int64_t)(it.row0 + c) * p.ldc;
                    }
                }
                const uint32_t b = blk % kWtAccs;
                bool go = ptx::mbar_wait_bounded(acc_full_bar(b), (blk / kWtAccs) & 1u, p.wait_limit_ns) && !*abort_flag;
                go = ptx::barrier_and<1, kDrain>(go);                        // also publishes the scales
                if (!go) {
                    report_wait_failure(kWaitAccFull);
                    *abort_flag = 1;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t t_lane = lane_base + b * kWtAccCols;
#pragma unroll 1
                for (int c0 = 0; c0 < it.nmma; c0 += 16) {
                    uint32_t r[16];
                    __syncwarp();
                    ptx::tmem_ld_32x32b_x16(t_lane + c0, r);
                    ptx::tmem_ld_wait();
                    if (c0 + 16 >= it.nmma) {
                        // the last columns are in registers: the accumulator can be overwritten
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(acc_empty_bar(b));
                    }
                    if (!STAGED && !n_ok) continue;
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        const float4 s4 = *reinterpret_cast<const float4*>(tok_scale + c0 + 4 * j4);
                        const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int c = c0 + 4 * j4 + j;
                            if (c < it.cnt) {
                                const float v = __fmul_rn(__fmul_rn(__int2float_rn((int)r[4 * j4 + j]), sv[j]), sbn);
                                if constexpr (STAGED)
                                    out_tile[c * 128 + wrow] = __float2bfloat16_rn(v);
                                else
                                    out[(int64_t)c * p.ldc] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                }
                if constexpr (STAGED) {
                    // The item's tile [tokens][128 weight rows] is in shared memory: every token's 256 bytes leave as
                    // sixteen 16-byte stores of neighbouring lanes, to the row's own destination (a remote store of
                    // 64 bytes, what a warp's 2-byte stores of one token amount to, uses a fraction of an NVLink
                    // packet).  The barrier at the top of the next item keeps the tile until everybody has read it.
                    asm volatile("bar.sync 2, %0;" ::"n"(kDrain) : "memory");
                    const int seg = dtid & 15;                       // 16-byte piece of the 256-byte row segment
                    const int nn = it.n0 + seg * 8;
#pragma unroll
                    for (int k = 0; k < kRowsPerThread; ++k) {
                        const int c = (dtid >> 4) + k * (kDrain / 16);
                        __nv_bfloat16* dst = dstp[k];
                        if (dst == nullptr) continue;
                        const uint4 v = *reinterpret_cast<const uint4*>(out_tile + c * 128 + seg * 8);
                        if (nn + 8 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
                            *reinterpret_cast<uint4*>(dst + nn) = v;
                        } else {
                            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
                            for (int j = 0; j < 8; ++j)
                                if (nn + j < p.N) dst[nn + j] = e[j];
                        }
                    }
                }
                ++blk;
            } else {
                // group scales: y[c] += float(acc_g[c]) * sa[row0 + c, g] for this warp's columns.  The tile's
                // columns are dealt to the four warps of a lane quarter eight at a time: warp `sub` takes the
                // 8-column pieces sub, sub + 4, sub + 8, ... (at most five).  Nothing here synchronises with
                // another drain warp; the block's token scales are in the ring that the producer warp fills.
                constexpr int NP = kWtPieces;
                float2 y2[NP][4];
#pragma unroll
                for (int v = 0; v < NP; ++v)
#pragma unroll
                    for (int j = 0; j < 4; ++j) y2[v][j] = make_float2(0.0f, 0.0f);
                // the warp's 8-column pieces: tile columns (4v + sub) * 8 < nmma, v = 0 .. npieces-1
                const int npieces = (it.nmma / 8 + 3 - sub) >> 2;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb, ++blk) {
                    const uint32_t b = blk % kWtAccs;
                    if (!ptx::mbar_wait_bounded(acc_full_bar(b), (blk / kWtAccs) & 1u, p.wait_limit_ns) || *abort_flag) {
                        report_wait_failure(kWaitAccFull);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    __syncwarp();   // tcgen05.ld is warp-collective; also publishes the ring writes inside the warp
                    const uint32_t t_lane = lane_base + b * kWtAccCols + sub * 8;
                    const float* sg = tok_scale + ((gb + kb) & 31) * kWtChunk + sub * 8;   // + 32 v: the warp's piece v
                    // int -> float by the conversion instruction: it runs on its own pipe, beside the packed FMAs
                    auto fold = [&](const uint32_t (&r)[8], int v) {
#pragma unroll
                        for (int j4 = 0; j4 < 2; ++j4) {
                            const float4 s4 = *reinterpret_cast<const float4*>(sg + v * 32 + 4 * j4);
                            const float2 f0 = make_float2(__int2float_rn((int)r[4 * j4 + 0]), __int2float_rn((int)r[4 * j4 + 1]));
                            const float2 f1 = make_float2(__int2float_rn((int)r[4 * j4 + 2]), __int2float_rn((int)r[4 * j4 + 3]));
                            y2[v][2 * j4] = __ffma2_rn(f0, make_float2(s4.x, s4.y), y2[v][2 * j4]);
                            y2[v][2 * j4 + 1] = __ffma2_rn(f1, make_float2(s4.z, s4.w), y2[v][2 * j4 + 1]);
                        }
                    };
                    auto release = [&]() {   // every column of this block is in registers: the accumulator can be overwritten
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(acc_empty_bar(b));
                    };
                    // eight columns per tensor-memory load; the next load is in flight while the current eight fold.
                    // One straight-line copy of the sequence per piece count, so that nothing in it is predicated.
                    uint32_t ra[8], rb[8];
                    auto pieces = [&](auto count) {
                        constexpr int CNT = decltype(count)::value;
                        ptx::tmem_ld_32x32b_x8(t_lane, ra);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int v = 0; v < CNT; v += 2) {
                            if (v + 1 < CNT) ptx::tmem_ld_32x32b_x8(t_lane + (v + 1) * 32, rb); else release();
                            fold(ra, v);
                            if (v + 1 < CNT) {
                                ptx::tmem_ld_wait();
                                if (v + 2 < CNT) ptx::tmem_ld_32x32b_x8(t_lane + (v + 2) * 32, ra); else release();
                                fold(rb, v + 1 < NP ? v + 1 : 0);
                                if (v + 2 < CNT) ptx::tmem_ld_wait();
                            }
                        }
                    };
                    static_assert(NP == 5, "one case per possible piece count below");
                    switch (npieces) {
                        case 5: pieces(std::integral_constant<int, 5>{}); break;
                        case 4: pieces(std::integral_constant<int, 4>{}); break;
                        case 3: pieces(std::integral_constant<int, 3>{}); break;
                        case 2: pieces(std::integral_constant<int, 2>{}); break;
                        case 1: pieces(std::integral_constant<int, 1>{}); break;
                        default: release(); break;
                    }
                }
                if (!ok) break;
                gb += (uint32_t)k_blocks;
                if (n_ok) {
#pragma unroll
                    for (int v = 0; v < NP; ++v) {
                        const int col0 = (4 * v + sub) * 8;
                        if (col0 >= it.cnt) continue;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int cidx = col0 + 2 * j;
                            if (cidx < it.cnt) out[(int64_t)cidx * p.ldc] = __float2bfloat16_rn(__fmul_rn(y2[v][j].x, sbn));
                            if (cidx + 1 < it.cnt) out[(int64_t)(cidx + 1) * p.ldc] = __float2bfloat16_rn(__fmul_rn(y2[v][j].y, sbn));
                        }
                    }
                }
            }
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

#endif  // W8A8_GEMM_I8_WT_KERNEL_CUH
