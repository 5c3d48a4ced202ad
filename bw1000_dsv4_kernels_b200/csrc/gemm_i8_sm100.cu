// W8A8 GEMM for sm_100a: C = bf16((float(A * B^T) * sa) * sb), int8 operands, int32
// accumulation on the 5th-generation tensor cores.
//
//   * A [M,K] and B [N,K] are both K-contiguous, so both MMA operands are "K-major".
//   * One CTA per SM, persistent over output tiles of 128 x BN.  Warp 0 issues TMA tile
//     loads (128-byte swizzle, 128 bytes of K per stage) into a ring of shared-memory
//     stages; warp 1 issues tcgen05.mma.kind::i8 (M128 x BN x K32) from one thread, four
//     per stage, accumulating in tensor memory; warps 2-5 drain the finished accumulator
//     with tcgen05.ld, apply the two scales and store bf16.  Tensor memory holds two
//     accumulators so that the drain of tile i overlaps the MMAs of tile i+1.
//   * The grouped (MoE) form walks expert segments: the tile list is derived inside the
//     kernel from expert_offsets (device memory), so no host synchronisation and no
//     scratch buffer is needed.  Rows of a tile that fall past the end of a segment are
//     computed and discarded.
//   * The group-scaled form (one activation scale per 128 of K) cannot defer scaling to
//     the end: each 128-wide K block is one accumulator that the drain warps fold into
//     fp32 registers as y = fma(float(acc), sa[row, g], y).
//   * Every wait on an mbarrier is bounded; a wait that gives up records a code in a
//     device status word and the CTA leaves its loops and frees its tensor memory.
//
// Arithmetic of the epilogue follows hip_kernels/w8a8_gemm_v5.hip:123 and
// hip_kernels/w8a8_gemm_intmm_fused.hip:34: (float(acc) * sa[row]) * sb[col] -> bf16.
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <mutex>

#include "launch_common.h"
#include "sm100_ptx.cuh"
#include "w8a8_arith.cuh"

namespace w8a8 {

// Sticky per-device status word written by kernels whose bounded waits ran out.
__device__ int g_device_status = 0;

// Process-wide option: launch the weight-streaming GEMMs (M <= 256) so that they may overlap the
// kernel before them on the stream (programmatic dependent launch).  Off by default.
static std::atomic<int> g_overlap_previous{0};
void set_overlap_previous_kernel(int on) { g_overlap_previous.store(on ? 1 : 0, std::memory_order_relaxed); }
int overlap_previous_kernel() { return g_overlap_previous.load(std::memory_order_relaxed); }

namespace {

constexpr int BM = 128;          // tile rows = MMA M = TMEM lanes
constexpr int BK = 128;          // bytes (= int8 elements) of K per pipeline stage
constexpr int UMMA_K = 32;       // K per tcgen05.mma for 8-bit operands
constexpr int kThreads = 192;    // producer warp, MMA warp, four drain warps
constexpr int kDrainThreads = 128;
constexpr int kMaxExperts = 1024;

enum WaitSite : int {
    kWaitEmptyStage = 101,
    kWaitFullStage = 102,
    kWaitAccEmpty = 103,
    kWaitAccFull = 104,
};

struct Params {
    const float* sa;
    const float* sb;
    void* C;
    const int* offsets;  // null: dense
    int M, N, K, E;
    int64_t ldc;         // row stride of C in elements (>= N)
    int sa_groups;
    int out_i32;
    // Fused all-gather: besides C, every output tile is also stored to these buffers (the same
    // slab of the other ranks' outputs, mapped into this process); same ldc.  npeers = 0: none.
    void* peerC[7];
    int npeers;
};

template <int BN, int STAGES>
struct Smem {
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTilesBytes = STAGES * kStageBytes;
    // after the tiles: one copy of the tile's column scales per drain warp, tile prefix,
    // barriers, tmem slot
    static constexpr int kSbOff = kTilesBytes;
    static constexpr int kPrefixOff = kSbOff + 4 * BN * 4;
    static constexpr int kBarOff = kPrefixOff + (kMaxExperts + 1) * 4 + 4;  // 8-byte aligned below
    static constexpr int kNumBars = 2 * STAGES + 8;  // stage full/empty + up to 4 accumulator full/empty pairs
    static constexpr int kTmemSlotOff = ((kBarOff + 7) & ~7) + kNumBars * 8;
    static constexpr int kAbortOff = kTmemSlotOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;  // slack to align the base to 1024
};

// Maps a linear tile index to (first A row, rows valid, first B row, first C column).
struct TileCoord {
    int a_row0;    // first row of A / C
    int row_end;   // one past the last valid row of this tile's segment
    int b_row0;    // first row of B (expert * N + n0 for the grouped form)
    int n0;        // first output column
    int expert;
};

struct Scheduler {
    const Params& p;
    const int* prefix;  // shared: prefix[e] = m-tiles of experts < e  (grouped only)
    int tiles_n;
    int total;

    __device__ Scheduler(const Params& p_, const int* prefix_, int bn) : p(p_), prefix(prefix_) {
        tiles_n = (p.N + bn - 1) / bn;
        if (p.offsets == nullptr) {
            total = ((p.M + BM - 1) / BM) * tiles_n;
        } else {
            total = prefix[p.E] * tiles_n;
        }
    }

    __device__ TileCoord at(int t, int bn) const {
        TileCoord c;
        if (p.offsets == nullptr) {
            const int tiles_m = (p.M + BM - 1) / BM;
            const int mt = t % tiles_m, nt = t / tiles_m;
            c.a_row0 = mt * BM;
            c.row_end = p.M;
            c.n0 = nt * bn;
            c.b_row0 = c.n0;
            c.expert = 0;
        } else {
            // largest e with prefix[e] * tiles_n <= t
            int lo = 0, hi = p.E;  // invariant: prefix[lo]*tiles_n <= t < prefix[hi]*tiles_n
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (prefix[mid] * tiles_n <= t) lo = mid; else hi = mid;
            }
            const int e = lo;
            const int cnt = prefix[e + 1] - prefix[e];
            const int local = t - prefix[e] * tiles_n;
            const int nt = local / cnt, mt = local % cnt;
            c.a_row0 = p.offsets[e] + mt * BM;
            c.row_end = p.offsets[e + 1];
            c.n0 = nt * bn;
            c.b_row0 = e * p.N + c.n0;
            c.expert = e;
        }
        return c;
    }
};

// One warp: prefix[e] = number of 128-row tiles of the experts before e, prefix[E] = all of them
// (exclusive scan of ceil(segment length / 128) over the experts, into shared memory).
__device__ __forceinline__ void build_tile_prefix(const Params& p, int* prefix, int lane) {
    int carry = 0;
    for (int e0 = 0; e0 < p.E; e0 += 32) {
        const int e = e0 + lane;
        int cnt = 0;
        if (e < p.E) cnt = (p.offsets[e + 1] - p.offsets[e] + BM - 1) / BM;
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

__device__ __forceinline__ void report_wait_failure(int site) {
    atomicCAS(&g_device_status, 0, site);
}


// Drains one finished accumulator: this thread owns TMEM lane (= tile row) `row` and walks
// NCOLS columns 32 at a time: tcgen05.ld -> (float(acc) * sa) * sb[col] -> bf16 -> global.
// `sbs` holds the tile's column scales in shared memory (private to the warp).
template <int NCOLS>
__device__ __forceinline__ void drain_accumulator(const Params& p, uint32_t t_lane, const float* sbs, int row,
                                                  bool row_ok, int n0, bool vec_ok) {
    const float sa = (row_ok && !p.out_i32) ? __ldg(p.sa + row) : 0.0f;
#pragma unroll 1
    for (int cc = 0; cc < NCOLS / 32; ++cc) {
        uint32_t r[32];
        __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the stores
        ptx::tmem_ld_32x32b_x32(t_lane + cc * 32, r);
        ptx::tmem_ld_wait();
        const int n = n0 + cc * 32;
        if (!row_ok || n >= p.N) continue;
        if (p.out_i32) {
            int* out = static_cast<int*>(p.C) + (int64_t)row * p.ldc + n;
            if (vec_ok && n + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<uint4*>(out + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (n + j < p.N) out[j] = (int)r[j];
            }
        } else {
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.C) + (int64_t)row * p.ldc + n;
            const float4* sb4 = reinterpret_cast<const float4*>(sbs + cc * 32);
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 s4 = sb4[j];
                const float v0 = __fmul_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 0]), sa), s4.x);
                const float v1 = __fmul_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 1]), sa), s4.y);
                const float v2 = __fmul_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 2]), sa), s4.z);
                const float v3 = __fmul_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 3]), sa), s4.w);
                packed[2 * j] = pack_bf16x2_rn(v0, v1);
                packed[2 * j + 1] = pack_bf16x2_rn(v2, v3);
            }
            if (vec_ok && n + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(out + 8 * j) =
                        make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                // the same 64 bytes to every peer's copy of the output (plain stores over NVLink)
#pragma unroll
                for (int d = 0; d < 7; ++d) {
                    if (d >= p.npeers) break;
                    __nv_bfloat16* po = static_cast<__nv_bfloat16*>(p.peerC[d]) + (int64_t)row * p.ldc + n;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint4*>(po + 8 * j) =
                            make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const uint32_t w = packed[j >> 1];
                    const uint16_t h = (j & 1) ? (uint16_t)(w >> 16) : (uint16_t)(w & 0xffffu);
                    if (n + j < p.N) reinterpret_cast<uint16_t*>(out)[j] = h;
                }
            }
        }
    }
}

__device__ __forceinline__ bool c_vector_stores_ok(const Params& p) {
    return (p.N % 8 == 0) && (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
}

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
    int* prefix = reinterpret_cast<int*>(smem + L::kPrefixOff);
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
    if (p.offsets != nullptr && warp == 2) build_tile_prefix(p, prefix, lane);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const Scheduler sched(p, prefix, BN);
    const int k_blocks = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
                const TileCoord c = sched.at(t, BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u) || *abort_flag) {
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
                if (!ptx::mbar_wait_bounded(acc_empty_bar(acc), acc_phase ^ 1u) || *abort_flag) {
                    report_wait_failure(kWaitAccEmpty);
                    *abort_flag = 1;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(full_bar(stage), phase) || *abort_flag) {
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
                const float* sb_row = p.sb + (int64_t)c.expert * p.N;
                for (int j = lane; j < BN; j += 32)
                    sbs[j] = (c.n0 + j < p.N) ? __ldg(sb_row + c.n0 + j) : 0.0f;
            }
            __syncwarp();
            bool got = ptx::mbar_wait_bounded(acc_full_bar(acc), acc_phase);
            if (!got || *abort_flag) {
                report_wait_failure(kWaitAccFull);
                *abort_flag = 1;
                break;
            }
            ptx::tc_fence_after_sync();
            const int row = c.a_row0 + quarter * 32 + lane;
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
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
    // output staging for the TMA-store epilogue: 4 slabs of [128 rows][64 bf16 = 128 B], 128B-swizzled
    static constexpr int kOutOff = kTilesBytes;
    static constexpr int kOutBytes = TMA_STORE ? 4 * 128 * 128 : 0;
    static constexpr int kSbOff = kOutOff + kOutBytes;          // 4 warps x 256 column scales
    static constexpr int kBarOff = kSbOff + 4 * 256 * 4;        // 8-byte aligned
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemSlotOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;
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
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int k_blocks = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += npairs) {
                const int mt = t % tiles_m, nt = t / tiles_m;
                const int a_row0 = mt * 256 + (int)rank * 128;
                const int b_row0 = nt * PBN + (int)rank * 128;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u) || *abort_flag) {
                        report_wait_failure(kWaitEmptyStage);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = tiles_base + stage * L::kStageBytes;
                    const uint32_t b_dst = a_dst + L::kABytes;
                    const uint32_t leader_full = ptx::map_to_cta(full_bar(stage), 0);
                    if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
                    ptx::tma_load_2d_pair(a_dst, &tmA, kb * BK, a_row0, leader_full);
                    ptx::tma_load_2d_pair(b_dst, &tmB, kb * BK, b_row0, leader_full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
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
                if (!ptx::mbar_wait_bounded(acc_empty_bar(acc), acc_phase ^ 1u) || *abort_flag) {
                    report_wait_failure(kWaitAccEmpty);
                    *abort_flag = 1;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * PBN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(full_bar(stage), phase) || *abort_flag) {
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
        const int quarter = warp & 3;
        float* sbs = sb_tile + (warp - 2) * PBN;
        int acc = 0;
        uint32_t acc_phase = 0;
        const bool vec_ok = c_vector_stores_ok(p);
        for (int t = pair; t < total; t += npairs) {
            const int mt = t % tiles_m, nt = t / tiles_m;
            const int n0 = nt * PBN;
            __syncwarp();
            if (!p.out_i32) {
                for (int j = lane; j < PBN; j += 32) sbs[j] = (n0 + j < p.N) ? __ldg(p.sb + n0 + j) : 0.0f;
            }
            __syncwarp();
            if (!ptx::mbar_wait_bounded(acc_full_bar(acc), acc_phase) || *abort_flag) {
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
                // Fused all-gather epilogue: the bf16 tile is staged in shared memory (four 64-column
                // slabs, 128-byte swizzle so that the 16-byte stores of a quarter-warp hit all banks) and
                // one thread sends it with TMA tile stores to this rank's buffer and to every peer's:
                // full 128-byte rows per request over NVLink, no store instruction per destination.
                const uint32_t out_base = tiles_base + L::kOutOff;
                const int r = quarter * 32 + lane;  // row inside this CTA's 128-row half tile
                const float sa = (row < p.M) ? __ldg(p.sa + row) : 0.0f;
                if (warp == 2 && lane == 0) ptx::bulk_wait_group_read0();  // previous tile's stores have read the staging
                asm volatile("bar.sync 2, %0;" ::"n"(kDrainThreads) : "memory");
#pragma unroll 1
                for (int cc = 0; cc < PBN / 32; ++cc) {
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
                    const uint32_t slab = out_base + (uint32_t)(cc >> 1) * (128u * 128u) + (uint32_t)r * 128u;
                    const uint32_t chunk0 = (uint32_t)(cc & 1) * 4u;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t phys = (chunk0 + j) ^ (uint32_t)(r & 7);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(slab + phys * 16u),
                                     "r"(packed[4 * j]), "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]),
                                     "r"(packed[4 * j + 3])
                                     : "memory");
                    }
                }
                ptx::fence_proxy_async_smem();  // the staged tile becomes visible to the TMA engine
                asm volatile("bar.sync 2, %0;" ::"n"(kDrainThreads) : "memory");
                if (warp == 2 && lane == 0) {
                    const int y = mt * 256 + (int)rank * 128;
                    for (int d = 0; d < smaps.count; ++d)
#pragma unroll
                        for (int sl = 0; sl < 4; ++sl)
                            if (n0 + sl * 64 < p.N)
                                ptx::tma_store_2d(&smaps.m[d], n0 + sl * 64, y, out_base + (uint32_t)sl * (128u * 128u));
                    ptx::bulk_commit_group();
                }
            }
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
                const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + b * GSN + half * HC;
                const float2 sg2 = splat2(sg), unbias = splat2(-12582912.0f);
#pragma unroll
                for (int cc = 0; cc < HC / 16; ++cc) {
                    uint32_t r0[16];
                    ptx::tmem_ld_32x32b_x16(t_lane + cc * 16, r0);
                    ptx::tmem_ld_wait();
                    if (cc == HC / 16 - 1) {
                        // the last columns are in registers: the accumulator can be overwritten
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(blk_empty_bar(b));
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float2 f = make_float2(__int_as_float((int)r0[2 * j] + 0x4B400000),
                                               __int_as_float((int)r0[2 * j + 1] + 0x4B400000));
                        y2[cc * 8 + j] = __ffma2_rn(__fadd2_rn(f, unbias), sg2, y2[cc * 8 + j]);
                    }
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


// Split-K epilogue of the weight-streaming kernels: sums the S partial tiles ([token][128 weight
// rows] int32, one in each peer CTA's shared memory, fixed order r = 0..S-1), applies the scales and
// stores.  Work item = (token column c, group of four weight rows): 16-byte loads through
// distributed shared memory, four outputs that are contiguous in C; consecutive threads take
// consecutive row groups of one column.  Four items are in flight per thread, because one item at a
// time would cost a full remote-load latency per item.
template <int MAXS>
__device__ __forceinline__ void reduce_partials_and_store(const Params& p, const uint32_t (&peer_base)[MAXS], int S,
                                                          int cols_lo, int cols_hi, int n0, int tid, int nthreads) {
    constexpr int U = 4;
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
                const float sa = __ldg(p.sa + c);
                float sbv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) sbv[j] = (n + j < p.N) ? __ldg(p.sb + n + j) : 0.0f;
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
    static constexpr int kBudget = 196 * 1024;
    static constexpr int kStages = kBudget / kStageBytes;
    static constexpr int kTilesBytes = kStages * kStageBytes;
    static constexpr int kPartialBytes = NTOK * 128 * 4;
    static_assert(kPartialBytes <= kTilesBytes, "the partial tile reuses the stage ring");
    static constexpr int kBarOff = kTilesBytes;
    static constexpr int kNumBars = 2 * kStages + 1;
    static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemSlotOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

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
        // drain warps: accumulator -> shared partial (or straight out when K is not split)
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
        reduce_partials_and_store<8>(p, peer_base, S, cols_lo, cols_hi, n0, threadIdx.x, kThreads);
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
    static constexpr int kBarOff = kTilesBytes;
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
        // drain warps of both CTAs: accumulator of this CTA's 128 weight rows -> shared partial
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
        reduce_partials_and_store<4>(p, peer_base, S, cols_lo, cols_hi, n0, threadIdx.x, kThreads);
    }

    // nobody leaves while a peer may still read its shared memory
    __syncthreads();
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// More than 48 KB of dynamic shared memory needs an opt-in per kernel and per device; done on the
// first launch of each kernel on each device.
template <typename Kernel>
bool opt_in_shared_memory(Kernel kernel, int bytes, bool (&done)[64]) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && done[dev]) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    if (dev >= 0 && dev < 64) done[dev] = true;
    return true;
}

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// 2-D uint8 tensor [rows, K] (K contiguous), box = 128 bytes of K x box_rows rows,
// 128-byte swizzle, out-of-range elements read as zero.
int make_tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(DSV4_ERR_DRIVER, "w8a8_gemm: cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {K};
    const cuuint32_t box[2] = {BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        static thread_local char msg[160];
        snprintf(msg, sizeof msg, "w8a8_gemm: cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu K=%llu)",
                 (int)r, (unsigned long long)rows, (unsigned long long)K);
        return fail(DSV4_ERR_DRIVER, msg);
    }
    return 0;
}

int sm_count() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev != cached_dev) {
        cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
        cached_dev = dev;
    }
    return cached;
}

template <int BN, int STAGES>
int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, int max_tiles,
                   cudaStream_t st) {
    using L = Smem<BN, STAGES>;
    static_assert(L::kDynamic <= 227 * 1024, "shared memory budget");
    static bool opted_in[64] = {};
    if (!opt_in_shared_memory(gemm_i8_kernel<BN, STAGES>, L::kDynamic, opted_in))
        return fail(DSV4_ERR_LAUNCH, "w8a8_gemm: cannot raise the dynamic shared memory limit");
    int grid = sm_count();
    if (grid <= 0) return fail(DSV4_ERR_LAUNCH, "w8a8_gemm: no CUDA device");
    if (max_tiles < grid) grid = max_tiles;
    if (grid < 1) grid = 1;
    gemm_i8_kernel<BN, STAGES><<<grid, kThreads, L::kDynamic, st>>>(tmA, tmB, p);
    return check_launch("w8a8_gemm");
}

template <int NTOK>
int launch_stream_variant(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int n_tiles, int splits,
                          cudaStream_t st) {
    using L = StreamSmem<NTOK>;
    static_assert(L::kDynamic <= 227 * 1024, "shared memory budget");
    static bool opted_in[64] = {};
    if (!opt_in_shared_memory(gemm_i8_stream_kernel<NTOK>, L::kDynamic, opted_in))
        return fail(DSV4_ERR_LAUNCH, "w8a8_gemm: cannot raise the dynamic shared memory limit");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_tiles * splits), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kDynamic;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_previous_kernel() ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, gemm_i8_stream_kernel<NTOK>, tmW, tmX, p);
    if (err != cudaSuccess) {
        cudaGetLastError();  // clear the sticky launch error
        static thread_local char msg[160];
        snprintf(msg, sizeof msg, "w8a8_gemm (weight streaming): %s", cudaGetErrorString(err));
        return fail(DSV4_ERR_LAUNCH, msg);
    }
    return check_launch("w8a8_gemm (weight streaming)");
}

// How many clusters of 2*splits CTAs of the pair streaming kernel the device can run at once (one
// CTA per SM, a cluster inside one GPC); asked once per device and cluster size.
int stream_pair_active_clusters(int splits) {
    static int cached[64][5] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || splits < 1 || splits > 4) return 0;
    if (cached[dev][splits] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(2 * splits * 64), 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = StreamPairSmem::kDynamic;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)(2 * splits);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_i8_stream_pair_kernel, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = -1;
        }
        cached[dev][splits] = n > 0 ? n : -1;
    }
    return cached[dev][splits] > 0 ? cached[dev][splits] : 0;
}

int launch_stream_pair(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int n_tiles, int splits,
                       cudaStream_t st) {
    using L = StreamPairSmem;
    static_assert(L::kDynamic <= 227 * 1024, "shared memory budget");
    static bool opted_in[64] = {};
    if (!opt_in_shared_memory(gemm_i8_stream_pair_kernel, L::kDynamic, opted_in))
        return fail(DSV4_ERR_LAUNCH, "w8a8_gemm: cannot raise the dynamic shared memory limit");
    // a cluster must fit into one GPC: take the widest K split whose clusters all run in one wave
    while (splits > 1 && stream_pair_active_clusters(splits) < n_tiles) --splits;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_tiles * 2 * splits), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kDynamic;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)(2 * splits);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_previous_kernel() ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, gemm_i8_stream_pair_kernel, tmW, tmX, p);
    if (err != cudaSuccess) {
        cudaGetLastError();  // clear the sticky launch error
        static thread_local char msg[160];
        snprintf(msg, sizeof msg, "w8a8_gemm (weight streaming, CTA pairs): %s", cudaGetErrorString(err));
        return fail(DSV4_ERR_LAUNCH, msg);
    }
    return check_launch("w8a8_gemm (weight streaming, CTA pairs)");
}

template <int STAGES>
int launch_gs_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, int max_tiles, cudaStream_t st) {
    using L = Smem<GSN, STAGES>;
    static_assert(L::kDynamic <= 227 * 1024, "shared memory budget");
    static bool opted_in[64] = {};
    if (!opt_in_shared_memory(gemm_i8_gs_kernel<STAGES>, L::kDynamic, opted_in))
        return fail(DSV4_ERR_LAUNCH, "grouped_gemm: cannot raise the dynamic shared memory limit");
    int grid = sm_count();
    if (grid <= 0) return fail(DSV4_ERR_LAUNCH, "grouped_gemm: no CUDA device");
    if (max_tiles < grid) grid = max_tiles;
    if (grid < 1) grid = 1;
    gemm_i8_gs_kernel<STAGES><<<grid, kGsThreads, L::kDynamic, st>>>(tmA, tmB, p);
    return check_launch("grouped_gemm (group-scaled)");
}

// bf16 [rows, cols] view with row stride ldc elements: box = 64 columns x 128 rows, 128-byte swizzle
int make_store_map(CUtensorMap* map, void* base, uint64_t rows, uint64_t cols, uint64_t ldc) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(DSV4_ERR_DRIVER, "w8a8_gemm: cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ldc * 2};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DSV4_ERR_DRIVER, "w8a8_gemm_allgather: cuTensorMapEncodeTiled failed for an output map");
    return 0;
}

template <int STAGES, bool TMA_STORE>
int launch_pair_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, const StoreMaps& smaps,
                        cudaStream_t st) {
    using L = PairSmem<STAGES, TMA_STORE>;
    static_assert(L::kDynamic <= 227 * 1024, "shared memory budget");
    static bool opted_in[64] = {};
    if (!opt_in_shared_memory(gemm_i8_pair_kernel<STAGES, TMA_STORE>, L::kDynamic, opted_in))
        return fail(DSV4_ERR_LAUNCH, "w8a8_gemm: cannot raise the dynamic shared memory limit");
    const int tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
    int pairs = sm_count() / 2;
    if (pairs <= 0) return fail(DSV4_ERR_LAUNCH, "w8a8_gemm: no CUDA device");
    if (tiles < pairs) pairs = tiles;
    gemm_i8_pair_kernel<STAGES, TMA_STORE><<<2 * pairs, kThreads, L::kDynamic, st>>>(tmA, tmB, p, smaps);
    return check_launch("w8a8_gemm");
}

}  // namespace

int gemm_i8(const GemmArgs& a, cudaStream_t st) {
    const bool grouped = a.offsets != nullptr;
    if (a.M < 0 || a.N < 0 || a.K < 0) return fail(DSV4_ERR_ARG, "w8a8_gemm: negative size");
    if (a.M == 0 || a.N == 0) return 0;
    if (a.K == 0) return fail(DSV4_ERR_ARG, "w8a8_gemm: K must be positive");
    if (a.A == nullptr || a.B == nullptr || a.C == nullptr) return fail(DSV4_ERR_ARG, "w8a8_gemm: null pointer");
    if (!a.out_i32 && (a.sa == nullptr || a.sb == nullptr)) return fail(DSV4_ERR_ARG, "w8a8_gemm: null scale pointer");
    if (a.K % 16 != 0) return fail(DSV4_ERR_ARG, "w8a8_gemm: K must be a multiple of 16 (TMA row stride)");
    if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15))
        return fail(DSV4_ERR_ARG, "w8a8_gemm: A and B must be 16-byte aligned");
    if (grouped && (a.E <= 0 || a.E > kMaxExperts)) return fail(DSV4_ERR_ARG, "grouped_gemm: E must be in 1..1024");
    if (a.sa_groups != 1) {
        if (a.out_i32) return fail(DSV4_ERR_ARG, "w8a8_gemm: raw accumulators exist only for per-token scaling");
        if (a.K % 128 != 0 || a.sa_groups != a.K / 128)
            return fail(DSV4_ERR_ARG, "grouped_gemm: group scales need K % 128 == 0 and sa_groups == K / 128");
    }

    Params p;
    p.sa = a.sa; p.sb = a.sb; p.C = a.C; p.offsets = a.offsets;
    p.M = a.M; p.N = a.N; p.K = a.K; p.E = grouped ? a.E : 1;
    p.ldc = a.ldc > 0 ? a.ldc : a.N;
    p.sa_groups = a.sa_groups; p.out_i32 = a.out_i32;
    if (p.ldc < a.N) return fail(DSV4_ERR_ARG, "w8a8_gemm: ldc smaller than N");
    p.npeers = 0;
    for (int d = 0; d < 7; ++d) p.peerC[d] = nullptr;
    if (a.npeers > 0) {
        if (a.npeers > 7 || grouped || a.out_i32 || a.sa_groups != 1)
            return fail(DSV4_ERR_ARG, "w8a8_gemm_allgather: at most 7 peers, dense per-token-scaled bf16 output only");
        if (a.N % 32 != 0 || p.ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(a.C) & 15))
            return fail(DSV4_ERR_ARG, "w8a8_gemm_allgather: N % 32 == 0, ldc % 8 == 0 and 16-byte aligned outputs required");
        for (int d = 0; d < a.npeers; ++d) {
            if (a.peerC[d] == nullptr || (reinterpret_cast<uintptr_t>(a.peerC[d]) & 15))
                return fail(DSV4_ERR_ARG, "w8a8_gemm_allgather: null or misaligned peer pointer");
            p.peerC[d] = a.peerC[d];
        }
        p.npeers = a.npeers;
    }

    const uint64_t b_rows = grouped ? (uint64_t)a.E * a.N : (uint64_t)a.N;
    const int sms = sm_count();
    const int tiles_m_bound = grouped ? (a.M / BM + a.E) : (a.M + BM - 1) / BM;

    // Tile width: 256 columns when that already gives every SM a tile, otherwise narrower
    // tiles so that a short, weight-streaming problem spreads over more SMs.
    int bn = 256;
    if ((int64_t)tiles_m_bound * ((a.N + 255) / 256) < sms) bn = 128;
    if (bn == 128 && (int64_t)tiles_m_bound * ((a.N + 127) / 128) < sms) bn = 64;
    if (bn == 64 && (int64_t)tiles_m_bound * ((a.N + 63) / 64) < sms) bn = 32;

    CUtensorMap tmA, tmB;
    if (a.sa_groups != 1) {
        int rc3 = make_tile_map(&tmA, a.A, (uint64_t)a.M, (uint64_t)a.K, BM);
        if (rc3) return rc3;
        rc3 = make_tile_map(&tmB, a.B, b_rows, (uint64_t)a.K, GSN);
        if (rc3) return rc3;
        return launch_gs_variant<4>(tmA, tmB, p, tiles_m_bound * ((a.N + GSN - 1) / GSN), st);
    }
    // Few tokens: stream the weight once, tokens on the MMA's N axis, K split over a cluster
    if (!grouped && a.M <= 256 && a.npeers == 0) {
        const int k_blocks = (a.K + BK - 1) / BK;
        if (a.M > 128 && a.N >= 256) {
            // 129..256 tokens: CTA pairs halve the token traffic per SM
            const int pair_tiles = (a.N + 255) / 256;
            int psplits = sms / (2 * pair_tiles);
            if (psplits > 4) psplits = 4;
            if (psplits > k_blocks) psplits = k_blocks;
            if (psplits < 1) psplits = 1;
            int rc5 = make_tile_map(&tmA, a.B, b_rows, (uint64_t)a.K, 128);   // weights
            if (rc5) return rc5;
            rc5 = make_tile_map(&tmB, a.A, (uint64_t)a.M, (uint64_t)a.K, 128);  // this CTA's half of the tokens
            if (rc5) return rc5;
            return launch_stream_pair(tmA, tmB, p, pair_tiles, psplits, st);
        }
        const int n_tiles = (a.N + 127) / 128;
        int splits = sms / n_tiles;
        if (splits > 8) splits = 8;
        if (splits > k_blocks) splits = k_blocks;
        if (splits < 1) splits = 1;
        const int ntok = a.M <= 16 ? 16 : a.M <= 32 ? 32 : a.M <= 64 ? 64 : a.M <= 128 ? 128 : 256;
        int rc4 = make_tile_map(&tmA, a.B, b_rows, (uint64_t)a.K, 128);   // weights
        if (rc4) return rc4;
        rc4 = make_tile_map(&tmB, a.A, (uint64_t)a.M, (uint64_t)a.K, (uint32_t)ntok);  // tokens
        if (rc4) return rc4;
        switch (ntok) {
            case 16: return launch_stream_variant<16>(tmA, tmB, p, n_tiles, splits, st);
            case 32: return launch_stream_variant<32>(tmA, tmB, p, n_tiles, splits, st);
            case 64: return launch_stream_variant<64>(tmA, tmB, p, n_tiles, splits, st);
            case 128: return launch_stream_variant<128>(tmA, tmB, p, n_tiles, splits, st);
            default: return launch_stream_variant<256>(tmA, tmB, p, n_tiles, splits, st);
        }
    }
    // Dense problems with more than one 128-row tile go to the CTA-pair kernel
    if (!grouped && a.M > 128 && (int64_t)((a.M + 255) / 256) * ((a.N + 255) / 256) >= sms / 4) {
        int rc2 = make_tile_map(&tmA, a.A, (uint64_t)a.M, (uint64_t)a.K, BM);
        if (rc2) return rc2;
        rc2 = make_tile_map(&tmB, a.B, b_rows, (uint64_t)a.K, 128);
        if (rc2) return rc2;
        StoreMaps smaps;
        smaps.count = 0;
        if (a.npeers > 0) {
            // fused all-gather: tile stores through tensor maps of this rank's slab and of every peer's
            rc2 = make_store_map(&smaps.m[0], a.C, (uint64_t)a.M, (uint64_t)a.N, (uint64_t)p.ldc);
            if (rc2) return rc2;
            for (int d = 0; d < a.npeers; ++d) {
                rc2 = make_store_map(&smaps.m[1 + d], a.peerC[d], (uint64_t)a.M, (uint64_t)a.N, (uint64_t)p.ldc);
                if (rc2) return rc2;
            }
            smaps.count = 1 + a.npeers;
            return launch_pair_variant<4, true>(tmA, tmB, p, smaps, st);
        }
        return launch_pair_variant<6, false>(tmA, tmB, p, smaps, st);
    }
    int rc = make_tile_map(&tmA, a.A, (uint64_t)a.M, (uint64_t)a.K, BM);
    if (rc) return rc;
    rc = make_tile_map(&tmB, a.B, b_rows, (uint64_t)a.K, (uint32_t)bn);
    if (rc) return rc;
    const int max_tiles = tiles_m_bound * ((a.N + bn - 1) / bn);
    switch (bn) {
        case 256: return launch_variant<256, 4>(tmA, tmB, p, max_tiles, st);
        case 128: return launch_variant<128, 6>(tmA, tmB, p, max_tiles, st);
        case 64: return launch_variant<64, 8>(tmA, tmB, p, max_tiles, st);
        default: return launch_variant<32, 10>(tmA, tmB, p, max_tiles, st);
    }
}

// ------------------------------------------------------------------------------------
// int32 [M,N] -> bf16 with the two scales (hip_kernels/w8a8_gemm_intmm_fused.hip:22-36)
// ------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(256) scale_convert_kernel(const int* __restrict__ acc,
                                                            const float* __restrict__ sa,
                                                            const float* __restrict__ sb,
                                                            __nv_bfloat16* __restrict__ out, int M, int N) {
    const int64_t total = (int64_t)M * N;
    for (int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; f < total;
         f += (int64_t)gridDim.x * blockDim.x) {
        const int row = (int)(f / N), col = (int)(f % N);
        out[f] = __float2bfloat16_rn(__fmul_rn(__fmul_rn(__int2float_rn(acc[f]), sa[row]), sb[col]));
    }
}
}  // namespace

int scale_convert(const void* acc, const void* sa, const void* sb, void* out, int M, int N, cudaStream_t st) {
    if (M == 0 || N == 0) return 0;
    int64_t blocks = ((int64_t)M * N + 255) / 256;
    if (blocks > (1 << 20)) blocks = 1 << 20;
    scale_convert_kernel<<<(int)blocks, 256, 0, st>>>(static_cast<const int*>(acc), static_cast<const float*>(sa),
                                                      static_cast<const float*>(sb),
                                                      static_cast<__nv_bfloat16*>(out), M, N);
    return check_launch("scale_convert");
}

int read_device_status(cudaStream_t st, int* out) {
    if (cudaStreamSynchronize(st) != cudaSuccess) return fail(DSV4_ERR_LAUNCH, "device_status: stream synchronise failed");
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess)
        return fail(DSV4_ERR_LAUNCH, "device_status: cannot read the status word");
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    }
    if (v == 0) {
        const int rc = read_row_status(&v);
        if (rc) return rc;
    }
    if (out) *out = v;
    return 0;
}

}  // namespace w8a8
