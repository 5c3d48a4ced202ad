// Private part of gemm_i8_sm100.cu (included by that translation unit only, hence the unnamed
// namespace): tile constants, kernel parameters, shared-memory layout, tile scheduler and the
// accumulator drain shared by the int8 GEMM kernels.
#ifndef W8A8_GEMM_I8_COMMON_CUH
#define W8A8_GEMM_I8_COMMON_CUH

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "launch_common.h"
#include "sm100_ptx.cuh"
#include "w8a8_arith.cuh"

namespace w8a8 {

// Sticky per-device status word written by kernels whose bounded waits ran out, and the address of
// its mirror in mapped host memory (set on the first GEMM launch on a device), which lets the next
// launch see the failure without synchronising.
__device__ int g_device_status = 0;
__device__ int* g_host_status_mirror = nullptr;

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
    const int* offsets;  // null: dense (or the masked layout)
    // masked layout: A and C are [E, max_m, .] and expert e owns the first masked_m[e] rows of its
    // block; null otherwise
    const int* masked_m;
    int max_m;
    int M, N, K, E;
    int64_t ldc;         // row stride of C in elements (>= N)
    int sa_groups;
    int out_i32;
    // Fused all-gather: besides C, every output tile is also stored to these buffers (the same
    // slab of the other ranks' outputs, mapped into this process); same ldc.  npeers = 0: none.
    void* peerC[7];
    int npeers;
    // CTA-pair kernel: m-tiles per group of its tile order (see PairTileOrder)
    int pair_group_m;
    // grouped GEMM with per-token scales only: row r of the result goes to row_ptr[r] (a bf16 row of N elements,
    // possibly in another GPU's memory) instead of C + r * ldc; null = C
    void* const* row_ptr;
    // every bounded wait of the launch gives up after this many nanoseconds
    unsigned long long wait_limit_ns;
    // test hook (never set through the public entry points): the producer issues no tile loads, so
    // every consumer wait of the launch runs out and the kernel leaves through its give-up path
    int withhold_loads;
};

template <int BN, int STAGES>
struct Smem {
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTilesBytes = STAGES * kStageBytes;
    // after the tiles: one copy of the tile's column scales per drain warp, barriers, tmem slot
    static constexpr int kSbOff = kTilesBytes;
    static constexpr int kBarOff = kSbOff + 4 * BN * 4;  // 8-byte aligned below
    static constexpr int kNumBars = 2 * STAGES + 8;  // stage full/empty + up to 4 accumulator full/empty pairs
    static constexpr int kTmemSlotOff = ((kBarOff + 7) & ~7) + kNumBars * 8;
    static constexpr int kAbortOff = kTmemSlotOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;  // slack to align the base to 1024
};

// Maps a linear tile index of a dense problem to its coordinates (M fastest).
struct TileCoord {
    int a_row0;    // first row of A / C
    int row_end;   // one past the last valid row
    int b_row0;    // first row of B
    int n0;        // first output column
};

struct Scheduler {
    const Params& p;
    int tiles_n;
    int total;

    __device__ Scheduler(const Params& p_, int bn) : p(p_) {
        tiles_n = (p.N + bn - 1) / bn;
        total = ((p.M + BM - 1) / BM) * tiles_n;
    }

    __device__ TileCoord at(int t, int bn) const {
        TileCoord c;
        const int tiles_m = (p.M + BM - 1) / BM;
        const int mt = t % tiles_m, nt = t / tiles_m;
        c.a_row0 = mt * BM;
        c.row_end = p.M;
        c.n0 = nt * bn;
        c.b_row0 = c.n0;
        return c;
    }
};

__device__ __forceinline__ void report_wait_failure(int site) {
    if (atomicCAS(&g_device_status, 0, site) == 0) {
        int* mirror = g_host_status_mirror;
        if (mirror != nullptr) {
            *reinterpret_cast<volatile int*>(mirror) = site;
            __threadfence_system();
        }
    }
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

}  // namespace
}  // namespace w8a8

#endif  // W8A8_GEMM_I8_COMMON_CUH
