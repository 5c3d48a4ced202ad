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
//   * The grouped (MoE) form puts an expert's weight rows on the MMA's M axis and its tokens
//     on the N axis (gemm_i8_wt_kernel.cuh); its work list is derived inside the kernel from
//     expert_offsets or masked_m (device memory), so no host synchronisation and no scratch
//     buffer is needed.
//   * Its group-scaled form (one activation scale per 128 of K) cannot defer scaling to
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
#include "gemm_i8_common.cuh"
#include "gemm_i8_tile_kernel.cuh"
#include "gemm_i8_pair_kernel.cuh"
#include "gemm_i8_stream_kernels.cuh"
#include "gemm_i8_wt_kernel.cuh"

namespace w8a8 {

// Option of the calling thread: launch the dense GEMMs (weight-streaming kernels for M <= 256, CTA-pair
// kernel above) so that they may overlap the kernel before them on the stream (programmatic dependent
// launch).  Off by default.  Per thread, so that one thread that captures a CUDA graph with the option
// on does not change what other threads launch meanwhile.
static thread_local int g_overlap_previous = 0;
void set_overlap_previous_kernel(int on) { g_overlap_previous = on ? 1 : 0; }
int overlap_previous_kernel() { return g_overlap_previous; }

namespace {

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
// Encoded tensor maps are kept per thread in a small table keyed by everything that goes into them (a
// descriptor holds an address and a shape, nothing that can go stale): a serving loop launches the same few
// GEMMs over the same buffers, and the grouped GEMM alone needs eleven maps per launch.
struct TileMapKey {
    const void* base;
    uint64_t rows, K;
    uint32_t box_rows;
    bool operator==(const TileMapKey& o) const {
        return base == o.base && rows == o.rows && K == o.K && box_rows == o.box_rows;
    }
};
struct TileMapCache {
    static constexpr int kEntries = 64;
    TileMapKey key[kEntries];
    CUtensorMap map[kEntries];
    int used = 0, next = 0;
};

int make_tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
    static thread_local TileMapCache cache;
    const TileMapKey k{base, rows, K, box_rows};
    for (int i = 0; i < cache.used; ++i) {
        if (cache.key[i] == k) {
            *map = cache.map[i];
            return 0;
        }
    }
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
    const int slot = cache.used < TileMapCache::kEntries ? cache.used++ : cache.next;
    cache.next = (slot + 1) % TileMapCache::kEntries;
    cache.key[slot] = k;
    cache.map[slot] = *map;
    return 0;
}

// The status word's mirror in mapped host memory: allocated (host memory only) and published to the
// device on the first GEMM launch on each device.  A kernel whose bounded wait gives up writes its
// code there as well, so a later launch can refuse to go on without synchronising anything.
volatile int* host_status_mirror() {
    static volatile int* mirror[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (mirror[dev] != nullptr) return mirror[dev];
    std::lock_guard<std::mutex> lock(mu);
    if (mirror[dev] != nullptr) return mirror[dev];
    int* host = nullptr;
    int* device_view = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void**>(&device_view), host, 0) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    *host = 0;
    if (cudaMemcpyToSymbol(g_host_status_mirror, &device_view, sizeof device_view) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    mirror[dev] = host;
    return mirror[dev];
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
    static_assert(L::kDynamic <= 227 * 1024, "shared memory limit");
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
    static_assert(L::kDynamic <= 227 * 1024, "shared memory limit");
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
    static_assert(L::kDynamic <= 227 * 1024, "shared memory limit");
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

// Grouped GEMM, weights on the MMA's M axis: one CTA per SM walks the (expert, token chunk, weight tile) items.
template <bool GS, bool STAGED = false>
int launch_wt_variant(const CUtensorMap& tmW, const WtMaps& xmaps, const Params& p, cudaStream_t st) {
    using L = WtSmem<GS, STAGED>;
    static_assert(L::kDynamic <= 227 * 1024, "shared memory limit");
    static bool opted_in[64] = {};
    if (!opt_in_shared_memory(gemm_i8_wt_kernel<GS, STAGED>, L::kDynamic, opted_in))
        return fail(DSV4_ERR_LAUNCH, "grouped_gemm: cannot raise the dynamic shared memory limit");
    int grid = sm_count();
    if (grid <= 0) return fail(DSV4_ERR_LAUNCH, "grouped_gemm: no CUDA device");
    // at most this many items exist, whatever the segment lengths turn out to be
    const int64_t bound = ((int64_t)p.M / kWtChunk + p.E) * ((p.N + 127) / 128);
    if (bound < grid) grid = (int)bound;
    if (grid < 1) grid = 1;
    gemm_i8_wt_kernel<GS, STAGED><<<grid, GS ? 576 : 192, L::kDynamic, st>>>(tmW, xmaps, p);
    return check_launch("grouped_gemm");
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
    static_assert(L::kDynamic <= 227 * 1024, "shared memory limit");
    static bool opted_in[64] = {};
    if (!opt_in_shared_memory(gemm_i8_pair_kernel<STAGES, TMA_STORE>, L::kDynamic, opted_in))
        return fail(DSV4_ERR_LAUNCH, "w8a8_gemm: cannot raise the dynamic shared memory limit");
    const int tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
    int pairs = sm_count() / 2;
    if (pairs <= 0) return fail(DSV4_ERR_LAUNCH, "w8a8_gemm: no CUDA device");
    if (tiles < pairs) pairs = tiles;
    if (!overlap_previous_kernel()) {
        gemm_i8_pair_kernel<STAGES, TMA_STORE><<<2 * pairs, kThreads, L::kDynamic, st>>>(tmA, tmB, p, smaps);
        return check_launch("w8a8_gemm");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kDynamic;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, gemm_i8_pair_kernel<STAGES, TMA_STORE>, tmA, tmB, p, smaps);
    if (err != cudaSuccess) {
        cudaGetLastError();  // clear the sticky launch error
        static thread_local char msg[160];
        snprintf(msg, sizeof msg, "w8a8_gemm (CTA pairs): %s", cudaGetErrorString(err));
        return fail(DSV4_ERR_LAUNCH, msg);
    }
    return check_launch("w8a8_gemm");
}

}  // namespace

int gemm_i8(const GemmArgs& a, cudaStream_t st) {
    const bool grouped = a.offsets != nullptr || a.masked_m != nullptr;
    if (a.M < 0 || a.N < 0 || a.K < 0) return fail(DSV4_ERR_ARG, "w8a8_gemm: negative size");
    if (a.M == 0 || a.N == 0) return 0;
    if (a.K == 0) return fail(DSV4_ERR_ARG, "w8a8_gemm: K must be positive");
    if (a.A == nullptr || a.B == nullptr || (a.C == nullptr && a.row_ptr == nullptr))
        return fail(DSV4_ERR_ARG, "w8a8_gemm: null pointer");
    if (a.row_ptr != nullptr && (!grouped || a.sa_groups != 1 || a.out_i32 || a.npeers != 0))
        return fail(DSV4_ERR_ARG, "grouped_gemm_scatter: row destinations exist only for the grouped GEMM with per-token scales");
    if (!a.out_i32 && (a.sa == nullptr || a.sb == nullptr)) return fail(DSV4_ERR_ARG, "w8a8_gemm: null scale pointer");
    if (a.K % 16 != 0) return fail(DSV4_ERR_ARG, "w8a8_gemm: K must be a multiple of 16 (TMA row stride)");
    if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15))
        return fail(DSV4_ERR_ARG, "w8a8_gemm: A and B must be 16-byte aligned");
    if (grouped && (a.E <= 0 || a.E > kMaxExperts)) return fail(DSV4_ERR_ARG, "grouped_gemm: E must be in 1..1024");
    if (a.sa_groups != 1) {
        if (!grouped) return fail(DSV4_ERR_ARG, "w8a8_gemm: group scales exist only for the grouped GEMM");
        if (a.out_i32) return fail(DSV4_ERR_ARG, "w8a8_gemm: raw accumulators exist only for per-token scaling");
        if (a.K % 128 != 0 || a.sa_groups != a.K / 128)
            return fail(DSV4_ERR_ARG, "grouped_gemm: group scales need K % 128 == 0 and sa_groups == K / 128");
    }

    // a kernel launched earlier on this device gave up a bounded wait: say so once instead of launching
    if (volatile int* mirror = host_status_mirror()) {
        const int site = *mirror;
        if (site != 0) {
            *mirror = 0;
            static thread_local char msg[160];
            snprintf(msg, sizeof msg, "w8a8_gemm: an earlier kernel on this device gave up a bounded wait (site %d); "
                     "nothing was launched; dsv4_device_status reads and clears the device's word", site);
            return fail(DSV4_ERR_DEVICE_WAIT, msg);
        }
    }

    Params p;
    p.wait_limit_ns = a.test_wait_limit_ns ? a.test_wait_limit_ns : ptx::kWaitLimitNs;
    p.withhold_loads = a.test_withhold_loads;
    p.sa = a.sa; p.sb = a.sb; p.C = a.C; p.offsets = a.offsets;
    p.masked_m = a.masked_m; p.max_m = a.max_m;
    p.row_ptr = a.row_ptr;
    p.M = a.M; p.N = a.N; p.K = a.K; p.E = grouped ? a.E : 1;
    p.ldc = a.ldc > 0 ? a.ldc : a.N;
    p.sa_groups = a.sa_groups; p.out_i32 = a.out_i32;
    if (p.ldc < a.N) return fail(DSV4_ERR_ARG, "w8a8_gemm: ldc smaller than N");
    {
        // groups of m-tiles whose rows of A (256 x K bytes each) take at most 32 MB, all about equally large
        const int tiles_m = (a.M + 255) / 256;
        const int64_t tile_bytes = (int64_t)256 * a.K;
        int gm_max = (int)((int64_t)32 * 1024 * 1024 / (tile_bytes > 0 ? tile_bytes : 1));
        if (gm_max < 1) gm_max = 1;
        const int groups = (tiles_m + gm_max - 1) / gm_max;
        p.pair_group_m = groups > 0 ? (tiles_m + groups - 1) / groups : 1;
        if (p.pair_group_m < 1) p.pair_group_m = 1;
    }
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
    const int tiles_m_bound = (a.M + BM - 1) / BM;

    // Tile width: 256 columns when that already gives every SM a tile, otherwise narrower
    // tiles so that a short, weight-streaming problem spreads over more SMs.
    int bn = 256;
    if ((int64_t)tiles_m_bound * ((a.N + 255) / 256) < sms) bn = 128;
    if (bn == 128 && (int64_t)tiles_m_bound * ((a.N + 127) / 128) < sms) bn = 64;
    if (bn == 64 && (int64_t)tiles_m_bound * ((a.N + 63) / 64) < sms) bn = 32;

    CUtensorMap tmA, tmB;
    if (grouped) {
        if (a.masked_m != nullptr && (a.offsets != nullptr || a.max_m <= 0 || (int64_t)a.E * a.max_m != a.M))
            return fail(DSV4_ERR_ARG, "grouped_gemm_masked: needs max_m > 0, M == E * max_m and no expert_offsets");
        if (a.out_i32) return fail(DSV4_ERR_ARG, "grouped_gemm: raw accumulators exist only for the dense GEMM");
        int rcw = make_tile_map(&tmB, a.B, b_rows, (uint64_t)a.K, 128);
        if (rcw) return rcw;
        WtMaps xmaps;
        for (int i = 0; i < kWtMaps; ++i) {
            rcw = make_tile_map(&xmaps.x[i], a.A, (uint64_t)a.M, (uint64_t)a.K, (uint32_t)(16 * (i + 1)));
            if (rcw) return rcw;
        }
        // Per-token scales: with a short K (the MoE down projection: 16 K blocks per item) the item's tile leaves
        // through shared memory in 256-byte row segments, which beats the sixth pipeline stage that the staging
        // tile displaces (0.72 against 0.79 ms on 256 experts of 128 rows, N = 7168, K = 2048); with a long K the
        // deeper pipeline wins (338 against 331 us on 64 experts, N = 4096, K = 7168).  Row destinations always
        // take the staged form.
        const bool short_k = (a.K + BK - 1) / BK <= 32 && p.ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(a.C) & 15) == 0;
        if (a.sa_groups == 1 && (a.row_ptr != nullptr || short_k)) return launch_wt_variant<false, true>(tmB, xmaps, p, st);
        return a.sa_groups != 1 ? launch_wt_variant<true>(tmB, xmaps, p, st) : launch_wt_variant<false>(tmB, xmaps, p, st);
    }
    // Few tokens: stream the weight once, tokens on the MMA's N axis, K split over a cluster
    if (a.M <= 256 && a.npeers == 0) {
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
    if (a.M > 128 && (int64_t)((a.M + 255) / 256) * ((a.N + 255) / 256) >= sms / 4) {
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
        if (volatile int* mirror = host_status_mirror()) *mirror = 0;
    }
    if (v == 0) {
        const int rc = read_row_status(&v);
        if (rc) return rc;
    }
    if (out) *out = v;
    return 0;
}

}  // namespace w8a8
