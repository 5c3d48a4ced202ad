// Expert segments for the MoE grouped GEMM, computed on the device from top-k routing
// ids: a stable counting sort by expert, written without atomics and without scratch
// memory so that the row order inside an expert is reproducible (increasing (token, slot)).
//
//   count   : CTA e counts the pairs routed to expert e        -> offsets[e+1] = count
//   scan    : one warp turns the counts into exclusive offsets -> offsets[0..E]
//   scatter : CTA e walks the id list again and numbers its pairs in order
//             -> src_row[offset_e + rank] = token, dst_slot[pair] = offset_e + rank
//
// The id list (T*topk int32, 128 KB at 4096 tokens x 8) stays in L2 across the E CTAs.
#include <cuda_runtime.h>
#include <cstdint>

#include "launch_common.h"

namespace w8a8 {
namespace {

constexpr int kSegThreads = 256;

__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    return v;
}

__global__ void __launch_bounds__(kSegThreads) seg_count_kernel(const int* __restrict__ ids, int R,
                                                                int* __restrict__ offsets) {
    __shared__ int red[kSegThreads / 32];
    const int e = blockIdx.x;
    int c = 0;
    for (int i = threadIdx.x; i < R; i += kSegThreads) c += (__ldg(ids + i) == e);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < kSegThreads / 32; ++w) t += red[w];
        offsets[e + 1] = t;
    }
}

__global__ void __launch_bounds__(32) seg_scan_kernel(int* __restrict__ offsets, int E) {
    const int lane = threadIdx.x;
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
        const int e = e0 + lane;
        const int cnt = (e < E) ? offsets[e + 1] : 0;
        const int incl = warp_incl_scan(cnt, lane);
        __syncwarp();
        if (e < E) offsets[e + 1] = carry + incl;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) offsets[0] = 0;
}

__global__ void __launch_bounds__(kSegThreads) seg_scatter_kernel(const int* __restrict__ ids, int R,
                                                                  int topk,
                                                                  const int* __restrict__ offsets,
                                                                  int* __restrict__ src_row,
                                                                  int* __restrict__ dst_slot) {
    __shared__ int warp_tot[kSegThreads / 32];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int base = offsets[e];
    for (int i0 = 0; i0 < R; i0 += kSegThreads) {
        const int i = i0 + threadIdx.x;
        const bool hit = (i < R) && (__ldg(ids + i) == e);
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        const int before = __popc(m & ((1u << lane) - 1u));
        if (lane == 0) warp_tot[warp] = __popc(m);
        __syncthreads();
        int wbase = 0, total = 0;
#pragma unroll
        for (int w = 0; w < kSegThreads / 32; ++w) {
            const int c = warp_tot[w];
            if (w < warp) wbase += c;
            total += c;
        }
        if (hit) {
            const int r = base + wbase + before;
            src_row[r] = i / topk;
            dst_slot[i] = r;
        }
        base += total;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(128) gather_rows_kernel(const uint4* __restrict__ src,
                                                          const int* __restrict__ src_row,
                                                          uint4* __restrict__ dst, int R, int vec_per_row,
                                                          const float* __restrict__ src_scale,
                                                          float* __restrict__ dst_scale, int spr) {
    for (int r = blockIdx.x; r < R; r += gridDim.x) {
        const int t = __ldg(src_row + r);
        const uint4* s = src + (int64_t)t * vec_per_row;
        uint4* d = dst + (int64_t)r * vec_per_row;
        for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) d[i] = __ldg(s + i);
        if (src_scale != nullptr)
            for (int i = threadIdx.x; i < spr; i += blockDim.x)
                dst_scale[(int64_t)r * spr + i] = __ldg(src_scale + (int64_t)t * spr + i);
    }
}

}  // namespace

int moe_segments(const int* topk_ids, int T, int topk, int E, int* offsets, int* src_row, int* dst_slot,
                 cudaStream_t st) {
    if (T < 0 || topk <= 0 || E <= 0) return fail(DSV4_ERR_ARG, "moe_segments: bad sizes");
    if (topk_ids == nullptr || offsets == nullptr || src_row == nullptr || dst_slot == nullptr)
        return fail(DSV4_ERR_ARG, "moe_segments: null pointer");
    const int64_t R64 = (int64_t)T * topk;
    if (R64 > INT32_MAX) return fail(DSV4_ERR_ARG, "moe_segments: T*topk exceeds int32");
    const int R = (int)R64;
    seg_count_kernel<<<E, kSegThreads, 0, st>>>(topk_ids, R, offsets);
    seg_scan_kernel<<<1, 32, 0, st>>>(offsets, E);
    seg_scatter_kernel<<<E, kSegThreads, 0, st>>>(topk_ids, R, topk, offsets, src_row, dst_slot);
    return check_launch("moe_segments");
}

int gather_rows(const void* src, const int* src_row, void* dst, int R, int row_bytes, const float* src_scale,
                float* dst_scale, int scales_per_row, cudaStream_t st) {
    if (R == 0) return 0;
    if (R < 0 || row_bytes <= 0 || row_bytes % 16 != 0) return fail(DSV4_ERR_ARG, "gather_rows: row_bytes must be a positive multiple of 16");
    if (src == nullptr || dst == nullptr || src_row == nullptr) return fail(DSV4_ERR_ARG, "gather_rows: null pointer");
    if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
        return fail(DSV4_ERR_ARG, "gather_rows: src and dst must be 16-byte aligned");
    gather_rows_kernel<<<R, 128, 0, st>>>(static_cast<const uint4*>(src), src_row, static_cast<uint4*>(dst), R,
                                          row_bytes / 16, src_scale, dst_scale, scales_per_row);
    return check_launch("gather_rows");
}

}  // namespace w8a8
