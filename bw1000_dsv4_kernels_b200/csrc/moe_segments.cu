// Expert segments for the MoE grouped GEMM, computed on the device from top-k routing
// ids: a stable counting sort by expert, written without atomics and without scratch
// memory so that the row order inside an expert is reproducible (increasing (token, slot)).
// Two forms with identical results: a chunked one for R >= 1024 routed pairs (below), and the
// per-expert one described next for small inputs.
// With expert_lo > 0 only experts [expert_lo, expert_lo + E) are sorted (expert parallelism);
// pairs routed elsewhere get slot -1.
//
//   count   : CTA e counts the pairs routed to expert e        -> offsets[e+1] = count
//   scan    : one warp turns the counts into exclusive offsets -> offsets[0..E]
//   scatter : CTA e walks the id list again and numbers its pairs in order
//             -> src_row[offset_e + rank] = token, dst_slot[pair] = offset_e + rank
//
// The id list (T*topk int32, 128 KB at 4096 tokens x 8) stays in L2 across the E CTAs.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
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
                                                                int expert_lo, int* __restrict__ offsets,
                                                                int* __restrict__ dst_slot) {
    __shared__ int red[kSegThreads / 32];
    const int e = blockIdx.x + expert_lo;
    // pairs routed to experts outside [expert_lo, expert_lo + E) keep slot -1
    for (int i = blockIdx.x * kSegThreads + threadIdx.x; i < R; i += gridDim.x * kSegThreads) dst_slot[i] = -1;
    int c = 0;
    for (int i = threadIdx.x; i < R; i += kSegThreads) c += (__ldg(ids + i) == e);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < kSegThreads / 32; ++w) t += red[w];
        offsets[blockIdx.x + 1] = t;
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
                                                                  int topk, int expert_lo,
                                                                  const int* __restrict__ offsets,
                                                                  int* __restrict__ src_row,
                                                                  int* __restrict__ dst_slot) {
    __shared__ int warp_tot[kSegThreads / 32];
    const int e = blockIdx.x + expert_lo;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int base = offsets[blockIdx.x];
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


// ---- chunked form (R >= 1024 pairs, E <= 1024): one warp per chunk -------------------------
// The chunk length is 256 pairs for up to 64 experts (short serial loops in the scatter), 512 up to 512
// experts, else 1024.
// count   : warp b builds the histogram of its chunk in shared memory and parks it in the
//           chunk's own stretch of dst_slot (dst_slot[chunk_begin + e], e < E <= chunk length)
// scan    : one warp (few experts) or one thread (many) per expert turns the per-chunk counts of
//           the expert into running bases (in place) and the totals into exclusive expert offsets
// scatter : warp b reads its bases (before it overwrites that stretch), then numbers its pairs
//           group of 32 by group of 32 in order, so rows stay sorted by (token, slot)
// Only a chunk's own warp ever writes its stretch of dst_slot, so the parked counts cannot be
// clobbered by another chunk; nothing outside the outputs is touched.
constexpr int kChunk = 1024;   // longest chunk; the form needs R >= kChunk

__device__ __forceinline__ void chunk_bounds(int b, int nchunks, int chunk, int R, int& lo, int& hi) {
    lo = b * chunk;
    hi = (b == nchunks - 1) ? R : lo + chunk;  // the last chunk takes the remainder as well
}

// The chunk's expert ids (rebased to the local expert range) go to shared memory first: the loads
// are independent and issued back to back, where a load inside the match loop would expose a full
// memory round trip in each of its iterations.  A chunk has fewer than 2 * kChunk pairs.
__device__ __forceinline__ void stage_chunk_ids(const int* __restrict__ ids, int lo, int hi, int expert_lo, int* sid,
                                                int lane) {
#pragma unroll 8
    for (int i = lo + lane; i < hi; i += 32) sid[i - lo] = __ldg(ids + i) - expert_lo;
}

__global__ void __launch_bounds__(32) seg_chunk_count_kernel(const int* __restrict__ ids, int R, int E, int chunk,
                                                             int expert_lo, int* __restrict__ dst_slot) {
    __shared__ int hist[1024];
    const int lane = threadIdx.x;
    int lo, hi;
    chunk_bounds(blockIdx.x, gridDim.x, chunk, R, lo, hi);
    for (int e = lane; e < E; e += 32) hist[e] = 0;
    __syncwarp();
    // counting needs no order: shared-memory atomics, every lane on its own pairs
#pragma unroll 8
    for (int i = lo + lane; i < hi; i += 32) {
        const int e = __ldg(ids + i) - expert_lo;
        if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) dst_slot[lo + e] = hist[e];
}

__global__ void __launch_bounds__(1024) seg_chunk_scan_kernel(int* __restrict__ dst_slot, int nchunks, int chunk, int E,
                                                              int* __restrict__ offsets) {
    __shared__ int totals[1024];
    __shared__ int warp_sums[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    totals[tid] = 0;
    __syncthreads();
    // warp w: experts w, w + 32, ...; lane = chunk (32 chunks per round, carried over the rounds)
    for (int e = warp; e < E; e += 32) {
        int run = 0;
        // four rounds of 32 chunks per batch: the loads of a batch are independent of the running sum
        for (int b0 = 0; b0 < nchunks; b0 += 128) {
            int c[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int b = b0 + 32 * j + lane;
                c[j] = b < nchunks ? dst_slot[(int64_t)b * chunk + e] : 0;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int b = b0 + 32 * j + lane;
                const int incl = warp_incl_scan(c[j], lane);
                if (b < nchunks) dst_slot[(int64_t)b * chunk + e] = run + incl - c[j];  // rows of expert e from earlier chunks
                run += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        if (lane == 0) totals[e] = run;
    }
    __syncthreads();
    // exclusive scan of the totals over the experts
    const int e = tid;
    int incl = warp_incl_scan(totals[e], lane);
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int ws = warp_sums[lane];
        const int wi = warp_incl_scan(ws, lane);
        warp_sums[lane] = wi - ws;
    }
    __syncthreads();
    const int excl = warp_sums[warp] + incl - totals[e];
    if (e < E) offsets[e] = excl;
    if (e == E - 1) offsets[E] = excl + totals[e];
}

// The same scan with one THREAD per expert (consecutive experts = consecutive addresses), for many
// experts: eight chunks at a time, the loads of a batch are independent of the running sum.
__global__ void __launch_bounds__(1024) seg_chunk_scan_wide_kernel(int* __restrict__ dst_slot, int nchunks, int chunk,
                                                                   int E, int* __restrict__ offsets) {
    __shared__ int totals[1024];
    __shared__ int warp_sums[32];
    const int e = threadIdx.x;
    int run = 0;
    if (e < E) {
        for (int b0 = 0; b0 < nchunks; b0 += 8) {
            int c[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) c[j] = (b0 + j < nchunks) ? dst_slot[(int64_t)(b0 + j) * chunk + e] : 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (b0 + j < nchunks) dst_slot[(int64_t)(b0 + j) * chunk + e] = run;
                run += c[j];
            }
        }
    }
    totals[e] = (e < E) ? run : 0;
    const int lane = e & 31, warp = e >> 5;
    int incl = warp_incl_scan(totals[e], lane);
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int ws = warp_sums[lane];
        const int wi = warp_incl_scan(ws, lane);
        warp_sums[lane] = wi - ws;
    }
    __syncthreads();
    const int excl = warp_sums[warp] + incl - totals[e];
    if (e < E) offsets[e] = excl;
    if (e == E - 1) offsets[E] = excl + totals[e];
}

__global__ void __launch_bounds__(32) seg_chunk_scatter_kernel(const int* __restrict__ ids, int R, int topk, int E,
                                                               int chunk, int expert_lo, const int* __restrict__ offsets,
                                                               int* __restrict__ src_row, int* __restrict__ dst_slot) {
    __shared__ int base[1024];
    __shared__ int sid[2 * kChunk];
    const int lane = threadIdx.x;
    int lo, hi;
    chunk_bounds(blockIdx.x, gridDim.x, chunk, R, lo, hi);
    for (int e = lane; e < E; e += 32) base[e] = offsets[e] + dst_slot[lo + e];
    stage_chunk_ids(ids, lo, hi, expert_lo, sid, lane);
    __syncwarp();
    for (int i0 = lo; i0 < hi; i0 += 32) {
        const int i = i0 + lane;
        const int e = (i < hi) ? sid[i - lo] : -1;
        const bool in = e >= 0 && e < E;
        const unsigned act = __ballot_sync(0xffffffffu, in);
        if (in) {
            const unsigned m = __match_any_sync(act, e);
            const int r = base[e] + __popc(m & ((1u << lane) - 1u));
            src_row[r] = i / topk;
            dst_slot[i] = r;
            __syncwarp(m);
            if (lane == __ffs(m) - 1) base[e] += __popc(m);
        } else if (i < hi) {
            dst_slot[i] = -1;
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(128) gather_rows_kernel(const uint4* __restrict__ src,
                                                          const int* __restrict__ src_row,
                                                          uint4* __restrict__ dst, int R, int vec_per_row,
                                                          const float* __restrict__ src_scale,
                                                          float* __restrict__ dst_scale, int spr,
                                                          const int* __restrict__ valid_rows) {
    if (valid_rows != nullptr) R = min(R, __ldg(valid_rows));
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

// out[t, :] = sum over the token's top-k slots j (in order) of w[t,j] * Z[dst_slot[t,j], :],
// accumulated in fp32 with fma; slots equal to -1 (expert not on this rank) are skipped.
template <bool OUT_F32>
__global__ void __launch_bounds__(128) moe_combine_kernel(const __nv_bfloat16* __restrict__ z,
                                                          const int* __restrict__ dst_slot,
                                                          const float* __restrict__ w, void* __restrict__ out, int T,
                                                          int topk, int H) {
    constexpr int kBatch = 8;                   // expert rows in flight per thread
    __shared__ const uint4* rowp[kBatch];
    __shared__ float wk[kBatch];
    const int V = H >> 3;
    const bool one_batch = topk <= kBatch;      // the usual case: the row pointers are set up once per token
    auto load_rows = [&](int t, int j0) {
        if (threadIdx.x < kBatch) {
            const int j = j0 + threadIdx.x;
            const uint4* ptr = nullptr;
            float wj = 0.0f;
            if (j < topk) {
                const int slot = __ldg(dst_slot + (int64_t)t * topk + j);
                wj = __ldg(w + (int64_t)t * topk + j);
                if (slot >= 0) ptr = reinterpret_cast<const uint4*>(z + (int64_t)slot * H);
            }
            rowp[threadIdx.x] = ptr;
            wk[threadIdx.x] = wj;
        }
    };
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        if (one_batch) {
            load_rows(t, 0);
            __syncthreads();
        }
        for (int vb = 0; vb < V; vb += 2 * 128) {
            float acc[2][8];                    // up to two 16-byte vectors per thread and pass
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i][e] = 0.0f;
            for (int j0 = 0; j0 < topk; j0 += kBatch) {
                if (!one_batch) {
                    __syncthreads();            // the previous batch's pointers have been used
                    load_rows(t, j0);
                    __syncthreads();
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int v = vb + i * 128 + threadIdx.x;
                    if (v >= V) break;
                    uint4 zv[kBatch];
#pragma unroll
                    for (int j = 0; j < kBatch; ++j)
                        zv[j] = rowp[j] != nullptr ? __ldg(rowp[j] + v) : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int j = 0; j < kBatch; ++j) {
                        if (rowp[j] == nullptr) continue;   // a skipped slot adds nothing, not even +0
                        const float wj = wk[j];
                        const uint32_t zw[4] = {zv[j].x, zv[j].y, zv[j].z, zv[j].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            acc[i][2 * e] = __fmaf_rn(wj, __uint_as_float(zw[e] << 16), acc[i][2 * e]);
                            acc[i][2 * e + 1] = __fmaf_rn(wj, __uint_as_float(zw[e] & 0xffff0000u), acc[i][2 * e + 1]);
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int v = vb + i * 128 + threadIdx.x;
                if (v >= V) break;
                if (OUT_F32) {
                    float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + (int64_t)t * H) + 2 * v;
                    o[0] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                    o[1] = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
                } else {
                    __nv_bfloat162 b[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) b[e] = __floats2bfloat162_rn(acc[i][2 * e], acc[i][2 * e + 1]);
                    reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + (int64_t)t * H)[v] =
                        *reinterpret_cast<uint4*>(b);
                }
            }
        }
        __syncthreads();
    }
}

// Expert-parallel combine fused with its exchange.  Every rank holds the outputs of its own experts
// (z, rows in its own segment order) and its own dst_slot map; all ranks' buffers are mapped into
// this GPU's address space.  The rank that owns token t pulls the token's top-k expert rows from
// whichever ranks hold them (peer loads), sums them in slot order with the same fp32 fma sequence as
// moe_combine -- so the result has the single-GPU bits -- and pushes the bf16 row into every rank's
// output (peer stores).  Per rank about T/G * topk rows come in and T/G * (G-1) rows go out, against
// an all-reduce of fp32 [T,H] partials.
constexpr int kMaxRanks = 8;
struct ExchangeArgs {
    const __nv_bfloat16* z[kMaxRanks];
    const int* slot[kMaxRanks];
    __nv_bfloat16* out[kMaxRanks];
};

__global__ void __launch_bounds__(128) moe_combine_exchange_kernel(ExchangeArgs a, const int* __restrict__ ids,
                                                                   const float* __restrict__ w, int G,
                                                                   int experts_per_rank, int t0, int t1, int topk,
                                                                   int H) {
    constexpr int kBatch = 8;                   // expert rows in flight per thread
    __shared__ const uint4* rowp[kBatch];
    __shared__ float wk[kBatch];
    const int V = H >> 3;
    const bool one_batch = topk <= kBatch;      // the usual case: the row pointers are set up once per token
    // expert id -> owning rank -> that rank's slot for this (token, j) -> address of the expert row
    auto load_rows = [&](int t, int j0) {
        if (threadIdx.x < kBatch) {
            const int j = j0 + threadIdx.x;
            const uint4* ptr = nullptr;
            float wj = 0.0f;
            if (j < topk) {
                const int64_t pair = (int64_t)t * topk + j;
                const int e = __ldg(ids + pair);
                const int rank = e >= 0 ? e / experts_per_rank : G;
                wj = __ldg(w + pair);
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r) {
                    if (r == rank && r < G) {
                        const int slot = a.slot[r][pair];
                        if (slot >= 0) ptr = reinterpret_cast<const uint4*>(a.z[r] + (int64_t)slot * H);
                    }
                }
            }
            rowp[threadIdx.x] = ptr;
            wk[threadIdx.x] = wj;
        }
    };
    for (int t = t0 + blockIdx.x; t < t1; t += gridDim.x) {
        float acc[4][8];                        // up to four 16-byte vectors per thread and pass
        if (one_batch) {
            load_rows(t, 0);
            __syncthreads();
        }
        for (int vb = 0; vb < V; vb += 4 * 128) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i][e] = 0.0f;
            for (int j0 = 0; j0 < topk; j0 += kBatch) {
                if (!one_batch) {
                    __syncthreads();            // the previous batch's pointers have been used
                    load_rows(t, j0);
                    __syncthreads();
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int v = vb + i * 128 + threadIdx.x;
                    if (v >= V) break;
                    uint4 zv[kBatch];
#pragma unroll
                    for (int j = 0; j < kBatch; ++j)
                        zv[j] = rowp[j] != nullptr ? rowp[j][v] : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int j = 0; j < kBatch; ++j) {
                        if (rowp[j] == nullptr) continue;   // a skipped slot adds nothing, not even +0
                        const float wj = wk[j];
                        const uint32_t zw[4] = {zv[j].x, zv[j].y, zv[j].z, zv[j].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            acc[i][2 * e] = __fmaf_rn(wj, __uint_as_float(zw[e] << 16), acc[i][2 * e]);
                            acc[i][2 * e + 1] = __fmaf_rn(wj, __uint_as_float(zw[e] & 0xffff0000u), acc[i][2 * e + 1]);
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int v = vb + i * 128 + threadIdx.x;
                if (v >= V) break;
                __nv_bfloat162 b[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) b[e] = __floats2bfloat162_rn(acc[i][2 * e], acc[i][2 * e + 1]);
                const uint4 packed = *reinterpret_cast<uint4*>(b);
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r)
                    if (r < G) reinterpret_cast<uint4*>(a.out[r] + (int64_t)t * H)[v] = packed;
            }
        }
        __syncthreads();
    }
}

// Router top-k: one warp per token.  Lane l holds logits l, l+32, ...; k rounds of a warp-wide
// arg-max (larger value wins, ties go to the lower expert index) pick the experts in descending
// order; the weights are the softmax over the k selected logits (exp computed in fp32 with the
// selected maximum subtracted, the engine's "renormalised top-k softmax").
template <int MAX_PER_LANE>
__global__ void __launch_bounds__(256) moe_topk_kernel(const float* __restrict__ logits, int T, int E, int k,
                                                       int* __restrict__ ids, float* __restrict__ weights) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
        const float* row = logits + (int64_t)t * E;
        float v[MAX_PER_LANE];
#pragma unroll
        for (int j = 0; j < MAX_PER_LANE; ++j) {
            const int e = lane + 32 * j;
            v[j] = (e < E) ? __ldg(row + e) : -INFINITY;
        }
        float first = 0.0f, denom = 0.0f, mine = 0.0f;
        for (int r = 0; r < k; ++r) {
            float best = -INFINITY;
            int best_e = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < MAX_PER_LANE; ++j) {
                const int e = lane + 32 * j;
                if (v[j] > best) { best = v[j]; best_e = e; }   // ascending e: the first maximum of the lane
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
                if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
            }
            if (r == 0) first = best;
            const float w = expf(best - first);
            denom += w;
            if (lane == r) mine = w;            // lane r keeps the r-th weight (k <= 32)
            if (lane == 0) ids[(int64_t)t * k + r] = best_e;
#pragma unroll
            for (int j = 0; j < MAX_PER_LANE; ++j)
                if (lane + 32 * j == best_e) v[j] = -INFINITY;
        }
        if (lane < k) weights[(int64_t)t * k + lane] = mine / denom;
    }
}

}  // namespace

int moe_topk(const float* logits, int T, int E, int k, int* ids, float* weights, cudaStream_t st) {
    if (T == 0) return 0;
    if (T < 0 || E <= 0 || k <= 0 || k > 32 || k > E || E > 1024)
        return fail(DSV4_ERR_ARG, "moe_topk: need 1 <= k <= min(32, E) and E <= 1024");
    if (logits == nullptr || ids == nullptr || weights == nullptr) return fail(DSV4_ERR_ARG, "moe_topk: null pointer");
    const int blocks = (T + 7) / 8;
    if (E <= 256)
        moe_topk_kernel<8><<<blocks, 256, 0, st>>>(logits, T, E, k, ids, weights);
    else
        moe_topk_kernel<32><<<blocks, 256, 0, st>>>(logits, T, E, k, ids, weights);
    return check_launch("moe_topk");
}

int moe_combine(const void* z, const int* dst_slot, const float* w, void* out, int T, int topk, int H, int out_f32,
                cudaStream_t st) {
    if (T == 0 || H == 0) return 0;
    if (T < 0 || topk <= 0 || H < 0 || H % 8 != 0) return fail(DSV4_ERR_ARG, "moe_combine: H must be a multiple of 8");
    if (z == nullptr || dst_slot == nullptr || w == nullptr || out == nullptr) return fail(DSV4_ERR_ARG, "moe_combine: null pointer");
    if ((reinterpret_cast<uintptr_t>(z) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return fail(DSV4_ERR_ARG, "moe_combine: z and out must be 16-byte aligned");
    if (out_f32)
        moe_combine_kernel<true><<<T, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(z), dst_slot, w, out, T, topk, H);
    else
        moe_combine_kernel<false><<<T, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(z), dst_slot, w, out, T, topk, H);
    return check_launch("moe_combine");
}

int moe_combine_exchange(const void* const* z_ranks, const int* const* slot_ranks, const int* topk_ids,
                         const float* topk_w, void* const* out_ranks, int G, int experts_per_rank, int t0, int t1,
                         int topk, int H, cudaStream_t st) {
    if (t1 <= t0 || H == 0) return 0;
    if (G < 1 || G > kMaxRanks) return fail(DSV4_ERR_ARG, "moe_combine_exchange: 1 to 8 ranks");
    if (t0 < 0 || topk <= 0 || experts_per_rank <= 0 || H < 0 || H % 8 != 0)
        return fail(DSV4_ERR_ARG, "moe_combine_exchange: bad sizes (H must be a multiple of 8)");
    if (z_ranks == nullptr || slot_ranks == nullptr || out_ranks == nullptr || topk_ids == nullptr || topk_w == nullptr)
        return fail(DSV4_ERR_ARG, "moe_combine_exchange: null pointer");
    ExchangeArgs a = {};
    for (int r = 0; r < G; ++r) {
        if (z_ranks[r] == nullptr || slot_ranks[r] == nullptr || out_ranks[r] == nullptr)
            return fail(DSV4_ERR_ARG, "moe_combine_exchange: null rank pointer");
        if ((reinterpret_cast<uintptr_t>(z_ranks[r]) & 15) || (reinterpret_cast<uintptr_t>(out_ranks[r]) & 15))
            return fail(DSV4_ERR_ARG, "moe_combine_exchange: z and out must be 16-byte aligned");
        a.z[r] = static_cast<const __nv_bfloat16*>(z_ranks[r]);
        a.slot[r] = slot_ranks[r];
        a.out[r] = static_cast<__nv_bfloat16*>(out_ranks[r]);
    }
    moe_combine_exchange_kernel<<<t1 - t0, 128, 0, st>>>(a, topk_ids, topk_w, G, experts_per_rank, t0, t1, topk, H);
    return check_launch("moe_combine_exchange");
}

// Where each of this rank's expert output rows has to go when the down GEMM itself delivers them (push
// instead of the owners' pull): the (token, slot) pair that sits in segment row r = dst_slot[pair] belongs to
// the rank that owns the token, rank = token / tokens_per_rank, and lands in that rank's inbox at row
// (token - rank * tokens_per_rank) * topk + slot.
struct InboxArgs {
    __nv_bfloat16* inbox[kMaxRanks];
};
__global__ void __launch_bounds__(256) moe_push_rows_kernel(InboxArgs a, const int* __restrict__ dst_slot, int pairs,
                                                            int topk, int tokens_per_rank, int G, int H,
                                                            void** __restrict__ row_ptr) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pairs) return;
    const int r = dst_slot[i];
    if (r < 0) return;
    const int t = i / topk, j = i - t * topk;
    int rank = t / tokens_per_rank;
    if (rank >= G) rank = G - 1;
    __nv_bfloat16* base = a.inbox[0];
#pragma unroll
    for (int g = 1; g < kMaxRanks; ++g)
        if (g == rank) base = a.inbox[g];
    row_ptr[r] = base + ((int64_t)(t - rank * tokens_per_rank) * topk + j) * H;
}

int moe_push_rows(const int* dst_slot, int T, int topk, int tokens_per_rank, void* const* inbox_ranks, int G, int H,
                  void** row_ptr, cudaStream_t st) {
    if (T == 0) return 0;
    if (G < 1 || G > kMaxRanks) return fail(DSV4_ERR_ARG, "moe_push_rows: 1 to 8 ranks");
    if (T < 0 || topk <= 0 || tokens_per_rank <= 0 || H <= 0 || (int64_t)T * topk > INT32_MAX)
        return fail(DSV4_ERR_ARG, "moe_push_rows: bad sizes");
    if ((int64_t)tokens_per_rank * G < T) return fail(DSV4_ERR_ARG, "moe_push_rows: tokens_per_rank * ranks < T");
    if (dst_slot == nullptr || inbox_ranks == nullptr || row_ptr == nullptr)
        return fail(DSV4_ERR_ARG, "moe_push_rows: null pointer");
    InboxArgs a = {};
    for (int g = 0; g < G; ++g) {
        if (inbox_ranks[g] == nullptr) return fail(DSV4_ERR_ARG, "moe_push_rows: null rank pointer");
        a.inbox[g] = static_cast<__nv_bfloat16*>(inbox_ranks[g]);
    }
    const int pairs = T * topk;
    moe_push_rows_kernel<<<(pairs + 255) / 256, 256, 0, st>>>(a, dst_slot, pairs, topk, tokens_per_rank, G, H, row_ptr);
    return check_launch("moe_push_rows");
}

int moe_segments(const int* topk_ids, int T, int topk, int E, int expert_lo, int* offsets, int* src_row,
                 int* dst_slot, cudaStream_t st) {
    if (T < 0 || topk <= 0 || E <= 0) return fail(DSV4_ERR_ARG, "moe_segments: bad sizes");
    if (topk_ids == nullptr || offsets == nullptr || src_row == nullptr || dst_slot == nullptr)
        return fail(DSV4_ERR_ARG, "moe_segments: null pointer");
    const int64_t R64 = (int64_t)T * topk;
    if (R64 > INT32_MAX) return fail(DSV4_ERR_ARG, "moe_segments: T*topk exceeds int32");
    const int R = (int)R64;
    if (R >= kChunk && E <= 1024) {
        // few experts (an expert-parallel rank): short chunks, one warp per expert in the scan; many
        // experts: long chunks, one thread per expert
        const bool few = E <= 64;
        const int chunk = few ? 256 : (E <= 512 ? 512 : kChunk);   // a chunk parks E counts in its own stretch: E <= chunk
        const int nchunks = R / chunk;
        seg_chunk_count_kernel<<<nchunks, 32, 0, st>>>(topk_ids, R, E, chunk, expert_lo, dst_slot);
        if (few)
            seg_chunk_scan_kernel<<<1, 1024, 0, st>>>(dst_slot, nchunks, chunk, E, offsets);
        else
            seg_chunk_scan_wide_kernel<<<1, 1024, 0, st>>>(dst_slot, nchunks, chunk, E, offsets);
        seg_chunk_scatter_kernel<<<nchunks, 32, 0, st>>>(topk_ids, R, topk, E, chunk, expert_lo, offsets, src_row,
                                                         dst_slot);
        return check_launch("moe_segments");
    }
    seg_count_kernel<<<E, kSegThreads, 0, st>>>(topk_ids, R, expert_lo, offsets, dst_slot);
    seg_scan_kernel<<<1, 32, 0, st>>>(offsets, E);
    seg_scatter_kernel<<<E, kSegThreads, 0, st>>>(topk_ids, R, topk, expert_lo, offsets, src_row, dst_slot);
    return check_launch("moe_segments");
}

int gather_rows(const void* src, const int* src_row, void* dst, int R, int row_bytes, const float* src_scale,
                float* dst_scale, int scales_per_row, const int* valid_rows, cudaStream_t st) {
    if (R == 0) return 0;
    if (R < 0 || row_bytes <= 0 || row_bytes % 16 != 0) return fail(DSV4_ERR_ARG, "gather_rows: row_bytes must be a positive multiple of 16");
    if (src == nullptr || dst == nullptr || src_row == nullptr) return fail(DSV4_ERR_ARG, "gather_rows: null pointer");
    if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
        return fail(DSV4_ERR_ARG, "gather_rows: src and dst must be 16-byte aligned");
    // With a device-side row count most of the R CTAs would find nothing to do; a grid of a few CTAs
    // per SM walks the rows instead.
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (sms > 0 && R > 16 * sms) ? 16 * sms : R;
    gather_rows_kernel<<<grid, 128, 0, st>>>(static_cast<const uint4*>(src), src_row, static_cast<uint4*>(dst), R,
                                          row_bytes / 16, src_scale, dst_scale, scales_per_row, valid_rows);
    return check_launch("gather_rows");
}

}  // namespace w8a8
