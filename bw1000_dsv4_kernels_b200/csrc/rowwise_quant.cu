// Row-wise activation kernels of the W8A8 path: per-token and per-group int8
// quantisers, residual-add + RMSNorm + quantise, SiLU*up + quantise, and the two
// unfused neighbours (rmsnorm, silu_and_mul).
//
// All of them are HBM-bound.  The fast kernels read each row once with 128-bit
// loads (8 bf16 per load), keep the row in registers between the reduction and
// the store, reduce with warp shuffles, and write int8 codes as 64-bit stores.
// A row is owned by one CTA; vector v of a row (elements 8v..8v+7) belongs to
// thread v mod blockDim.  The *_generic kernels accept any K and any alignment
// with scalar accesses and produce the same bits.
//
// Sum-of-squares order (add_rmsnorm_quant, rmsnorm): always 256 lanes.  Lane l
// accumulates its vectors v = l, l+256, ... in increasing v, and the 8 elements
// of a vector in increasing index, as acc = acc + a*a (separately rounded).  The
// 256 partials are reduced by an xor butterfly inside each group of 32 lanes and
// the 8 group sums are added left to right.  The order depends on K only.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>

#include "w8a8_arith.cuh"
#include "launch_common.h"
#include "sm100_ptx.cuh"

namespace w8a8 {

constexpr int kSumLanes = 256;

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_plain(const uint4* p) { return *p; }

// L2 eviction policy "evict first" for data that is touched once (activations streaming through a row
// kernel), so that it does not push a concurrently running GEMM's operand tiles out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint4 ld_stream_once(const uint4* p, uint64_t pol) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ uint4 ld_plain_once(const uint4* p, uint64_t pol) {
    uint4 v;
    asm volatile("ld.global.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(pol)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_once(uint4* p, const uint4& v, uint64_t pol) {
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w), "l"(pol)
                 : "memory");
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x);
    f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
    f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z);
    f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
}

__device__ __forceinline__ uint2 quant8_rn(const float (&f)[8], float inv) {
    uint2 o;
    o.x = pack_lowbytes(quant_rn_lowbyte(f[0], inv), quant_rn_lowbyte(f[1], inv), quant_rn_lowbyte(f[2], inv),
                        quant_rn_lowbyte(f[3], inv));
    o.y = pack_lowbytes(quant_rn_lowbyte(f[4], inv), quant_rn_lowbyte(f[5], inv), quant_rn_lowbyte(f[6], inv),
                        quant_rn_lowbyte(f[7], inv));
    return o;
}

// max |.| of the 8 bf16 in a 16-byte vector, done on packed bf16 pairs (exact)
__device__ __forceinline__ __nv_bfloat162 absmax_bf16x8(__nv_bfloat162 m, const uint4& v) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) m = __hmax2(m, __habs2(p[i]));
    return m;
}

// Block-wide max.  `red` has one slot per warp.  Every thread returns the result.
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float m = (lane < nwarps) ? red[lane] : 0.0f;
    return warp_max(m);
}

// Block-wide sum over exactly 256 threads in the fixed order described on top.
__device__ __forceinline__ float block_sum_256(float v, float* red) {
    v = warp_sum_butterfly(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int w = 1; w < kSumLanes / 32; ++w) t = __fadd_rn(t, red[w]);
    return t;
}

// ====================================================================================
// per_token_quant_int8  (reference: hip_kernels/dsv4_native_ext.cpp:24-40)
// ====================================================================================
template <int VPT>
__global__ void __launch_bounds__(1024) ptq_vec_kernel(const __nv_bfloat16* __restrict__ x,
                                                       int8_t* __restrict__ q,
                                                       float* __restrict__ s, int M, int K,
                                                       int64_t ldx) {
    ptx::grid_launch_dependents();  // a GEMM launched to overlap this kernel may start its set-up and weight loads
    __shared__ float red[32];
    const int V = K >> 3, T = blockDim.x, tid = threadIdx.x;
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)row * ldx);
        uint4 v[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = tid + i * T;
            v[i] = (idx < V) ? ld_stream(xr + idx) : make_uint4(0, 0, 0, 0);
        }
        __nv_bfloat162 m2 = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int i = 0; i < VPT; ++i) m2 = absmax_bf16x8(m2, v[i]);
        float am = fmaxf(__low2float(m2), __high2float(m2));
        am = block_max(am, red);
        float scale, inv;
        scale_from_amax(am, scale, inv);
        if (tid == 0) s[row] = scale;
        uint2* qr = reinterpret_cast<uint2*>(q + (int64_t)row * K);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = tid + i * T;
            if (idx < V) {
                float f[8];
                unpack8(v[i], f);
                qr[idx] = quant8_rn(f, inv);
            }
        }
        __syncthreads();  // `red` is reused by the next row
    }
}

// any K, any alignment; two reads of the row
__global__ void __launch_bounds__(256) ptq_generic_kernel(const __nv_bfloat16* __restrict__ x,
                                                          int8_t* __restrict__ q,
                                                          float* __restrict__ s, int M, int K,
                                                          int64_t ldx) {
    ptx::grid_launch_dependents();  // a GEMM launched to overlap this kernel may start its set-up and weight loads
    __shared__ float red[32];
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        const __nv_bfloat16* xr = x + (int64_t)row * ldx;
        float am = 0.0f;
        for (int j = threadIdx.x; j < K; j += blockDim.x) am = fmaxf(am, fabsf(__bfloat162float(xr[j])));
        am = block_max(am, red);
        float scale, inv;
        scale_from_amax(am, scale, inv);
        if (threadIdx.x == 0) s[row] = scale;
        int8_t* qr = q + (int64_t)row * K;
        for (int j = threadIdx.x; j < K; j += blockDim.x)
            qr[j] = (int8_t)quant_rn(__bfloat162float(xr[j]), inv);
        __syncthreads();
    }
}

// ====================================================================================
// per_token_group_quant_int8  (reference: hip_kernels/dsv4_all_hip_kernels.hip:49-86)
// Flat over all 16-byte vectors of a contiguous [M,K] tensor: vector f belongs to
// group f / LPG where LPG = group_size/8 lanes cooperate through shuffles.
// ====================================================================================
template <int LPG, int UNROLL>
__global__ void __launch_bounds__(256) ptgq_vec_kernel(const uint4* __restrict__ x,
                                                       uint2* __restrict__ q,
                                                       float* __restrict__ s, int64_t nvec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec;
         base += stride * UNROLL) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t f = base + u * stride;
            v[u] = (f < nvec) ? ld_stream(x + f) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t f = base + u * stride;
            __nv_bfloat162 m2 = absmax_bf16x8(__float2bfloat162_rn(0.0f), v[u]);
            float am = fmaxf(__low2float(m2), __high2float(m2));
            // nvec is a multiple of LPG and stride a multiple of 32, so the LPG lanes of
            // a group are all in range or all out of range together
#pragma unroll
            for (int o = LPG / 2; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            if (f < nvec) {
                const float scale = div127_rn(fmaxf(am, kAmaxFloor));
                const float rcp = __frcp_rn(scale);
                if ((threadIdx.x & (LPG - 1)) == 0) s[f / LPG] = scale;
                const float2 rcp2 = make_float2(rcp, rcp), nscale2 = make_float2(-scale, -scale);
                const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                uint32_t c[8];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    quant_trunc_div_rcp2(make_float2(bf16lo_to_f32(w[i]), bf16hi_to_f32(w[i])), nscale2, rcp2,
                                         c[2 * i], c[2 * i + 1]);
                uint2 o2;
                o2.x = pack_lowbytes(c[0], c[1], c[2], c[3]);
                o2.y = pack_lowbytes(c[4], c[5], c[6], c[7]);
                q[f] = o2;
            }
        }
    }
}

// one warp per (row, group); any group size, ragged last group allowed.
// Scales are laid out [M, ceil(K/gs)].
__global__ void __launch_bounds__(256) ptgq_generic_kernel(const __nv_bfloat16* __restrict__ x,
                                                           int8_t* __restrict__ q,
                                                           float* __restrict__ s, int M, int K,
                                                           int gs, int64_t ldx) {
    const int G = (K + gs - 1) / gs;
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < (int64_t)M * G; w += warps) {
        const int row = (int)(w / G), g = (int)(w % G);
        const int j0 = g * gs, j1 = min(j0 + gs, K);
        const __nv_bfloat16* xr = x + (int64_t)row * ldx;
        float am = 0.0f;
        for (int j = j0 + lane; j < j1; j += 32) am = fmaxf(am, fabsf(__bfloat162float(xr[j])));
        am = warp_max(am);
        const float scale = __fdiv_rn(fmaxf(am, kAmaxFloor), 127.0f);
        if (lane == 0) s[(int64_t)row * G + g] = scale;
        int8_t* qr = q + (int64_t)row * K;
        for (int j = j0 + lane; j < j1; j += 32)
            qr[j] = (int8_t)quant_trunc_div(__bfloat162float(xr[j]), scale);
    }
}

// ====================================================================================
// add_rmsnorm_quant  (reference: hip_kernels/dsv4_native_ext.cpp:103-132)
// 256 threads per row, VPT vectors per thread held in registers as fp32.
// ====================================================================================
template <int VPT>
__global__ void __launch_bounds__(kSumLanes) add_rmsnorm_quant_vec_kernel(
    __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ x,
    const __nv_bfloat16* __restrict__ w, int8_t* __restrict__ q, float* __restrict__ s, int M,
    int K, float eps) {
    ptx::grid_launch_dependents();  // a GEMM launched to overlap this kernel may start its set-up and weight loads
    __shared__ float red_sum[8];
    __shared__ float red_max[32];
    const int V = K >> 3, tid = threadIdx.x;
    const uint64_t once = l2_evict_first_policy();  // x and the residual pass through L2 once
    // 1.0f that the compiler cannot see through (K is positive): see quant_rn_lowbyte2
    const float2 one2 = splat2(__int_as_float(0x3f800000 | (K >> 31)));
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        uint4* rr = reinterpret_cast<uint4*>(res + (int64_t)row * K);
        const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)row * K);
        const uint4* wr = reinterpret_cast<const uint4*>(w);
        uint4 rv[VPT], xv[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = tid + i * kSumLanes;
            if (idx < V) {
                rv[i] = ld_plain_once(rr + idx, once);  // written back below: keep it on the coherent path
                xv[i] = ld_stream_once(xr + idx, once);
            } else {
                rv[i] = make_uint4(0, 0, 0, 0);
                xv[i] = make_uint4(0, 0, 0, 0);
            }
        }
        // Two elements per instruction where the order of operations allows it (packed f32x2: each half
        // is an independent, correctly rounded operation); the lane's sum of squares stays a sequential
        // chain of separately rounded adds in element order.
        float2 a[VPT][4];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const uint32_t rw[4] = {rv[i].x, rv[i].y, rv[i].z, rv[i].w}, xw[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                a[i][e] = __fadd2_rn(bf16x2_to_f32x2(rw[e]), bf16x2_to_f32x2(xw[e]));
                const float2 sq = __fmul2_rn(a[i][e], a[i][e]);
                ss = __fadd_rn(ss, sq.x);
                ss = __fadd_rn(ss, sq.y);
            }
            const int idx = tid + i * kSumLanes;
            if (idx < V) {
                uint4 o;
                o.x = pack_bf16x2_rn(a[i][0].x, a[i][0].y);
                o.y = pack_bf16x2_rn(a[i][1].x, a[i][1].y);
                o.z = pack_bf16x2_rn(a[i][2].x, a[i][2].y);
                o.w = pack_bf16x2_rn(a[i][3].x, a[i][3].y);
                st_once(rr + idx, o, once);
            }
        }
        const float total = block_sum_256(ss, red_sum);
        const float rrms = rrms_from_sumsq(total, K, eps);
        const float2 rrms2 = splat2(rrms);
        float am = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = tid + i * kSumLanes;
            const uint4 wv = (idx < V) ? __ldg(wr + idx) : make_uint4(0, 0, 0, 0);
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                a[i][e] = __fmul2_rn(__fmul2_rn(a[i][e], rrms2), bf16x2_to_f32x2(ww[e]));
                am = max3_abs(am, a[i][e].x, a[i][e].y);
            }
        }
        am = block_max(am, red_max);
        float scale, inv;
        scale_from_amax(am, scale, inv);
        if (tid == 0) s[row] = scale;
        const float2 inv2 = splat2(inv);
        uint2* qr = reinterpret_cast<uint2*>(q + (int64_t)row * K);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = tid + i * kSumLanes;
            if (idx < V) {
                const float2 c0 = quant_rn_lowbyte2(a[i][0], inv2, one2), c1 = quant_rn_lowbyte2(a[i][1], inv2, one2);
                const float2 c2 = quant_rn_lowbyte2(a[i][2], inv2, one2), c3 = quant_rn_lowbyte2(a[i][3], inv2, one2);
                uint2 o;
                o.x = pack_lowbytes(__float_as_uint(c0.x), __float_as_uint(c0.y), __float_as_uint(c1.x), __float_as_uint(c1.y));
                o.y = pack_lowbytes(__float_as_uint(c2.x), __float_as_uint(c2.y), __float_as_uint(c3.x), __float_as_uint(c3.y));
                qr[idx] = o;
            }
        }
        __syncthreads();
    }
}

// Element j of a row belongs to lane (j/8) mod 256; a lane walks its elements in
// increasing j.  Used by the *_generic kernels so that their sums associate exactly
// like the vector kernels'.
#define W8A8_FOR_LANE_ELEMENTS(j, K)                                              \
    for (int _v = threadIdx.x; _v * 8 < (K); _v += kSumLanes)                     \
        for (int j = _v * 8; j < min(_v * 8 + 8, (K)); ++j)

__global__ void __launch_bounds__(kSumLanes) add_rmsnorm_quant_generic_kernel(
    __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ x,
    const __nv_bfloat16* __restrict__ w, int8_t* __restrict__ q, float* __restrict__ s, int M,
    int K, float eps) {
    ptx::grid_launch_dependents();  // a GEMM launched to overlap this kernel may start its set-up and weight loads
    __shared__ float red_sum[8];
    __shared__ float red_max[32];
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        __nv_bfloat16* rr = res + (int64_t)row * K;
        const __nv_bfloat16* xr = x + (int64_t)row * K;
        float ss = 0.0f;
        W8A8_FOR_LANE_ELEMENTS(j, K) {
            const float a = __fadd_rn(__bfloat162float(rr[j]), __bfloat162float(xr[j]));
            ss = __fadd_rn(ss, __fmul_rn(a, a));
        }
        const float rrms = rrms_from_sumsq(block_sum_256(ss, red_sum), K, eps);
        float am = 0.0f;
        W8A8_FOR_LANE_ELEMENTS(j, K) {
            const float a = __fadd_rn(__bfloat162float(rr[j]), __bfloat162float(xr[j]));
            const float y = __fmul_rn(__fmul_rn(a, rrms), __bfloat162float(w[j]));
            am = fmaxf(am, fabsf(y));
        }
        am = block_max(am, red_max);
        float scale, inv;
        scale_from_amax(am, scale, inv);
        if (threadIdx.x == 0) s[row] = scale;
        int8_t* qr = q + (int64_t)row * K;
        W8A8_FOR_LANE_ELEMENTS(j, K) {
            const float a = __fadd_rn(__bfloat162float(rr[j]), __bfloat162float(xr[j]));
            const float y = __fmul_rn(__fmul_rn(a, rrms), __bfloat162float(w[j]));
            qr[j] = (int8_t)quant_rn(y, inv);
            rr[j] = __float2bfloat16_rn(a);  // last use of the old residual value
        }
        __syncthreads();
    }
}

// ====================================================================================
// rmsnorm, in place, no gamma  (reference: hip_kernels/dsv4_native_ext.cpp:45-60)
// ====================================================================================
template <int VPT>
__global__ void __launch_bounds__(kSumLanes) rmsnorm_vec_kernel(__nv_bfloat16* __restrict__ x, int M,
                                                                int K, float eps) {
    __shared__ float red_sum[8];
    const int V = K >> 3, tid = threadIdx.x;
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        uint4* xr = reinterpret_cast<uint4*>(x + (int64_t)row * K);
        float a[VPT][8];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = tid + i * kSumLanes;
            const uint4 v = (idx < V) ? ld_plain(xr + idx) : make_uint4(0, 0, 0, 0);
            unpack8(v, a[i]);
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = __fadd_rn(ss, __fmul_rn(a[i][e], a[i][e]));
        const float rrms = rrms_from_sumsq(block_sum_256(ss, red_sum), K, eps);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = tid + i * kSumLanes;
            if (idx < V) {
                uint4 o;
                o.x = pack_bf16x2_rn(__fmul_rn(a[i][0], rrms), __fmul_rn(a[i][1], rrms));
                o.y = pack_bf16x2_rn(__fmul_rn(a[i][2], rrms), __fmul_rn(a[i][3], rrms));
                o.z = pack_bf16x2_rn(__fmul_rn(a[i][4], rrms), __fmul_rn(a[i][5], rrms));
                o.w = pack_bf16x2_rn(__fmul_rn(a[i][6], rrms), __fmul_rn(a[i][7], rrms));
                xr[idx] = o;
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kSumLanes) rmsnorm_generic_kernel(__nv_bfloat16* __restrict__ x,
                                                                    int M, int K, float eps) {
    __shared__ float red_sum[8];
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        __nv_bfloat16* xr = x + (int64_t)row * K;
        float ss = 0.0f;
        W8A8_FOR_LANE_ELEMENTS(j, K) {
            const float a = __bfloat162float(xr[j]);
            ss = __fadd_rn(ss, __fmul_rn(a, a));
        }
        const float rrms = rrms_from_sumsq(block_sum_256(ss, red_sum), K, eps);
        W8A8_FOR_LANE_ELEMENTS(j, K) {
            xr[j] = __float2bfloat16_rn(__fmul_rn(__bfloat162float(xr[j]), rrms));
        }
        __syncthreads();
    }
}

// Which rows a masked launch touches: a per-row flag list (hip_kernels/dsv4_all_hip_kernels.hip:172-196),
// and/or the masked expert layout, where the rows are E blocks of max_m and expert e's block holds
// masked_m[e] valid rows at its start.  Skipped rows are neither read nor written.
struct RowFilter {
    const int* mask;       // null: no flag list
    const int* masked_m;   // null: no masked layout
    int max_m;
    __device__ __forceinline__ bool any() const { return mask != nullptr || masked_m != nullptr; }
    __device__ __forceinline__ bool active(int row) const {
        if (mask != nullptr && mask[row] == 0) return false;
        if (masked_m != nullptr) {
            const int e = row / max_m;
            return row - e * max_m < masked_m[e];
        }
        return true;
    }
};

// ====================================================================================
// silu_mul_quant (+ optional row mask)
// (reference: hip_kernels/dsv4_native_ext.cpp:79-98,
//             hip_kernels/dsv4_all_hip_kernels.hip:172-196 for the masked form)
// gate and up may be the two halves of one packed [M, 2N] tensor: ldg/ldu are row
// strides in elements.
// ====================================================================================
// One CTA per row.  h = silu(g)*u is computed once, in fp32, and parked in shared memory
// (N floats) between the amax reduction and the quantisation, so that registers only hold
// the loads in flight and several rows are resident per SM.  The arithmetic runs on
// float2 lanes (packed f32x2 instructions).
template <int T, int MINB>
__global__ void __launch_bounds__(T, MINB) silu_mul_quant_vec_kernel(
    const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
    const RowFilter mask, const int* __restrict__ valid_rows, int8_t* __restrict__ q,
    float* __restrict__ s, int M, int N, int64_t ldg, int64_t ldu) {
    ptx::grid_launch_dependents();  // a GEMM launched to overlap this kernel may start its set-up and weight loads
    extern __shared__ float4 h_row4[];  // N floats, 16-byte aligned
    __shared__ float red[32];
    const int V = N >> 3, tid = threadIdx.x;
    if (valid_rows != nullptr) M = min(M, __ldg(valid_rows));
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        if (!mask.active(row)) continue;  // uniform over the block
        const uint4* gr = reinterpret_cast<const uint4*>(g + (int64_t)row * ldg);
        const uint4* ur = reinterpret_cast<const uint4*>(u + (int64_t)row * ldu);
        float am = 0.0f;
        for (int base = tid; base < V; base += 2 * T) {
            // two vectors of each operand in flight per thread
            const int idx1 = base + T;
            const uint4 g0 = ld_stream(gr + base), u0 = ld_stream(ur + base);
            uint4 g1 = make_uint4(0, 0, 0, 0), u1 = g1;
            if (idx1 < V) {
                g1 = ld_stream(gr + idx1);
                u1 = ld_stream(ur + idx1);
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint4 gv = half ? g1 : g0, uv = half ? u1 : u0;
                const int idx = half ? idx1 : base;
                if (idx >= V) break;
                const float2 h0 = silu_mul2(bf16x2_to_f32x2(gv.x), bf16x2_to_f32x2(uv.x));
                const float2 h1 = silu_mul2(bf16x2_to_f32x2(gv.y), bf16x2_to_f32x2(uv.y));
                const float2 h2 = silu_mul2(bf16x2_to_f32x2(gv.z), bf16x2_to_f32x2(uv.z));
                const float2 h3 = silu_mul2(bf16x2_to_f32x2(gv.w), bf16x2_to_f32x2(uv.w));
                am = fmaxf(am, fmaxf(fmaxf(fabsf(h0.x), fabsf(h0.y)), fmaxf(fabsf(h1.x), fabsf(h1.y))));
                am = fmaxf(am, fmaxf(fmaxf(fabsf(h2.x), fabsf(h2.y)), fmaxf(fabsf(h3.x), fabsf(h3.y))));
                h_row4[2 * idx] = make_float4(h0.x, h0.y, h1.x, h1.y);
                h_row4[2 * idx + 1] = make_float4(h2.x, h2.y, h3.x, h3.y);
            }
        }
        am = block_max(am, red);  // also orders the shared-memory writes before the reads below
        float scale, inv;
        scale_from_amax(am, scale, inv);
        if (tid == 0) s[row] = scale;
        const float2 inv2 = splat2(inv);
        uint2* qr = reinterpret_cast<uint2*>(q + (int64_t)row * N);
        for (int idx = tid; idx < V; idx += T) {
            const float4 a = h_row4[2 * idx], b = h_row4[2 * idx + 1];
            const float2 c0 = quant_rn_lowbyte2(make_float2(a.x, a.y), inv2);
            const float2 c1 = quant_rn_lowbyte2(make_float2(a.z, a.w), inv2);
            const float2 c2 = quant_rn_lowbyte2(make_float2(b.x, b.y), inv2);
            const float2 c3 = quant_rn_lowbyte2(make_float2(b.z, b.w), inv2);
            uint2 o;
            o.x = pack_lowbytes(__float_as_uint(c0.x), __float_as_uint(c0.y), __float_as_uint(c1.x), __float_as_uint(c1.y));
            o.y = pack_lowbytes(__float_as_uint(c2.x), __float_as_uint(c2.y), __float_as_uint(c3.x), __float_as_uint(c3.y));
            qr[idx] = o;
        }
        __syncthreads();  // the row buffer and `red` are reused by the next row
    }
}

// Persistent form for many rows: a CTA first tabulates silu of every bf16 gate value with
// 2^-12 <= |g| < 2^20 in shared memory, then walks rows blockIdx.x, +gridDim.x, ...  The
// per-element work drops from ~30 to ~15 issue slots, which is what lets the kernel run at
// memory speed.  Shared memory: N floats for the row, then the 32 KB table.
template <int T, int MINB>
__global__ void __launch_bounds__(T, MINB) silu_mul_quant_table_kernel(
    const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
    const RowFilter mask, const int* __restrict__ valid_rows, int8_t* __restrict__ q,
    float* __restrict__ s, int M, int N, int64_t ldg, int64_t ldu) {
    ptx::grid_launch_dependents();  // a GEMM launched to overlap this kernel may start its set-up and weight loads
    extern __shared__ float4 h_row4[];
    __shared__ float red[32];
    float* tab = reinterpret_cast<float*>(h_row4) + N;
    const int V = N >> 3, tid = threadIdx.x;
    if (valid_rows != nullptr) M = min(M, __ldg(valid_rows));
    if ((int)blockIdx.x >= M) return;
    for (int i = tid; i < kSigTabEntries; i += T) tab[i] = silu_table_entry(i);
    __syncthreads();
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        if (!mask.active(row)) continue;  // uniform over the block
        const uint4* gr = reinterpret_cast<const uint4*>(g + (int64_t)row * ldg);
        const uint4* ur = reinterpret_cast<const uint4*>(u + (int64_t)row * ldu);
        float am = 0.0f;
        constexpr int NB = 3;  // vectors of each operand in flight per thread
        for (int base = tid; base < V; base += NB * T) {
            uint4 gv[NB], uv[NB];
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int idx = base + j * T;
                if (idx < V) {
                    gv[j] = ld_stream(gr + idx);
                    uv[j] = ld_stream(ur + idx);
                } else {
                    gv[j] = make_uint4(0, 0, 0, 0);
                    uv[j] = gv[j];
                }
            }
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int idx = base + j * T;
                if (idx >= V) break;
                float2 h[4];
                silu_mul8_table(gv[j], uv[j], tab, h);
                am = fmaxf(am, fmaxf(fmaxf(fabsf(h[0].x), fabsf(h[0].y)), fmaxf(fabsf(h[1].x), fabsf(h[1].y))));
                am = fmaxf(am, fmaxf(fmaxf(fabsf(h[2].x), fabsf(h[2].y)), fmaxf(fabsf(h[3].x), fabsf(h[3].y))));
                h_row4[2 * idx] = make_float4(h[0].x, h[0].y, h[1].x, h[1].y);
                h_row4[2 * idx + 1] = make_float4(h[2].x, h[2].y, h[3].x, h[3].y);
            }
        }
        am = block_max(am, red);
        float scale, inv;
        scale_from_amax(am, scale, inv);
        if (tid == 0) s[row] = scale;
        const float2 inv2 = splat2(inv);
        uint2* qr = reinterpret_cast<uint2*>(q + (int64_t)row * N);
        for (int idx = tid; idx < V; idx += T) {
            const float4 a = h_row4[2 * idx], b = h_row4[2 * idx + 1];
            const float2 c0 = quant_rn_lowbyte2(make_float2(a.x, a.y), inv2);
            const float2 c1 = quant_rn_lowbyte2(make_float2(a.z, a.w), inv2);
            const float2 c2 = quant_rn_lowbyte2(make_float2(b.x, b.y), inv2);
            const float2 c3 = quant_rn_lowbyte2(make_float2(b.z, b.w), inv2);
            uint2 o;
            o.x = pack_lowbytes(__float_as_uint(c0.x), __float_as_uint(c0.y), __float_as_uint(c1.x), __float_as_uint(c1.y));
            o.y = pack_lowbytes(__float_as_uint(c2.x), __float_as_uint(c2.y), __float_as_uint(c3.x), __float_as_uint(c3.y));
            qr[idx] = o;
        }
        __syncthreads();
    }
}

// Persistent form used for many rows.  One CTA of 1024 threads per SM = two independent groups of
// 512 threads that share the sigmoid table.  Each group owns a shared-memory row buffer and walks
// its own row blocks (RPB rows of N gates + N ups each):
//   wait (mbarrier) for the block's bulk copies -> the thread's gates and ups from shared memory
//   into registers -> group barrier -> one thread starts the bulk copies of the group's NEXT block
//   into the same buffer -> h = silu(g)*u in registers -> group barrier (publishes the per-warp
//   maxima) -> row maximum, quantise, store.
// The copies (cp.async.bulk, one per half row, completion counted on an mbarrier) therefore overlap
// all the arithmetic and the stores of the same group and everything the other group does, keep a
// whole row block in flight per group without registers or load/store-unit request slots, and the
// two groups are in different phases most of the time, so the shared-memory pipe (table gathers)
// and the arithmetic pipes (quantisation) are busy together.
__device__ int g_row_status = 0;  // non-zero: a bounded wait in a row kernel gave up

__device__ __forceinline__ void group_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int RPB, int VPT>
__global__ void __launch_bounds__(1024, 1) silu_mul_quant_async_kernel(
    const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
    const RowFilter mask, const int* __restrict__ valid_rows, int8_t* __restrict__ q,
    float* __restrict__ s, int M, int N, int64_t ldg, int64_t ldu) {
    ptx::grid_launch_dependents();  // a GEMM launched to overlap this kernel may start its set-up and weight loads
    constexpr int GROUP = 512, GT = GROUP / RPB, WPG = GT / 32;  // threads per group / per row, warps per row
    extern __shared__ uint4 smem4[];
    __shared__ float red[2][2][RPB][WPG];  // [group][parity][row][warp]
    __shared__ uint64_t bars[2];
    const int V = N >> 3;
    // [group][RPB][gate vectors V | up vectors V], then the sigmoid table
    float* tab = reinterpret_cast<float*>(smem4 + (size_t)2 * RPB * 2 * V);
    const int tid = threadIdx.x, grp = tid / GROUP, gtid = tid % GROUP;
    const int gi = gtid / GT, lt = gtid % GT, lane = tid & 31, wig = lt >> 5;
    if (valid_rows != nullptr) M = min(M, __ldg(valid_rows));
    const int nblocks = (M + RPB - 1) / RPB;
    const uint32_t bar = ptx::smem_u32(&bars[grp]);
    const uint32_t half_bytes = (uint32_t)N * 2u;  // one row of gates (or ups) in bf16
    uint4* my_buf = smem4 + (size_t)(grp * RPB) * 2 * V;
    // 1.0f that the compiler cannot see through (N is positive): see quant_rn_lowbyte2
    const float2 one2 = splat2(__int_as_float(0x3f800000 | (N >> 31)));

    auto row_active = [&](int row) { return row < M && mask.active(row); };
    // gate_up rows of a packed [M, 2N] tensor follow one another in memory exactly as in the buffer
    // ([row][gates | ups]): a block of short rows without a mask then comes in with ONE copy
    const bool block_copy = RPB > 1 && !mask.any() && u == g + N && ldg == ldu && ldg == 2 * (int64_t)N;
    // the group's first thread: arm the barrier with the bytes to come and start the copies.  The
    // buffer is only ever written by these copies; the kernel reads it.
    auto issue = [&](int rb) {
        if (block_copy && (rb + 1) * RPB <= M) {
            const uint32_t all = (uint32_t)RPB * 2u * half_bytes;
            ptx::mbar_arrive_expect_tx(bar, all);
            ptx::bulk_load(ptx::smem_u32(my_buf), g + (int64_t)rb * RPB * ldg, all, bar);
            return;
        }
        uint32_t bytes = 0;
        for (int r = 0; r < RPB; ++r) bytes += row_active(rb * RPB + r) ? 2u * half_bytes : 0u;
        ptx::mbar_arrive_expect_tx(bar, bytes);
        for (int r = 0; r < RPB; ++r) {
            const int row = rb * RPB + r;
            if (!row_active(row)) continue;
            const uint32_t gdst = ptx::smem_u32(my_buf + (size_t)(r * 2) * V);
            ptx::bulk_load(gdst, g + (int64_t)row * ldg, half_bytes, bar);
            ptx::bulk_load(gdst + half_bytes, u + (int64_t)row * ldu, half_bytes, bar);
        }
    };

    const int first = blockIdx.x * 2 + grp, stride = gridDim.x * 2;
    if (gtid == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_barrier_init();
        if (first < nblocks) issue(first);
    }
    for (int i = tid; i < kSigTabEntries; i += 1024) tab[i] = silu_table_entry(i);
    __syncthreads();  // table complete, barriers initialised

    uint32_t it = 0;
    for (int rb = first; rb < nblocks; rb += stride, ++it) {
        // every thread waits for the copies itself; whether the group goes on is decided together at the
        // first barrier below (a thread whose wait gave up skips its reads and votes no there)
        const bool arrived = ptx::mbar_wait_bounded(bar, it & 1u);
        const int row = rb * RPB + gi;
        const bool active = arrived && row_active(row);
        const uint4* gb = my_buf + (size_t)(gi * 2) * V;
        const uint4* ub = gb + V;
        // the thread's share of the row block goes to registers first, so that the buffer is free
        // and the next block's copies start before any arithmetic on this one; h later replaces
        // the raw words in the same registers
        uint32_t r[VPT][8];
        if (active) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int idx = lt + j * GT;
                if (idx < V) {
                    const uint4 gv = gb[idx], uv = ub[idx];
                    r[j][0] = gv.x; r[j][1] = gv.y; r[j][2] = gv.z; r[j][3] = gv.w;
                    r[j][4] = uv.x; r[j][5] = uv.y; r[j][6] = uv.z; r[j][7] = uv.w;
                }
            }
        }
        // the buffer has been read by everyone -- or somebody's wait gave up, and then the whole group leaves
        // here, before the named barriers further down
        if (!ptx::barrier_and_rt(1 + grp, GROUP, arrived)) {
            atomicCAS(&g_row_status, 0, 201);
            break;
        }
        if (gtid == 0 && rb + stride < nblocks) issue(rb + stride);
        float am = 0.0f;
        if (active) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int idx = lt + j * GT;
                if (idx < V) {
                    float2 h[4];
                    silu_mul8_table(make_uint4(r[j][0], r[j][1], r[j][2], r[j][3]),
                                    make_uint4(r[j][4], r[j][5], r[j][6], r[j][7]), tab, h);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        am = max3_abs(am, h[i].x, h[i].y);
                        r[j][2 * i] = __float_as_uint(h[i].x);
                        r[j][2 * i + 1] = __float_as_uint(h[i].y);
                    }
                }
            }
        }
        am = warp_max(am);
        if (lane == 0) red[grp][it & 1u][gi][wig] = am;
        group_barrier(3 + grp, GROUP);  // the per-warp maxima are visible
        float rowmax = (lane < WPG) ? red[grp][it & 1u][gi][lane] : 0.0f;
        rowmax = warp_max(rowmax);
        if (active) {
            float scale, inv;
            scale_from_amax(rowmax, scale, inv);
            if (lt == 0) s[row] = scale;
            const float2 inv2 = splat2(inv);
            uint2* qr = reinterpret_cast<uint2*>(q + (int64_t)row * N);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int idx = lt + j * GT;
                if (idx < V) {
                    float2 c[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        c[i] = quant_rn_lowbyte2(make_float2(__uint_as_float(r[j][2 * i]), __uint_as_float(r[j][2 * i + 1])),
                                                 inv2, one2);
                    const float2 c0 = c[0], c1 = c[1], c2 = c[2], c3 = c[3];
                    uint2 o;
                    o.x = pack_lowbytes(__float_as_uint(c0.x), __float_as_uint(c0.y), __float_as_uint(c1.x), __float_as_uint(c1.y));
                    o.y = pack_lowbytes(__float_as_uint(c2.x), __float_as_uint(c2.y), __float_as_uint(c3.x), __float_as_uint(c3.y));
                    qr[idx] = o;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(256) silu_mul_quant_generic_kernel(
    const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
    const RowFilter mask, const int* __restrict__ valid_rows, int8_t* __restrict__ q,
    float* __restrict__ s, int M, int N, int64_t ldg, int64_t ldu) {
    ptx::grid_launch_dependents();  // a GEMM launched to overlap this kernel may start its set-up and weight loads
    __shared__ float red[32];
    if (valid_rows != nullptr) M = min(M, __ldg(valid_rows));
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        if (!mask.active(row)) continue;
        const __nv_bfloat16* gr = g + (int64_t)row * ldg;
        const __nv_bfloat16* ur = u + (int64_t)row * ldu;
        float am = 0.0f;
        for (int j = threadIdx.x; j < N; j += blockDim.x)
            am = fmaxf(am, fabsf(silu_mul(__bfloat162float(gr[j]), __bfloat162float(ur[j]))));
        am = block_max(am, red);
        float scale, inv;
        scale_from_amax(am, scale, inv);
        if (threadIdx.x == 0) s[row] = scale;
        int8_t* qr = q + (int64_t)row * N;
        for (int j = threadIdx.x; j < N; j += blockDim.x)
            qr[j] = (int8_t)quant_rn(silu_mul(__bfloat162float(gr[j]), __bfloat162float(ur[j])), inv);
        __syncthreads();
    }
}

// ====================================================================================
// silu_and_mul -> bf16  (reference: hip_kernels/dsv4_native_ext.cpp:65-74)
// ====================================================================================
__global__ void __launch_bounds__(256) silu_mul_vec_kernel(const __nv_bfloat16* __restrict__ g,
                                                           const __nv_bfloat16* __restrict__ u,
                                                           __nv_bfloat16* __restrict__ out, int M,
                                                           int N, int64_t ldg, int64_t ldu) {
    const int V = N >> 3;
    const int64_t total = (int64_t)M * V;
    for (int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; f < total;
         f += (int64_t)gridDim.x * blockDim.x) {
        const int row = (int)(f / V), idx = (int)(f % V);
        const uint4 gv = ld_stream(reinterpret_cast<const uint4*>(g + (int64_t)row * ldg) + idx);
        const uint4 uv = ld_stream(reinterpret_cast<const uint4*>(u + (int64_t)row * ldu) + idx);
        float g8[8], u8[8], h[8];
        unpack8(gv, g8);
        unpack8(uv, u8);
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = silu_mul(g8[e], u8[e]);
        uint4 o;
        o.x = pack_bf16x2_rn(h[0], h[1]);
        o.y = pack_bf16x2_rn(h[2], h[3]);
        o.z = pack_bf16x2_rn(h[4], h[5]);
        o.w = pack_bf16x2_rn(h[6], h[7]);
        reinterpret_cast<uint4*>(out + (int64_t)row * N)[idx] = o;
    }
}

// Many elements: persistent CTAs that tabulate silu of every bf16 gate first (silu_mul8_table), then
// walk rows blockIdx.x, +gridDim.x, ...; the vectors of a row are dealt to the threads, two in flight
// per thread.  Same bits as silu_mul for every input.
__global__ void __launch_bounds__(512, 2) silu_mul_table_kernel(const __nv_bfloat16* __restrict__ g,
                                                                const __nv_bfloat16* __restrict__ u,
                                                                __nv_bfloat16* __restrict__ out, int M, int N,
                                                                int64_t ldg, int64_t ldu) {
    __shared__ float tab[kSigTabEntries];
    for (int i = threadIdx.x; i < kSigTabEntries; i += 512) tab[i] = silu_table_entry(i);
    __syncthreads();
    const int V = N >> 3;
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        const uint4* gr = reinterpret_cast<const uint4*>(g + (int64_t)row * ldg);
        const uint4* ur = reinterpret_cast<const uint4*>(u + (int64_t)row * ldu);
        uint4* orow = reinterpret_cast<uint4*>(out + (int64_t)row * N);
        for (int i0 = threadIdx.x; i0 < V; i0 += 2 * 512) {
            const int i1 = i0 + 512;
            const bool two = i1 < V;
            const uint4 g0 = ld_stream(gr + i0), u0 = ld_stream(ur + i0);
            const uint4 g1 = two ? ld_stream(gr + i1) : make_uint4(0, 0, 0, 0);
            const uint4 u1 = two ? ld_stream(ur + i1) : make_uint4(0, 0, 0, 0);
            float2 h[4];
            silu_mul8_table(g0, u0, tab, h);
            orow[i0] = make_uint4(pack_bf16x2_rn(h[0].x, h[0].y), pack_bf16x2_rn(h[1].x, h[1].y),
                                  pack_bf16x2_rn(h[2].x, h[2].y), pack_bf16x2_rn(h[3].x, h[3].y));
            if (two) {
                silu_mul8_table(g1, u1, tab, h);
                orow[i1] = make_uint4(pack_bf16x2_rn(h[0].x, h[0].y), pack_bf16x2_rn(h[1].x, h[1].y),
                                      pack_bf16x2_rn(h[2].x, h[2].y), pack_bf16x2_rn(h[3].x, h[3].y));
            }
        }
    }
}

__global__ void __launch_bounds__(256) silu_mul_generic_kernel(const __nv_bfloat16* __restrict__ g,
                                                               const __nv_bfloat16* __restrict__ u,
                                                               __nv_bfloat16* __restrict__ out,
                                                               int M, int N, int64_t ldg,
                                                               int64_t ldu) {
    const int64_t total = (int64_t)M * N;
    for (int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; f < total;
         f += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = f / N, j = f % N;
        out[f] = __float2bfloat16_rn(
            silu_mul(__bfloat162float(g[row * ldg + j]), __bfloat162float(u[row * ldu + j])));
    }
}

// ====================================================================================
// host-side launchers
// ====================================================================================
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static inline int round_up32(int v) { return (v + 31) & ~31; }
static inline int grid_rows(int M) { return M; }

int ptq(const void* x, void* q, void* s, int M, int K, int64_t ldx, cudaStream_t st) {
    if (M == 0 || K == 0) return 0;
    auto xp = static_cast<const __nv_bfloat16*>(x);
    auto qp = static_cast<int8_t*>(q);
    auto sp = static_cast<float*>(s);
    const bool vec = (K % 8 == 0) && (ldx % 8 == 0) && aligned16(x) && ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
    const int V = K / 8;
    if (vec && V <= 8 * 1024) {
        // vectors per thread: the smallest of 1,2,4,8 that keeps the CTA at 128 threads or fewer
        // (small CTAs -> many resident rows per SM, so that 2048 rows are one wave, and several 16-byte
        // loads in flight per thread; measured at K=7168: 112 threads x 8 vectors 7.2 us for 2048 rows
        // against 8.5 us with 224 threads x 4)
        const int vpt = V <= 128 ? 1 : V <= 256 ? 2 : V <= 512 ? 4 : 8;
        int T = round_up32((V + vpt - 1) / vpt);
        if (T < 64) T = 64;
        switch (vpt) {
            case 1: ptq_vec_kernel<1><<<grid_rows(M), T, 0, st>>>(xp, qp, sp, M, K, ldx); break;
            case 2: ptq_vec_kernel<2><<<grid_rows(M), T, 0, st>>>(xp, qp, sp, M, K, ldx); break;
            case 4: ptq_vec_kernel<4><<<grid_rows(M), T, 0, st>>>(xp, qp, sp, M, K, ldx); break;
            default: ptq_vec_kernel<8><<<grid_rows(M), T, 0, st>>>(xp, qp, sp, M, K, ldx); break;
        }
    } else {
        ptq_generic_kernel<<<grid_rows(M), 256, 0, st>>>(xp, qp, sp, M, K, ldx);
    }
    return check_launch("per_token_quant_int8");
}

int ptgq(const void* x, void* q, void* s, int M, int K, int gs, cudaStream_t st) {
    if (M == 0 || K == 0) return 0;
    if (gs <= 0) return fail(DSV4_ERR_ARG, "per_token_group_quant_int8: group_size must be positive");
    const bool vec = (K % gs == 0) && (gs % 8 == 0) && aligned16(x) &&
                     ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
    const int lpg = gs / 8;
    const int64_t nvec = (int64_t)M * (K / 8);
    auto xv = static_cast<const uint4*>(x);
    auto qv = static_cast<uint2*>(q);
    auto sp = static_cast<float*>(s);
    const int64_t want = (nvec + 256 * 4 - 1) / (256 * 4);
    const int grid = (int)(want < 1 ? 1 : (want > (1 << 20) ? (1 << 20) : want));
    bool done = false;
    if (vec) {
        done = true;
        switch (lpg) {
            case 1: ptgq_vec_kernel<1, 4><<<grid, 256, 0, st>>>(xv, qv, sp, nvec); break;
            case 2: ptgq_vec_kernel<2, 4><<<grid, 256, 0, st>>>(xv, qv, sp, nvec); break;
            case 4: ptgq_vec_kernel<4, 4><<<grid, 256, 0, st>>>(xv, qv, sp, nvec); break;
            case 8: ptgq_vec_kernel<8, 4><<<grid, 256, 0, st>>>(xv, qv, sp, nvec); break;
            case 16: ptgq_vec_kernel<16, 4><<<grid, 256, 0, st>>>(xv, qv, sp, nvec); break;
            case 32: ptgq_vec_kernel<32, 4><<<grid, 256, 0, st>>>(xv, qv, sp, nvec); break;
            default: done = false;
        }
    }
    if (!done) {
        const int64_t groups = (int64_t)M * ((K + gs - 1) / gs);
        const int64_t blocks = (groups + 7) / 8;
        ptgq_generic_kernel<<<(int)(blocks > (1 << 20) ? (1 << 20) : blocks), 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<int8_t*>(q), sp, M, K, gs, K);
    }
    return check_launch("per_token_group_quant_int8");
}

int add_rmsnorm_quant(void* res, const void* x, const void* w, void* q, void* s, int M, int K,
                      float eps, cudaStream_t st) {
    if (M == 0 || K == 0) return 0;
    auto rp = static_cast<__nv_bfloat16*>(res);
    auto xp = static_cast<const __nv_bfloat16*>(x);
    auto wp = static_cast<const __nv_bfloat16*>(w);
    auto qp = static_cast<int8_t*>(q);
    auto sp = static_cast<float*>(s);
    const bool vec = (K % 8 == 0) && aligned16(res) && aligned16(x) && aligned16(w) &&
                     ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
    const int V = K / 8;
    if (vec && V <= 8 * kSumLanes) {
        if (V <= kSumLanes)
            add_rmsnorm_quant_vec_kernel<1><<<grid_rows(M), kSumLanes, 0, st>>>(rp, xp, wp, qp, sp, M, K, eps);
        else if (V <= 2 * kSumLanes)
            add_rmsnorm_quant_vec_kernel<2><<<grid_rows(M), kSumLanes, 0, st>>>(rp, xp, wp, qp, sp, M, K, eps);
        else if (V <= 4 * kSumLanes)
            add_rmsnorm_quant_vec_kernel<4><<<grid_rows(M), kSumLanes, 0, st>>>(rp, xp, wp, qp, sp, M, K, eps);
        else
            add_rmsnorm_quant_vec_kernel<8><<<grid_rows(M), kSumLanes, 0, st>>>(rp, xp, wp, qp, sp, M, K, eps);
    } else {
        add_rmsnorm_quant_generic_kernel<<<grid_rows(M), kSumLanes, 0, st>>>(rp, xp, wp, qp, sp, M, K, eps);
    }
    return check_launch("add_rmsnorm_quant");
}

int rmsnorm(void* x, int M, int K, float eps, cudaStream_t st) {
    if (M == 0 || K == 0) return 0;
    auto xp = static_cast<__nv_bfloat16*>(x);
    const bool vec = (K % 8 == 0) && aligned16(x);
    const int V = K / 8;
    if (vec && V <= 8 * kSumLanes) {
        if (V <= kSumLanes) rmsnorm_vec_kernel<1><<<grid_rows(M), kSumLanes, 0, st>>>(xp, M, K, eps);
        else if (V <= 2 * kSumLanes) rmsnorm_vec_kernel<2><<<grid_rows(M), kSumLanes, 0, st>>>(xp, M, K, eps);
        else if (V <= 4 * kSumLanes) rmsnorm_vec_kernel<4><<<grid_rows(M), kSumLanes, 0, st>>>(xp, M, K, eps);
        else rmsnorm_vec_kernel<8><<<grid_rows(M), kSumLanes, 0, st>>>(xp, M, K, eps);
    } else {
        rmsnorm_generic_kernel<<<grid_rows(M), kSumLanes, 0, st>>>(xp, M, K, eps);
    }
    return check_launch("rmsnorm");
}

int silu_mul_quant(const void* g, const void* u, const int* row_mask, const int* valid_rows, void* q, void* s,
                   int M, int N, int64_t ldg, int64_t ldu, cudaStream_t st, const int* masked_m, int max_m) {
    if (M == 0 || N == 0) return 0;
    const RowFilter mask{row_mask, masked_m, max_m};
    auto gp = static_cast<const __nv_bfloat16*>(g);
    auto up = static_cast<const __nv_bfloat16*>(u);
    auto qp = static_cast<int8_t*>(q);
    auto sp = static_cast<float*>(s);
    const bool vec = (N % 8 == 0) && (ldg % 8 == 0) && (ldu % 8 == 0) && aligned16(g) &&
                     aligned16(u) && ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
    const int V = N / 8;
    const size_t row_smem = (size_t)N * sizeof(float);
    if (vec && row_smem <= 200 * 1024) {
        // the opt-in above 48 KB of dynamic shared memory is per device and per kernel
        static bool opted_in[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64 || !opted_in[dev]) {
            cudaFuncSetAttribute(silu_mul_quant_vec_kernel<128, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            cudaFuncSetAttribute(silu_mul_quant_vec_kernel<256, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            cudaFuncSetAttribute(silu_mul_quant_vec_kernel<384, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (dev >= 0 && dev < 64) opted_in[dev] = true;
        }
        const size_t tab_smem = row_smem + kSigTabEntries * sizeof(float);
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        // rows per group pass of the persistent kernel: as many (1, 2 or 4) as keep a group's 512
        // threads busy, while both groups' row buffers plus the table fit in shared memory
        // about 64 KB of row data per group pass (so that enough bytes are in flight), at most 8 rows
        int rpb = 1;
        while (rpb < 8 && (size_t)(2 * rpb) * row_smem <= 64 * 1024) rpb <<= 1;
        while (rpb > 1 && ((size_t)2 * rpb * row_smem + kSigTabEntries * sizeof(float) > 200 * 1024 ||
                           (V + 512 / rpb - 1) / (512 / rpb) > 5))
            rpb >>= 1;
        const size_t async_smem = (size_t)2 * rpb * row_smem + kSigTabEntries * sizeof(float);
        const int gt = 512 / rpb;
        const int vpt = (V + gt - 1) / gt;
        if (sms > 0 && async_smem <= 200 * 1024 && (int64_t)M >= (int64_t)4 * sms * rpb && V >= 64 && vpt <= 5) {
            const int nblocks = (M + rpb - 1) / rpb;
            const int grid = (nblocks + 1) / 2 < sms ? (nblocks + 1) / 2 : sms;
#define W8A8_LAUNCH_SILU_ASYNC(R, P)                                                                         \
    case R * 8 + P: {                                                                                        \
        static bool opted[64] = {};                                                                          \
        if (dev < 0 || dev >= 64 || !opted[dev]) {                                                           \
            cudaFuncSetAttribute(silu_mul_quant_async_kernel<R, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 200 * 1024);                                                                \
            if (dev >= 0 && dev < 64) opted[dev] = true;                                                     \
        }                                                                                                    \
        silu_mul_quant_async_kernel<R, P><<<grid, 1024, async_smem, st>>>(gp, up, mask, valid_rows, qp, sp, M, N, \
                                                                          ldg, ldu);                         \
    } break
#define W8A8_LAUNCH_SILU_ASYNC_ROWS(R)                                                                       \
    W8A8_LAUNCH_SILU_ASYNC(R, 1); W8A8_LAUNCH_SILU_ASYNC(R, 2); W8A8_LAUNCH_SILU_ASYNC(R, 3);                  \
    W8A8_LAUNCH_SILU_ASYNC(R, 4); W8A8_LAUNCH_SILU_ASYNC(R, 5)
            switch (rpb * 8 + vpt) {
                W8A8_LAUNCH_SILU_ASYNC_ROWS(1);
                W8A8_LAUNCH_SILU_ASYNC_ROWS(2);
                W8A8_LAUNCH_SILU_ASYNC_ROWS(4);
                W8A8_LAUNCH_SILU_ASYNC_ROWS(8);
                default: return fail(DSV4_ERR_LAUNCH, "silu_mul_quant: no kernel variant for this row length");
            }
#undef W8A8_LAUNCH_SILU_ASYNC_ROWS
#undef W8A8_LAUNCH_SILU_ASYNC
            return check_launch("silu_mul_quant");
        }
        if (sms > 0 && M >= 4 * sms && tab_smem <= 110 * 1024) {
            // many rows: persistent CTAs (two per SM) with the sigmoid table
            static bool tab_opted_in[64] = {};
            if (dev < 0 || dev >= 64 || !tab_opted_in[dev]) {
                cudaFuncSetAttribute(silu_mul_quant_table_kernel<512, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
                cudaFuncSetAttribute(silu_mul_quant_table_kernel<256, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
                if (dev >= 0 && dev < 64) tab_opted_in[dev] = true;
            }
            if (V > 512)
                silu_mul_quant_table_kernel<512, 2><<<2 * sms, 512, tab_smem, st>>>(gp, up, mask, valid_rows, qp, sp, M, N, ldg, ldu);
            else
                silu_mul_quant_table_kernel<256, 4><<<4 * sms, 256, tab_smem, st>>>(gp, up, mask, valid_rows, qp, sp, M, N, ldg, ldu);
            return check_launch("silu_mul_quant");
        }
        if (V <= 256)
            silu_mul_quant_vec_kernel<128, 8><<<grid_rows(M), 128, row_smem, st>>>(gp, up, mask, valid_rows, qp, sp, M, N, ldg, ldu);
        else if (V <= 1024)
            silu_mul_quant_vec_kernel<256, 4><<<grid_rows(M), 256, row_smem, st>>>(gp, up, mask, valid_rows, qp, sp, M, N, ldg, ldu);
        else
            silu_mul_quant_vec_kernel<384, 3><<<grid_rows(M), 384, row_smem, st>>>(gp, up, mask, valid_rows, qp, sp, M, N, ldg, ldu);
    } else {
        silu_mul_quant_generic_kernel<<<grid_rows(M), 256, 0, st>>>(gp, up, mask, valid_rows, qp, sp, M, N, ldg, ldu);
    }
    return check_launch("silu_mul_quant");
}

int read_row_status(int* out) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_row_status, sizeof(int)) != cudaSuccess)
        return fail(DSV4_ERR_LAUNCH, "device_status: cannot read the row-kernel status word");
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_row_status, &zero, sizeof(int));
    }
    *out = v;
    return 0;
}

int silu_mul(const void* g, const void* u, void* out, int M, int N, int64_t ldg, int64_t ldu,
             cudaStream_t st) {
    if (M == 0 || N == 0) return 0;
    auto gp = static_cast<const __nv_bfloat16*>(g);
    auto up = static_cast<const __nv_bfloat16*>(u);
    auto op = static_cast<__nv_bfloat16*>(out);
    const bool vec = (N % 8 == 0) && (ldg % 8 == 0) && (ldu % 8 == 0) && aligned16(g) &&
                     aligned16(u) && aligned16(out);
    const int64_t work = vec ? (int64_t)M * (N / 8) : (int64_t)M * N;
    int64_t blocks = (work + 255) / 256;
    if (blocks > (1 << 20)) blocks = 1 << 20;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (vec && sms > 0 && (int64_t)M * N >= (int64_t)(1 << 21) && M >= 2 * sms)
        silu_mul_table_kernel<<<2 * sms, 512, 0, st>>>(gp, up, op, M, N, ldg, ldu);
    else if (vec)
        silu_mul_vec_kernel<<<(int)blocks, 256, 0, st>>>(gp, up, op, M, N, ldg, ldu);
    else
        silu_mul_generic_kernel<<<(int)blocks, 256, 0, st>>>(gp, up, op, M, N, ldg, ldu);
    return check_launch("silu_and_mul");
}

}  // namespace w8a8
