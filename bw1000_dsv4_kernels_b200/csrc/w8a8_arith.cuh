// Scalar arithmetic of the W8A8 activation-quant chain, device side.
//
// Every floating-point step that decides an int8 code or an fp32 scale is written
// here with an explicitly rounded intrinsic (__fmul_rn, __fadd_rn, __fmaf_rn,
// __fdiv_rn, __fsqrt_rn) so that the compiler can neither contract a multiply and an
// add into an FMA nor substitute an approximate reciprocal / rsqrt / exp.  The same
// sequence of IEEE-754 binary32 operations is restated for the CPU in the test
// oracle; the two agree bit for bit because each step is a correctly rounded
// operation on both sides.
//
// Reference arithmetic this follows (hip_kernels/dsv4_native_ext.cpp):
//   quantiser        :24-40   am=max(amax,1e-10); s=am/127; inv=127/am; q=rint(x*inv)
//   add + rmsnorm    :103-132 a=res+x; rrms=rsqrt(sum(a*a)/N+eps); y=(a*rrms)*w
//   silu * up        :79-98   h=((1/(1+exp(-g)))*g)*u
//   group quantiser  hip_kernels/dsv4_all_hip_kernels.hip:49-86  q=trunc(clamp(x/s))
// Two deliberate differences, both needed for a reproducible result:
//   * rsqrt is computed as 1/sqrt with correctly rounded sqrt and divide;
//   * exp is the fixed polynomial below, not a vendor libm routine.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>

namespace w8a8 {

constexpr float kAmaxFloor = 1e-10f;

// ---- bf16 <-> f32 -----------------------------------------------------------------
// A 32-bit word holds two bf16 values; element 0 is the low half.
__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Round-to-nearest-even f32 -> bf16, two values packed (lo = a, hi = b).
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---- quantiser --------------------------------------------------------------------
// scale and inverse scale from a row (or group) absolute maximum
__device__ __forceinline__ void scale_from_amax(float amax, float& scale, float& inv) {
    float am = fmaxf(amax, kAmaxFloor);
    scale = __fdiv_rn(am, 127.0f);
    inv = __fdiv_rn(127.0f, am);
}

// round-half-even(x*inv), clamped to [-128,127]: the scalar form used by the generic
// kernels.  cvt.rni.s32 is rintf followed by an exact conversion.
__device__ __forceinline__ int quant_rn(float x, float inv) {
    int q = __float2int_rn(__fmul_rn(x, inv));
    return max(-128, min(127, q));
}

// The same code without a conversion instruction: t = x*inv (rounded), then t + 1.5*2^23
// rounds t to the nearest-even integer and leaves it, in two's complement, in the low
// mantissa bits, so the low byte of the sum's bit pattern IS the int8 code.  Valid while
// |t| < 2^22; for a finite row |t| <= 127*(1+2^-22) because inv came from the row's own
// amax, so the [-128,127] clamp of the scalar form can never bind and is dropped.  Rows
// that contain Inf or NaN give unspecified codes (as they do in the reference).
__device__ __forceinline__ uint32_t quant_rn_lowbyte(float x, float inv) {
    return __float_as_uint(__fadd_rn(__fmul_rn(x, inv), 12582912.0f));
}

// low bytes of four words -> one word (a in byte 0)
__device__ __forceinline__ uint32_t pack_lowbytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// group quantiser: true division by the stored scale, clamp, truncate toward zero
__device__ __forceinline__ int quant_trunc_div(float x, float scale) {
    float t = __fdiv_rn(x, scale);
    t = fmaxf(-128.0f, fminf(127.0f, t));
    return __float2int_rz(t);
}

// The same quotient without a division per element: with rcp = RN(1/scale) computed once per
// group, q0 = RN(x*rcp), r = fma(-q0, scale, x) (the exact residual, rounded once) and
// q1 = fma(r, rcp, q0) is the correctly rounded x/scale for operands in the normal range
// (the final step of the standard division algorithm); below 1 in magnitude the truncation is
// zero whatever the last bit.  Checked against true division in the GPU tests.
// Returns the code in the low byte of the result (two's complement).  No clamp: for a finite group
// |x| <= amax and scale = RN(amax/127), so |x/scale| <= 127*(1+2^-23) and the truncation is within
// [-127, 127]; groups containing Inf or NaN give unspecified codes.
__device__ __forceinline__ uint32_t quant_trunc_div_rcp(float x, float scale, float rcp) {
    const float q0 = __fmul_rn(x, rcp);
    const float r = __fmaf_rn(-q0, scale, x);
    const float q1 = __fmaf_rn(r, rcp, q0);
    return (uint32_t)__float2int_rz(q1);
}

// Two elements at once with the packed f32x2 instructions (same three roundings per element).
// nscale2 holds -scale in both halves: the packed fma has no negate modifier.
__device__ __forceinline__ void quant_trunc_div_rcp2(float2 x, float2 nscale2, float2 rcp2, uint32_t& lo,
                                                     uint32_t& hi) {
    const float2 q0 = __fmul2_rn(x, rcp2);
    const float2 r = __ffma2_rn(q0, nscale2, x);
    const float2 q1 = __ffma2_rn(r, rcp2, q0);
    lo = (uint32_t)__float2int_rz(q1.x);
    hi = (uint32_t)__float2int_rz(q1.y);
}

// RN(a / 127) without the division routine, for a >= kAmaxFloor: q0 = RN(a * RN(1/127)) is within
// one ulp of the quotient, the remainder a - 127*q0 is exact in one fma, and the corrected quotient
// rounds correctly (the same closing step as above).  Checked against __fdiv_rn for every bf16
// magnitude in the GPU tests.
constexpr float kRcp127 = 1.0f / 127.0f;   // correctly rounded: 0x3C010204
__device__ __forceinline__ float div127_rn(float a) {
    const float q0 = __fmul_rn(a, kRcp127);
    const float r = __fmaf_rn(q0, -127.0f, a);
    return __fmaf_rn(r, kRcp127, q0);
}

__device__ __forceinline__ uint32_t pack_i8x4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
           ((uint32_t)(d & 0xff) << 24);
}

// ---- exp / sigmoid ----------------------------------------------------------------
// exp_fixed(x) for x clamped to [-87, 87]:
//   z = fma(x, log2e, 1.5*2^23)        (round x*log2e to an integer n in the low bits)
//   n = z - 1.5*2^23
//   r = fma(n, -ln2_hi, x); r = fma(n, -ln2_lo, r)
//   p = 1 + r*(1 + r*(c2 + r*(c3 + r*(c4 + r*(c5 + r*c6)))))   (Horner, all fma)
//   result = p * 2^n   (added to the exponent field; p*2^n stays a normal number)
// Maximum observed error against a double-precision exp: 2.6 ulp of the result.
constexpr float kExpClamp = 87.0f;
constexpr float kLog2e = 1.44269502162933349609375f;        // 0x3FB8AA3B
constexpr float kRoundMagic = 12582912.0f;                  // 1.5 * 2^23
constexpr float kLn2Hi = 0.693145751953125f;                // 0x3F317200
constexpr float kLn2Lo = 1.428606765330187045e-06f;         // 0x35BFBE8E
constexpr float kExpC2 = 0.5f;
constexpr float kExpC3 = 0.16666667163372039794921875f;     // 0x3E2AAAAB
constexpr float kExpC4 = 0.0416666679084300994873046875f;   // 0x3D2AAAAB
constexpr float kExpC5 = 0.008333333767950534820556640625f; // 0x3C088889
constexpr float kExpC6 = 0.001388888922519981861114501953125f;  // 0x3AB60B61

__device__ __forceinline__ float exp_fixed(float x) {
    x = fminf(fmaxf(x, -kExpClamp), kExpClamp);
    float z = __fmaf_rn(x, kLog2e, kRoundMagic);
    float n = __fadd_rn(z, -kRoundMagic);
    float r = __fmaf_rn(n, -kLn2Hi, x);
    r = __fmaf_rn(n, -kLn2Lo, r);
    float p = __fmaf_rn(r, kExpC6, kExpC5);
    p = __fmaf_rn(r, p, kExpC4);
    p = __fmaf_rn(r, p, kExpC3);
    p = __fmaf_rn(r, p, kExpC2);
    p = __fmaf_rn(r, p, 1.0f);
    p = __fmaf_rn(r, p, 1.0f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(z) << 23));
}

// sigmoid(g) = 1/(1+exp(-g)); __frcp_rn is the correctly rounded reciprocal == IEEE 1.0f / x
__device__ __forceinline__ float sigmoid_fixed(float g) {
    return __frcp_rn(__fadd_rn(1.0f, exp_fixed(-g)));
}

// h = ((1/(1+exp(-g))) * g) * u, each step rounded to f32
__device__ __forceinline__ float silu_mul(float g, float u) {
    return __fmul_rn(__fmul_rn(sigmoid_fixed(g), g), u);
}

// ---- silu by table ------------------------------------------------------------------------
// The gate is bf16: only 65536 inputs exist.  A kernel may tabulate silu(g) = RN(sigmoid_fixed(g)*g)
// for the inputs with 2^-12 <= |g| < 2^20 (4096 bit patterns per sign, 8192 floats = 32 KB of shared
// memory) and look values up instead of recomputing them; inputs outside that range (zeros,
// tiny, huge, Inf, NaN) are computed.  The table holds the computation's own results, so a lookup
// returns exactly the same bits.
constexpr uint32_t kSigTabLo = 0x3980u;    // bf16 bits of 2^-12
constexpr int kSigTabEntries = 8192;

// Entry i < 4096 holds silu(g) = RN(sigmoid_fixed(g) * g) for the positive gate with bf16 bits
// kSigTabLo + i; entry i >= 4096 the negative gate with magnitude bits kSigTabLo + (8191 - i).
// With t = gate bits - kSigTabLo (mod 2^16) that is entry (t ^ (sign ? 0xffff : 0)) & 0x1fff.
// Two thirds of the range need no exp: for g >= 32, exp_fixed(-g) < 2^-24, so 1 + exp rounds to 1 and
// sigmoid_fixed(g) is exactly 1 (silu = g); for g <= -88 the exponent argument is clamped, so
// sigmoid_fixed(g) is the one constant sigmoid_fixed(-88).  Same bits as the general formula.
__device__ __forceinline__ float silu_table_entry(int i) {
    const uint32_t bits = i < 4096 ? (kSigTabLo + (uint32_t)i) : (0x8000u | (kSigTabLo + (uint32_t)(8191 - i)));
    const float g = __uint_as_float(bits << 16);
    if (g >= 32.0f) return g;
    if (g <= -88.0f) return __fmul_rn(sigmoid_fixed(-88.0f), g);
    return __fmul_rn(sigmoid_fixed(g), g);
}

// ---- two-lane forms ------------------------------------------------------------------
// The same operation sequences on float2 with the packed fma.rn.f32x2 / mul / add of
// sm_100: each half is an independent, correctly rounded binary32 operation, so results
// are bit-identical to the scalar forms while needing half the issue slots.
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }

__device__ __forceinline__ float2 bf16x2_to_f32x2(uint32_t w) {
    return make_float2(bf16lo_to_f32(w), bf16hi_to_f32(w));
}

__device__ __forceinline__ float2 exp_fixed2(float2 x) {
    x.x = fminf(fmaxf(x.x, -kExpClamp), kExpClamp);
    x.y = fminf(fmaxf(x.y, -kExpClamp), kExpClamp);
    const float2 z = __ffma2_rn(x, splat2(kLog2e), splat2(kRoundMagic));
    const float2 n = __fadd2_rn(z, splat2(-kRoundMagic));
    float2 r = __ffma2_rn(n, splat2(-kLn2Hi), x);
    r = __ffma2_rn(n, splat2(-kLn2Lo), r);
    float2 p = __ffma2_rn(r, splat2(kExpC6), splat2(kExpC5));
    p = __ffma2_rn(r, p, splat2(kExpC4));
    p = __ffma2_rn(r, p, splat2(kExpC3));
    p = __ffma2_rn(r, p, splat2(kExpC2));
    p = __ffma2_rn(r, p, splat2(1.0f));
    p = __ffma2_rn(r, p, splat2(1.0f));
    return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(z.x) << 23)),
                       __int_as_float(__float_as_int(p.y) + (__float_as_int(z.y) << 23)));
}

__device__ __forceinline__ float2 silu_mul2(float2 g, float2 u) {
    const float2 e = exp_fixed2(make_float2(-g.x, -g.y));
    const float2 d = __fadd2_rn(splat2(1.0f), e);
    const float2 sig = make_float2(__frcp_rn(d.x), __frcp_rn(d.y));
    return __fmul2_rn(__fmul2_rn(sig, g), u);
}

// int8 codes of two values in the low bytes of the two returned words (see quant_rn_lowbyte).
// Deliberately the scalar rounded multiply and add, not the packed f32x2 pair: the product must be
// rounded before the add (x*inv can land exactly on a half after rounding and then rounds to even),
// and a packed mul followed by a packed add came out of the assembler as one fused operation,
// which rounds the unrounded product instead (1 code in 3 M differed, always on such ties).
__device__ __forceinline__ float2 quant_rn_lowbyte2(float2 x, float2 inv2) {
    return make_float2(__fadd_rn(__fmul_rn(x.x, inv2.x), kRoundMagic), __fadd_rn(__fmul_rn(x.y, inv2.y), kRoundMagic));
}

// The same rounding sequence with the packed instructions: RN(x*inv) by the packed multiply, then
// the magic constant added by a packed fma whose multiplier `one2` is 1.0 taken from a run-time
// value, so the assembler sees an ordinary fma of an already rounded product and cannot merge the
// two steps.  RN(p * 1 + magic) = RN(p + magic).
__device__ __forceinline__ float2 quant_rn_lowbyte2(float2 x, float2 inv2, float2 one2) {
    return __ffma2_rn(__fmul2_rn(x, inv2), one2, splat2(kRoundMagic));
}

// max(a, |b|, |c|) in one instruction (three-input max of sm_100)
__device__ __forceinline__ float max3_abs(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(fabsf(b)), "f"(fabsf(c)));
    return d;
}

// 0xffffffff if bit 15 of w is set, else 0: prmt with the sign-replicate flag (selector nibble 8 | 1)
// on all four result bytes.
__device__ __forceinline__ uint32_t sign_of_byte1(uint32_t w) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, 0x9999;" : "=r"(d) : "r"(w), "r"(0u));
    return d;
}

// h for the 8 gates / ups of one 16-byte vector pair; tab is the silu table.
// Both halves of a word are rebased with one subtraction (a borrow out of the low half only happens
// for a low gate below the table, which is a miss anyway) and one range test covers the vector:
// a gate hits iff bits 12..14 of its rebased pattern are clear (bit 15 is the sign).  If all 8
// gates hit, silu(g) is looked up, otherwise (rare: zeros, tiny or huge gates) the whole vector is
// computed.  Both give the same bits.
__device__ __forceinline__ void silu_mul8_table(const uint4& gv, const uint4& uv, const float* __restrict__ tab,
                                                float2 (&h)[4]) {
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    constexpr uint32_t kRebase = kSigTabLo | (kSigTabLo << 16);
    uint32_t t[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) t[i] = gw[i] - kRebase;
    if (((t[0] | t[1] | t[2] | t[3]) & 0x70007000u) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // the index is masked to the table's 8192 entries whatever the gate bits are
            const uint32_t sign_lo = sign_of_byte1(t[i]);
            const uint32_t sign_hi = (uint32_t)((int)t[i] >> 31);
            const uint32_t lo = (t[i] ^ sign_lo) & 0x1fffu;
            const uint32_t hi = ((t[i] >> 16) ^ sign_hi) & 0x1fffu;
            h[i] = __fmul2_rn(make_float2(tab[lo], tab[hi]), bf16x2_to_f32x2(uw[i]));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = silu_mul2(bf16x2_to_f32x2(gw[i]), bf16x2_to_f32x2(uw[i]));
    }
}

// rrms = 1 / sqrt(sumsq / n + eps)
__device__ __forceinline__ float rrms_from_sumsq(float sumsq, int n, float eps) {
    float mean = __fdiv_rn(sumsq, (float)n);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

// ---- reductions -------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// xor butterfly, offsets 16,8,4,2,1: after it every lane holds the same sum, and the
// association order is fixed (the oracle applies the same tree to 32 lane partials).
__device__ __forceinline__ float warp_sum_butterfly(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace w8a8
