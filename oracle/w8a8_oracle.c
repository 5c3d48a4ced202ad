/* CPU oracle for the W8A8 linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic of the reference's HIP kernels, used by the
 * tests, by the smoke check and by the benchmark's CPU-baseline legs as the checker
 * the CUDA kernels are compared with.  Nothing in the shipped package may call it.
 *
 * PARITY PIN.  The reference ships no executable tests, no golden vectors and no CPU
 * implementation for this path, and its sources are HIP for a device that is not
 * available, so the reference itself cannot be run: at byte level the parity of this
 * oracle is UNPINNED.  What pins it instead:
 *   - each function follows the cited reference lines step by step;
 *   - the order-independent parts (absolute maximum, int8 x int8 -> int32 dot products,
 *     the quantiser, the epilogue) are checked bit for bit against independent
 *     numpy / torch formulas in the CPU tests;
 *   - the order- or libm-dependent parts (sum of squares, 1/sqrt, exp) are checked
 *     against double-precision formulas with the tolerance the reference's own recorded
 *     runs had (int8 codes differing by at most 1).
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fPIC -shared  (see oracle/build_oracle.py).
 * -ffp-contract=off matters: a*b+c must round twice unless fmaf() is written.
 *
 * bf16 values travel as uint16_t bit patterns.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Number of OpenMP threads for the loops below (launchers often export OMP_NUM_THREADS=1);
 * n <= 0 leaves the current setting.  Returns the thread count now in effect. */
int oracle_set_num_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
}

/* ---- bf16 ------------------------------------------------------------------------- */
static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round to nearest even; NaN -> 0x7FFF (what the device conversion returns) */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* fmaxf as the device computes it: NaN operands are ignored */
static inline float max_ignoring_nan(float a, float b) { return fmaxf(a, b); }

/* ---- the per-row quantiser (hip_kernels/dsv4_native_ext.cpp:34-39) ----------------
 * am = max(amax, 1e-10); s = am/127; inv = 127/am; q = clamp(rint(x*inv), -128, 127) */
static inline void scale_from_amax(float amax, float* scale, float* inv) {
    float am = max_ignoring_nan(amax, 1e-10f);
    *scale = am / 127.0f;
    *inv = 127.0f / am;
}

static inline int8_t quant_rn(float x, float inv) {
    float r = rintf(x * inv); /* default rounding mode: nearest even */
    int q = (int)r;
    if (q < -128) q = -128;
    if (q > 127) q = 127;
    return (int8_t)q;
}

/* per_token_quant_int8: hip_kernels/dsv4_native_ext.cpp:24-40 */
void oracle_ptq(const uint16_t* x, int64_t ldx, int8_t* q, float* s, int M, int N) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const uint16_t* xr = x + (int64_t)m * ldx;
        float amax = 0.0f;
        for (int j = 0; j < N; ++j) amax = max_ignoring_nan(amax, fabsf(bf16_to_f32(xr[j])));
        float scale, inv;
        scale_from_amax(amax, &scale, &inv);
        s[m] = scale;
        for (int j = 0; j < N; ++j) q[(int64_t)m * N + j] = quant_rn(bf16_to_f32(xr[j]), inv);
    }
}

/* The wording of the benchmark configuration instead of the kernel's: s = amax/127,
 * q = clamp(round_half_even(x / s), -127, 127).  Kept to count how often the two
 * definitions disagree; it is not the primary definition. */
void oracle_ptq_divide_form(const uint16_t* x, int64_t ldx, int8_t* q, float* s, int M, int N) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const uint16_t* xr = x + (int64_t)m * ldx;
        float amax = 0.0f;
        for (int j = 0; j < N; ++j) amax = max_ignoring_nan(amax, fabsf(bf16_to_f32(xr[j])));
        float scale = max_ignoring_nan(amax, 1e-10f) / 127.0f;
        s[m] = scale;
        for (int j = 0; j < N; ++j) {
            int v = (int)rintf(bf16_to_f32(xr[j]) / scale);
            if (v < -127) v = -127;
            if (v > 127) v = 127;
            q[(int64_t)m * N + j] = (int8_t)v;
        }
    }
}

/* per_token_group_quant_int8: hip_kernels/dsv4_all_hip_kernels.hip:49-86.
 * Per (row, group): s = max(amax,1e-10)/127; q = (int8)(int)clamp(x / s, -128, 127),
 * i.e. division by the stored scale and truncation toward zero (:81-84).
 * Scales are [M, ceil(N/gs)]; the reference indexes rows by N/gs (:76), which is the
 * same whenever gs divides N. */
void oracle_ptgq(const uint16_t* x, int8_t* q, float* s, int M, int N, int gs) {
    const int G = (N + gs - 1) / gs;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        for (int g = 0; g < G; ++g) {
            const int j0 = g * gs, j1 = (j0 + gs < N) ? j0 + gs : N;
            float amax = 0.0f;
            for (int j = j0; j < j1; ++j)
                amax = max_ignoring_nan(amax, fabsf(bf16_to_f32(x[(int64_t)m * N + j])));
            const float scale = max_ignoring_nan(amax, 1e-10f) / 127.0f;
            s[(int64_t)m * G + g] = scale;
            for (int j = j0; j < j1; ++j) {
                float t = bf16_to_f32(x[(int64_t)m * N + j]) / scale;
                t = fmaxf(-128.0f, fminf(127.0f, t));
                q[(int64_t)m * N + j] = (int8_t)(int)t;
            }
        }
    }
}

/* ---- sum of squares in the build's fixed order --------------------------------------
 * The reference reduces with 64-lane wavefront shuffles (dsv4_native_ext.cpp:114-117),
 * an order that only exists on its hardware.  The order defined here depends on N only:
 * 256 lanes; element j belongs to lane (j/8) mod 256; a lane adds its elements in
 * increasing j as acc = acc + a*a; lanes are combined by an xor butterfly (offsets 16, 8,
 * 4, 2, 1) inside each group of 32, and the 8 group sums are added left to right. */
static float sum_squares_fixed_order(const float* a, int N) {
    float lane[256];
    for (int l = 0; l < 256; ++l) lane[l] = 0.0f;
    for (int v = 0; v * 8 < N; ++v) {
        const int l = v & 255;
        const int j1 = (v * 8 + 8 < N) ? v * 8 + 8 : N;
        float acc = lane[l];
        for (int j = v * 8; j < j1; ++j) {
            const float sq = a[j] * a[j];
            acc = acc + sq;
        }
        lane[l] = acc;
    }
    for (int o = 16; o > 0; o >>= 1) {
        float next[256];
        for (int l = 0; l < 256; ++l) next[l] = lane[l] + lane[l ^ o];
        memcpy(lane, next, sizeof lane);
    }
    float total = lane[0];
    for (int w = 1; w < 8; ++w) total = total + lane[32 * w];
    return total;
}

/* rrms = 1/sqrt(sum/N + eps).  The reference calls rsqrtf (:117), whose last bits are
 * device-specific; here sqrt and the division are the correctly rounded IEEE ones. */
static inline float rrms_from_sum(float sum, int N, float eps) {
    const float mean = sum / (float)N;
    return 1.0f / sqrtf(mean + eps);
}

/* add_rmsnorm_quant: hip_kernels/dsv4_native_ext.cpp:103-132.
 * a = res + x in fp32; res <- bf16(a) in place; the unrounded a feeds the norm (:112-113);
 * y = (a*rrms)*w (:121); then the per-row quantiser on y (:124-131). */
void oracle_add_rmsnorm_quant(uint16_t* res, const uint16_t* x, const uint16_t* w, int8_t* q, float* s,
                              int M, int N, float eps) {
#pragma omp parallel
    {
        float* a = (float*)malloc(sizeof(float) * (size_t)(N > 0 ? N : 1));
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            uint16_t* rr = res + (int64_t)m * N;
            const uint16_t* xr = x + (int64_t)m * N;
            for (int j = 0; j < N; ++j) {
                a[j] = bf16_to_f32(rr[j]) + bf16_to_f32(xr[j]);
                rr[j] = f32_to_bf16(a[j]);
            }
            const float rrms = rrms_from_sum(sum_squares_fixed_order(a, N), N, eps);
            float amax = 0.0f;
            for (int j = 0; j < N; ++j) {
                const float t = a[j] * rrms;
                a[j] = t * bf16_to_f32(w[j]);
                amax = max_ignoring_nan(amax, fabsf(a[j]));
            }
            float scale, inv;
            scale_from_amax(amax, &scale, &inv);
            s[m] = scale;
            for (int j = 0; j < N; ++j) q[(int64_t)m * N + j] = quant_rn(a[j], inv);
        }
        free(a);
    }
}

/* rmsnorm, in place, no gamma: hip_kernels/dsv4_native_ext.cpp:45-60 */
void oracle_rmsnorm(uint16_t* x, int M, int N, float eps) {
#pragma omp parallel
    {
        float* a = (float*)malloc(sizeof(float) * (size_t)(N > 0 ? N : 1));
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            uint16_t* xr = x + (int64_t)m * N;
            for (int j = 0; j < N; ++j) a[j] = bf16_to_f32(xr[j]);
            const float rrms = rrms_from_sum(sum_squares_fixed_order(a, N), N, eps);
            for (int j = 0; j < N; ++j) xr[j] = f32_to_bf16(a[j] * rrms);
        }
        free(a);
    }
}

/* ---- exp with a fixed operation sequence --------------------------------------------
 * The reference calls expf (:88), which differs in the last bits between math libraries.
 * This build defines exp as the following sequence of correctly rounded operations:
 *   x clamped to [-87, 87]
 *   z = fma(x, log2e, 1.5*2^23); n = z - 1.5*2^23          (n = nearest integer to x*log2e)
 *   r = fma(n, -ln2_hi, x); r = fma(n, -ln2_lo, r)
 *   p = 1 + r(1 + r(1/2 + r(1/6 + r(1/24 + r(1/120 + r/720)))))   Horner, every step an fma
 *   result = p * 2^n, formed by adding n to the exponent field of p. */
float oracle_exp(float x) {
    if (x < -87.0f) x = -87.0f;
    if (x > 87.0f) x = 87.0f;
    const float z = fmaf(x, 0x1.715476p+0f, 0x1.8p+23f);
    const float n = z - 0x1.8p+23f;
    float r = fmaf(n, -0x1.62e4p-1f, x);
    r = fmaf(n, -0x1.7f7d1cp-20f, r);
    float p = fmaf(r, 0x1.6c16c2p-10f, 0x1.111112p-7f);
    p = fmaf(r, p, 0x1.555556p-5f);
    p = fmaf(r, p, 0x1.555556p-3f);
    p = fmaf(r, p, 0.5f);
    p = fmaf(r, p, 1.0f);
    p = fmaf(r, p, 1.0f);
    uint32_t pb, zb;
    memcpy(&pb, &p, 4);
    memcpy(&zb, &z, 4);
    pb += zb << 23;
    float out;
    memcpy(&out, &pb, 4);
    return out;
}

/* h = ((1/(1+exp(-g)))*g)*u, every step rounded to fp32: dsv4_native_ext.cpp:88-89 */
static inline float silu_mul(float g, float u) {
    const float e = oracle_exp(-g);
    const float sig = 1.0f / (1.0f + e);
    const float t = sig * g;
    return t * u;
}

/* silu_and_mul -> bf16: hip_kernels/dsv4_native_ext.cpp:65-74 */
void oracle_silu_mul(const uint16_t* g, int64_t ldg, const uint16_t* u, int64_t ldu, uint16_t* out, int M,
                     int N) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int j = 0; j < N; ++j)
            out[(int64_t)m * N + j] =
                f32_to_bf16(silu_mul(bf16_to_f32(g[m * ldg + j]), bf16_to_f32(u[m * ldu + j])));
}

/* silu_mul_quant: hip_kernels/dsv4_native_ext.cpp:79-98; with mask != NULL it is
 * silu_mul_masked_quant, hip_kernels/dsv4_all_hip_kernels.hip:172-196 (rows with
 * mask[row]==0 are skipped, their outputs untouched). */
void oracle_silu_mul_quant(const uint16_t* g, int64_t ldg, const uint16_t* u, int64_t ldu, const int* mask,
                           int8_t* q, float* s, int M, int N) {
#pragma omp parallel
    {
        float* h = (float*)malloc(sizeof(float) * (size_t)(N > 0 ? N : 1));
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            if (mask && mask[m] == 0) continue;
            float amax = 0.0f;
            for (int j = 0; j < N; ++j) {
                h[j] = silu_mul(bf16_to_f32(g[m * ldg + j]), bf16_to_f32(u[m * ldu + j]));
                amax = max_ignoring_nan(amax, fabsf(h[j]));
            }
            float scale, inv;
            scale_from_amax(amax, &scale, &inv);
            s[m] = scale;
            for (int j = 0; j < N; ++j) q[(int64_t)m * N + j] = quant_rn(h[j], inv);
        }
        free(h);
    }
}

/* ---- GEMM ----------------------------------------------------------------------------
 * acc[m,n] = sum_k A[m,k]*B[n,k] in int32 (exact; the inner loop of
 * hip_kernels/dsv4_native_ext.cpp:181-185 and w8a8_gemm_v5.hip:103-108). */
void oracle_gemm_i32(const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            const int8_t* a = A + (int64_t)m * K;
            const int8_t* b = B + (int64_t)n * K;
            int32_t acc = 0;
            for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            C[(int64_t)m * N + n] = acc;
        }
}

/* out = bf16((float(acc)*sa[row])*sb[col]): hip_kernels/w8a8_gemm_intmm_fused.hip:34,
 * w8a8_gemm_v5.hip:123, dsv4_native_ext.cpp:190.  (float) of an int32 rounds to nearest
 * even, which matters once |acc| exceeds 2^24. */
void oracle_scale_convert(const int32_t* acc, const float* sa, const float* sb, uint16_t* out, int M, int N) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            const float t = (float)acc[(int64_t)m * N + n] * sa[m];
            out[(int64_t)m * N + n] = f32_to_bf16(t * sb[n]);
        }
}

void oracle_w8a8_gemm(const int8_t* A, const int8_t* B, const float* sa, const float* sb, uint16_t* out, int M,
                      int N, int K) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            const int8_t* a = A + (int64_t)m * K;
            const int8_t* b = B + (int64_t)n * K;
            int32_t acc = 0;
            for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            const float t = (float)acc * sa[m];
            out[(int64_t)m * N + n] = f32_to_bf16(t * sb[n]);
        }
}

/* MoE grouped GEMM.  The reference lists it without source (README.md:66); the definition
 * is the benchmark configuration's: rows [off[e], off[e+1]) of A use expert e's weights
 * W[e] ([N,K]) and channel scales sw[e].
 *   sa_groups == 1  : out = bf16((float(acc)*sa[r])*sw[e,n])
 *   sa_groups == K/128 : y = 0; for each 128-wide block g of K in order:
 *                        y = fma(float(acc_g), sa[r,g], y); out = bf16(y*sw[e,n]) */
void oracle_grouped_gemm(const int8_t* A, const int8_t* W, const float* sa, const float* sw,
                         const int32_t* off, uint16_t* out, int R, int E, int N, int K, int sa_groups) {
    (void)R;
    for (int e = 0; e < E; ++e) {
        const int r0 = off[e], r1 = off[e + 1];
#pragma omp parallel for collapse(2) schedule(static)
        for (int r = r0; r < r1; ++r)
            for (int n = 0; n < N; ++n) {
                const int8_t* a = A + (int64_t)r * K;
                const int8_t* b = W + ((int64_t)e * N + n) * K;
                float y;
                if (sa_groups == 1) {
                    int32_t acc = 0;
                    for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
                    y = (float)acc * sa[r];
                } else {
                    y = 0.0f;
                    for (int g = 0; g < sa_groups; ++g) {
                        const int k1 = (g * 128 + 128 < K) ? g * 128 + 128 : K;
                        int32_t acc = 0;
                        for (int k = g * 128; k < k1; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
                        y = fmaf((float)acc, sa[(int64_t)r * sa_groups + g], y);
                    }
                }
                out[(int64_t)r * N + n] = f32_to_bf16(y * sw[(int64_t)e * N + n]);
            }
    }
}

/* Stable counting sort of (token, slot) pairs by expert id, restricted to the experts
 * [lo, lo + E): pairs routed elsewhere get dst_slot -1 and no row. */
void oracle_moe_segments(const int32_t* ids, int T, int topk, int E, int lo, int32_t* off, int32_t* src_row,
                         int32_t* dst_slot) {
    const int R = T * topk;
    for (int e = 0; e <= E; ++e) off[e] = 0;
    for (int i = 0; i < R; ++i) {
        const int e = ids[i] - lo;
        if (e >= 0 && e < E) off[e + 1]++;
    }
    for (int e = 0; e < E; ++e) off[e + 1] += off[e];
    int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * (size_t)E);
    for (int e = 0; e < E; ++e) cur[e] = off[e];
    for (int i = 0; i < R; ++i) {
        const int e = ids[i] - lo;
        if (e >= 0 && e < E) {
            const int r = cur[e]++;
            src_row[r] = i / topk;
            dst_slot[i] = r;
        } else {
            dst_slot[i] = -1;
        }
    }
    free(cur);
}

/* Weighted sum of a token's expert outputs (the engine's moe_sum step,
 * DSV4_OPERATOR_ANALYSIS.md:48): acc = fma(w[t,j], z[slot], acc) over j in order, fp32;
 * out_bf16 (RNE) or out_f32, whichever is not NULL. */
void oracle_moe_combine(const uint16_t* z, const int32_t* dst_slot, const float* w, uint16_t* out_bf16,
                        float* out_f32, int T, int topk, int H) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < H; ++h) {
            float acc = 0.0f;
            for (int j = 0; j < topk; ++j) {
                const int slot = dst_slot[(int64_t)t * topk + j];
                if (slot < 0) continue;
                acc = fmaf(w[(int64_t)t * topk + j], bf16_to_f32(z[(int64_t)slot * H + h]), acc);
            }
            if (out_f32) out_f32[(int64_t)t * H + h] = acc;
            if (out_bf16) out_bf16[(int64_t)t * H + h] = f32_to_bf16(acc);
        }
}

/* The same weighted sum when the expert outputs are spread over G ranks (expert parallelism; the
 * reference leaves multi-GPU execution to the engine, README.md:104): expert e lives on rank
 * e / experts_per_rank, z_ranks[r] holds rank r's rows and slot_ranks[r] its own dst_slot map
 * (-1 for experts of other ranks).  Tokens t0 <= t < t1 only; rows outside are left untouched. */
void oracle_moe_combine_exchange(const uint16_t* const* z_ranks, const int32_t* const* slot_ranks,
                                 const int32_t* ids, const float* w, uint16_t* out_bf16, int G,
                                 int experts_per_rank, int t0, int t1, int topk, int H) {
#pragma omp parallel for schedule(static)
    for (int t = t0; t < t1; ++t)
        for (int h = 0; h < H; ++h) {
            float acc = 0.0f;
            for (int j = 0; j < topk; ++j) {
                const int64_t pair = (int64_t)t * topk + j;
                const int e = ids[pair];
                if (e < 0) continue;
                const int r = e / experts_per_rank;
                if (r >= G) continue;
                const int slot = slot_ranks[r][pair];
                if (slot < 0) continue;
                acc = fmaf(w[pair], bf16_to_f32(z_ranks[r][(int64_t)slot * H + h]), acc);
            }
            out_bf16[(int64_t)t * H + h] = f32_to_bf16(acc);
        }
}

/* Router top-k (the engine's routing step, DSV4_OPERATOR_ANALYSIS.md:40): k rounds of arg-max,
 * larger logit first, ties to the lower expert index; weights = softmax over the selected logits
 * with the first (largest) one subtracted, exp in fp32 (expf), sum in selection order. */
void oracle_moe_topk(const float* logits, int T, int E, int k, int32_t* ids, float* w) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        const float* row = logits + (int64_t)t * E;
        char* taken = (char*)calloc((size_t)E, 1);
        float first = 0.0f, denom = 0.0f;
        for (int r = 0; r < k; ++r) {
            int best = -1;
            for (int e = 0; e < E; ++e)
                if (!taken[e] && (best < 0 || row[e] > row[best])) best = e;
            taken[best] = 1;
            ids[(int64_t)t * k + r] = best;
            if (r == 0) first = row[best];
            const float x = expf(row[best] - first);
            w[(int64_t)t * k + r] = x;
            denom += x;
        }
        for (int r = 0; r < k; ++r) w[(int64_t)t * k + r] = w[(int64_t)t * k + r] / denom;
        free(taken);
    }
}
