/* C-ABI of the B200 (sm_100a) W8A8 linear path.
 *
 * This is the boundary a host program binds instead of the reference's HIP launchers.
 * Every entry point takes plain device pointers and sizes, launches asynchronously on
 * the given CUDA stream (0 = the legacy default stream), never synchronises the host
 * and never allocates device memory.  All of them return an int status: 0 on success,
 * one of the DSV4_ERR_* codes otherwise; dsv4_last_error() then gives a message for
 * the calling thread.  (The reference launchers return void and report nothing.)
 *
 * Layouts: activations bf16 row-major; int8 codes row-major with the shape of the
 * activation; scales fp32.  "M" is rows (tokens), "N" the row length of the
 * quantisers (the reference's naming) and the output width of the GEMMs.
 *
 * Citations are file:line in the reference project (hip_kernels/...).
 */
#ifndef DSV4_W8A8_H
#define DSV4_W8A8_H

#include <stdint.h>

#if defined(__GNUC__)
#define DSV4_API __attribute__((visibility("default")))
#else
#define DSV4_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without pulling in the CUDA headers */
typedef struct CUstream_st* dsv4_stream_t;

enum {
    DSV4_OK = 0,
    DSV4_ERR_ARG = 1,         /* null pointer, negative size, unsupported stride/alignment */
    DSV4_ERR_LAUNCH = 2,      /* the CUDA runtime rejected the launch */
    DSV4_ERR_DRIVER = 3,      /* tensor-map creation failed / driver entry point missing */
    DSV4_ERR_DEVICE_WAIT = 4  /* a bounded wait in an earlier GEMM kernel on this device gave up; returned once by
                                 the next GEMM launch, which launches nothing (see dsv4_device_status) */
};

#define DSV4_ABI_VERSION 1
DSV4_API int dsv4_abi_version(void);

/* Message for the last non-zero status returned on this thread ("" if none). */
DSV4_API const char* dsv4_last_error(void);

/* Synchronises `stream`, then reads and clears the current device's sticky status word
 * that the GEMM kernels set when one of their bounded waits ran out (0 = none).
 * Intended for tests and post-mortems; the launch path never calls it. */
DSV4_API int dsv4_device_status(dsv4_stream_t stream, int* status_out);

/* Option of the CALLING THREAD, off by default (no reference counterpart): it affects the launches this
 * thread makes afterwards, on any stream, and nobody else's.  When enabled, the dense GEMM
 * launchers (not the grouped ones) start with programmatic dependent launch: the
 * kernel may begin while the kernel before it on the stream is still running, sets itself up and
 * starts streaming the WEIGHT, and waits for that kernel to complete only before it reads the
 * activations and their scales or writes its output.  The row kernels of this library let such a
 * dependent start as soon as they are running.  Contract when enabled: the weight and its channel
 * scales must not be written by the kernel that directly precedes the GEMM on the stream (a weight
 * update, a dequantisation, a LoRA merge): the GEMM would read them before that kernel has finished,
 * and nothing reports it. */
DSV4_API void dsv4_set_overlap_previous_kernel(int enable);
DSV4_API int dsv4_get_overlap_previous_kernel(void);

/* ---- activation quantisers ------------------------------------------------------ */

/* per_token_quant_int8.  x bf16 [M,N] contiguous -> q int8 [M,N], s fp32 [M].
 * Replaces launch_ptq, dsv4_all_hip_kernels.hip:343-345 (kernel :27-43). */
DSV4_API int launch_ptq(const void* x, void* q, void* s, int M, int N, dsv4_stream_t stream);

/* Same, with a row stride for x in elements (x may be a column slice of a wider tensor). */
DSV4_API int launch_ptq_strided(const void* x, int64_t ldx, void* q, void* s, int M, int N,
                       dsv4_stream_t stream);

/* per_token_group_quant_int8.  x bf16 [M,N] contiguous -> q int8 [M,N],
 * s fp32 [M, ceil(N/gs)] row-major.  q = trunc(clamp(x / s, -128, 127)).
 * Replaces launch_ptgq, dsv4_all_hip_kernels.hip:346-350 (kernel :49-86). */
DSV4_API int launch_ptgq(const void* x, void* q, void* s, int M, int N, int gs, dsv4_stream_t stream);

/* add_rmsnorm_quant.  res <- res + x (bf16, in place); y = rmsnorm(res + x) * w;
 * q,s = per-token quantisation of y.  res,x bf16 [M,N]; w bf16 [N].
 * Replaces launch_add_rmsnorm_quant exported by libdsv4_ops_hip.so
 * (kernel dsv4_native_ext.cpp:103-132). */
DSV4_API int launch_add_rmsnorm_quant(void* res, const void* x, const void* w, void* q, void* s, int M,
                             int N, float eps, dsv4_stream_t stream);

/* silu_mul_quant.  h = silu(g) * u in fp32, then per-token quantisation.
 * Replaces launch_silu_mul_quant exported by libdsv4_ops_hip.so
 * (kernel dsv4_native_ext.cpp:79-98). */
DSV4_API int launch_silu_mul_quant(const void* g, const void* u, void* q, void* s, int M, int N,
                          dsv4_stream_t stream);

/* Same with a row mask: rows whose mask[row] == 0 are skipped (q and s untouched).
 * Replaces launch_silu_mul_masked_quant, dsv4_all_hip_kernels.hip:362-366. */
DSV4_API int launch_silu_mul_masked_quant(const void* g, const void* u, const int* mask, void* q, void* s,
                                 int M, int N, dsv4_stream_t stream);

/* Same with row strides (elements) so that g and u can be the halves of one packed
 * [M, 2N] gate_up tensor.  mask may be null.  valid_rows may be null; otherwise it points to
 * one int32 ON THE DEVICE and only rows below min(M, *valid_rows) are processed (the row count
 * of an expert-parallel rank is only known on the device). */
DSV4_API int launch_silu_mul_quant_strided(const void* g, int64_t ldg, const void* u, int64_t ldu,
                                  const int* mask, const int* valid_rows, void* q, void* s, int M,
                                  int N, dsv4_stream_t stream);

/* The same on the masked expert layout of an expert-parallel prefill: the rows are E blocks of max_m
 * (g, u: [E * max_m, N] with row strides ldg, ldu, e.g. the halves of one packed [E, max_m, 2N] tensor),
 * masked_m int32 [E] ON THE DEVICE, and only the first masked_m[e] rows of block e are processed
 * (q int8 [E * max_m, N] and s fp32 [E * max_m] of the other rows are untouched; values above max_m
 * count as max_m).  The engine's silu_and_mul_masked_post_quant (DSV4_OPERATOR_ANALYSIS.md:45), whose
 * kernel in the reference takes a per-row flag list instead (dsv4_all_hip_kernels.hip:172-196). */
DSV4_API int launch_silu_mul_quant_masked_layout(const void* g, int64_t ldg, const void* u, int64_t ldu,
                                        const int* masked_m, void* q, void* s, int E, int max_m, int N,
                                        dsv4_stream_t stream);

/* ---- unfused neighbours --------------------------------------------------------- */

/* x <- x * rsqrt(mean(x^2) + eps), in place, no gamma.
 * Replaces launch_rmsnorm (libdsv4_ops_hip.so) / launch_rmsnorm_self,
 * dsv4_all_hip_kernels.hip:351-353. */
DSV4_API int launch_rmsnorm(void* x, int M, int N, float eps, dsv4_stream_t stream);
DSV4_API int launch_rmsnorm_self(void* x, int M, int N, float eps, dsv4_stream_t stream);

/* out = bf16(silu(g) * u).  Replaces launch_silu_mul, dsv4_all_hip_kernels.hip:359-361. */
DSV4_API int launch_silu_mul(const void* g, const void* u, void* out, int M, int N, dsv4_stream_t stream);
/* Same with row strides ldg / ldu (elements) for gate and up, e.g. the two halves of a packed
 * gate_up [M, 2N] tensor as the reference's wrapper slices them (dsv4_native_ext.cpp:327-346);
 * out is dense [M, N]. */
DSV4_API int launch_silu_mul_strided(const void* g, long long ldg, const void* u, long long ldu, void* out, int M,
                       int N, dsv4_stream_t stream);

/* ---- int8 GEMM ------------------------------------------------------------------ */

/* C[m,n] = bf16((float(sum_k A[m,k]*B[n,k]) * sa[m]) * sb[n]).
 * A int8 [M,K], B int8 [N,K] (both K contiguous), sa fp32 [M], sb fp32 [N], C bf16 [M,N].
 * K must be a multiple of 16 and A, B 16-byte aligned (TMA requirements).
 * Replaces launch_w8a8_gemm_v5, w8a8_gemm_v5.hip:128-145. */
DSV4_API int launch_w8a8_gemm(const void* A, const void* B, const void* sa, const void* sb, void* C, int M,
                     int N, int K, dsv4_stream_t stream);
DSV4_API int launch_w8a8_gemm_v5(const void* A, const void* B, const void* sa, const void* sb, void* C,
                        int M, int N, int K, dsv4_stream_t stream);

/* Same with a row stride for C in elements (ldc >= N): the result can be written straight
 * into a column slab of a wider [M, ldc] buffer, as a column-sharded linear layer needs. */
DSV4_API int launch_w8a8_gemm_ld(const void* A, const void* B, const void* sa, const void* sb, void* C,
                        int64_t ldc, int M, int N, int K, dsv4_stream_t stream);

/* Fused GEMM + all-gather for a column-sharded linear layer.  The tile epilogue stages the bf16 tile in
 * shared memory, 64 columns at a time, and sends every piece with TMA tile stores to C_local and, over
 * NVLink, to the npeers <= 7 buffers in C_peers (in the order given): host array of DEVICE pointers into
 * the other ranks' output buffers, mapped into this process (CUDA IPC / symmetric memory), each already
 * offset to this rank's column slab; all share the row stride ldc.  (Problems too small for the CTA-pair
 * kernel store 64-byte pieces with plain stores instead.)  N % 32 == 0.  The caller orders the ranks
 * afterwards (a barrier) before anyone reads a full row.  No counterpart in the reference, which has no
 * collective code. */
DSV4_API int launch_w8a8_gemm_allgather(const void* A, const void* B, const void* sa, const void* sb,
                               void* C_local, void* const* C_peers, int npeers, int64_t ldc, int M,
                               int N, int K, dsv4_stream_t stream);

/* Raw accumulators: C int32 [M,N] = sum_k A[m,k]*B[n,k].  The product torch._int_mm
 * supplies in w8a8_gemm_intmm_fused.hip:38-39. */
DSV4_API int launch_w8a8_gemm_i32(const void* A, const void* B, void* C, int M, int N, int K,
                         dsv4_stream_t stream);

/* bf_out[m,n] = bf16((float(int_out[m,n]) * sa[m]) * sb[n]).
 * Replaces launch_scale_convert, w8a8_gemm_intmm_fused.hip:40-52. */
DSV4_API int launch_scale_convert(const void* int_out, const void* sa, const void* sb, void* bf_out, int M,
                         int N, dsv4_stream_t stream);

/* ---- MoE grouped GEMM ----------------------------------------------------------- */

/* Rows of A are sorted by expert; expert e owns rows [expert_offsets[e], expert_offsets[e+1])
 * (int32, on the device, E+1 entries, non-decreasing, last <= R; rows past R and experts whose
 * entries decrease are skipped rather than trusted).
 *   sa_groups == 1 : C[r,n] = bf16((float(acc[r,n]) * sa[r]) * sw[e,n])
 *   sa_groups == K/128 : sa is [R, K/128];
 *       C[r,n] = bf16(y * sw[e,n]),  y = fma(float(acc_g[r,n]), sa[r,g], y) for g = 0,1,...
 *       where acc_g is the exact int32 sum over the g-th 128 columns of K.
 * A int8 [R,K]; W int8 [E,N,K]; sw fp32 [E,N]; C bf16 [R,N].
 * The reference lists grouped_gemm without source (README.md:66); the layout follows its
 * engine-side description (DSV4_OPERATOR_ANALYSIS.md:42-43). */
DSV4_API int launch_grouped_gemm(const void* A, const void* W, const void* sa, const void* sw,
                        const int* expert_offsets, void* C, int R, int E, int N, int K,
                        int sa_groups, dsv4_stream_t stream);

/* The same product on the masked expert layout that the engine's prefill GEMM
 * m_grouped_w8a8_gemm_nt_masked takes (DSV4_OPERATOR_ANALYSIS.md:43; the reference has no source for
 * it): A int8 [E, max_m, K], W int8 [E, N, K], sw fp32 [E, N], C bf16 [E, max_m, N], masked_m int32 [E]
 * ON THE DEVICE; expert e multiplies the first masked_m[e] rows of its block (values above max_m count
 * as max_m) and leaves the other rows of C untouched.  sa fp32 [E * max_m] (sa_groups == 1) or
 * [E * max_m, K/128] (sa_groups == K/128), arithmetic as above. */
DSV4_API int launch_grouped_gemm_masked(const void* A, const void* W, const void* sa, const void* sw,
                               const int* masked_m, void* C, int E, int max_m, int N, int K, int sa_groups,
                               dsv4_stream_t stream);

/* Router top-k.  logits fp32 [T,E] (E <= 1024) -> topk_ids int32 [T,k] in descending order of logit
 * (ties: lower expert index first), topk_w fp32 [T,k] = softmax over the k selected logits.
 * The engine's routing step (DSV4_OPERATOR_ANALYSIS.md:40); the reference has no kernel for it. */
DSV4_API int launch_moe_topk(const float* logits, int T, int E, int k, int* topk_ids, float* topk_w,
                    dsv4_stream_t stream);

/* Segment offsets and the token permutation from top-k routing ids.
 * topk_ids int32 [T, topk] -> expert_offsets int32 [E+1] for the E experts
 * [expert_lo, expert_lo + E) (expert_lo = 0 and E = all experts on one GPU; a slice under
 * expert parallelism);
 * src_row int32 [T*topk]: routed row r (in expert-sorted order) came from token src_row[r],
 *   valid for r < expert_offsets[E];
 * dst_slot int32 [T*topk]: pair (t, j) landed at routed row dst_slot[t*topk + j], or -1 when
 *   its expert is outside the slice.
 * Within an expert, rows keep increasing (t, j) order.  Uses no scratch memory. */
DSV4_API int launch_moe_segments(const int* topk_ids, int T, int topk, int E, int expert_lo,
                        int* expert_offsets, int* src_row, int* dst_slot, dsv4_stream_t stream);

/* dst[r, :] = src[src_row[r], :] for r < R (and r < *valid_rows when valid_rows, a device
 * pointer, is not null); rows of row_bytes bytes (multiple of 16); optionally the same gather
 * for fp32 scales with scales_per_row entries per row. */
DSV4_API int launch_gather_rows(const void* src, const int* src_row, void* dst, int R, int row_bytes,
                       const float* src_scale, float* dst_scale, int scales_per_row,
                       const int* valid_rows, dsv4_stream_t stream);

/* out[t, :] = sum_j topk_w[t,j] * z[dst_slot[t,j], :] over the token's top-k slots in order
 * (fp32 fma accumulation; slots equal to -1 are skipped).  z bf16 [R,H]; out bf16 [T,H], or
 * fp32 [T,H] when out_f32 != 0 (the partial sum an expert-parallel rank contributes). */
DSV4_API int launch_moe_combine(const void* z, const int* dst_slot, const float* topk_w, void* out, int T,
                       int topk, int H, int out_f32, dsv4_stream_t stream);

/* Expert-parallel combine fused with its exchange over peer memory (no reference counterpart: the
 * reference has no collective code, README.md:104).  num_ranks (1..8) ranks each hold z (their own
 * experts' outputs, bf16 [*,H]) and dst_slot (int32 [T*topk], -1 for experts of other ranks), the
 * expert e living on rank e / experts_per_rank; z_ranks / slot_ranks / out_ranks are HOST arrays of
 * num_ranks device pointers, all dereferenceable from this GPU (peer mappings).  For the tokens
 * t0 <= t < t1 this call computes out[t,:] = sum_j topk_w[t,j] * z_rank(j)[slot(j),:] in slot order
 * (the arithmetic of launch_moe_combine) and stores the bf16 row into every rank's out [T,H].  The
 * caller orders it after all ranks' z are complete and makes the stores visible afterwards (e.g.
 * symmetric-memory barriers on the stream). */
DSV4_API int launch_moe_combine_exchange(const void* const* z_ranks, const int* const* slot_ranks,
                       const int* topk_ids, const float* topk_w, void* const* out_ranks, int num_ranks,
                       int experts_per_rank, int t0, int t1, int topk, int H, dsv4_stream_t stream);

/* Expert-parallel down projection that delivers its rows itself (no reference counterpart, as above).
 * launch_grouped_gemm with per-token scales, except that row r of the result is stored to row_ptr[r]
 * (device array of R device addresses, each a bf16 row of N elements, possibly in another GPU's memory
 * mapped into this process; 16-byte aligned rows leave in 256-byte segments, others element by element)
 * instead of C + r * N.  With the table that
 * launch_moe_push_rows builds, every expert output row lands in the inbox of the rank that owns its token
 * while the GEMM is still streaming weights, so the owners' combine reads local memory only. */
DSV4_API int launch_grouped_gemm_scatter(const void* A, const void* W, const void* sa, const void* sw,
                       const int* expert_offsets, void* const* row_ptr, int R, int E, int N, int K,
                       dsv4_stream_t stream);
/* row_ptr[dst_slot[t*topk+j]] = inbox_ranks[g] + ((t - g*tokens_per_rank)*topk + j) * H elements, g = the
 * rank that owns token t (t / tokens_per_rank), for every pair whose dst_slot is not -1.  inbox_ranks is a
 * HOST array of num_ranks device pointers (bf16 [tokens_per_rank*topk, H] each); row_ptr is a device array
 * with one entry per segment row of this rank. */
DSV4_API int launch_moe_push_rows(const int* dst_slot, int T, int topk, int tokens_per_rank,
                       void* const* inbox_ranks, int num_ranks, int H, void** row_ptr, dsv4_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* DSV4_W8A8_H */
