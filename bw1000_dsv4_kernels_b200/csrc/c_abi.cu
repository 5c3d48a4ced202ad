// extern "C" entry points declared in include/dsv4_w8a8.h: argument checks, then the
// launchers.  Nothing here allocates, synchronises or touches torch.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>

#include "launch_common.h"

namespace w8a8 {
namespace {
thread_local char g_last_error[256] = "";
}

int fail(int code, const char* msg) {
    std::snprintf(g_last_error, sizeof g_last_error, "%s", msg);
    return code;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    std::snprintf(g_last_error, sizeof g_last_error, "%s: %s", what, cudaGetErrorString(e));
    return DSV4_ERR_LAUNCH;
}

namespace {
inline cudaStream_t cs(dsv4_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

int check_rows(const char* op, int M, int N) {
    if (M < 0 || N < 0) {
        char msg[128];
        std::snprintf(msg, sizeof msg, "%s: negative size (M=%d, N=%d)", op, M, N);
        return fail(DSV4_ERR_ARG, msg);
    }
    return 0;
}
#define DSV4_REQUIRE_PTR(op, ptr)                                                  \
    if ((ptr) == nullptr) return fail(DSV4_ERR_ARG, op ": null pointer " #ptr)
}  // namespace
}  // namespace w8a8

using namespace w8a8;

extern "C" {

int dsv4_abi_version(void) { return DSV4_ABI_VERSION; }
void dsv4_set_overlap_previous_kernel(int enable) { set_overlap_previous_kernel(enable); }
int dsv4_get_overlap_previous_kernel(void) { return overlap_previous_kernel(); }

const char* dsv4_last_error(void) { return g_last_error; }

int dsv4_device_status(dsv4_stream_t stream, int* status_out) { return read_device_status(cs(stream), status_out); }

int launch_ptq_strided(const void* x, int64_t ldx, void* q, void* s, int M, int N, dsv4_stream_t stream) {
    if (int rc = check_rows("per_token_quant_int8", M, N)) return rc;
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("per_token_quant_int8", x);
    DSV4_REQUIRE_PTR("per_token_quant_int8", q);
    DSV4_REQUIRE_PTR("per_token_quant_int8", s);
    if (ldx < N) return fail(DSV4_ERR_ARG, "per_token_quant_int8: row stride smaller than N");
    return ptq(x, q, s, M, N, ldx, cs(stream));
}

int launch_ptq(const void* x, void* q, void* s, int M, int N, dsv4_stream_t stream) {
    return launch_ptq_strided(x, N, q, s, M, N, stream);
}

int launch_ptgq(const void* x, void* q, void* s, int M, int N, int gs, dsv4_stream_t stream) {
    if (int rc = check_rows("per_token_group_quant_int8", M, N)) return rc;
    if (gs <= 0) return fail(DSV4_ERR_ARG, "per_token_group_quant_int8: group_size must be positive");
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("per_token_group_quant_int8", x);
    DSV4_REQUIRE_PTR("per_token_group_quant_int8", q);
    DSV4_REQUIRE_PTR("per_token_group_quant_int8", s);
    return ptgq(x, q, s, M, N, gs, cs(stream));
}

int launch_add_rmsnorm_quant(void* res, const void* x, const void* w, void* q, void* s, int M, int N,
                             float eps, dsv4_stream_t stream) {
    if (int rc = check_rows("add_rmsnorm_quant", M, N)) return rc;
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("add_rmsnorm_quant", res);
    DSV4_REQUIRE_PTR("add_rmsnorm_quant", x);
    DSV4_REQUIRE_PTR("add_rmsnorm_quant", w);
    DSV4_REQUIRE_PTR("add_rmsnorm_quant", q);
    DSV4_REQUIRE_PTR("add_rmsnorm_quant", s);
    return add_rmsnorm_quant(res, x, w, q, s, M, N, eps, cs(stream));
}

int launch_silu_mul_quant_strided(const void* g, int64_t ldg, const void* u, int64_t ldu, const int* mask,
                                  const int* valid_rows, void* q, void* s, int M, int N, dsv4_stream_t stream) {
    if (int rc = check_rows("silu_mul_quant", M, N)) return rc;
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("silu_mul_quant", g);
    DSV4_REQUIRE_PTR("silu_mul_quant", u);
    DSV4_REQUIRE_PTR("silu_mul_quant", q);
    DSV4_REQUIRE_PTR("silu_mul_quant", s);
    if (ldg < N || ldu < N) return fail(DSV4_ERR_ARG, "silu_mul_quant: row stride smaller than N");
    return silu_mul_quant(g, u, mask, valid_rows, q, s, M, N, ldg, ldu, cs(stream));
}

int launch_silu_mul_quant(const void* g, const void* u, void* q, void* s, int M, int N, dsv4_stream_t stream) {
    return launch_silu_mul_quant_strided(g, N, u, N, nullptr, nullptr, q, s, M, N, stream);
}

int launch_silu_mul_masked_quant(const void* g, const void* u, const int* mask, void* q, void* s, int M, int N,
                                 dsv4_stream_t stream) {
    return launch_silu_mul_quant_strided(g, N, u, N, mask, nullptr, q, s, M, N, stream);
}

int launch_silu_mul_quant_masked_layout(const void* g, int64_t ldg, const void* u, int64_t ldu, const int* masked_m,
                                        void* q, void* s, int E, int max_m, int N, dsv4_stream_t stream) {
    if (E < 0 || max_m < 0 || (int64_t)E * max_m > INT32_MAX)
        return fail(DSV4_ERR_ARG, "silu_and_mul_masked_post_quant: E and max_m must be non-negative and E * max_m fit in int32");
    const int M = E * max_m;
    if (int rc = check_rows("silu_and_mul_masked_post_quant", M, N)) return rc;
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("silu_and_mul_masked_post_quant", g);
    DSV4_REQUIRE_PTR("silu_and_mul_masked_post_quant", u);
    DSV4_REQUIRE_PTR("silu_and_mul_masked_post_quant", masked_m);
    DSV4_REQUIRE_PTR("silu_and_mul_masked_post_quant", q);
    DSV4_REQUIRE_PTR("silu_and_mul_masked_post_quant", s);
    if (ldg < N || ldu < N) return fail(DSV4_ERR_ARG, "silu_and_mul_masked_post_quant: row stride smaller than N");
    return silu_mul_quant(g, u, nullptr, nullptr, q, s, M, N, ldg, ldu, cs(stream), masked_m, max_m);
}

int launch_rmsnorm(void* x, int M, int N, float eps, dsv4_stream_t stream) {
    if (int rc = check_rows("rmsnorm", M, N)) return rc;
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("rmsnorm", x);
    return rmsnorm(x, M, N, eps, cs(stream));
}

int launch_rmsnorm_self(void* x, int M, int N, float eps, dsv4_stream_t stream) {
    return launch_rmsnorm(x, M, N, eps, stream);
}

int launch_silu_mul(const void* g, const void* u, void* out, int M, int N, dsv4_stream_t stream) {
    if (int rc = check_rows("silu_and_mul", M, N)) return rc;
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("silu_and_mul", g);
    DSV4_REQUIRE_PTR("silu_and_mul", u);
    DSV4_REQUIRE_PTR("silu_and_mul", out);
    return silu_mul(g, u, out, M, N, N, N, cs(stream));
}

int launch_silu_mul_strided(const void* g, long long ldg, const void* u, long long ldu, void* out, int M, int N,
                            dsv4_stream_t stream) {
    if (int rc = check_rows("silu_and_mul", M, N)) return rc;
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("silu_and_mul", g);
    DSV4_REQUIRE_PTR("silu_and_mul", u);
    DSV4_REQUIRE_PTR("silu_and_mul", out);
    if (ldg < N || ldu < N) return fail(DSV4_ERR_ARG, "silu_and_mul: row stride smaller than N");
    return silu_mul(g, u, out, M, N, ldg, ldu, cs(stream));
}

int launch_w8a8_gemm(const void* A, const void* B, const void* sa, const void* sb, void* C, int M, int N, int K,
                     dsv4_stream_t stream) {
    GemmArgs a{};
    a.A = A; a.B = B; a.sa = static_cast<const float*>(sa); a.sb = static_cast<const float*>(sb); a.C = C;
    a.offsets = nullptr; a.M = M; a.N = N; a.K = K; a.E = 1; a.sa_groups = 1; a.out_i32 = 0;
    return gemm_i8(a, cs(stream));
}

// Test hook, deliberately not declared in include/dsv4_w8a8.h: the same launch as launch_w8a8_gemm (or
// launch_grouped_gemm when expert_offsets is not null), except that the kernel's producer issues no tile
// loads and every bounded wait gives up after wait_limit_ns.  All consumer waits of the launch therefore
// run out: the kernel must record the wait site in the device status word, leave through its normal
// teardown (tensor memory freed) and return; nothing is written to C.  The launch itself returns 0.
DSV4_API int dsv4_test_gemm_wait_expiry(const void* A, const void* B, const void* sa, const void* sb, void* C, int M,
                                        int N, int K, const int* expert_offsets, int E,
                                        unsigned long long wait_limit_ns, dsv4_stream_t stream) {
    GemmArgs a{};
    a.A = A; a.B = B; a.sa = static_cast<const float*>(sa); a.sb = static_cast<const float*>(sb); a.C = C;
    a.offsets = expert_offsets; a.M = M; a.N = N; a.K = K; a.E = expert_offsets ? E : 1; a.sa_groups = 1; a.out_i32 = 0;
    a.test_withhold_loads = 1;
    a.test_wait_limit_ns = wait_limit_ns ? wait_limit_ns : 1000000ull;
    return gemm_i8(a, cs(stream));
}

int launch_w8a8_gemm_v5(const void* A, const void* B, const void* sa, const void* sb, void* C, int M, int N,
                        int K, dsv4_stream_t stream) {
    return launch_w8a8_gemm(A, B, sa, sb, C, M, N, K, stream);
}

int launch_w8a8_gemm_i32(const void* A, const void* B, void* C, int M, int N, int K, dsv4_stream_t stream) {
    GemmArgs a{};
    a.A = A; a.B = B; a.sa = nullptr; a.sb = nullptr; a.C = C;
    a.offsets = nullptr; a.M = M; a.N = N; a.K = K; a.E = 1; a.sa_groups = 1; a.out_i32 = 1;
    return gemm_i8(a, cs(stream));
}

int launch_scale_convert(const void* int_out, const void* sa, const void* sb, void* bf_out, int M, int N,
                         dsv4_stream_t stream) {
    if (int rc = check_rows("scale_convert", M, N)) return rc;
    if (M == 0 || N == 0) return 0;
    DSV4_REQUIRE_PTR("scale_convert", int_out);
    DSV4_REQUIRE_PTR("scale_convert", sa);
    DSV4_REQUIRE_PTR("scale_convert", sb);
    DSV4_REQUIRE_PTR("scale_convert", bf_out);
    return scale_convert(int_out, sa, sb, bf_out, M, N, cs(stream));
}

int launch_grouped_gemm(const void* A, const void* W, const void* sa, const void* sw, const int* expert_offsets,
                        void* C, int R, int E, int N, int K, int sa_groups, dsv4_stream_t stream) {
    if (expert_offsets == nullptr) return fail(DSV4_ERR_ARG, "grouped_gemm: null pointer expert_offsets");
    GemmArgs a{};
    a.A = A; a.B = W; a.sa = static_cast<const float*>(sa); a.sb = static_cast<const float*>(sw); a.C = C;
    a.offsets = expert_offsets; a.M = R; a.N = N; a.K = K; a.E = E; a.sa_groups = sa_groups; a.out_i32 = 0;
    return gemm_i8(a, cs(stream));
}

int launch_grouped_gemm_scatter(const void* A, const void* W, const void* sa, const void* sw, const int* expert_offsets,
                                void* const* row_ptr, int R, int E, int N, int K, dsv4_stream_t stream) {
    if (expert_offsets == nullptr) return fail(DSV4_ERR_ARG, "grouped_gemm_scatter: null pointer expert_offsets");
    if (row_ptr == nullptr) return fail(DSV4_ERR_ARG, "grouped_gemm_scatter: null pointer row_ptr");
    GemmArgs a{};
    a.A = A; a.B = W; a.sa = static_cast<const float*>(sa); a.sb = static_cast<const float*>(sw); a.C = nullptr;
    a.row_ptr = row_ptr;
    a.offsets = expert_offsets; a.M = R; a.N = N; a.K = K; a.E = E; a.sa_groups = 1; a.out_i32 = 0;
    return gemm_i8(a, cs(stream));
}

int launch_moe_push_rows(const int* dst_slot, int T, int topk, int tokens_per_rank, void* const* inbox_ranks,
                         int num_ranks, int H, void** row_ptr, dsv4_stream_t stream) {
    return moe_push_rows(dst_slot, T, topk, tokens_per_rank, inbox_ranks, num_ranks, H, row_ptr, cs(stream));
}

int launch_grouped_gemm_masked(const void* A, const void* W, const void* sa, const void* sw, const int* masked_m,
                               void* C, int E, int max_m, int N, int K, int sa_groups, dsv4_stream_t stream) {
    if (masked_m == nullptr) return fail(DSV4_ERR_ARG, "grouped_gemm_masked: null pointer masked_m");
    if (E <= 0 || max_m < 0 || (int64_t)E * max_m > INT32_MAX)
        return fail(DSV4_ERR_ARG, "grouped_gemm_masked: E must be positive, max_m non-negative and E * max_m fit in int32");
    if (max_m == 0) return 0;
    GemmArgs a{};
    a.A = A; a.B = W; a.sa = static_cast<const float*>(sa); a.sb = static_cast<const float*>(sw); a.C = C;
    a.offsets = nullptr; a.masked_m = masked_m; a.max_m = max_m;
    a.M = E * max_m; a.N = N; a.K = K; a.E = E; a.sa_groups = sa_groups; a.out_i32 = 0;
    return gemm_i8(a, cs(stream));
}

int launch_moe_segments(const int* topk_ids, int T, int topk, int E, int expert_lo, int* expert_offsets,
                        int* src_row, int* dst_slot, dsv4_stream_t stream) {
    if (expert_lo < 0) return fail(DSV4_ERR_ARG, "moe_segments: expert_lo must not be negative");
    return moe_segments(topk_ids, T, topk, E, expert_lo, expert_offsets, src_row, dst_slot, cs(stream));
}

int launch_gather_rows(const void* src, const int* src_row, void* dst, int R, int row_bytes,
                       const float* src_scale, float* dst_scale, int scales_per_row, const int* valid_rows,
                       dsv4_stream_t stream) {
    return gather_rows(src, src_row, dst, R, row_bytes, src_scale, dst_scale, scales_per_row, valid_rows, cs(stream));
}

int launch_moe_topk(const float* logits, int T, int E, int k, int* topk_ids, float* topk_w, dsv4_stream_t stream) {
    return moe_topk(logits, T, E, k, topk_ids, topk_w, cs(stream));
}

int launch_moe_combine(const void* z, const int* dst_slot, const float* topk_w, void* out, int T, int topk, int H,
                       int out_f32, dsv4_stream_t stream) {
    return moe_combine(z, dst_slot, topk_w, out, T, topk, H, out_f32, cs(stream));
}

int launch_moe_combine_exchange(const void* const* z_ranks, const int* const* slot_ranks, const int* topk_ids,
                                const float* topk_w, void* const* out_ranks, int num_ranks, int experts_per_rank,
                                int t0, int t1, int topk, int H, dsv4_stream_t stream) {
    return moe_combine_exchange(z_ranks, slot_ranks, topk_ids, topk_w, out_ranks, num_ranks, experts_per_rank, t0, t1,
                                topk, H, cs(stream));
}

int launch_w8a8_gemm_allgather(const void* A, const void* B, const void* sa, const void* sb, void* C_local,
                               void* const* C_peers, int npeers, int64_t ldc, int M, int N, int K,
                               dsv4_stream_t stream) {
    if (npeers < 0 || npeers > 7) return fail(DSV4_ERR_ARG, "w8a8_gemm_allgather: npeers must be in 0..7");
    if (npeers > 0 && C_peers == nullptr) return fail(DSV4_ERR_ARG, "w8a8_gemm_allgather: null pointer C_peers");
    GemmArgs a{};
    a.A = A; a.B = B; a.sa = static_cast<const float*>(sa); a.sb = static_cast<const float*>(sb); a.C = C_local;
    a.offsets = nullptr; a.M = M; a.N = N; a.K = K; a.E = 1; a.ldc = ldc; a.sa_groups = 1; a.out_i32 = 0;
    a.npeers = npeers;
    for (int d = 0; d < npeers; ++d) a.peerC[d] = C_peers[d];
    return gemm_i8(a, cs(stream));
}

int launch_w8a8_gemm_ld(const void* A, const void* B, const void* sa, const void* sb, void* C, int64_t ldc, int M,
                        int N, int K, dsv4_stream_t stream) {
    GemmArgs a{};
    a.A = A; a.B = B; a.sa = static_cast<const float*>(sa); a.sb = static_cast<const float*>(sb); a.C = C;
    a.offsets = nullptr; a.M = M; a.N = N; a.K = K; a.E = 1; a.ldc = ldc; a.sa_groups = 1; a.out_i32 = 0;
    return gemm_i8(a, cs(stream));
}

}  // extern "C"
