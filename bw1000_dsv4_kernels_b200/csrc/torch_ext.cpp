// Python operator boundary: the pybind11 module `dsv4_native_ext`.
//
// It keeps the operator names, argument order, return shapes and the RuntimeError
// behaviour of the reference module (hip_kernels/dsv4_native_ext.cpp:314-444): every op
// exists as `name(...)` and as `name_stream(..., stream_ptr)` where stream_ptr is the raw
// stream handle (torch.cuda.current_stream().cuda_stream).  Each wrapper only checks its
// arguments, allocates the outputs with torch and forwards plain pointers to the C-ABI
// (include/dsv4_w8a8.h); there is no CPU path: a non-CUDA tensor raises.
//
// Streams: `name(...)` launches on torch's current stream; `name_stream(..., stream_ptr)` launches on the
// given stream and copies nothing, but its outputs still come from torch's caching allocator, which ties
// them to the CURRENT stream: a caller that passes another stream keeps the outputs alive (or calls
// record_stream on them) until that stream has run the kernel, as with any tensor used across streams.
//
// Differences from the reference, all additive or stricter:
//   * `name(...)` launches on torch's current stream rather than on stream 0;
//   * dtype / device / shape / alignment are checked (the reference checks contiguity only);
//   * silu ops accept row-strided 2-D views, so the halves of a packed gate_up work;
//   * new names: w8a8_gemm (alias), w8a8_gemm_i32, scale_convert,
//     per_token_group_quant_int8, silu_mul_masked_quant, grouped_gemm, moe_segments,
//     gather_rows, device_status;
//   * flash_mla_decode is not part of the W8A8 path and is not provided.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <string>
#include <vector>

#include "../../include/dsv4_w8a8.h"

namespace {

using torch::Tensor;

// `name(...)` variants pass this sentinel; it is resolved to torch's current stream on the
// tensors' device after the argument checks and the device guard.
constexpr int64_t kCurrentStream = INT64_MIN;
inline int64_t current_stream_ptr() { return kCurrentStream; }
inline dsv4_stream_t as_stream(int64_t stream_ptr) {
    if (stream_ptr == kCurrentStream) return reinterpret_cast<dsv4_stream_t>(at::cuda::getCurrentCUDAStream().stream());
    return reinterpret_cast<dsv4_stream_t>(stream_ptr);
}

void check_status(int rc) {
    TORCH_CHECK(rc == 0, "dsv4_native_ext: ", dsv4_last_error(), " (status ", rc, ")");
}

void check_cuda(const Tensor& t, const char* name, c10::ScalarType dtype) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (this extension has no CPU path)");
    TORCH_CHECK(t.scalar_type() == dtype, name, " must have dtype ", dtype, ", got ", t.scalar_type());
}

void check_same_device(const Tensor& a, const Tensor& b, const char* what) {
    TORCH_CHECK(a.device() == b.device(), what, ": tensors are on different devices");
}

int to_int(int64_t v, const char* what) {
    TORCH_CHECK(v >= 0 && v <= INT32_MAX, what, " does not fit in int32: ", v);
    return static_cast<int>(v);
}

struct Rows {
    int M, N;
};
Rows rows_of(const Tensor& x) {
    TORCH_CHECK(x.dim() >= 1, "expected at least one dimension");
    const int64_t n = x.size(-1);
    const int64_t m = n == 0 ? 0 : x.numel() / n;
    return {to_int(m, "rows"), to_int(n, "row length")};
}

// ---- per_token_quant_int8 (reference wrapper :314-324) ----------------------------
std::vector<Tensor> per_token_quant_int8_stream(Tensor x, int64_t stream_ptr) {
    TORCH_CHECK(x.is_contiguous());
    check_cuda(x, "x", torch::kBFloat16);
    c10::cuda::CUDAGuard guard(x.device());
    const Rows r = rows_of(x);
    auto q = torch::empty_like(x, x.options().dtype(torch::kInt8));
    auto s = torch::empty({r.M}, x.options().dtype(torch::kFloat32));
    check_status(launch_ptq(x.data_ptr(), q.data_ptr(), s.data_ptr(), r.M, r.N, as_stream(stream_ptr)));
    return {q, s.unsqueeze(-1)};
}

// ---- per_token_group_quant_int8 (launcher dsv4_all_hip_kernels.hip:346-350) -------
std::vector<Tensor> per_token_group_quant_int8_stream(Tensor x, int64_t group_size, int64_t stream_ptr) {
    TORCH_CHECK(x.is_contiguous());
    check_cuda(x, "x", torch::kBFloat16);
    TORCH_CHECK(group_size > 0, "group_size must be positive");
    c10::cuda::CUDAGuard guard(x.device());
    const Rows r = rows_of(x);
    const int64_t groups = (r.N + group_size - 1) / group_size;
    auto q = torch::empty_like(x, x.options().dtype(torch::kInt8));
    auto s = torch::empty({r.M, groups}, x.options().dtype(torch::kFloat32));
    check_status(launch_ptgq(x.data_ptr(), q.data_ptr(), s.data_ptr(), r.M, r.N, to_int(group_size, "group_size"),
                             as_stream(stream_ptr)));
    return {q, s};
}

// ---- rmsnorm (reference wrapper :326-334): in place, returns x --------------------
Tensor rmsnorm_stream(Tensor x, double eps, int64_t stream_ptr) {
    TORCH_CHECK(x.is_contiguous());
    check_cuda(x, "x", torch::kBFloat16);
    TORCH_CHECK(x.dim() == 2, "rmsnorm expects a 2-D tensor");
    c10::cuda::CUDAGuard guard(x.device());
    check_status(launch_rmsnorm(x.data_ptr(), to_int(x.size(0), "M"), to_int(x.size(1), "N"), (float)eps,
                                as_stream(stream_ptr)));
    return x;
}

struct GateUp {
    int M, N;
    int64_t ldg, ldu;
};
GateUp check_gate_up(const Tensor& gate, const Tensor& up) {
    check_cuda(gate, "gate", torch::kBFloat16);
    check_cuda(up, "up", torch::kBFloat16);
    check_same_device(gate, up, "gate/up");
    TORCH_CHECK(gate.dim() == 2 && up.dim() == 2, "gate and up must be 2-D");
    TORCH_CHECK(gate.sizes() == up.sizes(), "gate and up must have the same shape");
    // the reference requires gate.is_contiguous(); a unit inner stride is enough here
    TORCH_CHECK(gate.size(1) == 0 || (gate.stride(1) == 1 && up.stride(1) == 1),
                "gate and up must have unit stride in the last dimension");
    return {to_int(gate.size(0), "M"), to_int(gate.size(1), "N"), gate.stride(0), up.stride(0)};
}

// ---- silu_and_mul (reference wrapper :336-346) -------------------------------------
Tensor silu_and_mul_stream(Tensor gate, Tensor up, int64_t stream_ptr) {
    const GateUp g = check_gate_up(gate, up);
    c10::cuda::CUDAGuard guard(gate.device());
    auto out = torch::empty({g.M, g.N}, gate.options());
    check_status(launch_silu_mul_strided(gate.data_ptr(), g.ldg, up.data_ptr(), g.ldu, out.data_ptr(), g.M, g.N,
                                         as_stream(stream_ptr)));
    return out;
}

// ---- silu_mul_quant (reference wrapper :348-359) -----------------------------------
std::vector<Tensor> silu_mul_quant_stream(Tensor gate, Tensor up, int64_t stream_ptr) {
    const GateUp g = check_gate_up(gate, up);
    c10::cuda::CUDAGuard guard(gate.device());
    auto q = torch::empty({g.M, g.N}, gate.options().dtype(torch::kInt8));
    auto s = torch::empty({g.M}, gate.options().dtype(torch::kFloat32));
    check_status(launch_silu_mul_quant_strided(gate.data_ptr(), g.ldg, up.data_ptr(), g.ldu, nullptr, nullptr,
                                               q.data_ptr(), s.data_ptr(), g.M, g.N, as_stream(stream_ptr)));
    return {q, s.unsqueeze(-1)};
}

// Same, but only the first min(M, valid_rows[0]) rows are processed; valid_rows is a one-element
// int32 CUDA tensor (the routed-row count of an expert-parallel rank lives on the device).
// Rows beyond it are left unwritten (their content is unspecified, as in gather_rows): a zero fill
// of the whole [M, N] output would cost more than the kernel when few rows are valid.
std::vector<Tensor> silu_mul_quant_rows_stream(Tensor gate, Tensor up, Tensor valid_rows, int64_t stream_ptr) {
    const GateUp g = check_gate_up(gate, up);
    check_cuda(valid_rows, "valid_rows", torch::kInt32);
    check_same_device(gate, valid_rows, "gate/valid_rows");
    TORCH_CHECK(valid_rows.numel() >= 1, "valid_rows must hold one int32");
    c10::cuda::CUDAGuard guard(gate.device());
    auto q = torch::empty({g.M, g.N}, gate.options().dtype(torch::kInt8));
    auto s = torch::empty({g.M}, gate.options().dtype(torch::kFloat32));
    check_status(launch_silu_mul_quant_strided(gate.data_ptr(), g.ldg, up.data_ptr(), g.ldu, nullptr,
                                               static_cast<const int*>(valid_rows.data_ptr()), q.data_ptr(),
                                               s.data_ptr(), g.M, g.N, as_stream(stream_ptr)));
    return {q, s.unsqueeze(-1)};
}

// masked form (launcher dsv4_all_hip_kernels.hip:362-366): rows with mask == 0 are skipped;
// their q and s entries are returned as zero.
std::vector<Tensor> silu_mul_masked_quant_stream(Tensor gate, Tensor up, Tensor mask, int64_t stream_ptr) {
    const GateUp g = check_gate_up(gate, up);
    check_cuda(mask, "mask", torch::kInt32);
    check_same_device(gate, mask, "gate/mask");
    TORCH_CHECK(mask.is_contiguous() && mask.numel() == g.M, "mask must be a contiguous int32 tensor of M entries");
    c10::cuda::CUDAGuard guard(gate.device());
    auto q = torch::zeros({g.M, g.N}, gate.options().dtype(torch::kInt8));
    auto s = torch::zeros({g.M}, gate.options().dtype(torch::kFloat32));
    check_status(launch_silu_mul_quant_strided(gate.data_ptr(), g.ldg, up.data_ptr(), g.ldu,
                                               static_cast<const int*>(mask.data_ptr()), nullptr, q.data_ptr(),
                                               s.data_ptr(), g.M, g.N, as_stream(stream_ptr)));
    return {q, s.unsqueeze(-1)};
}

// masked expert layout (the engine's silu_and_mul_masked_post_quant, DSV4_OPERATOR_ANALYSIS.md:45):
// gate, up [E, max_m, N] (e.g. the halves of a packed [E, max_m, 2N] tensor), masked_m int32 [E];
// only the first masked_m[e] rows of expert e are processed, the rest of q and s is returned as zero.
std::vector<Tensor> silu_and_mul_masked_post_quant_stream(Tensor gate, Tensor up, Tensor masked_m, int64_t stream_ptr) {
    check_cuda(gate, "gate", torch::kBFloat16);
    check_cuda(up, "up", torch::kBFloat16);
    check_cuda(masked_m, "masked_m", torch::kInt32);
    check_same_device(gate, up, "gate/up");
    check_same_device(gate, masked_m, "gate/masked_m");
    TORCH_CHECK(gate.dim() == 3 && up.dim() == 3 && gate.sizes() == up.sizes(), "gate and up must be [E, max_m, N]");
    const int64_t E = gate.size(0), max_m = gate.size(1), N = gate.size(2);
    TORCH_CHECK(masked_m.is_contiguous() && masked_m.numel() == E, "masked_m must be a contiguous int32 tensor of E entries");
    // rows of all experts must form one strided 2-D view: [E * max_m, N] with a single row stride
    TORCH_CHECK(N == 0 || (gate.stride(2) == 1 && up.stride(2) == 1), "gate and up must have unit stride in the last dimension");
    TORCH_CHECK(max_m <= 1 || E <= 1 || (gate.stride(0) == max_m * gate.stride(1) && up.stride(0) == max_m * up.stride(1)),
                "gate and up must be views whose expert blocks follow one another (stride(0) == max_m * stride(1))");
    c10::cuda::CUDAGuard guard(gate.device());
    auto q = torch::zeros({E, max_m, N}, gate.options().dtype(torch::kInt8));
    auto s = torch::zeros({E, max_m}, gate.options().dtype(torch::kFloat32));
    check_status(launch_silu_mul_quant_masked_layout(gate.data_ptr(), gate.stride(1), up.data_ptr(), up.stride(1),
                                                     static_cast<const int*>(masked_m.data_ptr()), q.data_ptr(),
                                                     s.data_ptr(), to_int(E, "E"), to_int(max_m, "max_m"), to_int(N, "N"),
                                                     as_stream(stream_ptr)));
    return {q, s.unsqueeze(-1)};
}

// ---- add_rmsnorm_quant (reference wrapper :361-373): res is overwritten with res+x --
std::vector<Tensor> add_rmsnorm_quant_stream(Tensor res, Tensor x, Tensor w, double eps, int64_t stream_ptr) {
    TORCH_CHECK(res.is_contiguous());
    check_cuda(res, "res", torch::kBFloat16);
    check_cuda(x, "x", torch::kBFloat16);
    check_cuda(w, "w", torch::kBFloat16);
    check_same_device(res, x, "res/x");
    check_same_device(res, w, "res/w");
    TORCH_CHECK(x.dim() == 2, "x must be 2-D");
    TORCH_CHECK(x.is_contiguous() && w.is_contiguous(), "x and w must be contiguous");
    TORCH_CHECK(res.sizes() == x.sizes(), "res and x must have the same shape");
    TORCH_CHECK(w.numel() == x.size(1), "w must have N entries");
    c10::cuda::CUDAGuard guard(x.device());
    const int M = to_int(x.size(0), "M"), N = to_int(x.size(1), "N");
    auto q = torch::empty_like(x, x.options().dtype(torch::kInt8));
    auto s = torch::empty({M}, x.options().dtype(torch::kFloat32));
    check_status(launch_add_rmsnorm_quant(res.data_ptr(), x.data_ptr(), w.data_ptr(), q.data_ptr(), s.data_ptr(), M,
                                          N, (float)eps, as_stream(stream_ptr)));
    return {q, s.unsqueeze(-1)};
}

// ---- w8a8_scaled_gemm (reference wrapper :375-387) ---------------------------------
struct GemmShape {
    int M, N, K;
};
GemmShape check_gemm_operands(const Tensor& A, const Tensor& B) {
    check_cuda(A, "A", torch::kInt8);
    check_cuda(B, "B", torch::kInt8);
    check_same_device(A, B, "A/B");
    TORCH_CHECK(A.dim() == 2 && B.dim() == 2, "A must be [M,K] and B [N,K]");
    TORCH_CHECK(A.is_contiguous() && B.is_contiguous(), "A and B must be contiguous");
    TORCH_CHECK(A.size(1) == B.size(1), "A and B disagree on K: ", A.size(1), " vs ", B.size(1));
    return {to_int(A.size(0), "M"), to_int(B.size(0), "N"), to_int(A.size(1), "K")};
}
// A scale vector as the launchers take it: fp32, n entries, dense, on the operands' device.  Nothing is
// copied here: a hidden copy would run on torch's current stream, which need not be the stream the
// `_stream` variants launch on.
const Tensor& flat_scale(const Tensor& s, int64_t n, const char* name, const Tensor& operand) {
    check_cuda(s, name, torch::kFloat32);
    check_same_device(s, operand, name);
    TORCH_CHECK(s.numel() == n, name, " must have ", n, " entries, got ", s.numel());
    TORCH_CHECK(s.is_contiguous(), name, " must be contiguous");
    return s;
}

Tensor w8a8_scaled_gemm_stream(Tensor A, Tensor B, Tensor sa, Tensor sb, int64_t stream_ptr) {
    const GemmShape g = check_gemm_operands(A, B);
    const Tensor& sa_c = flat_scale(sa, g.M, "sa", A);
    const Tensor& sb_c = flat_scale(sb, g.N, "sb", A);
    c10::cuda::CUDAGuard guard(A.device());
    auto C = torch::empty({g.M, g.N}, A.options().dtype(torch::kBFloat16));
    check_status(launch_w8a8_gemm(A.data_ptr(), B.data_ptr(), sa_c.data_ptr(), sb_c.data_ptr(), C.data_ptr(), g.M,
                                  g.N, g.K, as_stream(stream_ptr)));
    return C;
}

Tensor w8a8_gemm_i32_stream(Tensor A, Tensor B, int64_t stream_ptr) {
    const GemmShape g = check_gemm_operands(A, B);
    c10::cuda::CUDAGuard guard(A.device());
    auto C = torch::empty({g.M, g.N}, A.options().dtype(torch::kInt32));
    check_status(launch_w8a8_gemm_i32(A.data_ptr(), B.data_ptr(), C.data_ptr(), g.M, g.N, g.K, as_stream(stream_ptr)));
    return C;
}

Tensor scale_convert_stream(Tensor acc, Tensor sa, Tensor sb, int64_t stream_ptr) {
    check_cuda(acc, "acc", torch::kInt32);
    TORCH_CHECK(acc.dim() == 2 && acc.is_contiguous(), "acc must be a contiguous [M,N] tensor");
    const Tensor& sa_c = flat_scale(sa, acc.size(0), "sa", acc);
    const Tensor& sb_c = flat_scale(sb, acc.size(1), "sb", acc);
    c10::cuda::CUDAGuard guard(acc.device());
    auto out = torch::empty_like(acc, acc.options().dtype(torch::kBFloat16));
    check_status(launch_scale_convert(acc.data_ptr(), sa_c.data_ptr(), sb_c.data_ptr(), out.data_ptr(),
                                      to_int(acc.size(0), "M"), to_int(acc.size(1), "N"), as_stream(stream_ptr)));
    return out;
}

// ---- grouped_gemm ------------------------------------------------------------------
Tensor grouped_gemm_impl(Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor expert_offsets, c10::optional<Tensor> out,
                         int64_t stream_ptr) {
    check_cuda(A, "A", torch::kInt8);
    check_cuda(W, "W", torch::kInt8);
    check_cuda(sa, "sa", torch::kFloat32);
    check_cuda(sw, "sw", torch::kFloat32);
    check_cuda(expert_offsets, "expert_offsets", torch::kInt32);
    check_same_device(A, W, "A/W");
    check_same_device(A, sa, "A/sa");
    check_same_device(A, sw, "A/sw");
    check_same_device(A, expert_offsets, "A/expert_offsets");
    TORCH_CHECK(A.dim() == 2 && W.dim() == 3, "A must be [R,K] and W [E,N,K]");
    TORCH_CHECK(A.is_contiguous() && W.is_contiguous() && sw.is_contiguous() && expert_offsets.is_contiguous(),
                "A, W, sw and expert_offsets must be contiguous");
    const int R = to_int(A.size(0), "R"), K = to_int(A.size(1), "K");
    const int E = to_int(W.size(0), "E"), N = to_int(W.size(1), "N");
    TORCH_CHECK(W.size(2) == K, "A and W disagree on K");
    TORCH_CHECK(sw.numel() == (int64_t)E * N, "sw must be [E,N]");
    TORCH_CHECK(expert_offsets.numel() == E + 1, "expert_offsets must have E+1 entries");
    TORCH_CHECK(sa.is_contiguous(), "sa must be contiguous");
    const Tensor& sa_c = sa;
    int groups = 1;
    if (sa_c.numel() != R) {
        TORCH_CHECK(K % 128 == 0 && sa_c.numel() == (int64_t)R * (K / 128),
                    "sa must have R entries (per token) or be [R, K/128] (per 128-wide group)");
        groups = K / 128;
    }
    c10::cuda::CUDAGuard guard(A.device());
    Tensor C;
    if (out.has_value()) {   // e.g. a buffer in symmetric memory that peers read
        C = *out;
        check_cuda(C, "out", torch::kBFloat16);
        TORCH_CHECK(C.dim() == 2 && C.is_contiguous() && C.size(0) >= R && C.size(1) == N,
                    "out must be a contiguous bf16 [>= R, N] tensor");
    } else {
        C = torch::empty({R, N}, A.options().dtype(torch::kBFloat16));
    }
    check_status(launch_grouped_gemm(A.data_ptr(), W.data_ptr(), sa_c.data_ptr(), sw.data_ptr(),
                                     static_cast<const int*>(expert_offsets.data_ptr()), C.data_ptr(), R, E, N, K,
                                     groups, as_stream(stream_ptr)));
    return C;
}

Tensor grouped_gemm_stream(Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor expert_offsets, int64_t stream_ptr) {
    return grouped_gemm_impl(A, W, sa, sw, expert_offsets, c10::nullopt, stream_ptr);
}

// masked expert layout (the engine's m_grouped_w8a8_gemm_nt_masked, DSV4_OPERATOR_ANALYSIS.md:43):
// A int8 [E, max_m, K], W int8 [E, N, K], sa fp32 [E, max_m(, 1)] or [E, max_m, K/128], sw fp32 [E, N],
// masked_m int32 [E] -> bf16 [E, max_m, N]; rows at or beyond masked_m[e] keep what `out` held (zero
// when the operator allocates the output).
Tensor grouped_gemm_masked_stream(Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor masked_m, c10::optional<Tensor> out,
                                  int64_t stream_ptr) {
    check_cuda(A, "A", torch::kInt8);
    check_cuda(W, "W", torch::kInt8);
    check_cuda(sa, "sa", torch::kFloat32);
    check_cuda(sw, "sw", torch::kFloat32);
    check_cuda(masked_m, "masked_m", torch::kInt32);
    check_same_device(A, W, "A/W");
    check_same_device(A, sa, "A/sa");
    check_same_device(A, sw, "A/sw");
    check_same_device(A, masked_m, "A/masked_m");
    TORCH_CHECK(A.dim() == 3 && W.dim() == 3, "A must be [E,max_m,K] and W [E,N,K]");
    TORCH_CHECK(A.is_contiguous() && W.is_contiguous() && sa.is_contiguous() && sw.is_contiguous() && masked_m.is_contiguous(),
                "A, W, sa, sw and masked_m must be contiguous");
    const int E = to_int(A.size(0), "E"), max_m = to_int(A.size(1), "max_m"), K = to_int(A.size(2), "K");
    const int N = to_int(W.size(1), "N");
    TORCH_CHECK(W.size(0) == E && W.size(2) == K, "A and W disagree on E or K");
    TORCH_CHECK(sw.numel() == (int64_t)E * N, "sw must be [E,N]");
    TORCH_CHECK(masked_m.numel() == E, "masked_m must have E entries");
    int groups = 1;
    if (sa.numel() != (int64_t)E * max_m) {
        TORCH_CHECK(K % 128 == 0 && sa.numel() == (int64_t)E * max_m * (K / 128),
                    "sa must have E*max_m entries (per token) or be [E, max_m, K/128] (per 128-wide group)");
        groups = K / 128;
    }
    c10::cuda::CUDAGuard guard(A.device());
    Tensor C;
    if (out.has_value()) {
        C = *out;
        check_cuda(C, "out", torch::kBFloat16);
        check_same_device(A, C, "A/out");
        TORCH_CHECK(C.is_contiguous() && C.dim() == 3 && C.size(0) == E && C.size(1) == max_m && C.size(2) == N,
                    "out must be a contiguous bf16 [E, max_m, N] tensor");
    } else {
        C = torch::zeros({E, max_m, N}, A.options().dtype(torch::kBFloat16));
    }
    if (E == 0 || max_m == 0 || N == 0) return C;
    check_status(launch_grouped_gemm_masked(A.data_ptr(), W.data_ptr(), sa.data_ptr(), sw.data_ptr(),
                                            static_cast<const int*>(masked_m.data_ptr()), C.data_ptr(), E, max_m, N, K,
                                            groups, as_stream(stream_ptr)));
    return C;
}

std::vector<Tensor> moe_segments_impl(Tensor topk_ids, int64_t num_experts, int64_t expert_lo,
                                      c10::optional<Tensor> slot_out, int64_t stream_ptr);
std::vector<Tensor> moe_segments_stream(Tensor topk_ids, int64_t num_experts, int64_t expert_lo, int64_t stream_ptr) {
    return moe_segments_impl(topk_ids, num_experts, expert_lo, c10::nullopt, stream_ptr);
}

std::vector<Tensor> moe_segments_impl(Tensor topk_ids, int64_t num_experts, int64_t expert_lo,
                                      c10::optional<Tensor> slot_out, int64_t stream_ptr) {
    check_cuda(topk_ids, "topk_ids", torch::kInt32);
    TORCH_CHECK(topk_ids.dim() == 2 && topk_ids.is_contiguous(), "topk_ids must be a contiguous [T,topk] tensor");
    c10::cuda::CUDAGuard guard(topk_ids.device());
    const int T = to_int(topk_ids.size(0), "T"), topk = to_int(topk_ids.size(1), "topk");
    auto opt = topk_ids.options();
    auto offsets = torch::empty({num_experts + 1}, opt);
    auto src_row = torch::empty({(int64_t)T * topk}, opt);
    Tensor dst_slot;
    if (slot_out.has_value()) {   // e.g. a buffer in symmetric memory that peers read
        check_cuda(*slot_out, "dst_slot", torch::kInt32);
        TORCH_CHECK(slot_out->is_contiguous() && slot_out->numel() >= (int64_t)T * topk,
                    "dst_slot must be a contiguous int32 tensor with at least T*topk entries");
        dst_slot = slot_out->view({-1}).narrow(0, 0, (int64_t)T * topk);
    } else {
        dst_slot = torch::empty({(int64_t)T * topk}, opt);
    }
    if (T == 0) {
        offsets.zero_();
        return {offsets, src_row, dst_slot};
    }
    check_status(launch_moe_segments(static_cast<const int*>(topk_ids.data_ptr()), T, topk,
                                     to_int(num_experts, "num_experts"), to_int(expert_lo, "expert_lo"),
                                     static_cast<int*>(offsets.data_ptr()),
                                     static_cast<int*>(src_row.data_ptr()), static_cast<int*>(dst_slot.data_ptr()),
                                     as_stream(stream_ptr)));
    return {offsets, src_row, dst_slot};
}

// rows of `src` ([T, row]) gathered by src_row; `scales` ([T, spr] or [T,1]) optional
std::vector<Tensor> gather_rows_stream(Tensor src, Tensor src_row, c10::optional<Tensor> scales,
                                       c10::optional<Tensor> valid_rows, int64_t stream_ptr) {
    TORCH_CHECK(src.is_cuda() && src.dim() == 2 && src.is_contiguous(), "src must be a contiguous 2-D CUDA tensor");
    check_cuda(src_row, "src_row", torch::kInt32);
    TORCH_CHECK(src_row.is_contiguous(), "src_row must be contiguous");
    c10::cuda::CUDAGuard guard(src.device());
    const int R = to_int(src_row.numel(), "R");
    const int64_t row_bytes = src.size(1) * src.element_size();
    auto dst = torch::empty({R, src.size(1)}, src.options());
    Tensor dscale;
    const float* sp = nullptr;
    float* dp = nullptr;
    int spr = 0;
    Tensor sc;
    if (scales.has_value()) {
        sc = scales->contiguous();
        check_cuda(sc, "scales", torch::kFloat32);
        TORCH_CHECK(sc.dim() == 2 && sc.size(0) == src.size(0), "scales must be [T, n]");
        spr = to_int(sc.size(1), "scales per row");
        dscale = torch::empty({R, sc.size(1)}, sc.options());
        sp = static_cast<const float*>(sc.data_ptr());
        dp = static_cast<float*>(dscale.data_ptr());
    }
    const int* vr = nullptr;
    if (valid_rows.has_value()) {
        check_cuda(*valid_rows, "valid_rows", torch::kInt32);
        vr = static_cast<const int*>(valid_rows->data_ptr());
    }
    check_status(launch_gather_rows(src.data_ptr(), static_cast<const int*>(src_row.data_ptr()), dst.data_ptr(), R,
                                    to_int(row_bytes, "row bytes"), sp, dp, spr, vr, as_stream(stream_ptr)));
    if (scales.has_value()) return {dst, dscale};
    return {dst};
}

// router top-k: logits fp32 [T,E] -> [ids int32 [T,k], weights fp32 [T,k]]
std::vector<Tensor> moe_topk_stream(Tensor logits, int64_t k, int64_t stream_ptr) {
    check_cuda(logits, "logits", torch::kFloat32);
    TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous(), "logits must be a contiguous [T,E] tensor");
    c10::cuda::CUDAGuard guard(logits.device());
    const int T = to_int(logits.size(0), "T"), E = to_int(logits.size(1), "E");
    auto ids = torch::empty({T, k}, logits.options().dtype(torch::kInt32));
    auto w = torch::empty({T, k}, logits.options());
    check_status(launch_moe_topk(static_cast<const float*>(logits.data_ptr()), T, E, to_int(k, "k"),
                                 static_cast<int*>(ids.data_ptr()), static_cast<float*>(w.data_ptr()),
                                 as_stream(stream_ptr)));
    return {ids, w};
}

// out[t] = sum_j w[t,j] * z[dst_slot[t,j]]  (bf16, or fp32 partial sums when out_f32)
Tensor moe_combine_stream(Tensor z, Tensor dst_slot, Tensor topk_w, bool out_f32, int64_t stream_ptr) {
    check_cuda(z, "z", torch::kBFloat16);
    check_cuda(dst_slot, "dst_slot", torch::kInt32);
    check_cuda(topk_w, "topk_w", torch::kFloat32);
    TORCH_CHECK(z.dim() == 2 && z.is_contiguous() && topk_w.dim() == 2 && topk_w.is_contiguous() &&
                dst_slot.is_contiguous() && dst_slot.numel() == topk_w.numel(),
                "z must be [R,H], topk_w [T,topk], dst_slot T*topk entries, all contiguous");
    c10::cuda::CUDAGuard guard(z.device());
    const int T = to_int(topk_w.size(0), "T"), topk = to_int(topk_w.size(1), "topk"), H = to_int(z.size(1), "H");
    auto out = torch::empty({T, H}, z.options().dtype(out_f32 ? torch::kFloat32 : torch::kBFloat16));
    check_status(launch_moe_combine(z.data_ptr(), static_cast<const int*>(dst_slot.data_ptr()),
                                    static_cast<const float*>(topk_w.data_ptr()), out.data_ptr(), T, topk, H,
                                    out_f32 ? 1 : 0, as_stream(stream_ptr)));
    return out;
}

// Expert-parallel combine + exchange: pointers (as integers) to every rank's z, dst_slot and out
// buffers, mapped into this GPU's address space (symmetric memory buffer_ptrs); tokens [t0, t1).
void moe_combine_exchange_stream(std::vector<int64_t> z_ptrs, std::vector<int64_t> slot_ptrs, Tensor topk_ids,
                                 Tensor topk_w, std::vector<int64_t> out_ptrs, int64_t experts_per_rank, int64_t t0,
                                 int64_t t1, int64_t H, int64_t stream_ptr) {
    check_cuda(topk_ids, "topk_ids", torch::kInt32);
    check_cuda(topk_w, "topk_w", torch::kFloat32);
    TORCH_CHECK(topk_ids.dim() == 2 && topk_ids.is_contiguous() && topk_w.is_contiguous() &&
                topk_w.sizes() == topk_ids.sizes(), "topk_ids and topk_w must be contiguous [T,topk]");
    const size_t G = z_ptrs.size();
    TORCH_CHECK(G >= 1 && G <= 8 && slot_ptrs.size() == G && out_ptrs.size() == G, "1 to 8 ranks, three pointer lists");
    TORCH_CHECK(t0 >= 0 && t1 <= topk_ids.size(0), "token range outside [0, T)");
    c10::cuda::CUDAGuard guard(topk_ids.device());
    std::vector<const void*> z(G);
    std::vector<const int*> slot(G);
    std::vector<void*> out(G);
    for (size_t r = 0; r < G; ++r) {
        z[r] = reinterpret_cast<const void*>(z_ptrs[r]);
        slot[r] = reinterpret_cast<const int*>(slot_ptrs[r]);
        out[r] = reinterpret_cast<void*>(out_ptrs[r]);
    }
    check_status(launch_moe_combine_exchange(z.data(), slot.data(), static_cast<const int*>(topk_ids.data_ptr()),
                                             static_cast<const float*>(topk_w.data_ptr()), out.data(), (int)G,
                                             to_int(experts_per_rank, "experts_per_rank"), to_int(t0, "t0"),
                                             to_int(t1, "t1"), to_int(topk_ids.size(1), "topk"), to_int(H, "H"),
                                             as_stream(stream_ptr)));
}

// Grouped GEMM (per-token scales) whose result row r is stored to the address row_ptr[r] (int64 device tensor of
// R addresses, e.g. rows of other ranks' inboxes in symmetric memory) instead of a dense [R,N] tensor.
void grouped_gemm_scatter_stream(Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor expert_offsets, Tensor row_ptr,
                                 int64_t stream_ptr) {
    check_cuda(A, "A", torch::kInt8);
    check_cuda(W, "W", torch::kInt8);
    check_cuda(sa, "sa", torch::kFloat32);
    check_cuda(sw, "sw", torch::kFloat32);
    check_cuda(expert_offsets, "expert_offsets", torch::kInt32);
    check_cuda(row_ptr, "row_ptr", torch::kInt64);
    check_same_device(A, W, "A/W");
    check_same_device(A, sa, "A/sa");
    check_same_device(A, sw, "A/sw");
    check_same_device(A, expert_offsets, "A/expert_offsets");
    check_same_device(A, row_ptr, "A/row_ptr");
    TORCH_CHECK(A.dim() == 2 && W.dim() == 3, "A must be [R,K] and W [E,N,K]");
    TORCH_CHECK(A.is_contiguous() && W.is_contiguous() && sw.is_contiguous() && sa.is_contiguous() &&
                expert_offsets.is_contiguous() && row_ptr.is_contiguous(), "all operands must be contiguous");
    const int R = to_int(A.size(0), "R"), K = to_int(A.size(1), "K");
    const int E = to_int(W.size(0), "E"), N = to_int(W.size(1), "N");
    TORCH_CHECK(W.size(2) == K, "A and W disagree on K");
    TORCH_CHECK(sw.numel() == (int64_t)E * N, "sw must be [E,N]");
    TORCH_CHECK(sa.numel() == R, "sa must have R entries (per-token scales)");
    TORCH_CHECK(expert_offsets.numel() == E + 1, "expert_offsets must have E+1 entries");
    TORCH_CHECK(row_ptr.numel() >= R, "row_ptr must have an address for every row");
    c10::cuda::CUDAGuard guard(A.device());
    check_status(launch_grouped_gemm_scatter(A.data_ptr(), W.data_ptr(), sa.data_ptr(), sw.data_ptr(),
                                             static_cast<const int*>(expert_offsets.data_ptr()),
                                             reinterpret_cast<void* const*>(row_ptr.data_ptr()), R, E, N, K,
                                             as_stream(stream_ptr)));
}

// row_ptr[dst_slot[pair]] = address of the pair's row in the inbox of the rank that owns its token
void moe_push_rows_stream(Tensor dst_slot, int64_t topk, int64_t tokens_per_rank, std::vector<int64_t> inbox_ptrs,
                          int64_t H, Tensor row_ptr, int64_t stream_ptr) {
    check_cuda(dst_slot, "dst_slot", torch::kInt32);
    check_cuda(row_ptr, "row_ptr", torch::kInt64);
    check_same_device(dst_slot, row_ptr, "dst_slot/row_ptr");
    TORCH_CHECK(dst_slot.is_contiguous() && row_ptr.is_contiguous(), "dst_slot and row_ptr must be contiguous");
    TORCH_CHECK(topk > 0 && dst_slot.numel() % topk == 0, "dst_slot must have T*topk entries");
    TORCH_CHECK(row_ptr.numel() >= dst_slot.numel(), "row_ptr must have T*topk entries");
    const size_t G = inbox_ptrs.size();
    TORCH_CHECK(G >= 1 && G <= 8, "1 to 8 ranks");
    std::vector<void*> inbox(G);
    for (size_t g = 0; g < G; ++g) inbox[g] = reinterpret_cast<void*>(inbox_ptrs[g]);
    c10::cuda::CUDAGuard guard(dst_slot.device());
    check_status(launch_moe_push_rows(static_cast<const int*>(dst_slot.data_ptr()), to_int(dst_slot.numel() / topk, "T"),
                                      to_int(topk, "topk"), to_int(tokens_per_rank, "tokens_per_rank"), inbox.data(),
                                      (int)G, to_int(H, "H"), reinterpret_cast<void**>(row_ptr.data_ptr()),
                                      as_stream(stream_ptr)));
}

// w8a8 GEMM written into columns [col0, col0 + N) of an existing bf16 [M, ldc] buffer
void w8a8_gemm_into_stream(Tensor A, Tensor B, Tensor sa, Tensor sb, Tensor out, int64_t col0, int64_t stream_ptr) {
    const GemmShape g = check_gemm_operands(A, B);
    const Tensor& sa_c = flat_scale(sa, g.M, "sa", A);
    const Tensor& sb_c = flat_scale(sb, g.N, "sb", A);
    check_cuda(out, "out", torch::kBFloat16);
    TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.size(0) == g.M && col0 >= 0 && col0 + g.N <= out.size(1),
                "out must be a [M, >= col0 + N] bf16 tensor with unit inner stride");
    c10::cuda::CUDAGuard guard(A.device());
    auto* base = static_cast<at::BFloat16*>(out.data_ptr()) + col0;
    check_status(launch_w8a8_gemm_ld(A.data_ptr(), B.data_ptr(), sa_c.data_ptr(), sb_c.data_ptr(), base, out.stride(0),
                                     g.M, g.N, g.K, as_stream(stream_ptr)));
}

// Fused GEMM + all-gather: the result goes to columns [col0, col0+N) of `out` and of every buffer
// whose base address is listed in peer_ptrs (device pointers to the other ranks' [M, ldc] outputs,
// e.g. torch.distributed._symmetric_memory buffer_ptrs), all with out's row stride.
void w8a8_gemm_allgather_stream(Tensor A, Tensor B, Tensor sa, Tensor sb, Tensor out, int64_t col0,
                                std::vector<int64_t> peer_ptrs, int64_t stream_ptr) {
    const GemmShape g = check_gemm_operands(A, B);
    const Tensor& sa_c = flat_scale(sa, g.M, "sa", A);
    const Tensor& sb_c = flat_scale(sb, g.N, "sb", A);
    check_cuda(out, "out", torch::kBFloat16);
    TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.size(0) == g.M && col0 >= 0 && col0 + g.N <= out.size(1),
                "out must be a [M, >= col0 + N] bf16 tensor with unit inner stride");
    TORCH_CHECK(peer_ptrs.size() <= 7, "at most 7 peers");
    c10::cuda::CUDAGuard guard(A.device());
    std::vector<void*> peers;
    for (int64_t ptr : peer_ptrs) peers.push_back(reinterpret_cast<at::BFloat16*>(ptr) + col0);
    auto* base = static_cast<at::BFloat16*>(out.data_ptr()) + col0;
    check_status(launch_w8a8_gemm_allgather(A.data_ptr(), B.data_ptr(), sa_c.data_ptr(), sb_c.data_ptr(), base,
                                            peers.data(), (int)peers.size(), out.stride(0), g.M, g.N, g.K,
                                            as_stream(stream_ptr)));
}

int64_t device_status() {
    int v = 0;
    check_status(dsv4_device_status(as_stream(current_stream_ptr()), &v));
    return v;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "B200 (sm_100a) W8A8 linear path behind the dsv4_native_ext operator names";
    // the reference's names (hip_kernels/dsv4_native_ext.cpp:429-444)
    m.def("per_token_quant_int8", [](Tensor x) { return per_token_quant_int8_stream(x, current_stream_ptr()); });
    m.def("per_token_quant_int8_stream", &per_token_quant_int8_stream);
    m.def("rmsnorm", [](Tensor x, double eps) { return rmsnorm_stream(x, eps, current_stream_ptr()); });
    m.def("rmsnorm_stream", &rmsnorm_stream);
    m.def("silu_and_mul", [](Tensor g, Tensor u) { return silu_and_mul_stream(g, u, current_stream_ptr()); });
    m.def("silu_and_mul_stream", &silu_and_mul_stream);
    m.def("silu_mul_quant", [](Tensor g, Tensor u) { return silu_mul_quant_stream(g, u, current_stream_ptr()); });
    m.def("silu_mul_quant_stream", &silu_mul_quant_stream);
    m.def("add_rmsnorm_quant", [](Tensor res, Tensor x, Tensor w, double eps) {
        return add_rmsnorm_quant_stream(res, x, w, eps, current_stream_ptr());
    });
    m.def("add_rmsnorm_quant_stream", &add_rmsnorm_quant_stream);
    m.def("w8a8_scaled_gemm", [](Tensor A, Tensor B, Tensor sa, Tensor sb) {
        return w8a8_scaled_gemm_stream(A, B, sa, sb, current_stream_ptr());
    });
    m.def("w8a8_scaled_gemm_stream", &w8a8_scaled_gemm_stream);
    // additions
    m.def("w8a8_gemm", [](Tensor A, Tensor B, Tensor sa, Tensor sb) {
        return w8a8_scaled_gemm_stream(A, B, sa, sb, current_stream_ptr());
    });
    m.def("w8a8_gemm_stream", &w8a8_scaled_gemm_stream);
    m.def("w8a8_gemm_i32", [](Tensor A, Tensor B) { return w8a8_gemm_i32_stream(A, B, current_stream_ptr()); });
    m.def("w8a8_gemm_i32_stream", &w8a8_gemm_i32_stream);
    m.def("scale_convert", [](Tensor acc, Tensor sa, Tensor sb) {
        return scale_convert_stream(acc, sa, sb, current_stream_ptr());
    });
    m.def("scale_convert_stream", &scale_convert_stream);
    m.def("per_token_group_quant_int8", [](Tensor x, int64_t gs) {
        return per_token_group_quant_int8_stream(x, gs, current_stream_ptr());
    }, py::arg("x"), py::arg("group_size") = 128);
    m.def("per_token_group_quant_int8_stream", &per_token_group_quant_int8_stream);
    m.def("silu_mul_masked_quant", [](Tensor g, Tensor u, Tensor mask) {
        return silu_mul_masked_quant_stream(g, u, mask, current_stream_ptr());
    });
    m.def("silu_mul_masked_quant_stream", &silu_mul_masked_quant_stream);
    m.def("grouped_gemm", [](Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor off) {
        return grouped_gemm_stream(A, W, sa, sw, off, current_stream_ptr());
    });
    m.def("grouped_gemm_stream", &grouped_gemm_stream);
    m.def("grouped_gemm_masked", [](Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor masked_m, c10::optional<Tensor> out) {
        return grouped_gemm_masked_stream(A, W, sa, sw, masked_m, out, current_stream_ptr());
    }, py::arg("A"), py::arg("W"), py::arg("sa"), py::arg("sw"), py::arg("masked_m"), py::arg("out") = py::none());
    m.def("grouped_gemm_masked_stream", &grouped_gemm_masked_stream);
    // the engine's names for the two masked-layout operators
    m.def("m_grouped_w8a8_gemm_nt_masked", [](Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor masked_m, c10::optional<Tensor> out) {
        return grouped_gemm_masked_stream(A, W, sa, sw, masked_m, out, current_stream_ptr());
    }, py::arg("A"), py::arg("W"), py::arg("sa"), py::arg("sw"), py::arg("masked_m"), py::arg("out") = py::none());
    m.def("silu_and_mul_masked_post_quant", [](Tensor g, Tensor u, Tensor masked_m) {
        return silu_and_mul_masked_post_quant_stream(g, u, masked_m, current_stream_ptr());
    });
    m.def("silu_and_mul_masked_post_quant_stream", &silu_and_mul_masked_post_quant_stream);
    m.def("grouped_gemm_into", [](Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor off, Tensor out) {
        return grouped_gemm_impl(A, W, sa, sw, off, out, current_stream_ptr());
    });
    m.def("moe_segments_into", [](Tensor ids, int64_t E, int64_t lo, Tensor slot_out) {
        return moe_segments_impl(ids, E, lo, slot_out, current_stream_ptr());
    });
    m.def("moe_combine_exchange", [](std::vector<int64_t> z, std::vector<int64_t> slot, Tensor ids, Tensor w,
                                     std::vector<int64_t> out, int64_t epr, int64_t t0, int64_t t1, int64_t H) {
        moe_combine_exchange_stream(z, slot, ids, w, out, epr, t0, t1, H, current_stream_ptr());
    });
    m.def("moe_combine_exchange_stream", &moe_combine_exchange_stream);
    m.def("grouped_gemm_scatter", [](Tensor A, Tensor W, Tensor sa, Tensor sw, Tensor off, Tensor row_ptr) {
        grouped_gemm_scatter_stream(A, W, sa, sw, off, row_ptr, current_stream_ptr());
    });
    m.def("grouped_gemm_scatter_stream", &grouped_gemm_scatter_stream);
    m.def("moe_push_rows", [](Tensor dst_slot, int64_t topk, int64_t per, std::vector<int64_t> inbox, int64_t H,
                              Tensor row_ptr) {
        moe_push_rows_stream(dst_slot, topk, per, inbox, H, row_ptr, current_stream_ptr());
    });
    m.def("moe_push_rows_stream", &moe_push_rows_stream);
    m.def("moe_segments", [](Tensor ids, int64_t E, int64_t lo) {
        return moe_segments_stream(ids, E, lo, current_stream_ptr());
    }, py::arg("topk_ids"), py::arg("num_experts"), py::arg("expert_lo") = 0);
    m.def("moe_segments_stream", &moe_segments_stream);
    m.def("gather_rows", [](Tensor src, Tensor src_row, c10::optional<Tensor> scales, c10::optional<Tensor> valid) {
        return gather_rows_stream(src, src_row, scales, valid, current_stream_ptr());
    }, py::arg("src"), py::arg("src_row"), py::arg("scales") = py::none(), py::arg("valid_rows") = py::none());
    m.def("gather_rows_stream", &gather_rows_stream);
    m.def("silu_mul_quant_rows", [](Tensor g, Tensor u, Tensor valid) {
        return silu_mul_quant_rows_stream(g, u, valid, current_stream_ptr());
    });
    m.def("silu_mul_quant_rows_stream", &silu_mul_quant_rows_stream);
    m.def("moe_topk", [](Tensor logits, int64_t k) { return moe_topk_stream(logits, k, current_stream_ptr()); });
    m.def("moe_topk_stream", &moe_topk_stream);
    m.def("moe_combine", [](Tensor z, Tensor slot, Tensor w, bool f32) {
        return moe_combine_stream(z, slot, w, f32, current_stream_ptr());
    }, py::arg("z"), py::arg("dst_slot"), py::arg("topk_w"), py::arg("out_f32") = false);
    m.def("moe_combine_stream", &moe_combine_stream);
    m.def("w8a8_gemm_into", [](Tensor A, Tensor B, Tensor sa, Tensor sb, Tensor out, int64_t col0) {
        w8a8_gemm_into_stream(A, B, sa, sb, out, col0, current_stream_ptr());
    });
    m.def("w8a8_gemm_into_stream", &w8a8_gemm_into_stream);
    m.def("w8a8_gemm_allgather", [](Tensor A, Tensor B, Tensor sa, Tensor sb, Tensor out, int64_t col0,
                                    std::vector<int64_t> peers) {
        w8a8_gemm_allgather_stream(A, B, sa, sb, out, col0, peers, current_stream_ptr());
    });
    m.def("w8a8_gemm_allgather_stream", &w8a8_gemm_allgather_stream);
    m.def("device_status", &device_status);
    m.def("abi_version", [] { return dsv4_abi_version(); });
    m.def("set_overlap_previous_kernel", [](bool on) { dsv4_set_overlap_previous_kernel(on ? 1 : 0); },
          "GEMMs with M <= 256 may start (set-up, weight loads) while the previous kernel on the stream still runs");
    m.def("get_overlap_previous_kernel", [] { return dsv4_get_overlap_previous_kernel() != 0; });
}
