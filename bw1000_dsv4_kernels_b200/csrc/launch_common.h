// Status codes and error reporting shared by the launchers behind the C-ABI.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/dsv4_w8a8.h"

namespace w8a8 {

// Records `msg` as the calling thread's last error and returns `code`.
int fail(int code, const char* msg);
// cudaGetLastError() after a launch; records "<what>: <cuda error string>" on failure.
int check_launch(const char* what);

// ---- launchers implemented in rowwise_quant.cu -----------------------------------
int ptq(const void* x, void* q, void* s, int M, int K, int64_t ldx, cudaStream_t st);
int ptgq(const void* x, void* q, void* s, int M, int K, int gs, cudaStream_t st);
int add_rmsnorm_quant(void* res, const void* x, const void* w, void* q, void* s, int M, int K,
                      float eps, cudaStream_t st);
int rmsnorm(void* x, int M, int K, float eps, cudaStream_t st);
// masked_m / max_m: masked expert layout (rows are E blocks of max_m rows, the first masked_m[e] of block e valid)
int silu_mul_quant(const void* g, const void* u, const int* mask, const int* valid_rows, void* q, void* s,
                   int M, int N, int64_t ldg, int64_t ldu, cudaStream_t st, const int* masked_m = nullptr,
                   int max_m = 0);
int silu_mul(const void* g, const void* u, void* out, int M, int N, int64_t ldg, int64_t ldu,
             cudaStream_t st);

// ---- launchers implemented in gemm_i8_sm100.cu ------------------------------------
struct GemmArgs {
    const void* A;        // int8 [M or R, K]
    const void* B;        // int8 [N, K] or [E, N, K]
    const float* sa;      // [M] per token, or [M, K/128] when sa_groups > 1
    const float* sb;      // [N] or [E, N]; may be null only when out_i32
    void* C;              // bf16 [M, N] or int32 [M, N]
    const int* offsets;   // null for a dense GEMM, else expert_offsets[E+1]
    const int* masked_m = nullptr;  // masked layout instead of offsets: A, C are [E, max_m, .], masked_m[E] on the device
    int max_m = 0;
    int M, N, K, E;
    int64_t ldc;          // row stride of C in elements; 0 = N
    int sa_groups;        // 1 = per-token scale; K/128 = one scale per 128 of K
    int out_i32;          // 1 = write raw int32 accumulators
    void* const* row_ptr = nullptr;  // grouped GEMM, per-token scales: device array, one destination row per result row (C unused)
    void* peerC[7];       // fused all-gather: the other ranks' mapped output slabs
    int npeers;           // 0 = none
    // Test hook, zero through every public entry point: the tile producers of the launch issue no
    // loads and every bounded wait gives up after test_wait_limit_ns, so the kernel's give-up path runs.
    int test_withhold_loads = 0;
    unsigned long long test_wait_limit_ns = 0;
};
int gemm_i8(const GemmArgs& a, cudaStream_t st);
int scale_convert(const void* acc, const void* sa, const void* sb, void* out, int M, int N,
                  cudaStream_t st);

// ---- launchers implemented in moe_segments.cu -------------------------------------
int moe_segments(const int* topk_ids, int T, int topk, int E, int expert_lo, int* offsets, int* src_row,
                 int* dst_slot, cudaStream_t st);
int gather_rows(const void* src, const int* src_row, void* dst, int R, int row_bytes,
                const float* src_scale, float* dst_scale, int scales_per_row, const int* valid_rows,
                cudaStream_t st);
int moe_topk(const float* logits, int T, int E, int k, int* ids, float* weights, cudaStream_t st);
int moe_combine(const void* z, const int* dst_slot, const float* w, void* out, int T, int topk, int H,
                int out_f32, cudaStream_t st);
void set_overlap_previous_kernel(int on);
int overlap_previous_kernel();
int moe_combine_exchange(const void* const* z_ranks, const int* const* slot_ranks, const int* topk_ids,
                         const float* topk_w, void* const* out_ranks, int G, int experts_per_rank, int t0, int t1,
                         int topk, int H, cudaStream_t st);
int moe_push_rows(const int* dst_slot, int T, int topk, int tokens_per_rank, void* const* inbox_ranks, int G, int H,
                  void** row_ptr, cudaStream_t st);
int read_device_status(cudaStream_t st, int* out);
int read_row_status(int* out);  // status word of the row kernels (after the stream was synchronised)

}  // namespace w8a8
