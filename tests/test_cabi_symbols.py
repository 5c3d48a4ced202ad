"""The C-ABI library loads without a GPU and exports every symbol that include/dsv4_w8a8.h
declares; argument errors are reported before anything touches the device."""
import ctypes
import os
import re

import bw1000_dsv4_kernels_b200 as pkg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dsv4_w8a8.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"DSV4_API\s+(?:const\s+char\s*\*|int)\s+(\w+)\s*\(", text)


def test_every_declared_symbol_is_exported():
    names = declared_symbols()
    assert len(names) >= 20 and "launch_ptq" in names and "launch_grouped_gemm" in names
    lib = ctypes.CDLL(pkg.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    # the launcher names the reference exports (dsv4_all_hip_kernels.hip:342-381, w8a8_gemm_v5.hip:129,
    # w8a8_gemm_intmm_fused.hip:41, and the shipped libdsv4_ops_hip.so)
    for ref_name in ("launch_ptq", "launch_ptgq", "launch_rmsnorm_self", "launch_rmsnorm", "launch_silu_mul",
                     "launch_silu_mul_quant", "launch_silu_mul_masked_quant", "launch_add_rmsnorm_quant",
                     "launch_w8a8_gemm_v5", "launch_scale_convert"):
        assert ref_name in names


def test_abi_version_and_argument_errors_without_a_device():
    lib = ctypes.CDLL(pkg.LIB_PATH)
    lib.dsv4_last_error.restype = ctypes.c_char_p
    assert lib.dsv4_abi_version() == 1
    null = ctypes.c_void_p(0)
    assert lib.launch_ptq(null, null, null, 0, 128, null) == 0             # empty input: nothing to do
    assert lib.launch_ptq(null, null, null, 4, 128, null) == 1             # DSV4_ERR_ARG
    assert b"null pointer" in lib.dsv4_last_error()
    assert lib.launch_ptq(null, null, null, -1, 128, null) == 1
    assert b"negative" in lib.dsv4_last_error()
    assert lib.launch_ptgq(null, null, null, 4, 128, 0, null) == 1
    assert lib.launch_w8a8_gemm(null, null, null, null, null, 4, 8, 32, null) == 1
    assert lib.launch_w8a8_gemm(null, null, null, null, null, 0, 8, 32, null) == 0
    one = ctypes.c_void_p(16)
    assert lib.launch_w8a8_gemm(one, one, one, one, one, 4, 8, 24, null) == 1
    assert b"multiple of 16" in lib.dsv4_last_error()
    assert lib.launch_grouped_gemm(one, one, one, one, null, one, 4, 2, 8, 32, 1, null) == 1
    assert lib.launch_moe_segments(null, 4, 2, 8, 0, null, null, null, null) == 1
    assert lib.launch_gather_rows(one, one, one, 4, 24, null, null, 0, null, null) == 1
    # additions without a reference counterpart: same argument discipline
    assert lib.launch_silu_mul_strided(one, ctypes.c_longlong(4), one, ctypes.c_longlong(8), one, 2, 8, null) == 1
    assert b"stride" in lib.dsv4_last_error()
    assert lib.launch_moe_combine_exchange(null, null, null, null, null, 2, 4, 0, 4, 2, 64, null) == 1
    assert lib.launch_moe_combine_exchange(null, null, null, null, null, 2, 4, 4, 4, 2, 64, null) == 0   # no tokens
    ptrs = (ctypes.c_void_p * 9)(*([16] * 9))
    assert lib.launch_moe_combine_exchange(ptrs, ptrs, one, one, ptrs, 9, 4, 0, 4, 2, 64, null) == 1     # > 8 ranks
    # the overlap option is a process-wide switch, off by default
    assert lib.dsv4_get_overlap_previous_kernel() == 0
    lib.dsv4_set_overlap_previous_kernel(1)
    assert lib.dsv4_get_overlap_previous_kernel() == 1
    lib.dsv4_set_overlap_previous_kernel(0)
    assert lib.dsv4_get_overlap_previous_kernel() == 0


def test_operator_module_lists_the_reference_names():
    ext = pkg.dsv4_native_ext
    for name in ("per_token_quant_int8", "rmsnorm", "silu_and_mul", "silu_mul_quant", "add_rmsnorm_quant",
                 "w8a8_scaled_gemm"):
        assert hasattr(ext, name) and hasattr(ext, name + "_stream")      # dsv4_native_ext.cpp:429-442
    for name in ("w8a8_gemm", "per_token_group_quant_int8", "grouped_gemm", "moe_segments", "moe_combine", "moe_topk",
                 "moe_combine_exchange", "gather_rows", "w8a8_gemm_allgather", "set_overlap_previous_kernel"):
        assert hasattr(ext, name)
