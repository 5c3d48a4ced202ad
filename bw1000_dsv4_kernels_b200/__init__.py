"""B200 (sm_100a) implementation of the DeepSeek-V4 W8A8 linear path behind the
`dsv4_native_ext` operator names.

    from bw1000_dsv4_kernels_b200 import dsv4_native_ext as ext
    q, s = ext.per_token_quant_int8(x)            # x: bf16 CUDA tensor
    y = ext.w8a8_scaled_gemm(q, w_int8, s, s_ch)  # bf16 [M, N]

The operator module is a compiled extension kept next to this file; build it with
`python -m bw1000_dsv4_kernels_b200.build`.  There is no Python or CPU fallback: if the
extension is missing the import fails, and every operator raises on non-CUDA tensors.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdsv4_w8a8.so")



def _load_ext():
    import importlib

    import torch  # noqa: F401  (the extension links against libtorch)
    try:
        return importlib.import_module(__name__ + ".dsv4_native_ext")
    except ImportError as exc:
        raise ImportError(
            "bw1000_dsv4_kernels_b200: the compiled operator module dsv4_native_ext is missing or "
            "cannot be loaded (" + str(exc) + "). Build it with "
            "`python -m bw1000_dsv4_kernels_b200.build`; there is no fallback path.") from exc


def __getattr__(name):
    # The operator module is imported on first use so that `python -m <package>.build` can run
    # before it exists; a missing module is an ImportError at that first use, never a fallback.
    if name == "dsv4_native_ext":
        ext = _load_ext()
        globals()[name] = ext
        return ext
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def c_abi() -> ctypes.CDLL:
    """The C-ABI library (include/dsv4_w8a8.h) as a ctypes handle."""
    return ctypes.CDLL(LIB_PATH)


__all__ = ["dsv4_native_ext", "c_abi", "LIB_PATH"]
