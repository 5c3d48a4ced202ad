"""Engine integration: rebinds lmslim's `per_token_quant_int8` to this package's kernel.

The counterpart of the reference's `hip_kernels/hip_graph_safe.py:16-35`: the serving engine
calls `lmslim.layers.gemm.int8_utils.per_token_quant_int8(x, scale_dtype=None, cal_sum=False)`
before every W8A8 linear layer; the patch replaces it with a wrapper of the same signature that
launches `per_token_quant_int8_stream` on torch's current stream, so the call is captured like any
other kernel when the engine records its CUDA graphs.

Enable it the way the reference is enabled: set `SGLANG_USE_HIP_QUANT=1` (the reference's
switch, kept so that existing launch scripts work) or `SGLANG_USE_B200_QUANT=1`, and import this
module (for example from a `.pth` file in site-packages, as `README.md:97-100` of the reference
does).  Without lmslim installed the patch reports that and does nothing.
"""
import importlib
import os

ENV_SWITCHES = ("SGLANG_USE_B200_QUANT", "SGLANG_USE_HIP_QUANT")
TARGET_MODULE = "lmslim.layers.gemm.int8_utils"
_MARK = "_b200_graph_safe_patched"


def make_wrapper(ext, current_stream_ptr):
    """The replacement function.  `scale_dtype` and `cal_sum` are accepted and ignored, exactly as
    the reference's wrapper does (hip_graph_safe.py:25-28)."""

    def b200_wrapper(x, scale_dtype=None, cal_sum=False):
        return ext.per_token_quant_int8_stream(x, current_stream_ptr())

    return b200_wrapper


def apply_patch(ext=None, log=print) -> bool:
    """Returns True if the engine function was (or already had been) rebound."""
    try:
        target = importlib.import_module(TARGET_MODULE)
    except ImportError:
        log("[B200-GRAPH-SAFE] lmslim is not installed, nothing to patch")
        return False
    if getattr(target, _MARK, False):
        return True
    if ext is None:
        import bw1000_dsv4_kernels_b200 as pkg
        ext = pkg.dsv4_native_ext          # raises ImportError if the extension has not been built
    import torch

    target._orig_per_token_quant_int8 = target.per_token_quant_int8
    target.per_token_quant_int8 = make_wrapper(ext, lambda: torch.cuda.current_stream().cuda_stream)
    setattr(target, _MARK, True)
    log("[B200-GRAPH-SAFE] Patched lmslim.per_token_quant_int8 -> dsv4_native_ext (sm_100a) with stream")
    return True


def remove_patch() -> bool:
    try:
        target = importlib.import_module(TARGET_MODULE)
    except ImportError:
        return False
    if not getattr(target, _MARK, False):
        return False
    target.per_token_quant_int8 = target._orig_per_token_quant_int8
    setattr(target, _MARK, False)
    return True


if any(os.environ.get(name, "0") == "1" for name in ENV_SWITCHES):
    apply_patch()
