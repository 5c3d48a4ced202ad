"""The engine patch against a fake lmslim module (no GPU, no lmslim needed)."""
import sys
import types

import pytest


@pytest.fixture
def fake_lmslim(monkeypatch):
    pkg = types.ModuleType("lmslim")
    layers = types.ModuleType("lmslim.layers")
    gemm = types.ModuleType("lmslim.layers.gemm")
    utils = types.ModuleType("lmslim.layers.gemm.int8_utils")
    utils.per_token_quant_int8 = lambda x, scale_dtype=None, cal_sum=False: ("engine", x)
    for name, mod in (("lmslim", pkg), ("lmslim.layers", layers), ("lmslim.layers.gemm", gemm),
                      ("lmslim.layers.gemm.int8_utils", utils)):
        monkeypatch.setitem(sys.modules, name, mod)
    return utils


class FakeExt:
    def __init__(self):
        self.calls = []

    def per_token_quant_int8_stream(self, x, stream_ptr):
        self.calls.append((x, stream_ptr))
        return ["q", "s"]


def test_patch_rebinds_with_reference_signature(fake_lmslim):
    from bw1000_dsv4_kernels_b200 import lmslim_patch
    ext = FakeExt()
    msgs = []
    wrapper = lmslim_patch.make_wrapper(ext, lambda: 1234)
    assert wrapper("x", scale_dtype="float32", cal_sum=True) == ["q", "s"]
    assert ext.calls == [("x", 1234)]
    assert lmslim_patch.apply_patch(ext=ext, log=msgs.append) is True
    assert fake_lmslim.per_token_quant_int8.__name__ == "b200_wrapper"
    assert fake_lmslim._orig_per_token_quant_int8("y")[0] == "engine"
    assert lmslim_patch.apply_patch(ext=ext, log=msgs.append) is True      # idempotent
    assert len(msgs) == 1 and "Patched" in msgs[0]
    assert lmslim_patch.remove_patch() is True
    assert fake_lmslim.per_token_quant_int8("z")[0] == "engine"


def test_patch_without_lmslim_is_a_no_op(monkeypatch):
    from bw1000_dsv4_kernels_b200 import lmslim_patch
    monkeypatch.setitem(sys.modules, "lmslim", None)
    msgs = []
    assert lmslim_patch.apply_patch(ext=FakeExt(), log=msgs.append) is False
    assert "not installed" in msgs[0]
