"""The C-ABI library: it loads, exports every symbol include/monofab.h declares,
reports the operand-block layouts of the reference, and fails loudly (never
falls back) without a GPU."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported():
    from monoserve_b200 import _C
    header = open(os.path.join(ROOT, "include", "monofab.h")).read()
    declared = set(re.findall(r"\b(monofab_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_C.EXPORTS)
    for name in declared:
        assert getattr(_C.lib, name) is not None
    assert _C.lib.monofab_version() >= 100


def test_struct_layouts_have_the_reference_sizes():
    from monoserve_b200 import _C
    L = _C.struct_layouts()
    # sizes: csrc/fabric/model_types.h:66,96,114,128,205,216,229
    want = {"GemmArgs": 128, "AttnArgs": 128, "NormArgs": 128, "StepArgs": 64, "ReduceArgs": 64,
            "PermuteArgs": 128, "SampleArgs": 64}
    for name, size in want.items():
        assert L[name][0] == size
    for name in ("QkArgs", "RouterArgs", "ExpandArgs", "AttnPlanArgs"):
        assert L[name][0] % 64 == 0
    g = L["GemmArgs"][1]
    assert g["out"] == (0, "u64") and g["ld_out"] == (40, "u32") and g["w_fp8"] == (68, "u32")
    assert L["RouterArgs"][1]["scale"][1] == "f32"
    assert L["AttnArgs"][1]["scale_log2"] == (72, "f32")


def test_gemm_args_packs_by_layout():
    import struct
    from monoserve_b200 import _C
    b = _C.gemm_args(out=0x1234, ld_out=7, k_tiles=3, epi=2, bm=64, n_limit=99, pair_token=5, up_offset=11)
    assert len(b) == 128
    assert struct.unpack_from("<Q", b, 0)[0] == 0x1234 and struct.unpack_from("<I", b, 40)[0] == 7
    assert struct.unpack_from("<I", b, 64)[0] == 11
    from monoserve_b200.fabric.args import pack
    with pytest.raises(KeyError):
        pack("GemmArgs", nonsense=1)


def test_argument_errors_are_reported():
    from monoserve_b200 import _C
    cfg = _C.MoEConfigC(hidden=100, intermediate=64, experts=8, top_k=2, max_tokens=4)
    h = ctypes.c_void_p()
    assert _C.lib.monofab_moe_create(ctypes.byref(cfg), ctypes.byref(h)) == -1
    assert b"hidden" in _C.lib.monofab_last_error()
    with pytest.raises(RuntimeError, match="monofab: .*experts"):
        cfg = _C.MoEConfigC(hidden=256, intermediate=64, experts=300, top_k=2, max_tokens=4)
        _C.check(_C.lib.monofab_moe_create(ctypes.byref(cfg), ctypes.byref(h)))
    assert _C.lib.monofab_router_topk(None, None, None, None, None, None, None, 1, 8, 2, 0, 1, 1.0, 0, None) == -1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback():
    from monoserve_b200 import _C
    cfg = _C.MoEConfigC(hidden=256, intermediate=64, experts=8, top_k=2, max_tokens=4)
    h = ctypes.c_void_p()
    assert _C.lib.monofab_moe_create(ctypes.byref(cfg), ctypes.byref(h)) == -2   # MONOFAB_ECUDA
    from monoserve_b200.moe import MoELayer
    with pytest.raises(RuntimeError, match="CUDA device is required"):
        MoELayer(256, 64, 8, 2, 4)


def test_releases_wait_for_a_resident_fabric():
    """The deferred-release registry without a GPU: a release handed in while a fabric counts as
    running on the device is queued, survives the stop of one of two fabrics, and is carried out
    when the last one stops; with none running it is carried out at once."""
    import ctypes
    from monoserve_b200 import _C
    dev = 63    # a device index nothing else in the tests uses

    def state():
        out = (ctypes.c_uint64 * 3)()
        assert _C.lib.monofab_release_debug(3, dev, ctypes.byref(out)) == 0
        return list(out)

    queued0, done0, running0 = state()
    assert (queued0, running0) == (0, 0)
    assert _C.lib.monofab_release_debug(2, dev, None) == 0            # nothing resident: at once
    assert state() == [0, done0 + 1, 0]
    _C.lib.monofab_release_debug(0, dev, None)                         # two fabrics start
    _C.lib.monofab_release_debug(0, dev, None)
    for _ in range(3):
        _C.lib.monofab_release_debug(2, dev, None)
    assert state() == [3, done0 + 1, 2]
    _C.lib.monofab_release_debug(1, dev, None)                         # one stops: still queued
    assert state() == [3, done0 + 1, 1]
    _C.lib.monofab_release_debug(1, dev, None)                         # the last one stops: drained
    assert state() == [0, done0 + 4, 0]
    assert _C.lib.monofab_release_debug(3, 64, None) != 0              # device index out of range
