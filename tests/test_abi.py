"""CPU checks of the drop-in boundary: the shared library loads, exports every entry point that
include/splash_b200.h declares, refuses compute without a device instead of falling back, and plans
projections as documented."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "splash_b200.h")).read()
    return sorted(set(re.findall(r"SB_API\s+[\w\s\*]+?\b(sb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from splash_b200 import lib
    l = lib.load()
    names = declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(l, n)]
    assert not missing, missing


def test_no_cpu_fallback_without_a_device():
    from splash_b200 import lib
    if lib.device_count() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(lib.SbError):
        lib.init(0)
    with pytest.raises(lib.SbError):
        lib.DeviceBuffer(1024)
    with pytest.raises(lib.SbError):
        lib.linear(1 << 20, 1 << 20, 1 << 20, 0, 64, 1024, 16)


def test_linear_plans_of_the_27b_projections():
    from splash_b200 import lib
    l = lib.load()
    l.sb_linear_plan.argtypes = [ctypes.c_uint32] * 5 + [ctypes.POINTER(lib.SbLinearPlan)]
    p = lib.SbLinearPlan()
    # gate/up: K = 5120 = 20 super-blocks in 2 slices of 10, 544 tiles of 32 columns
    assert l.sb_linear_plan(lib.FMT_Q4K, 17408, 5120, 16, lib.EP_GATE_UP, ctypes.byref(p)) == 0
    assert (p.slices, p.tiles, p.slice_blocks_max, p.ctas) == (2, 544, 10, 148) and p.smem_bytes <= 227 * 1024 and p.stages >= 2
    # the tensor-memory kernel: 136 tiles of 128 columns (the tensor-memory lanes)
    l.sb_linear_plan_flags.argtypes = [ctypes.c_uint32] * 6 + [ctypes.POINTER(lib.SbLinearPlan)]
    T = lib.LINEAR_TCGEN05
    assert l.sb_linear_plan_flags(lib.FMT_Q4K, 17408, 5120, 16, lib.EP_GATE_UP, T, ctypes.byref(p)) == 0
    assert (p.slices, p.tiles, p.tile_rows, p.slice_blocks_max, p.ctas) == (2, 136, 128, 10, 148)
    assert p.smem_bytes <= 227 * 1024 and p.stages >= 3 and p.stages % 3 == 0
    # every Q4_K projection of the 27B shape gets a plan whose slices cover K and whose grid is whole slice groups
    for n, k in ((14336, 5120), (16384, 5120), (5120, 6144), (5120, 17408), (248320, 5120)):
        assert l.sb_linear_plan_flags(lib.FMT_Q4K, n, k, 16, 0, T, ctypes.byref(p)) == 0
        assert p.slices * p.slice_blocks_max >= k // 256 and p.ctas % p.slices == 0 and p.ctas <= 148
        assert p.smem_bytes <= 227 * 1024 and p.stages % 3 == 0 and p.tiles == (n + 127) // 128
    # down: Q6_K, K = 17408 = 68 super-blocks
    assert l.sb_linear_plan(lib.FMT_Q6K, 5120, 17408, 16, lib.EP_RESIDUAL, ctypes.byref(p)) == 0
    assert p.slices * p.slice_blocks_max >= 68 and p.ctas % p.slices == 0 and p.smem_bytes <= 227 * 1024
    # argument errors are values, not crashes
    assert l.sb_linear_plan(lib.FMT_Q4K, 17408, 5000, 16, 0, ctypes.byref(p)) == -1
    assert l.sb_linear_plan(3, 64, 1024, 16, 0, ctypes.byref(p)) == -1
    assert b"format" in l.sb_last_error()


def test_row_bytes():
    from splash_b200 import lib
    l = lib.load()
    assert l.sb_row_bytes(lib.FMT_Q4K, 5120) == 20 * 144
    assert l.sb_row_bytes(lib.FMT_Q6K, 17408) == 68 * 210
    assert l.sb_row_bytes(lib.FMT_Q80, 5120) == 160 * 34
    assert l.sb_row_bytes(lib.FMT_Q4K, 100) == 0


def test_ctypes_mirrors_have_the_headers_structure_sizes():
    """Every argument structure the harness mirrors in ctypes has the size the library was compiled with."""
    import ctypes
    from splash_b200 import lib, target, tp
    l = lib.load()
    l.sb_struct_bytes.restype = ctypes.c_uint64
    l.sb_struct_bytes.argtypes = [ctypes.c_char_p]
    mirrors = dict(SbLinearArgs=lib.SbLinearArgs, SbLinearPlan=lib.SbLinearPlan, SbKvLayer=lib.SbKvLayer, SbAttnStoreArgs=lib.SbAttnStoreArgs,
                   SbAttnArgs=lib.SbAttnArgs, SbGdnTape=lib.SbGdnTape, SbGdnArgs=lib.SbGdnArgs, SbSampleArgs=lib.SbSampleArgs,
                   SbPenaltyArgs=lib.SbPenaltyArgs, SbAcceptArgs=lib.SbAcceptArgs, SbSelectAcceptArgs=lib.SbSelectAcceptArgs, SbAdmitArgs=lib.SbAdmitArgs, SbLanePolicy=lib.SbLanePolicy, SbMoeRouteArgs=lib.SbMoeRouteArgs,
                   SbMoeExpertArgs=lib.SbMoeExpertArgs, SbTargetConfig=target.SbTargetConfig, SbTargetShare=tp.SbTargetShare)
    for name, mirror in mirrors.items():
        assert int(l.sb_struct_bytes(name.encode())) == ctypes.sizeof(mirror), name
    assert int(l.sb_struct_bytes(b"NoSuchStruct")) == 0
