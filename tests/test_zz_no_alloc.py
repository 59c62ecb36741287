"""sb_gdn_verify_static, the Gated-DeltaNet verify step for hosts that may not allocate device memory (a process
that gave its whole GPU to its own arena, a plugin inside one, code under a fixed memory budget): called through the
C ABI twice in a row and compared with sb_gdn_verify on the same inputs. Both run the same kernel, so the outputs
must be identical bit for bit, on the first call (which looks up the built-in scratch's address) and on the second
(which finds the previous call's contents in the scratch)."""
import ctypes

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu


def _inputs(rng, key_heads, value_heads):
    D = 128
    KW, VW = key_heads * D, value_heads * D
    C = 2 * KW + VW
    bf = lambda shape, s: ol.f2bf((rng.standard_normal(shape) * s).astype(np.float32))
    return dict(
        C=C, KW=KW, VW=VW, stride=C + VW,
        qkvz=bf((16, C + VW), 1.0), b=bf((16, value_heads), 1.0), a=bf((16, value_heads), 1.0), conv_w=bf((C, 4), 0.4),
        a_scale=(-np.exp(rng.uniform(-3, 0.5, value_heads))).astype(np.float32), dt_bias=bf((value_heads,), 0.5),
        norm_w=(1 + 0.1 * rng.standard_normal(D)).astype(np.float32), cs_in=bf((3, C), 1.0),
        state=(rng.standard_normal((value_heads, D, D)) * 0.05).astype(np.float32),
        pend=dict(inputs=bf((16, C), 1.0), k=bf((16, KW), 0.09), v=bf((16, VW), 0.5),
                  beta=ol.f2bf(rng.uniform(0.1, 0.9, (16, value_heads)).astype(np.float32)),
                  decay=rng.uniform(0.5, 1.0, (16, value_heads)).astype(np.float32)))


def _run(lib, l, entry, x, key_heads, value_heads, rows, pending_rows):
    up = lib.DeviceBuffer.from_numpy
    d = {n: up(x[n]) for n in ("qkvz", "b", "a", "conv_w", "a_scale", "dt_bias", "norm_w", "cs_in", "state")}
    dp = {n: up(v) for n, v in x["pend"].items()}
    sizes = dict(inputs=16 * x["C"] * 2, k=16 * x["KW"] * 2, v=16 * x["VW"] * 2, beta=16 * value_heads * 2, decay=16 * value_heads * 4)
    ds = {n: lib.DeviceBuffer(b) for n, b in sizes.items()}
    for b in ds.values():
        b.fill(0)
    dcs, dst, dh = lib.DeviceBuffer(x["cs_in"].nbytes), lib.DeviceBuffer(x["state"].nbytes), lib.DeviceBuffer(16 * x["VW"] * 2)
    dh.fill(0)
    tape = lambda t: lib.SbGdnTape(t["inputs"].ptr, t["k"].ptr, t["v"].ptr, t["beta"].ptr, t["decay"].ptr)
    args = lib.SbGdnArgs(d["qkvz"].ptr, d["b"].ptr, d["a"].ptr, d["conv_w"].ptr, d["a_scale"].ptr, d["dt_bias"].ptr, d["norm_w"].ptr,
                         d["cs_in"].ptr, dcs.ptr, d["state"].ptr, dst.ptr, tape(dp), tape(ds), dh.ptr, None,
                         rows, pending_rows, key_heads, value_heads, x["stride"], value_heads, x["VW"], 0)
    lib.check(entry(None, ctypes.byref(args)))
    lib.stream_sync()
    assert lib.device_status() == 0
    out = dict(cs=dcs.to_numpy(np.uint16, x["cs_in"].shape), state=dst.to_numpy(np.float32, x["state"].shape),
               hidden=dh.to_numpy(np.uint16, (16, x["VW"])))
    out.update({n: ds[n].to_numpy(np.uint8, (sizes[n],)) for n in sizes})
    return out


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    from splash_b200 import lib
    lib.init(0)
    l = lib.ops()
    for call, (seed, kh, vh, rows, pending) in enumerate([(21, 16, 48, 16, 7), (22, 2, 6, 9, 16)]):
        x = _inputs(np.random.default_rng(seed), kh, vh)
        want = _run(lib, l, l.sb_gdn_verify, x, kh, vh, rows, pending)
        got = _run(lib, l, l.sb_gdn_verify_static, x, kh, vh, rows, pending)
        for name in want:
            assert np.array_equal(got[name], want[name]), (call, name)
        assert np.abs(ol.bf2f(got["hidden"][:rows])).max() > 0  # the step did produce rows


def test_static_scratch_entry_point_rejects_shapes_beyond_its_array():
    from splash_b200 import lib
    lib.init(0)
    l = lib.ops()
    args = lib.SbGdnArgs(*([1 << 20] * 11), lib.SbGdnTape(*([1 << 20] * 5)), lib.SbGdnTape(*([1 << 20] * 5)), 1 << 20, None,
                         16, 0, 16, 80, 80 * 128 * 4, 80, 80 * 128, 0)
    assert l.sb_gdn_verify_static(None, ctypes.byref(args)) == -1
    assert b"64" in l.sb_last_error()
