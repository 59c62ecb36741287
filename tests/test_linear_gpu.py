"""Parity of sb_linear (CUDA, through the C ABI) with the oracle on seeded inputs.

Gate, as in the reference's projection test (dev/tests/engine/gguf_projection_test.mm:226-245): every
output must lie in [round(v - e), round(v + e)] where v is the fp64 dot product of the oracle and e
its projectionBound; Q4_K uses the bound of exactly represented weights, Q6_K / Q8_0 the bound that
admits one rounding of each weight to half."""
import ctypes

import numpy as np
import pytest

import oracle_lib as ol
import quant_fixtures as qf

pytestmark = pytest.mark.gpu


def _setup():
    from splash_b200 import lib
    lib.init(0)
    return lib


def oracle_f64(fmt, W, n, k, X, rows):
    o = ol.load()
    val = np.empty((rows, n), np.float64)
    be = np.empty_like(val)
    bs = np.empty_like(val)
    assert o.so_linear_f64(fmt, ol.ptr(W), n, k, ol.ptr(X), rows, ol.ptr(val), ol.ptr(be), ol.ptr(bs)) == 0
    return val, be, bs


def check_interval(got_bits, lo_val, hi_val):
    lo = ol.bf2f(ol.f2bf(lo_val.astype(np.float32)))
    hi = ol.bf2f(ol.f2bf(hi_val.astype(np.float32)))
    got = ol.bf2f(got_bits)
    bad = ~((got >= lo) & (got <= hi))
    assert not bad.any(), f"{bad.sum()} of {bad.size} outputs outside the bound; worst |got-v|={np.abs(got - (lo_val+hi_val)/2)[bad].max()}"


def run_linear(lib, fmt, W, n, k, X, rows, **kw):
    wd = lib.DeviceBuffer.from_numpy(W)
    xd = lib.DeviceBuffer.from_numpy(X)
    f32 = kw.get("out_f32", False)
    od = lib.DeviceBuffer(rows * n * (4 if f32 else 2) + 512)
    od.fill(0xFF)
    lib.linear(wd.ptr, xd.ptr, od.ptr, fmt, n, k, rows, **kw)
    lib.stream_sync()
    assert lib.device_status() == 0
    return od.to_numpy(np.float32 if f32 else np.uint16, (rows, n))


@pytest.mark.parametrize("fmt,n,k,rows", [
    (0, 512, 1024, 16), (0, 320, 5120, 16), (0, 192, 6144, 5), (0, 64, 17408, 16), (0, 96, 2816, 16),
    (4, 256, 1024, 16), (4, 128, 17408, 16), (4, 192, 5120, 3),
    (6, 256, 1024, 16), (6, 128, 5120, 7),
])
def test_linear_plain(fmt, n, k, rows):
    lib = _setup()
    W = qf.realistic(fmt, n, k, seed=n + k)
    X = qf.activations(rows, k, seed=rows)
    got = run_linear(lib, fmt, W, n, k, X, rows)
    v, be, bs = oracle_f64(fmt, W, n, k, X, rows)
    e = be if fmt == 0 else bs
    check_interval(got, v - e, v + e)


def test_linear_config0_q4k():
    """The benchmark's single-projection configuration: X bf16 [16, 5120] ~ N(0,1), W [17408, 5120] Q4_K."""
    lib = _setup()
    n, k, rows = 17408, 5120, 16
    W = qf.config0_q4k(n, k, seed=0)
    X = qf.activations(rows, k, seed=0)
    got = run_linear(lib, 0, W, n, k, X, rows)
    v, be, _ = oracle_f64(0, W, n, k, X, rows)
    check_interval(got, v - be, v + be)
    # north-star tolerance as well: 2e-3 relative to the output's scale
    rel = np.abs(ol.bf2f(got) - v) / np.maximum(np.abs(v), np.abs(v).mean())
    assert rel.max() < 4e-3  # bf16 rounding alone is 2^-9 = 1.95e-3


def test_linear_f32_destination_rounds_to_bf16_destination():
    lib = _setup()
    n, k, rows = 256, 5120, 16
    W = qf.realistic(0, n, k)
    X = qf.activations(rows, k)
    a = run_linear(lib, 0, W, n, k, X, rows)
    b = run_linear(lib, 0, W, n, k, X, rows, out_f32=True)
    assert np.array_equal(a, ol.f2bf(b))


def test_linear_rows_independent_of_batch():
    """A row's output does not depend on how many other rows share the launch, nor on NaN in them."""
    lib = _setup()
    n, k = 256, 5120
    W = qf.realistic(0, n, k)
    X = qf.activations(16, k)
    full = run_linear(lib, 0, W, n, k, X, 16)
    one = run_linear(lib, 0, W, n, k, X[:1].copy(), 1)
    assert np.array_equal(full[:1], one)
    Xn = X.copy()
    Xn[5:] = 0x7FC0
    part = run_linear(lib, 0, W, n, k, Xn, 16)
    assert np.array_equal(full[:5], part[:5])


@pytest.mark.parametrize("fmt", [0, 4])
def test_linear_residual_and_gate(fmt):
    lib = _setup()
    n, k, rows = 256, 5120, 16
    W = qf.realistic(fmt, n, k)
    X = qf.activations(rows, k)
    rng = np.random.default_rng(3)
    aux = ol.f2bf(rng.standard_normal((rows, n)).astype(np.float32) * 4)
    auxd = lib.DeviceBuffer.from_numpy(aux)
    plain = run_linear(lib, fmt, W, n, k, X, rows, out_f32=True)
    res = run_linear(lib, fmt, W, n, k, X, rows, aux=auxd.ptr, epilogue=lib.EP_RESIDUAL)
    assert np.array_equal(res, ol.f2bf(plain + ol.bf2f(aux)))
    up = run_linear(lib, fmt, W, n, k, X, rows, aux=auxd.ptr, epilogue=lib.EP_UP_WITH_GATE)
    g = ol.bf2f(aux)
    want = ol.bf2f(ol.f2bf(plain)) * (g / (1.0 + np.exp2(-1.44269504089 * g).astype(np.float32)))
    # the device's exp2 differs from numpy's in the last ulp: allow one bf16 ulp
    d = np.abs(ol.bf2f(up).astype(np.float64) - want)
    assert (d <= np.abs(want) * 2.0 ** -7 + 1e-30).all()


def test_linear_one_pass_gate_up_equals_two_passes():
    lib = _setup()
    n, k, rows = 256, 5120, 16
    Wg = qf.realistic(0, n, k, seed=1)
    Wu = qf.realistic(0, n, k, seed=2)
    X = qf.activations(rows, k)
    gate = run_linear(lib, 0, Wg, n, k, X, rows)
    gd = lib.DeviceBuffer.from_numpy(gate)
    two = run_linear(lib, 0, Wu, n, k, X, rows, aux=gd.ptr, epilogue=lib.EP_UP_WITH_GATE)
    wud = lib.DeviceBuffer.from_numpy(Wu)
    one = run_linear(lib, 0, Wg, n, k, X, rows, weights2=wud.ptr, epilogue=lib.EP_GATE_UP)
    assert np.array_equal(one, two)


def test_linear_fused_rmsnorm_matches_oracle_norm():
    lib = _setup()
    n, k, rows = 256, 5120, 16
    W = qf.realistic(0, n, k)
    X = qf.activations(rows, k)
    rng = np.random.default_rng(9)
    wn = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    x = ol.bf2f(X).astype(np.float64)
    inv = 1.0 / np.sqrt((x * x).mean(axis=1, keepdims=True) + 1e-6)
    Xn = ol.f2bf(((x * inv).astype(np.float32) * wn).astype(np.float32))
    wnd = lib.DeviceBuffer.from_numpy(wn)
    fused = run_linear(lib, 0, W, n, k, X, rows, norm_weight=wnd.ptr, out_f32=True)
    separate = run_linear(lib, 0, W, n, k, Xn, rows, out_f32=True)
    # the normalized inputs may differ by one bf16 ulp where fp32 and fp64 inverse RMS round apart
    assert np.abs(fused - separate).max() <= 2e-2 * np.abs(separate).max()
    assert np.median(np.abs(fused - separate)) <= 1e-3 * np.abs(separate).max()


def test_linear_rejects_bad_arguments():
    lib = _setup()
    with pytest.raises(lib.SbError):
        lib.linear(1 << 20, 1 << 20, 1 << 20, 0, 64, 1000, 16)  # k not whole super-blocks
    with pytest.raises(lib.SbError):
        lib.linear(1 << 20, 1 << 20, 1 << 20, 0, 64, 1024, 0)  # no rows
    with pytest.raises(lib.SbError):
        lib.linear(1 << 20, 1 << 20, 1 << 20, 4, 64, 1024, 17)  # more than 16 rows go to the many-row kernel, which multiplies Q4_K only
    with pytest.raises(lib.SbError):
        lib.linear(1 << 20, 1 << 20, 1 << 20, 3, 64, 1024, 16)  # unsupported format


# ---- the same contract on the tcgen05 kernel (SB_LINEAR_TCGEN05: weights expanded into tensor memory) ----

@pytest.mark.parametrize("n,k,rows", [(512, 1024, 16), (320, 5120, 16), (192, 6144, 5), (64, 17408, 16), (96, 2816, 16), (4096, 256, 1)])
def test_linear_tcgen05_plain(n, k, rows):
    lib = _setup()
    W = qf.realistic(0, n, k, seed=n + k)
    X = qf.activations(rows, k, seed=rows)
    got = run_linear(lib, 0, W, n, k, X, rows, flags=lib.LINEAR_TCGEN05)
    v, be, _ = oracle_f64(0, W, n, k, X, rows)
    check_interval(got, v - be, v + be)


def test_linear_tcgen05_config0_and_agreement_with_warp_kernel():
    """Benchmark configuration 0 on the tensor-memory kernel; both kernels feed the tensor cores the same exact
    integer operands, so they may differ only by the order of fp32 additions."""
    lib = _setup()
    n, k, rows = 17408, 5120, 16
    W = qf.config0_q4k(n, k, seed=0)
    X = qf.activations(rows, k, seed=0)
    got = run_linear(lib, 0, W, n, k, X, rows, flags=lib.LINEAR_TCGEN05, out_f32=True)
    v, be, _ = oracle_f64(0, W, n, k, X, rows)
    check_interval(ol.f2bf(got), v - be, v + be)
    warp = run_linear(lib, 0, W, n, k, X, rows, out_f32=True)
    assert np.abs(got - warp).max() <= 1e-5 * np.abs(warp).max()


def test_linear_tcgen05_epilogues():
    lib = _setup()
    n, k, rows = 384, 5120, 16
    T = lib.LINEAR_TCGEN05
    Wg = qf.realistic(0, n, k, seed=1)
    Wu = qf.realistic(0, n, k, seed=2)
    X = qf.activations(rows, k)
    rng = np.random.default_rng(3)
    aux = ol.f2bf(rng.standard_normal((rows, n)).astype(np.float32) * 4)
    auxd = lib.DeviceBuffer.from_numpy(aux)
    plain = run_linear(lib, 0, Wg, n, k, X, rows, out_f32=True, flags=T)
    assert np.array_equal(run_linear(lib, 0, Wg, n, k, X, rows, flags=T), ol.f2bf(plain))
    res = run_linear(lib, 0, Wg, n, k, X, rows, aux=auxd.ptr, epilogue=lib.EP_RESIDUAL, flags=T)
    assert np.array_equal(res, ol.f2bf(plain + ol.bf2f(aux)))
    gate = run_linear(lib, 0, Wg, n, k, X, rows, flags=T)
    gd = lib.DeviceBuffer.from_numpy(gate)
    two = run_linear(lib, 0, Wu, n, k, X, rows, aux=gd.ptr, epilogue=lib.EP_UP_WITH_GATE, flags=T)
    wud = lib.DeviceBuffer.from_numpy(Wu)
    one = run_linear(lib, 0, Wg, n, k, X, rows, weights2=wud.ptr, epilogue=lib.EP_GATE_UP, flags=T)
    assert np.array_equal(one, two)


def test_linear_tcgen05_rows_independent_of_batch():
    lib = _setup()
    n, k = 256, 5120
    W = qf.realistic(0, n, k)
    X = qf.activations(16, k)
    T = lib.LINEAR_TCGEN05
    full = run_linear(lib, 0, W, n, k, X, 16, flags=T)
    one = run_linear(lib, 0, W, n, k, X[:1].copy(), 1, flags=T)
    assert np.array_equal(full[:1], one)
    Xn = X.copy()
    Xn[5:] = 0x7FC0
    part = run_linear(lib, 0, W, n, k, Xn, 16, flags=T)
    assert np.array_equal(full[:5], part[:5])


@pytest.mark.parametrize("fmt,n,k", [(0, 5120, 6144), (4, 1024, 17408), (0, 256, 1024)])
def test_linear_partial_sums_then_prepare_sum_equal_the_residual_epilogue(fmt, n, k):
    """SB_EPILOGUE_PARTIALS leaves the k-slices' sums; sb_linear_prepare_sum adds them and the residual in the same
    order as the in-kernel reduction, so the new hidden state has the same bits, and so has what is prepared from it."""
    lib = _setup()
    L = lib.load()
    rows = 16
    W = qf.realistic(fmt, n, k, seed=5)
    X = qf.activations(rows, k, seed=6)
    rng = np.random.default_rng(7)
    res = ol.f2bf(rng.standard_normal((rows, n)).astype(np.float32) * 2)
    resd = lib.DeviceBuffer.from_numpy(res)
    want = run_linear(lib, fmt, W, n, k, X, rows, aux=resd.ptr, epilogue=lib.EP_RESIDUAL)
    plan = lib.SbLinearPlan()
    L.sb_linear_plan.argtypes = [ctypes.c_uint32] * 5 + [ctypes.POINTER(lib.SbLinearPlan)]
    lib.check(L.sb_linear_plan(fmt, n, k, rows, lib.EP_PARTIALS, ctypes.byref(plan)))
    wd, xd = lib.DeviceBuffer.from_numpy(W), lib.DeviceBuffer.from_numpy(X)
    parts = lib.DeviceBuffer(plan.slices * 16 * n * 4)
    parts.fill(0xFF)
    lib.linear(wd.ptr, xd.ptr, parts.ptr, fmt, n, k, rows, epilogue=lib.EP_PARTIALS, out_f32=True)
    # consumer side: a Q4_K projection of the new hidden state (n must be whole super-blocks)
    prep_a, prep_b = lib.DeviceBuffer(int(L.sb_linear_prepared_bytes(n))), lib.DeviceBuffer(int(L.sb_linear_prepared_bytes(n)))
    hidden = lib.DeviceBuffer(rows * n * 2)
    wn = lib.DeviceBuffer.from_numpy((1 + 0.1 * rng.standard_normal(n)).astype(np.float32))
    lib.check(L.sb_linear_prepare_sum(None, parts.ptr, plan.slices, n, resd.ptr, n, hidden.ptr, n, rows, n, wn.ptr, lib.FMT_Q4K, prep_a.ptr, None, 0))
    lib.stream_sync()
    assert lib.device_status() == 0
    got = hidden.to_numpy(np.uint16, (rows, n))
    assert np.array_equal(got, want)
    wantd = lib.DeviceBuffer.from_numpy(want)
    lib.check(L.sb_linear_prepare(None, wantd.ptr, rows, n, n, wn.ptr, lib.FMT_Q4K, prep_b.ptr, None, 0))
    lib.stream_sync()
    assert np.array_equal(prep_a.to_numpy(np.uint8, (int(L.sb_linear_prepared_bytes(n)),)), prep_b.to_numpy(np.uint8, (int(L.sb_linear_prepared_bytes(n)),)))


@pytest.mark.parametrize("fmt,n,k", [(0, 17408, 5120), (0, 2816, 1024), (4, 512, 2048), (6, 256, 1024)])
def test_gate_up_partial_sums_then_prepare_equal_the_one_pass_epilogue(fmt, n, k):
    """SB_EPILOGUE_GATE_UP_PARTIALS leaves the pair's k-slice sums; sb_linear_prepare_gate_up adds them in slice order and
    applies the activation: the SwiGLU result and what is prepared from it have the bits of the one-pass epilogue."""
    lib = _setup()
    L = lib.load()
    rows = 16
    Wg, Wu = qf.realistic(fmt, n, k, seed=11), qf.realistic(fmt, n, k, seed=12)
    X = qf.activations(rows, k, seed=13)
    gd, ud, xd = lib.DeviceBuffer.from_numpy(Wg), lib.DeviceBuffer.from_numpy(Wu), lib.DeviceBuffer.from_numpy(X)
    act = lib.DeviceBuffer(rows * n * 2 + 256)
    lib.linear(gd.ptr, xd.ptr, act.ptr, fmt, n, k, rows, weights2=ud.ptr, epilogue=lib.EP_GATE_UP)
    lib.stream_sync()
    want = act.to_numpy(np.uint16, (rows, n))
    plan = lib.SbLinearPlan()
    L.sb_linear_plan.argtypes = [ctypes.c_uint32] * 5 + [ctypes.POINTER(lib.SbLinearPlan)]
    lib.check(L.sb_linear_plan(fmt, n, k, rows, lib.EP_GATE_UP_PARTIALS, ctypes.byref(plan)))
    parts = lib.DeviceBuffer(plan.slices * 16 * 2 * n * 4)
    parts.fill(0xFF)
    lib.linear(gd.ptr, xd.ptr, parts.ptr, fmt, n, k, rows, weights2=ud.ptr, epilogue=lib.EP_GATE_UP_PARTIALS, out_f32=True, out_stride=2 * n)
    nb = (n + 255) // 256 * 256
    if nb != n:
        return  # the conversion takes whole super-blocks; the partial sums above were still written without a fault
    P, U = ctypes.c_void_p, ctypes.c_uint32
    L.sb_linear_prepare_gate_up.argtypes = [P, P, U, U, U, P, U, U, U, P, U]
    size = int(L.sb_linear_prepared_bytes(n))
    prep_a, prep_b = lib.DeviceBuffer(size), lib.DeviceBuffer(size)
    got_act = lib.DeviceBuffer(rows * n * 2 + 256)
    lib.check(L.sb_linear_prepare_gate_up(None, parts.ptr, plan.slices, 2 * n, n, got_act.ptr, n, rows, lib.FMT_Q6K, prep_a.ptr, 0))
    lib.stream_sync()
    assert lib.device_status() == 0
    got = got_act.to_numpy(np.uint16, (rows, n))
    # -0 and +0 are the same activation; everything else bit for bit
    same = (got == want) | (((got | want) & 0x7FFF) == 0)
    assert same.all()
    lib.check(L.sb_linear_prepare(None, act.ptr, rows, n, n, None, lib.FMT_Q6K, prep_b.ptr, None, 0))
    lib.stream_sync()
    a, b = prep_a.to_numpy(np.uint8, (size,)), prep_b.to_numpy(np.uint8, (size,))
    assert np.array_equal(a.view(np.float16) == 0, b.view(np.float16) == 0)
    assert np.array_equal(a.view(np.uint16) & 0x7FFF, b.view(np.uint16) & 0x7FFF) or np.array_equal(a, b)
    # the contract: fp32 rows of 2 n columns
    bad = lib.SbLinearArgs(gd.ptr, ud.ptr, xd.ptr, None, None, parts.ptr, None, fmt, n, k, rows, k, 0, n, lib.EP_GATE_UP_PARTIALS, 1, 0)
    assert L.sb_linear(None, ctypes.byref(bad)) == -1
