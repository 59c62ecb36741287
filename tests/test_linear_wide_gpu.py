"""Parity of the many-row projection (sb_linear with more than 16 rows -> sb_linear_wide: weights dequantized to half,
tcgen05 tensor cores, accumulators in tensor memory) with the oracle's fp64 products, through the C ABI.

Gate, as in the reference's projection test for its staged tile (dev/tests/engine/gguf_projection_test.mm:226-245):
every output lies in [round(v - e), round(v + e)], v the fp64 dot product and e the bound that admits weights rounded to
half (2^-16 sum|x| max|w| + 2^-11 sum|x w| + 2^-25 sum|x|, dev/tests/engine/GgufFormatReference.hpp:728-742). This
kernel rounds the weight's two factors (d sc, dmin mn) to half before their fused multiply-add, so each weight carries
up to three half roundings where the reference's tile carries one: the middle term is taken three times. The north
star's 2e-3 of the output's scale is checked as well."""
import numpy as np
import pytest

import oracle_lib as ol
import quant_fixtures as qf
from test_linear_gpu import check_interval, oracle_f64, run_linear

pytestmark = pytest.mark.gpu


def _setup():
    from splash_b200 import lib
    lib.init(0)
    return lib


def wide_bound(fmt, W, n, k, X, rows):
    v, be, bs = oracle_f64(fmt, W, n, k, X, rows)
    return v, be + 3.0 * (bs - be)


@pytest.mark.parametrize("n,k,rows", [
    (512, 1024, 128), (256, 5120, 64), (392, 2048, 17), (1024, 1024, 100), (256, 1024, 130), (768, 2048, 256), (128, 17408, 48),
])
def test_wide_plain(n, k, rows):
    lib = _setup()
    W = qf.realistic(0, n, k, seed=n + k)
    X = qf.activations(rows, k, seed=rows)
    got = run_linear(lib, 0, W, n, k, X, rows)
    v, e = wide_bound(0, W, n, k, X, rows)
    check_interval(got, v - e, v + e)
    # the north star's tolerance on the fp32 sums (the bf16 destination's own rounding is up to 2^-9 = 1.95e-3 more)
    got32 = run_linear(lib, 0, W, n, k, X, rows, out_f32=True)
    rel = np.abs(got32 - v) / np.maximum(np.abs(v), np.abs(v).mean())
    assert rel.max() < 2e-3 and np.median(rel) < 4e-4
    assert np.array_equal(got, ol.f2bf(got32))


def test_wide_config0_shape_at_128_rows():
    """The gate projection of the 27B shape at 128 rows (8 lanes of 16): X ~ N(0,1), W [17408, 5120] Q4_K by the benchmark's recipe."""
    lib = _setup()
    n, k, rows = 17408, 5120, 128
    W = qf.config0_q4k(n, k, seed=0)
    X = qf.activations(rows, k, seed=0)
    got = run_linear(lib, 0, W, n, k, X, rows)
    v, e = wide_bound(0, W, n, k, X, rows)
    check_interval(got, v - e, v + e)


def test_wide_f32_destination_rounds_to_bf16_destination():
    lib = _setup()
    n, k, rows = 512, 2048, 96
    W = qf.realistic(0, n, k)
    X = qf.activations(rows, k)
    a = run_linear(lib, 0, W, n, k, X, rows)
    b = run_linear(lib, 0, W, n, k, X, rows, out_f32=True)
    assert np.array_equal(a, ol.f2bf(b))


def test_wide_rows_independent_of_the_other_rows():
    """A row's output does not depend on how many other rows share the launch or the pass, nor on NaN in them."""
    lib = _setup()
    n, k = 256, 2048
    W = qf.realistic(0, n, k)
    X = qf.activations(160, k)
    full = run_linear(lib, 0, W, n, k, X, 160)
    some = run_linear(lib, 0, W, n, k, X[:40].copy(), 40)
    assert np.array_equal(full[:40], some)
    tail = run_linear(lib, 0, W, n, k, X[128:160].copy(), 32)   # the second pass's rows, alone
    assert np.array_equal(full[128:160], tail)
    Xn = X[:64].copy()
    Xn[30:] = 0x7FC0
    part = run_linear(lib, 0, W, n, k, Xn, 64)
    assert np.array_equal(full[:30], part[:30])


def test_wide_residual_gate_and_one_pass_gate_up():
    lib = _setup()
    n, k, rows = 384, 2048, 80
    rng = np.random.default_rng(3)
    W, W2 = qf.realistic(0, n, k, seed=1), qf.realistic(0, n, k, seed=2)
    X = qf.activations(rows, k)
    aux = ol.f2bf(rng.standard_normal((rows, n)).astype(np.float32))
    plain = run_linear(lib, 0, W, n, k, X, rows, out_f32=True)
    ad = lib.DeviceBuffer.from_numpy(aux)
    res = run_linear(lib, 0, W, n, k, X, rows, aux=ad.ptr, epilogue=lib.EP_RESIDUAL)
    assert np.array_equal(res, ol.f2bf(plain + ol.bf2f(aux)))
    silu = lambda x: x / (1.0 + np.exp2(np.float32(-1.44269504089) * x))
    gated = run_linear(lib, 0, W, n, k, X, rows, aux=ad.ptr, epilogue=lib.EP_UP_WITH_GATE)
    want = ol.bf2f(ol.f2bf(plain)) * silu(ol.bf2f(aux))
    d = np.abs(ol.bf2f(gated) - want)
    assert (d <= 2.0 ** -7 * np.abs(want) + 1e-30).all()          # within a bf16 step (the quotient is the approximate one)
    # one pass over gate and up rows == the separate gate pass feeding the up pass
    w2d = lib.DeviceBuffer.from_numpy(W2)
    one = run_linear(lib, 0, W, n, k, X, rows, weights2=w2d.ptr, epilogue=lib.EP_GATE_UP)
    gate = run_linear(lib, 0, W, n, k, X, rows)
    gd = lib.DeviceBuffer.from_numpy(gate)
    two = run_linear(lib, 0, W2, n, k, X, rows, aux=gd.ptr, epilogue=lib.EP_UP_WITH_GATE)
    assert np.array_equal(one, two)


@pytest.mark.parametrize("n,k,rows", [(512, 6144, 128), (1024, 17408, 80), (256, 1024, 40), (1280, 2816, 200)])
def test_wide_k_split_sums_then_the_conversion_that_adds_them(n, k, rows):
    """SB_EPILOGUE_PARTIALS leaves every k-range's sums; sb_linear_wide_prepare_sum adds them onto the residual in split order,
    writes the new hidden rows and converts them. The hidden rows against the oracle's bound, and the conversion equal to a
    plain conversion of those rows."""
    import ctypes
    lib = _setup()
    l = lib.load()
    l.sb_linear_wide_splits.argtypes = [ctypes.c_uint32] * 2
    l.sb_linear_wide_prepare_sum.argtypes = ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32,
                                              ctypes.c_void_p] + [ctypes.c_uint32] * 3 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32])
    rng = np.random.default_rng(n + rows)
    W = qf.realistic(0, n, k, seed=k)
    X = qf.activations(rows, k, seed=3)
    res = ol.f2bf(rng.standard_normal((rows, n)).astype(np.float32))
    splits = int(l.sb_linear_wide_splits(n, k))
    assert 1 <= splits <= 64 and (splits > 1 or k < 1536 or n >= 148 * 256)
    wd, xd, rd = lib.DeviceBuffer.from_numpy(W), lib.DeviceBuffer.from_numpy(X), lib.DeviceBuffer.from_numpy(res)
    parts = lib.DeviceBuffer(splits * rows * n * 4)
    parts.fill(0xFF)
    lib.linear(wd.ptr, xd.ptr, parts.ptr, 0, n, k, rows, epilogue=lib.EP_PARTIALS, out_f32=True)
    summed, norm_w = lib.DeviceBuffer(rows * n * 2), lib.DeviceBuffer.from_numpy((1 + 0.1 * rng.standard_normal(n)).astype(np.float32))
    nbytes = int(l.sb_linear_wide_prepared_bytes(rows, n))
    conv, conv2 = lib.DeviceBuffer(nbytes), lib.DeviceBuffer(nbytes)
    conv.fill(0), conv2.fill(0)
    lib.check(l.sb_linear_wide_prepare_sum(None, parts.ptr, splits, n, rd.ptr, n, summed.ptr, n, rows, n, norm_w.ptr, conv.ptr, 0))
    lib.stream_sync()
    assert lib.device_status() == 0
    p = parts.to_numpy(np.float32, (splits, rows, n))
    got = summed.to_numpy(np.uint16, (rows, n))
    total = np.zeros((rows, n), np.float32)
    for sp in range(splits):
        total += p[sp]
    assert np.array_equal(got, ol.f2bf(total + ol.bf2f(res)))              # the sum as stated: split order, then the residual
    v, e = wide_bound(0, W, n, k, X, rows)
    e = e + 2.0 ** -22 * splits * np.abs(v).max()                          # (fp32 additions of the splits)
    assert (total >= v - e).all() and (total <= v + e).all()
    lib.check(l.sb_linear_wide_prepare(None, summed.ptr, rows, n, n, norm_w.ptr, conv2.ptr, 0))
    lib.stream_sync()
    assert np.array_equal(conv.to_numpy(np.uint8, (nbytes,)), conv2.to_numpy(np.uint8, (nbytes,)))


def image_of(lib, fmt, W, n, k):
    wd = lib.DeviceBuffer.from_numpy(W)
    img = lib.DeviceBuffer(int(lib.load().sb_linear_wide_image_bytes(fmt, n, k)))
    lib.check(lib.load().sb_linear_wide_image(None, fmt, wd.ptr, n, k, img.ptr))
    lib.stream_sync()
    return img


def run_image(lib, fmt, img, n, k, X, rows, img2=None, **kw):
    xd = lib.DeviceBuffer.from_numpy(X)
    f32 = kw.get("out_f32", False)
    od = lib.DeviceBuffer(rows * n * (4 if f32 else 2) + 512)
    od.fill(0xFF)
    lib.linear(img.ptr, xd.ptr, od.ptr, fmt, n, k, rows, weights2=img2.ptr if img2 else None, flags=lib.LINEAR_WIDE_IMAGE, **kw)
    lib.stream_sync()
    assert lib.device_status() == 0
    return od.to_numpy(np.float32 if f32 else np.uint16, (rows, n))


@pytest.mark.parametrize("fmt", [4, 6, 37])
@pytest.mark.parametrize("n,k,rows", [(512, 1024, 128), (392, 2816, 17), (256, 5120, 64), (128, 17408, 48), (640, 2048, 200)])
def test_wide_q6k_and_nvfp4_images(fmt, n, k, rows):
    """Q6_K, Q8_0 and NVFP4 rows through their images: the weight's half is fl16(code * fl16(scale)), two roundings, so the
    middle term of the reference's bound for half-rounded weights is taken twice."""
    lib = _setup()
    W = qf.realistic(fmt, n, k, seed=n + k + fmt)
    X = qf.activations(rows, k, seed=rows)
    img = image_of(lib, fmt, W, n, k)
    v, be, bs = oracle_f64(fmt, W, n, k, X, rows)
    e = be + 2.0 * (bs - be)
    got = run_image(lib, fmt, img, n, k, X, rows)
    check_interval(got, v - e, v + e)
    got32 = run_image(lib, fmt, img, n, k, X, rows, out_f32=True)
    rel = np.abs(got32 - v) / np.maximum(np.abs(v), np.abs(v).mean())
    assert rel.max() < (4e-3 if fmt == 37 else 2e-3) and np.median(rel) < 4e-4    # (e2m1 codes: heavier tails than the 6- and 8-bit codes)
    assert np.array_equal(got, ol.f2bf(got32))


@pytest.mark.parametrize("fmt", [4, 37])
def test_wide_image_rows_with_scales_far_apart(fmt):
    """Rows whose scales differ by 2^40 from row to row, and by 2^12 inside a row: the power of two taken out of each row
    keeps every row's halves in range."""
    lib = _setup()
    n, k, rows = 256, 2048, 32
    rng = np.random.default_rng(9)
    W = qf.realistic(fmt, n, k, seed=3).reshape(n, k // 256, -1).copy()
    for r in range(n):
        row_pow = float(2.0 ** rng.integers(-20, 21))
        for sb in range(k // 256):
            inner = float(2.0 ** -rng.integers(0, 13))
            if fmt == 4:
                d = np.float16(min(6e4, max(6.2e-5, 1e-3 * row_pow * inner)))
                W[r, sb, 208:210] = np.frombuffer(d.tobytes(), np.uint8)
            else:
                W[r, sb, 16:20] = np.frombuffer(np.float32(1e-3 * row_pow * inner).tobytes(), np.uint8)
    W = W.reshape(n, -1)
    X = qf.activations(rows, k, seed=1)
    img = image_of(lib, fmt, W, n, k)
    v, be, bs = oracle_f64(fmt, W, n, k, X, rows)
    e = be + 2.0 * (bs - be)
    got32 = run_image(lib, fmt, img, n, k, X, rows, out_f32=True)
    assert np.isfinite(got32).all()
    assert (got32 >= v - e - 1e-30).all() and (got32 <= v + e + 1e-30).all()


def test_wide_image_gate_up_and_k_split_sums():
    lib = _setup()
    n, k, rows = 384, 2048, 80
    W, W2 = qf.realistic(37, n, k, seed=1), qf.realistic(37, n, k, seed=2)
    X = qf.activations(rows, k)
    g, u = image_of(lib, 37, W, n, k), image_of(lib, 37, W2, n, k)
    one = run_image(lib, 37, g, n, k, X, rows, img2=u, epilogue=lib.EP_GATE_UP)
    gate = run_image(lib, 37, g, n, k, X, rows)
    gd = lib.DeviceBuffer.from_numpy(gate)
    two = run_image(lib, 37, u, n, k, X, rows, aux=gd.ptr, epilogue=lib.EP_UP_WITH_GATE)
    assert np.array_equal(one, two)
    # the k-split sums of a Q6_K image add up to the plain product (fp32, up to the order of the additions)
    W6 = qf.realistic(4, 512, 6144, seed=5)
    X6 = qf.activations(rows, 6144)
    i6 = image_of(lib, 4, W6, 512, 6144)
    plain = run_image(lib, 4, i6, 512, 6144, X6, rows, out_f32=True)
    import ctypes
    lib.load().sb_linear_wide_splits.argtypes = [ctypes.c_uint32] * 2
    splits = int(lib.load().sb_linear_wide_splits(512, 6144))
    xd, parts = lib.DeviceBuffer.from_numpy(X6), lib.DeviceBuffer(splits * rows * 512 * 4)
    lib.linear(i6.ptr, xd.ptr, parts.ptr, 4, 512, 6144, rows, epilogue=lib.EP_PARTIALS, out_f32=True, flags=lib.LINEAR_WIDE_IMAGE)
    lib.stream_sync()
    total = parts.to_numpy(np.float32, (splits, rows, 512)).astype(np.float64).sum(axis=0)
    assert splits > 1 and np.abs(total - plain).max() <= 1e-5 * np.abs(plain).max()


def test_wide_rejects_what_it_does_not_multiply():
    lib = _setup()
    d = lib.DeviceBuffer(1 << 20)
    with pytest.raises(lib.SbError):
        lib.linear(d.ptr, d.ptr, d.ptr, lib.FMT_Q6K, 256, 1024, 64)       # Q6_K rows as they are: the kernel reads their image
    with pytest.raises(lib.SbError):
        lib.linear(d.ptr, d.ptr, d.ptr, lib.FMT_Q4K, 256, 1024, 64, flags=lib.LINEAR_WIDE_IMAGE)   # Q4_K has no image
    with pytest.raises(lib.SbError):
        lib.linear(d.ptr, d.ptr, d.ptr, lib.FMT_Q80, 256, 1024, 64)       # Q8_0 rows as they are: likewise
    with pytest.raises(lib.SbError):
        lib.linear(d.ptr, d.ptr, d.ptr, lib.FMT_Q4K, 256, 1000, 64)       # k not whole super-blocks
