"""Device dequantization (sb_dequant, through the C ABI) against the reference's golden hashes and the oracle.

The reference's own check is bit equality of the dequantized weights (dev/tests/engine/gguf_dequant_test.mm:50-56);
its recorded SHA-256 values of upstream ggml's output (dev/tests/fixtures/weight-goldens/goldens.json, copied to
tests/golden/weight_goldens.json) pin Q4_K, Q6_K and Q8_0 here without the reference tree. NVFP4, for which no hash
was recorded, and the fp16-rounded mode are held bit for bit against the oracle, itself pinned to the reference's
CPU code (tests/test_oracle_formats.py)."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle_lib as ol
import quant_fixtures as qf

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "weight_goldens.json")))


def _device_dequant(lib, fmt, native, rows, k, f16=False):
    wd = lib.DeviceBuffer.from_numpy(native)
    od = lib.DeviceBuffer(rows * k * (2 if f16 else 4))
    od.fill(0xFF)
    lib.check(lib.load().sb_dequant(None, fmt, wd.ptr, rows, k, od.ptr, int(f16)))
    lib.stream_sync()
    assert lib.device_status() == 0
    return od.to_numpy(np.float16 if f16 else np.float32, (rows, k))


@pytest.mark.parametrize("name", ["q4k", "q6k", "q80"])
def test_device_dequant_matches_golden_hash(name):
    from splash_b200 import lib
    lib.init(0)
    o = ol.load()
    g = GOLD["gguf_dequantization"][name]
    rows, k, fmt = GOLD["rows"], GOLD["columns"], g["format"]
    native = np.zeros(rows * ol.row_bytes(o, fmt, k), np.uint8)
    assert o.so_golden_fixture(fmt, rows, k, GOLD["seed_base"] + fmt, ol.ptr(native)) == 0
    values = _device_dequant(lib, fmt, native, rows, k)
    assert hashlib.sha256(values.tobytes()).hexdigest() == g["sha256"]


def _nvfp4_rows(rng, rows, k):
    """Rows of the loader's NVFP4 block (148 bytes per 256 weights: 16 E4M3 group scales, the fp32 tensor scale, 128
    bytes of E2M1 codes) with scales in the range of the reference's fixtures (GgufFormatReference.hpp:292-324)."""
    nb = k // 256
    blk = rng.integers(0, 256, (rows, nb, 148), dtype=np.uint8)
    blk[..., 0:16] = rng.integers(0x38, 0x68, (rows, nb, 16), dtype=np.uint8)
    g = rng.uniform(8e-6, 6e-5, (rows, nb)).astype(np.float32)
    blk[..., 16:20] = g.view(np.uint8).reshape(rows, nb, 4)
    return blk.reshape(rows, nb * 148)


@pytest.mark.parametrize("fmt", [0, 4, 6, 37])
@pytest.mark.parametrize("f16", [False, True])
def test_device_dequant_matches_oracle_bit_for_bit(fmt, f16):
    from splash_b200 import lib
    lib.init(0)
    o = ol.load()
    rows, k = 96, 2304 if fmt != 6 else 2304 + 32
    rng = np.random.default_rng(100 + fmt)
    native = _nvfp4_rows(rng, rows, k) if fmt == 37 else qf.realistic(fmt, rows, k, seed=100 + fmt)
    assert native.shape[1] == ol.row_bytes(o, fmt, k)
    want = ol.dequant(o, fmt, np.ascontiguousarray(native).reshape(-1), rows, k)
    got = _device_dequant(lib, fmt, native, rows, k, f16)
    if f16:
        # one more rounding of the fp32 value, as the reference's staged tile stores it (gguf_staged.h:11-17)
        assert np.array_equal(got.view(np.uint16), want.astype(np.float16).view(np.uint16))
    else:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_device_dequant_rejects_partial_blocks():
    from splash_b200 import lib
    lib.init(0)
    d = lib.DeviceBuffer(4096)
    assert lib.load().sb_dequant(None, 0, d.ptr, 1, 100, d.ptr, 0) == -1
    assert lib.load().sb_dequant(None, 99, d.ptr, 1, 256, d.ptr, 0) == -1
