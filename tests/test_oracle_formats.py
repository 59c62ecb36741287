"""The oracle's GGUF dequantization against the reference's golden hashes (SHA-256 of upstream
ggml output) and, where the reference shim was built, against the reference's CPU code bit for bit."""
import hashlib
import json
import os

import numpy as np
import pytest

from oracle_lib import dequant, load, load_ref, ptr, row_bytes

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "weight_goldens.json")))


@pytest.mark.parametrize("name", ["q4k", "q6k", "q80"])
def test_dequant_matches_golden_hash(name):
    lib = load()
    g = GOLD["gguf_dequantization"][name]
    rows, K, fmt = GOLD["rows"], GOLD["columns"], g["format"]
    native = np.zeros(rows * row_bytes(lib, fmt, K), np.uint8)
    assert lib.so_golden_fixture(fmt, rows, K, GOLD["seed_base"] + fmt, ptr(native)) == 0
    values = dequant(lib, fmt, native, rows, K)
    assert hashlib.sha256(values.tobytes()).hexdigest() == g["sha256"]


@pytest.mark.parametrize("fmt", [0, 4, 6, 37])
def test_dequant_matches_reference_code(fmt):
    ref = load_ref()
    if ref is None:
        pytest.skip("reference shim not built (reference tree absent)")
    lib = load()
    rows, K = 64, 2048
    native = np.zeros(rows * row_bytes(lib, fmt, K), np.uint8)
    assert ref.ref_realistic(fmt, rows, K, 42, ptr(native)) == 0
    assert ref.ref_row_bytes(fmt, K) == row_bytes(lib, fmt, K)
    mine = dequant(lib, fmt, native, rows, K)
    theirs = np.empty_like(mine)
    assert ref.ref_row_values(fmt, ptr(native), rows, K, ptr(theirs)) == 0
    assert np.array_equal(mine.view(np.uint32), theirs.view(np.uint32))


def test_row_bytes():
    lib = load()
    assert row_bytes(lib, 0, 5120) == 20 * 144
    assert row_bytes(lib, 4, 5120) == 20 * 210
    assert row_bytes(lib, 6, 5120) == 160 * 34
    assert row_bytes(lib, 0, 100) == 0
