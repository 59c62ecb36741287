"""The prompt-lookup index (host code: runs without a GPU) against the reference's own: vectors written from the reference's
compiled LookupIndex (tests/golden/lookup_goldens.json), the compiled reference itself after every token where it was built
here, the replay fixture of the reference's test where the reference tree is present, and a statement of the match by
exhaustive search."""
import ctypes
import json
import os
import time

import numpy as np
import pytest

import oracle_lib as ol

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lookup_goldens.json")


def brute_match(tokens, n):
    """The match after tokens[:n]: the longest suffix (up to 64, at least 3 tokens) that ended earlier, most recent first."""
    best, end = 0, 0
    for e in range(n - 2, -1, -1):
        k = 0
        while k < 64 and k <= e and tokens[e - k] == tokens[n - 1 - k]:
            k += 1
        if k > best:
            best, end = k, e
        if best == 64:
            break
    return (best, end) if best >= 3 else (0, 0)


def trace(tokens):
    from splash_b200 import lookup
    index = lookup.LookupIndex()
    out = []
    for t in tokens:
        index.append([t])
        out.append(index.match())
    return index, out


def test_index_reproduces_the_vectors_written_from_the_reference():
    cases = json.load(open(GOLDEN))["cases"]
    assert len(cases) == 8
    matched = 0
    for case in cases:
        _, got = trace(case["tokens"])
        want = list(zip(case["lengths"], case["ends"]))
        assert got == want, case["name"]
        matched += sum(1 for n, _ in want if n)
    assert matched > 4000


def test_index_equals_exhaustive_search_and_proposes_what_followed():
    from splash_b200 import lookup
    rng = np.random.default_rng(5)
    for alphabet, n in ((2, 300), (4, 500), (30, 700)):
        tokens = rng.integers(0, alphabet, n).astype(np.uint32)
        index, got = trace(tokens)
        for i, m in enumerate(got):
            assert m == brute_match(tokens, i + 1), (alphabet, i)
        length, end = index.match()
        if length:
            assert np.array_equal(index.proposals(31), tokens[end + 1:end + 32])
            assert len(index.proposals(10 ** 6)) == n - 1 - end          # at most as far as the latest token
        assert len(index) == n
    # appending a block at once is appending its tokens one by one
    a, b = lookup.LookupIndex(), lookup.LookupIndex()
    a.append(tokens)
    for t in tokens:
        b.append([t])
    assert a.match() == b.match() and np.array_equal(a.proposals(16), b.proposals(16))
    # nothing before the third token, and nothing for tokens that never repeat
    fresh = lookup.LookupIndex()
    fresh.append(np.arange(100))
    assert fresh.match() == (0, 0) and len(fresh.proposals(16)) == 0
    assert lookup.agreement(5, 0, np.arange(5, 21)) == 0 and lookup.agreement(9, 0, np.arange(5, 21)) == 1
    assert lookup.agreement(99, 0, np.arange(5, 21)) == 2 and lookup.agreement(5, 1, np.arange(5, 21)) == 3


def _reference():
    path = os.path.join(ol.ORACLE_DIR, "_ref", "libsplash_ref_lookup.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libsplash_ref_lookup.so was not built (no reference tree here)")
    ref = ctypes.CDLL(path)
    ref.ref_lookup_trace.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    return ref


def test_index_equals_the_compiled_reference_after_every_token():
    ref = _reference()
    rng = np.random.default_rng(11)
    for alphabet, n in ((2, 3000), (3, 3000), (7, 4000), (300, 5000)):
        tokens = rng.integers(0, alphabet, n).astype(np.uint32)
        if alphabet == 300:                           # spans copied from earlier places, as a rewrite of a file would
            for _ in range(30):
                a, k, at = rng.integers(0, n - 200), rng.integers(3, 150), rng.integers(200, n - 200)
                tokens[at:at + k] = tokens[a:a + k]
        lengths, ends = np.zeros(n, np.uint32), np.zeros(n, np.uint32)
        ref.ref_lookup_trace(tokens.ctypes.data, n, lengths.ctypes.data, ends.ctypes.data)
        _, got = trace(tokens)
        assert got == list(zip(lengths.tolist(), ends.tolist())), alphabet


def test_index_follows_the_references_replay_fixture():
    """The decode traces the reference's own test replays (dev/tests/engine/lookup_replay_fixture.txt, read where it lies):
    at every cycle's anchor the match and the chain of up to 31 tokens are the offline replay's."""
    # (the reference tree: SPLASH_REFERENCE, else a `reference` folder beside the repository)
    root = os.environ.get("SPLASH_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(ol.ORACLE_DIR)), "reference")
    path = os.path.join(root, "dev", "tests", "engine", "lookup_replay_fixture.txt")
    if not os.path.exists(path):
        pytest.skip("the reference tree is not here")
    from splash_b200 import lookup
    words = [w for line in open(path) if not line.startswith("#") for w in line.split()]
    at, requests, cycles, matched = 0, 0, 0, 0
    while at < len(words):
        assert words[at] == "request"
        prompt, total = int(words[at + 1]), int(words[at + 2])
        tokens = [int(w) for w in words[at + 3:at + 3 + total]]
        at += 3 + total
        requests += 1
        index, filed = lookup.LookupIndex(), 0
        while at < len(words) and words[at] != "request":
            assert words[at] == "cycle"
            anchor, length, end, count = (int(w) for w in words[at + 1:at + 5])
            chain = [int(w) for w in words[at + 5:at + 5 + count]]
            at += 5 + count
            index.append(tokens[filed:anchor + 1])
            filed = anchor + 1
            got_length, got_end = index.match()
            assert got_length == min(length, 64), (requests, anchor)      # (the replay counts up to 4096 tokens)
            if length:
                assert got_end == end and index.proposals(31).tolist() == chain, (requests, anchor)
                matched += 1
            else:
                assert count == 0 and len(index.proposals(31)) == 0
            cycles += 1
    assert (requests, cycles, matched) == (2, 239, 147)     # what the reference's test counts in its fixture


def test_index_takes_long_and_degenerate_requests_in_bounded_time():
    from splash_b200 import lookup
    rng = np.random.default_rng(3)
    for tokens in (rng.integers(0, 150000, 100000), np.full(100000, 7), np.tile(np.arange(3), 33334), rng.integers(0, 4, 100000)):
        index = lookup.LookupIndex()
        t0 = time.time()
        index.append(tokens)
        assert time.time() - t0 < 20.0
        assert index.match() == brute_match(tokens.tolist(), len(tokens))
