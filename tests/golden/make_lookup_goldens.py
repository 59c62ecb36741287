"""Writes tests/golden/lookup_goldens.json from the reference's own prompt-lookup index (runtime/model/LookupProposals.cpp
compiled into oracle/_ref/libsplash_ref_lookup.so by `make -C oracle ref`): for seeded token streams, the match (length, end)
after every token. Run where the reference tree is present; the vectors travel, the reference does not."""
import ctypes
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "..", "..", "oracle", "_ref", "libsplash_ref_lookup.so")


def streams():
    """Seeded streams whose suffixes repeat in different ways: small alphabets, copied spans, runs, periodic text."""
    out = []
    for seed, (alphabet, n) in enumerate([(2, 400), (3, 600), (5, 800), (50, 1200), (1000, 1500)]):
        rng = np.random.default_rng(seed)
        out.append((f"uniform over {alphabet} tokens", rng.integers(0, alphabet, n)))
    rng = np.random.default_rng(77)
    t = list(rng.integers(0, 5000, 300))
    for _ in range(40):                               # spans copied from earlier places, some with a changed token
        a = int(rng.integers(0, len(t) - 80))
        span = t[a:a + int(rng.integers(3, 80))]
        if rng.random() < 0.3:
            span[int(rng.integers(len(span)))] = int(rng.integers(5000))
        t += span + list(rng.integers(0, 5000, int(rng.integers(0, 6))))
    out.append(("copied spans", np.array(t)))
    out.append(("runs of one token", np.array([7] * 200 + [9] + [7] * 150 + [9, 9, 9] + [7] * 70)))
    out.append(("period 5 then period 7", np.array(list(range(5)) * 60 + list(range(10, 17)) * 40 + list(range(5)) * 30)))
    return [(name, np.ascontiguousarray(tokens, np.uint32)) for name, tokens in out]


def main():
    ref = ctypes.CDLL(REF)
    ref.ref_lookup_trace.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    cases = []
    for name, tokens in streams():
        lengths, ends = np.zeros(len(tokens), np.uint32), np.zeros(len(tokens), np.uint32)
        ref.ref_lookup_trace(tokens.ctypes.data, len(tokens), lengths.ctypes.data, ends.ctypes.data)
        cases.append(dict(name=name, tokens=tokens.tolist(), lengths=lengths.tolist(), ends=ends.tolist()))
    with open(os.path.join(HERE, "lookup_goldens.json"), "w") as f:
        json.dump(dict(source="runtime/model/LookupProposals.cpp through oracle/ref_lookup_shim.cpp", cases=cases), f, separators=(",", ":"))
    print(sum(len(c["tokens"]) for c in cases), "tokens in", len(cases), "streams;", sum(sum(1 for x in c["lengths"] if x) for c in cases), "matches")


if __name__ == "__main__":
    main()
