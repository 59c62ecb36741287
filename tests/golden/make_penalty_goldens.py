"""Writes tests/golden/penalty_goldens.json: the reference's own host statement of the sampling penalties
(dev/tests/engine/PenaltyReference.hpp, through oracle/_ref/libsplash_ref.so, built by `make -C oracle ref`) on seeded
logits, counts and policies. Run where the reference tree is present; the tests then hold the oracle's restatement
against these vectors anywhere."""
import ctypes
import json
import os
import struct

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ref = ctypes.CDLL(os.path.join(HERE, "..", "..", "oracle", "_ref", "libsplash_ref.so"))
ref.ref_penalty.restype = ctypes.c_float
ref.ref_penalty.argtypes = [ctypes.c_float, ctypes.c_uint32, ctypes.c_int] + [ctypes.c_float] * 3

bits = lambda f: struct.unpack("<I", struct.pack("<f", f))[0]
rng = np.random.default_rng(20)
values = list(rng.standard_normal(40).astype(np.float32) * 8) + [0.0, -0.0, 3.0e38, -3.0e38, 1e-30, float("inf"), float("-inf"), float("nan")]
policies = [(1.0, 0.0, 0.0), (1.3, 0.0, 0.0), (0.8, 0.0, 0.0), (1.0, 0.7, 0.0), (1.0, 0.0, 0.25), (1.15, 0.4, 0.1), (1e-39, 0.0, 0.0), (2.0, 3e38, 3e38)]
cases = []
for rep, pres, freq in policies:
    for v in values:
        for count, prompt in ((0, 0), (0, 1), (1, 0), (3, 1), (1000, 0)):
            out = ref.ref_penalty(float(v), count, prompt, rep, pres, freq)
            cases.append([bits(float(v)), count, prompt, bits(np.float32(rep)), bits(np.float32(pres)), bits(np.float32(freq)), bits(out)])
json.dump({"source": "splash::test::referencePenalty (dev/tests/engine/PenaltyReference.hpp:28-40)",
           "columns": ["value", "count", "prompt", "repetition", "presence", "frequency", "result"], "float_bits": True, "cases": cases},
          open(os.path.join(HERE, "penalty_goldens.json"), "w"))
print(len(cases), "cases")
