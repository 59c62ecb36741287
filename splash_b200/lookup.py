"""ctypes harness of the prompt-lookup index (sb_lookup_* of include/splash_b200.h)."""
import ctypes

import numpy as np

from . import lib

_P, _U = ctypes.c_void_p, ctypes.c_uint32


def _bind():
    l = lib.load()
    if getattr(l, "_lookup_bound", False):
        return l
    l.sb_lookup_create.argtypes = [ctypes.POINTER(_P)]
    l.sb_lookup_destroy.argtypes = [_P]
    l.sb_lookup_append.argtypes = [_P, _P, ctypes.c_uint64]
    l.sb_lookup_match.argtypes = [_P, ctypes.POINTER(_U), ctypes.POINTER(_U)]
    l.sb_lookup_proposals.argtypes = [_P, _U, _P, ctypes.POINTER(_U)]
    l.sb_lookup_size.argtypes = [_P, ctypes.POINTER(ctypes.c_uint64)]
    l.sb_lookup_agreement.argtypes = [_U, _U, _P, ctypes.c_uint64, ctypes.POINTER(_U)]
    l._lookup_bound = True
    return l


class LookupIndex:
    def __init__(self):
        self.handle = None
        self.l = _bind()
        h = _P()
        lib.check(self.l.sb_lookup_create(ctypes.byref(h)))
        self.handle = h.value

    def __del__(self):
        if self.handle:
            self.l.sb_lookup_destroy(self.handle)
            self.handle = None

    def append(self, tokens):
        t = np.ascontiguousarray(tokens, np.uint32).reshape(-1)
        lib.check(self.l.sb_lookup_append(self.handle, t.ctypes.data_as(_P), t.size))

    def match(self):
        """(length, end): length 0 without a match; end the index of the earlier occurrence's last token."""
        n, e = _U(), _U()
        lib.check(self.l.sb_lookup_match(self.handle, ctypes.byref(n), ctypes.byref(e)))
        return int(n.value), int(e.value)

    def proposals(self, count):
        out, n = np.zeros(max(count, 1), np.uint32), _U()
        lib.check(self.l.sb_lookup_proposals(self.handle, count, out.ctypes.data_as(_P), ctypes.byref(n)))
        return out[:n.value].copy()

    def __len__(self):
        n = ctypes.c_uint64()
        lib.check(self.l.sb_lookup_size(self.handle, ctypes.byref(n)))
        return int(n.value)


def agreement(token, depth, candidates):
    c = np.ascontiguousarray(candidates, np.uint32).reshape(-1)
    out = _U()
    lib.check(_bind().sb_lookup_agreement(token, depth, c.ctypes.data_as(_P), c.size, ctypes.byref(out)))
    return int(out.value)
