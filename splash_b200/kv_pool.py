"""ctypes harness of the KV page pool (sb_kv_pool_* of include/splash_b200.h)."""
import ctypes

import numpy as np

from . import lib

_P, _U = ctypes.c_void_p, ctypes.c_uint32


def _bind():
    l = lib.load()
    if getattr(l, "_pool_bound", False):
        return l
    l.sb_kv_pool_create.argtypes = [_U, _U, _U, _U, ctypes.POINTER(_P)]
    l.sb_kv_pool_for_target.argtypes = [_P, ctypes.POINTER(_P)]
    l.sb_kv_pool_destroy.argtypes = [_P]
    l.sb_kv_pool_acquire.argtypes = [_P, _U, ctypes.c_uint64]
    l.sb_kv_pool_release.argtypes = [_P, _U]
    l.sb_kv_pool_table.argtypes = [_P, _U, ctypes.POINTER(ctypes.POINTER(_U)), ctypes.POINTER(_U)]
    l.sb_kv_pool_counts.argtypes = [_P, ctypes.POINTER(_U), ctypes.POINTER(_U)]
    l.sb_kv_pool_write_tables.argtypes = [_P, _P]
    l._pool_bound = True
    return l


class KvPool:
    def __init__(self, pages=0, lanes=0, lane_cap_pages=0, page_tokens=0, target=None):
        self.handle = None
        self.l = _bind()
        h = _P()
        if target is not None:
            lib.check(self.l.sb_kv_pool_for_target(target.handle, ctypes.byref(h)))
        else:
            lib.check(self.l.sb_kv_pool_create(pages, lanes, lane_cap_pages, page_tokens, ctypes.byref(h)))
        self.handle = h.value

    def __del__(self):
        if self.handle:
            self.l.sb_kv_pool_destroy(self.handle)
            self.handle = None

    def acquire(self, lane, tokens):
        """True when the lane now holds the pages of `tokens` tokens; False (nothing taken) when the pool cannot give them."""
        st = self.l.sb_kv_pool_acquire(self.handle, lane, tokens)
        if st == -4:
            return False
        lib.check(st)
        return True

    def release(self, lane):
        lib.check(self.l.sb_kv_pool_release(self.handle, lane))

    def table(self, lane):
        p, n = ctypes.POINTER(_U)(), _U()
        lib.check(self.l.sb_kv_pool_table(self.handle, lane, ctypes.byref(p), ctypes.byref(n)))
        return np.array([p[i] for i in range(n.value)], np.uint32)

    def counts(self):
        f, h = _U(), _U()
        lib.check(self.l.sb_kv_pool_counts(self.handle, ctypes.byref(f), ctypes.byref(h)))
        return int(f.value), int(h.value)

    def write_tables(self, target):
        lib.check(self.l.sb_kv_pool_write_tables(self.handle, target.handle))
