"""ctypes harness of the GGUF reader and loader (sb_gguf_* and sb_target_load_gguf of include/splash_b200.h)."""
import ctypes

import numpy as np

from . import lib
from .target import SbTargetConfig, Target

_P, _U = ctypes.c_void_p, ctypes.c_uint32


class SbGgufTensor(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("type", _U), ("n_dims", _U), ("dims", ctypes.c_uint64 * 4), ("data", _P),
                ("bytes", ctypes.c_uint64)]


def _bind():
    l = lib.load()
    if getattr(l, "_gguf_bound", False):
        return l
    l.sb_gguf_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(_P)]
    l.sb_gguf_close.argtypes = [_P]
    l.sb_gguf_tensor_count.argtypes = [_P, ctypes.POINTER(ctypes.c_uint64)]
    l.sb_gguf_tensor.argtypes = [_P, ctypes.c_uint64, ctypes.POINTER(SbGgufTensor)]
    l.sb_gguf_find.argtypes = [_P, ctypes.c_char_p, ctypes.POINTER(SbGgufTensor)]
    l.sb_gguf_meta_u64.argtypes = [_P, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint64)]
    l.sb_gguf_meta_f64.argtypes = [_P, ctypes.c_char_p, ctypes.POINTER(ctypes.c_double)]
    l.sb_gguf_meta_str.argtypes = [_P, ctypes.c_char_p, ctypes.POINTER(ctypes.c_char_p)]
    l.sb_gguf_target_config.argtypes = [_P, ctypes.POINTER(SbTargetConfig)]
    l.sb_target_load_gguf.argtypes = [_P, _P]
    l.sb_target_config.argtypes = [_P, ctypes.POINTER(SbTargetConfig)]
    l._gguf_bound = True
    return l


class GgufFile:
    def __init__(self, path):
        """path: one file, or the parts of a split GGUF in split order (a list)."""
        self.handle = None
        self.l = _bind()
        h = _P()
        if isinstance(path, (list, tuple)):
            paths = (ctypes.c_char_p * len(path))(*[str(p).encode() for p in path])
            self.l.sb_gguf_open_parts.argtypes = [ctypes.POINTER(ctypes.c_char_p), _U, ctypes.POINTER(_P)]
            lib.check(self.l.sb_gguf_open_parts(paths, len(path), ctypes.byref(h)))
        else:
            lib.check(self.l.sb_gguf_open(str(path).encode(), ctypes.byref(h)))
        self.handle = h.value

    def array(self, key):
        """A numeric metadata array as float64 values; None without such a key."""
        values, n = ctypes.POINTER(ctypes.c_double)(), ctypes.c_uint64()
        self.l.sb_gguf_meta_array.argtypes = [_P, ctypes.c_char_p, ctypes.POINTER(ctypes.POINTER(ctypes.c_double)), ctypes.POINTER(ctypes.c_uint64)]
        if self.l.sb_gguf_meta_array(self.handle, key.encode(), ctypes.byref(values), ctypes.byref(n)) != 0:
            return None
        return np.array([values[i] for i in range(n.value)], np.float64)

    def close(self):
        if self.handle:
            self.l.sb_gguf_close(self.handle)
            self.handle = None

    def __del__(self):
        self.close()

    @staticmethod
    def _view(t):
        dims = [int(t.dims[d]) for d in range(t.n_dims)]
        data = np.ctypeslib.as_array(ctypes.cast(t.data, ctypes.POINTER(ctypes.c_uint8)), (int(t.bytes),)) if t.bytes else np.zeros(0, np.uint8)
        return dict(name=t.name.decode(errors="replace"), type=int(t.type), dims=dims, data=data)

    def tensors(self):
        n = ctypes.c_uint64()
        lib.check(self.l.sb_gguf_tensor_count(self.handle, ctypes.byref(n)))
        out = []
        for i in range(n.value):
            t = SbGgufTensor()
            lib.check(self.l.sb_gguf_tensor(self.handle, i, ctypes.byref(t)))
            out.append(self._view(t))
        return out

    def find(self, name):
        t = SbGgufTensor()
        if self.l.sb_gguf_find(self.handle, name.encode(), ctypes.byref(t)) != 0:
            return None
        return self._view(t)

    def meta(self, key):
        """The key's value as int, float or str; None without such a key."""
        u, f, s = ctypes.c_uint64(), ctypes.c_double(), ctypes.c_char_p()
        if self.l.sb_gguf_meta_u64(self.handle, key.encode(), ctypes.byref(u)) == 0:
            return int(u.value)
        if self.l.sb_gguf_meta_f64(self.handle, key.encode(), ctypes.byref(f)) == 0:
            return float(f.value)
        if self.l.sb_gguf_meta_str(self.handle, key.encode(), ctypes.byref(s)) == 0:
            return s.value.decode()
        return None

    def target_config(self, **runtime):
        """The model's configuration from the file, the fields the file does not hold (page_tokens, kv_scale_f16, max_context,
        lanes, ...) from `runtime`; as a dict for Target(**config)."""
        cfg = SbTargetConfig(**runtime)
        lib.check(self.l.sb_gguf_target_config(self.handle, ctypes.byref(cfg)))
        return {name: getattr(cfg, name) for name, _ in SbTargetConfig._fields_}


def load_target(path, **runtime):
    """A target created for the GGUF (its configuration, every projection tensor in the file's format) and filled with its
    tensors; `runtime` gives the fields a file does not hold (page_tokens, kv_scale_f16, max_context, lanes). Returns
    (target, file)."""
    f = GgufFile(path)
    cfg = SbTargetConfig(**runtime)
    h = _P()
    f.l.sb_target_create_from_gguf.argtypes = [_P, ctypes.POINTER(SbTargetConfig), ctypes.POINTER(_P)]
    lib.check(f.l.sb_target_create_from_gguf(f.handle, ctypes.byref(cfg), ctypes.byref(h)))
    return Target.from_handle(h.value), f


def load_into(target, f):
    """Fills an existing target from an open GgufFile (sb_target_load_gguf)."""
    lib.check(f.l.sb_target_load_gguf(target.handle, f.handle))
