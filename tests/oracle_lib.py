"""ctypes loader of the CPU oracle (oracle/liboracle.so) and, when it was built, of the reference
shim (oracle/_ref/libsplash_ref.so). Test infrastructure only."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

FMT_Q4K, FMT_Q6K, FMT_Q80, FMT_NVFP4, FMT_BF16, FMT_F16, FMT_F32 = 0, 4, 6, 37, 41, 42, 64


def _build():
    subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)


def load():
    path = os.path.join(ORACLE_DIR, "liboracle.so")
    srcs = [os.path.join(ORACLE_DIR, f) for f in os.listdir(ORACLE_DIR) if f.startswith("so_")]
    if not os.path.exists(path) or any(os.path.getmtime(s) > os.path.getmtime(path) for s in srcs):
        _build()
    lib = ctypes.CDLL(path)
    lib.so_row_bytes.restype = ctypes.c_uint64
    return lib


def load_ref():
    """The reference's own CPU code behind a C shim; None when it was not built here."""
    path = os.path.join(ORACLE_DIR, "_ref", "libsplash_ref.so")
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    lib.ref_kv_scale.restype = ctypes.c_float
    lib.ref_kv_scale.argtypes = [ctypes.c_float]
    lib.ref_kv_code.argtypes = [ctypes.c_float, ctypes.c_float]
    return lib


def ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def row_bytes(lib, fmt, K):
    return int(lib.so_row_bytes(fmt, K))


def dequant(lib, fmt, native, rows, K):
    out = np.empty((rows, K), np.float32)
    assert lib.so_dequant(fmt, ptr(native), rows, K, ptr(out)) == 0
    return out


# bf16 helpers on numpy arrays (round to nearest even).
def f2bf(x):
    v = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return (((v + 0x7FFF + ((v >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf2f(u):
    return (np.ascontiguousarray(u, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- structures of oracle/so_ops.cpp and oracle/so_gdn.cpp ----
_P, _U = ctypes.c_void_p, ctypes.c_uint32


class SoKvLayer(ctypes.Structure):
    _fields_ = [("k", _P), ("v", _P), ("k_scale", _P), ("v_scale", _P),
                ("kv_heads", _U), ("head_dim", _U), ("page_tokens", _U), ("scale_f16", _U)]


class SoGdnTape(ctypes.Structure):
    _fields_ = [("inputs", _P), ("k", _P), ("v", _P), ("beta", _P), ("decay", _P)]


class SoGdnArgs(ctypes.Structure):
    _fields_ = [("qkvz", _P), ("b", _P), ("a", _P), ("conv_w", _P), ("a_scale", _P), ("dt_bias", _P), ("norm_w", _P),
                ("conv_state_in", _P), ("conv_state_out", _P), ("state_in", _P), ("state_out", _P),
                ("pending", SoGdnTape), ("step", SoGdnTape), ("hidden", _P),
                ("rows", _U), ("pending_rows", _U), ("key_heads", _U), ("value_heads", _U), ("qkvz_stride", _U),
                ("ab_stride", _U), ("hidden_stride", _U), ("tiled", _U), ("tree", _P), ("pending_path", _U)]


class HostKv:
    """A host-side INT8 cache of one layer in the product's layout, with its oracle descriptor."""

    def __init__(self, pages, kv_heads, head_dim, page_tokens, scale_f16):
        self.k = np.zeros((pages, kv_heads, page_tokens, head_dim), np.int8)
        self.v = np.zeros_like(self.k)
        st = np.float16 if scale_f16 else np.float32
        self.ks = np.zeros((pages, kv_heads, page_tokens), st)
        self.vs = np.zeros_like(self.ks)
        self.geom = (kv_heads, head_dim, page_tokens, int(bool(scale_f16)))

    def desc(self):
        return SoKvLayer(ptr(self.k), ptr(self.v), ptr(self.ks), ptr(self.vs), *self.geom)

    def fill_random(self, rng, tokens_per_page_filled=None):
        self.k[...] = rng.integers(-127, 128, self.k.shape, dtype=np.int8)
        self.v[...] = rng.integers(-127, 128, self.v.shape, dtype=np.int8)
        self.ks[...] = rng.uniform(0.005, 0.03, self.ks.shape).astype(self.ks.dtype)
        self.vs[...] = rng.uniform(0.005, 0.03, self.vs.shape).astype(self.vs.dtype)


def bind_ops(lib):
    F = ctypes.c_float
    lib.so_kv_scale.restype = F
    lib.so_kv_scale.argtypes = [F]
    lib.so_kv_code.argtypes = [F, F]
    lib.so_rope_tables.argtypes = [_P, _U, _P, _U, F, _P, _P]
    lib.so_kv_path_commit.argtypes = [_P, _P, _U, _U]
    lib.so_moe_route.argtypes = [_P, _U, _U, _U, _U, _U, _P, _U, _P, _P, _P]
    lib.so_moe_experts.argtypes = [_P, _P, _P, _P, _P, _P, _P, _U, _U, _U, _U, _U, _P, _P]
    lib.so_penalize_logit.restype = F
    lib.so_penalize_logit.argtypes = [F, _U, F, F, F, F]
    lib.so_sample_penalize.argtypes = [_P, _U, _U, _U, _P, _P, _P, F, F, F]
    lib.so_sample_verify.argtypes = [_P, _U, _U, _U, _P, F, _P, _P, _P]
    lib.so_sample_verify_filtered.argtypes = [_P, _U, _U, _U, _P, F, F, _U, F, _P, _P, _P, _P]
    return lib
