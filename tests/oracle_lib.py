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
