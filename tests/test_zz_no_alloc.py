"""sb_gdn_verify_static, the Gated-DeltaNet verify step for hosts that may not allocate device memory (a process
that gave its whole GPU to its own arena, a plugin inside one, code under a fixed memory budget): called through the
C ABI twice in a row and compared with sb_gdn_verify on the same inputs. Both run the same kernel, so the outputs
must be identical bit for bit, on the first call (which looks up the built-in scratch's address) and on the second
(which finds the previous call's contents in the scratch). The variants with the fused gate projection and with tree
rows go the same way, and one case runs in a fresh process that never calls sb_init, which is how such a host would
use the entry point."""
import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _inputs(rng, key_heads, value_heads, gate_k=0):
    D = 128
    KW, VW = key_heads * D, value_heads * D
    C = 2 * KW + VW
    bf = lambda shape, s: ol.f2bf((rng.standard_normal(shape) * s).astype(np.float32))
    x = dict(
        C=C, KW=KW, VW=VW, stride=C + VW,
        qkvz=bf((16, C + VW), 1.0), b=bf((16, value_heads), 1.0), a=bf((16, value_heads), 1.0), conv_w=bf((C, 4), 0.4),
        a_scale=(-np.exp(rng.uniform(-3, 0.5, value_heads))).astype(np.float32), dt_bias=bf((value_heads,), 0.5),
        norm_w=(1 + 0.1 * rng.standard_normal(D)).astype(np.float32), cs_in=bf((3, C), 1.0),
        state=(rng.standard_normal((value_heads, D, D)) * 0.05).astype(np.float32),
        pend=dict(inputs=bf((16, C), 1.0), k=bf((16, KW), 0.09), v=bf((16, VW), 0.5),
                  beta=ol.f2bf(rng.uniform(0.1, 0.9, (16, value_heads)).astype(np.float32)),
                  decay=rng.uniform(0.5, 1.0, (16, value_heads)).astype(np.float32)))
    if gate_k:
        x["gate_w"] = (rng.standard_normal((2 * value_heads, gate_k)) / np.sqrt(gate_k)).astype(np.float32)
        x["gate_x"] = bf((16, gate_k), 1.0)
    return x


def _sizes(x, value_heads):
    return dict(inputs=16 * x["C"] * 2, k=16 * x["KW"] * 2, v=16 * x["VW"] * 2, beta=16 * value_heads * 2, decay=16 * value_heads * 4)


def _tree_rows(parent):
    tree = np.zeros((len(parent), 2), np.uint32)
    for r in range(len(parent)):
        tree[r, 0] = (1 << r) | (tree[parent[r], 0] if r else 0)
        tree[r, 1] = parent[r] | ((bin(int(tree[r, 0])).count("1") - 1) << 16)
    return tree


def _run(lib, l, entry, x, key_heads, value_heads, rows, pending_rows, tree=None, pending_path=0):
    up = lib.DeviceBuffer.from_numpy
    d = {n: up(x[n]) for n in ("qkvz", "b", "a", "conv_w", "a_scale", "dt_bias", "norm_w", "cs_in", "state")}
    dp = {n: up(v) for n, v in x["pend"].items()}
    sizes = _sizes(x, value_heads)
    ds = {n: lib.DeviceBuffer(b) for n, b in sizes.items()}
    for b in ds.values():
        b.fill(0)
    dcs, dst, dh = lib.DeviceBuffer(x["cs_in"].nbytes), lib.DeviceBuffer(x["state"].nbytes), lib.DeviceBuffer(16 * x["VW"] * 2)
    dh.fill(0)
    tape = lambda t: lib.SbGdnTape(t["inputs"].ptr, t["k"].ptr, t["v"].ptr, t["beta"].ptr, t["decay"].ptr)
    args = lib.SbGdnArgs(d["qkvz"].ptr, d["b"].ptr, d["a"].ptr, d["conv_w"].ptr, d["a_scale"].ptr, d["dt_bias"].ptr, d["norm_w"].ptr,
                         d["cs_in"].ptr, dcs.ptr, d["state"].ptr, dst.ptr, tape(dp), tape(ds), dh.ptr, None,
                         rows, pending_rows, key_heads, value_heads, x["stride"], value_heads, x["VW"], 0)
    keep = []
    if "gate_w" in x:  # the kernel projects b and a itself
        gw, gx = up(x["gate_w"]), up(x["gate_x"])
        keep += [gw, gx]
        args.b = args.a = None
        args.gate_weight, args.gate_input, args.gate_k, args.gate_input_stride = gw.ptr, gx.ptr, x["gate_w"].shape[1], x["gate_w"].shape[1]
    if tree is not None:
        td = up(tree)
        keep.append(td)
        args.tree = td.ptr
    args.pending_path = pending_path
    lib.check(entry(None, ctypes.byref(args)))
    lib.stream_sync()
    assert lib.device_status() == 0
    out = dict(cs=dcs.to_numpy(np.uint16, x["cs_in"].shape), state=dst.to_numpy(np.float32, x["state"].shape),
               hidden=dh.to_numpy(np.uint16, (16, x["VW"])))
    out.update({n: ds[n].to_numpy(np.uint8, (sizes[n],)) for n in sizes})
    return out


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    from splash_b200 import lib
    lib.init(0)
    l = lib.ops()
    for call, (seed, kh, vh, rows, pending) in enumerate([(21, 16, 48, 16, 7), (22, 2, 6, 9, 16)]):
        x = _inputs(np.random.default_rng(seed), kh, vh)
        want = _run(lib, l, l.sb_gdn_verify, x, kh, vh, rows, pending)
        got = _run(lib, l, l.sb_gdn_verify_static, x, kh, vh, rows, pending)
        for name in want:
            assert np.array_equal(got[name], want[name]), (call, name)
        assert np.abs(ol.bf2f(got["hidden"][:rows])).max() > 0  # the step did produce rows


def test_static_scratch_entry_point_with_fused_gates_and_with_tree_rows():
    """The kernel's own alpha / beta projection and the tree kernel run from the built-in scratch too."""
    from splash_b200 import lib
    lib.init(0)
    l = lib.ops()
    x = _inputs(np.random.default_rng(23), 4, 12, gate_k=1024)
    want = _run(lib, l, l.sb_gdn_verify, x, 4, 12, 16, 5)
    got = _run(lib, l, l.sb_gdn_verify_static, x, 4, 12, 16, 5)
    for name in want:
        assert np.array_equal(got[name], want[name]), ("fused gates", name)
    parent = [0, 0, 1, 2, 0, 4, 5, 6, 6, 8, 9]
    x = _inputs(np.random.default_rng(24), 2, 6)
    want = _run(lib, l, l.sb_gdn_verify, x, 2, 6, len(parent), 0, tree=_tree_rows(parent), pending_path=0b100101)
    got = _run(lib, l, l.sb_gdn_verify_static, x, 2, 6, len(parent), 0, tree=_tree_rows(parent), pending_path=0b100101)
    for name in want:
        assert np.array_equal(got[name], want[name]), ("tree", name)
    assert np.abs(ol.bf2f(got["hidden"][:len(parent)])).max() > 0


def test_static_scratch_entry_point_rejects_shapes_beyond_its_array():
    from splash_b200 import lib
    lib.init(0)
    l = lib.ops()
    args = lib.SbGdnArgs(*([1 << 20] * 11), lib.SbGdnTape(*([1 << 20] * 5)), lib.SbGdnTape(*([1 << 20] * 5)), 1 << 20, None,
                         16, 0, 16, 80, 80 * 128 * 4, 80, 80 * 128, 0)
    assert l.sb_gdn_verify_static(None, ctypes.byref(args)) == -1
    assert b"64" in l.sb_last_error()


# The child below is the host this entry point is for: it owns its device memory (taken from the CUDA runtime
# directly, as an arena would have been) and never calls sb_init, sb_alloc or any other allocating routine of the
# library. It writes what the call produced to a file for the parent to compare.
_CHILD = r"""
import ctypes, sys
import numpy as np
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
import test_zz_no_alloc as t
from splash_b200 import lib
rt = None
for name in ("libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so", "libcudart.so"):
    try:
        rt = ctypes.CDLL(name)
        break
    except OSError:
        pass
assert rt is not None, "no CUDA runtime library to allocate with"
rt.cudaMalloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t]
rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
rt.cudaMemset.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t]
assert rt.cudaSetDevice(0) == 0

def alloc(nbytes):
    p = ctypes.c_void_p()
    assert rt.cudaMalloc(ctypes.byref(p), nbytes + 256) == 0
    assert rt.cudaMemset(p, 0, nbytes + 256) == 0
    return p.value

def up(a):
    a = np.ascontiguousarray(a)
    p = alloc(a.nbytes)
    assert rt.cudaMemcpy(p, a.ctypes.data_as(ctypes.c_void_p), a.nbytes, 1) == 0
    return p

def down(p, dtype, shape):
    out = np.empty(shape, dtype)
    assert rt.cudaMemcpy(out.ctypes.data_as(ctypes.c_void_p), p, out.nbytes, 2) == 0
    return out

kh, vh, rows, pending = 2, 6, 16, 4
x = t._inputs(np.random.default_rng(25), kh, vh)
l = lib.ops()
d = {n: up(x[n]) for n in ("qkvz", "b", "a", "conv_w", "a_scale", "dt_bias", "norm_w", "cs_in", "state")}
dp = {n: up(v) for n, v in x["pend"].items()}
sizes = t._sizes(x, vh)
ds = {n: alloc(b) for n, b in sizes.items()}
dcs, dst, dh = alloc(x["cs_in"].nbytes), alloc(x["state"].nbytes), alloc(16 * x["VW"] * 2)
tape = lambda q: lib.SbGdnTape(q["inputs"], q["k"], q["v"], q["beta"], q["decay"])
args = lib.SbGdnArgs(d["qkvz"], d["b"], d["a"], d["conv_w"], d["a_scale"], d["dt_bias"], d["norm_w"], d["cs_in"], dcs, d["state"], dst,
                     tape(dp), tape(ds), dh, None, rows, pending, kh, vh, x["stride"], vh, x["VW"], 0)
outs = {}
for call in range(2):   # twice: the second call finds the first one's contents in the scratch
    st = l.sb_gdn_verify_static(None, ctypes.byref(args))
    assert st == 0, l.sb_last_error()
    assert rt.cudaDeviceSynchronize() == 0
    outs[f"cs{call}"] = down(dcs, np.uint16, x["cs_in"].shape)
    outs[f"state{call}"] = down(dst, np.float32, x["state"].shape)
    outs[f"hidden{call}"] = down(dh, np.uint16, (16, x["VW"]))
    outs[f"k{call}"] = down(ds["k"], np.uint8, (sizes["k"],))
np.savez(sys.argv[3], **outs)
"""


def test_static_scratch_entry_point_in_a_process_that_never_calls_sb_init():
    from splash_b200 import lib
    lib.init(0)
    l = lib.ops()
    kh, vh, rows, pending = 2, 6, 16, 4
    x = _inputs(np.random.default_rng(25), kh, vh)
    want = _run(lib, l, l.sb_gdn_verify, x, kh, vh, rows, pending)
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "child.npz")
        r = subprocess.run([sys.executable, "-c", _CHILD, HERE, os.path.dirname(HERE), out], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        got = np.load(out)
        for call in range(2):
            assert np.array_equal(got[f"cs{call}"], want["cs"]), call
            assert np.array_equal(got[f"state{call}"], want["state"]), call
            assert np.array_equal(got[f"hidden{call}"], want["hidden"]), call
            assert np.array_equal(got[f"k{call}"], want["k"]), call
