"""Tensor parallelism of the verify step on the host side: a rank's share of the model (sb_target_share), the cut of
whole tensors and state into a rank's share (what a loader does with a whole model's GGUF tensors), and the
rendezvous of the ranks' exchange windows. Tensor names are sb_target_tensor's."""
import ctypes

import numpy as np

from . import lib
from . import target as _target

_U = ctypes.c_uint32
HANDLE_BYTES = 64
_BLOCK = {lib.FMT_Q4K: (256, 144), lib.FMT_Q6K: (256, 210), lib.FMT_Q80: (32, 34)}


class SbTargetShare(ctypes.Structure):
    _fields_ = [(n, _U) for n in ("q_heads", "q_head0", "kv_heads", "kv_head0", "gdn_key_heads", "gdn_key_head0",
                                  "gdn_value_heads", "gdn_value_head0", "intermediate", "intermediate0", "vocab", "vocab0")]


def share(config, world, rank):
    """Rank `rank`'s share of the whole model's dimensions, as a dict."""
    l = lib.load()
    l.sb_target_share.argtypes = [ctypes.POINTER(_target.SbTargetConfig), ctypes.POINTER(SbTargetShare)]
    cfg = _target.SbTargetConfig(**{**config, "tp_world": world, "tp_rank": rank})
    out = SbTargetShare()
    lib.check(l.sb_target_share(ctypes.byref(cfg), ctypes.byref(out)))
    return {n: getattr(out, n) for n, _ in SbTargetShare._fields_}


def _rows(a, *ranges):
    return np.concatenate([a[b:e] for b, e in ranges], axis=0)


def _k_range(rows, fmt, first, count):
    """Input columns [first, first + count) of native quantized rows: whole blocks of each row."""
    elements, nbytes = _BLOCK[fmt]
    assert first % elements == 0 and count % elements == 0
    n = rows.shape[0]
    blocks = rows.reshape(n, -1, nbytes)
    return np.ascontiguousarray(blocks[:, first // elements:(first + count) // elements]).reshape(n, -1)


def shard(config, sh, layer, name, array):
    """The share `sh` of the whole tensor (or state array) `name` of `layer` (-1: the model's own tensors)."""
    c = config
    D = c["head_dim"]
    a = np.asarray(array)
    if layer < 0:
        if name == "output":
            return np.ascontiguousarray(a[sh["vocab0"]:sh["vocab0"] + sh["vocab"]])
        return a  # token_embd, output_norm: whole
    attention = (layer + 1) % c["attention_interval"] == 0
    if name in ("attn_norm", "ffn_norm", "q_norm", "k_norm", "ssm_norm"):
        return a
    if name in ("ffn_gate", "ffn_up"):
        return np.ascontiguousarray(a[sh["intermediate0"]:sh["intermediate0"] + sh["intermediate"]])
    if name == "ffn_down":
        return _k_range(a, c["fmt_down"], sh["intermediate0"], sh["intermediate"])
    if attention:
        hq = 2 * D if c["gated_attention"] else D
        Q, K = c["q_heads"], c["kv_heads"]
        q0, ql, k0, kl = sh["q_head0"], sh["q_heads"], sh["kv_head0"], sh["kv_heads"]
        if name == "in_proj":
            kb, vb = Q * hq, Q * hq + K * D
            return _rows(a, (q0 * hq, (q0 + ql) * hq), (kb + k0 * D, kb + (k0 + kl) * D), (vb + k0 * D, vb + (k0 + kl) * D))
        if name == "out_proj":
            return _k_range(a, c["fmt_proj"], q0 * D, ql * D)
        if name in ("kv_k", "kv_v", "kv_ks", "kv_vs"):
            return np.ascontiguousarray(a[:, k0:k0 + kl])
        raise KeyError(name)
    KH, VH = c["gdn_key_heads"], c["gdn_value_heads"]
    k0, kl, v0, vl = sh["gdn_key_head0"], sh["gdn_key_heads"], sh["gdn_value_head0"], sh["gdn_value_heads"]
    q_r, k_r = (k0 * 128, (k0 + kl) * 128), (KH * 128 + k0 * 128, KH * 128 + (k0 + kl) * 128)
    v_r = (2 * KH * 128 + v0 * 128, 2 * KH * 128 + (v0 + vl) * 128)
    z_r = ((2 * KH + VH) * 128 + v0 * 128, (2 * KH + VH) * 128 + (v0 + vl) * 128)
    channels = lambda x, axis: np.ascontiguousarray(np.concatenate([x.take(range(*r), axis=axis) for r in (q_r, k_r, v_r)], axis=axis))
    heads = lambda x, first, count, width: np.ascontiguousarray(x[:, first * width:(first + count) * width])
    if name == "in_proj":
        return _rows(a, q_r, k_r, v_r, z_r)
    if name == "out_proj":
        if not c["tiled_heads"]:
            return _k_range(a, c["fmt_proj"], v0 * 128, vl * 128)
        # tiled output columns: value head h = key head * per_key + j writes column block j * KH + key head, so a rank's
        # heads are per_key runs of its key heads' blocks; the same rule on its own heads gives its local column order
        per_key = VH // KH
        return np.concatenate([_k_range(a, c["fmt_proj"], (j * KH + k0) * 128, kl * 128) for j in range(per_key)], axis=1)
    if name == "ssm_ab":
        return _rows(a, (v0, v0 + vl), (VH + v0, VH + v0 + vl))
    if name == "ssm_conv":
        return channels(a, 0)
    if name in ("ssm_a", "ssm_dt_bias"):
        return np.ascontiguousarray(a[v0:v0 + vl])
    if name in ("state0", "state1"):
        return np.ascontiguousarray(a[v0:v0 + vl])
    if name in ("conv0", "conv1") or name.startswith("tape_inputs"):
        return channels(a, 1)
    if name.startswith("tape_k"):
        return heads(a, k0, kl, 128)
    if name.startswith("tape_v"):
        return heads(a, v0, vl, 128)
    if name.startswith("tape_beta") or name.startswith("tape_decay"):
        return heads(a, v0, vl, 1)
    raise KeyError(name)


def connect(t, all_gather):
    """Connects the tensor-parallel target `t` to its peers. `all_gather(bytes) -> [bytes of every rank, in rank order]`
    is the host transport (torch.distributed.all_gather_object, a pipe, a file: anything)."""
    l = t.l
    l.sb_target_tp_export.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    l.sb_target_tp_connect.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    mine = ctypes.create_string_buffer(HANDLE_BYTES)
    lib.check(l.sb_target_tp_export(t.handle, mine))
    handles = all_gather(mine.raw)
    assert all(len(h) == HANDLE_BYTES for h in handles)
    blob = b"".join(handles)
    lib.check(l.sb_target_tp_connect(t.handle, blob))


class Group:
    """One rank's end of the node's exchange at operator level (sb_tp_* of include/splash_b200.h)."""

    def __init__(self, world, rank, width, gather_width, all_gather):
        P, U = ctypes.c_void_p, _U
        l = self.l = lib.load()
        l.sb_tp_create.argtypes = [U, U, U, U, ctypes.POINTER(P)]
        l.sb_tp_destroy.argtypes = [P]
        l.sb_tp_export.argtypes = [P, P]
        l.sb_tp_connect.argtypes = [P, P]
        l.sb_tp_gather_matrix.argtypes = [P, ctypes.POINTER(P), ctypes.POINTER(ctypes.c_uint64)]
        l.sb_tp_prepare_sum.argtypes = [P, P, U, P, U, U, P, U, P, U, U, U, P, U, P, P, U]
        l.sb_tp_all_gather.argtypes = [P, P, U, U, U, U]
        l.sb_tp_advance.argtypes = [P, P, U]
        h = P()
        lib.check(l.sb_tp_create(world, rank, width, gather_width, ctypes.byref(h)))
        self.handle, self.world, self.rank = h.value, world, rank
        mine = ctypes.create_string_buffer(HANDLE_BYTES)
        lib.check(l.sb_tp_export(self.handle, mine))
        lib.check(l.sb_tp_connect(self.handle, b"".join(all_gather(mine.raw))))
        p, n = P(), ctypes.c_uint64()
        lib.check(l.sb_tp_gather_matrix(self.handle, ctypes.byref(p), ctypes.byref(n)))
        self.gather_ptr, self.gather_bytes = p.value, n.value

    def prepare_sum(self, stream, index, partials, slices, partial_stride, residual, sum_out, rows, k, norm_weight, fmt, prepared, flags=0):
        lib.check(self.l.sb_tp_prepare_sum(stream, self.handle, index, partials, slices, partial_stride, residual, k, sum_out, k, rows, k,
                                           norm_weight, fmt, prepared, None, flags))

    def all_gather(self, stream, index, rows, column0, columns):
        lib.check(self.l.sb_tp_all_gather(stream, self.handle, index, rows, column0, columns))

    def advance(self, stream, exchanges):
        lib.check(self.l.sb_tp_advance(stream, self.handle, exchanges))

    def close(self):
        if self.handle:
            self.l.sb_tp_destroy(self.handle)
            self.handle = None
