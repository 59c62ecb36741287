"""ctypes harness of the target model's verify step (sb_target_* of include/splash_b200.h)."""
import ctypes

import numpy as np

from . import lib

_P, _U, _F = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_float
ADVANCE, GRAPH, TREE, KEEP_PENDING, DRAWS, PROMPT = 1, 2, 4, 8, 16, 32


class SbTargetConfig(ctypes.Structure):
    _fields_ = [("layers", _U), ("hidden", _U), ("vocab", _U), ("intermediate", _U),
                ("q_heads", _U), ("kv_heads", _U), ("head_dim", _U), ("rotary_pairs", _U), ("rope_theta", _F),
                ("gdn_key_heads", _U), ("gdn_value_heads", _U), ("attention_interval", _U),
                ("page_tokens", _U), ("kv_scale_f16", _U), ("max_context", _U),
                ("fmt_proj", _U), ("fmt_down", _U), ("fmt_head", _U), ("fmt_embed", _U),
                ("gated_attention", _U), ("tiled_heads", _U), ("tp_world", _U), ("tp_rank", _U),
                ("moe_experts", _U), ("moe_top_k", _U), ("moe_intermediate", _U), ("lanes", _U),
                ("ep_world", _U), ("ep_rank", _U)]


# The benchmark configurations' shapes (weights are synthetic; see quant fixtures and sb_target_randomize).
TINY = dict(layers=4, hidden=1024, vocab=32000, intermediate=2816, q_heads=8, kv_heads=2, head_dim=128, rotary_pairs=16,
            rope_theta=1e6, gdn_key_heads=8, gdn_value_heads=8, attention_interval=4, page_tokens=256, kv_scale_f16=1,
            max_context=4096, fmt_proj=lib.FMT_Q4K, fmt_down=lib.FMT_Q4K, fmt_head=lib.FMT_Q6K, fmt_embed=lib.FMT_Q6K,
            gated_attention=1, tiled_heads=0)
QWEN27B = dict(layers=64, hidden=5120, vocab=151936, intermediate=17408, q_heads=24, kv_heads=4, head_dim=256,
               rotary_pairs=32, rope_theta=1e7, gdn_key_heads=16, gdn_value_heads=48, attention_interval=4, page_tokens=256,
               kv_scale_f16=1, max_context=32768 + 1024, fmt_proj=lib.FMT_Q4K, fmt_down=lib.FMT_Q6K, fmt_head=lib.FMT_Q6K,
               fmt_embed=lib.FMT_Q6K, gated_attention=1, tiled_heads=1)


# The MoE configuration's shape (35B-A3B: 40 layers at 3:1, hidden 2048, 16 query / 2 KV heads of 256, 256 experts of
# width 512 plus a shared one, top 8); the GDN head counts are this harness's choice (the configuration names none).
QWEN35B_A3B = dict(layers=40, hidden=2048, vocab=151936, intermediate=512, q_heads=16, kv_heads=2, head_dim=256, rotary_pairs=32,
                   rope_theta=1e7, gdn_key_heads=16, gdn_value_heads=32, attention_interval=4, page_tokens=256, kv_scale_f16=1,
                   max_context=8192 + 1024, fmt_proj=lib.FMT_Q4K, fmt_down=lib.FMT_Q4K, fmt_head=lib.FMT_Q6K, fmt_embed=lib.FMT_Q6K,
                   gated_attention=1, tiled_heads=1, moe_experts=256, moe_top_k=8, moe_intermediate=512)


def _bind():
    l = lib.ops()
    if getattr(l, "_target_bound", False):
        return l
    l.sb_target_create.argtypes = [ctypes.POINTER(SbTargetConfig), ctypes.POINTER(_P)]
    l.sb_target_destroy.argtypes = [_P]
    l.sb_target_tensor.argtypes = [_P, ctypes.c_int, ctypes.c_char_p, ctypes.POINTER(_P), ctypes.POINTER(ctypes.c_uint64)]
    l.sb_target_randomize.argtypes = [_P, ctypes.c_uint64, _U]
    l.sb_target_reset.argtypes = [_P, _U]
    l.sb_target_set_penalties.argtypes = [_P, _F, _F, _F]
    l.sb_target_set_router_scores.argtypes = [_P, ctypes.c_int]
    l.sb_target_step.argtypes = [_P, _P, _U, _F, _U]
    l.sb_target_verify.argtypes = [_P, _P, _P, _P, _U, _F, _U, _P, _P]
    l.sb_target_verify_tree.argtypes = [_P, _P, _P, _P, _P, _U, _F, _U, _P, _P]
    l.sb_target_reset_lanes.argtypes = [_P, _P]
    l.sb_target_verify_lanes.argtypes = [_P, _P, _P, _P, _U, _F, _U, _P, _P]
    l.sb_target_stats.argtypes = [_P, _U, ctypes.POINTER(_U), ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64),
                                  ctypes.POINTER(ctypes.c_uint64)]
    l._target_bound = True
    return l


class Target:
    def __init__(self, **config):
        self.l = _bind()
        self.config = dict(config)
        self.cfg = SbTargetConfig(**config)
        h = _P()
        lib.check(self.l.sb_target_create(ctypes.byref(self.cfg), ctypes.byref(h)))
        self.handle = h.value

    @classmethod
    def from_handle(cls, handle):
        """Wraps a target created by the library (sb_target_create_from_gguf)."""
        self = cls.__new__(cls)
        self.l = _bind()
        self.handle = handle
        self.cfg = SbTargetConfig()
        self.l.sb_target_config.argtypes = [_P, ctypes.POINTER(SbTargetConfig)]
        lib.check(self.l.sb_target_config(handle, ctypes.byref(self.cfg)))
        self.config = {name: getattr(self.cfg, name) for name, _ in SbTargetConfig._fields_}
        return self

    def tensor_format(self, layer, name):
        f = _U()
        self.l.sb_target_tensor_format.argtypes = [_P, ctypes.c_int, ctypes.c_char_p, ctypes.POINTER(_U)]
        lib.check(self.l.sb_target_tensor_format(self.handle, layer, name.encode(), ctypes.byref(f)))
        return int(f.value)

    def close(self):
        if self.handle:
            self.l.sb_target_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor(self, layer, name):
        p, n = _P(), ctypes.c_uint64()
        lib.check(self.l.sb_target_tensor(self.handle, layer, name.encode(), ctypes.byref(p), ctypes.byref(n)))
        return p.value, n.value

    def upload(self, layer, name, array, lane=0):
        """`lane`: the lane's share of a per-lane tensor (the tensor is an array over the lanes)."""
        a = np.ascontiguousarray(array)
        p, n = self.tensor(layer, name)
        share = n // max(1, self.cfg.lanes) if lane else n
        assert a.nbytes <= share, (name, a.nbytes, share)
        lib.check(self.l.sb_upload(p + lane * share, a.ctypes.data_as(_P), a.nbytes, None))
        lib.stream_sync()

    def download(self, layer, name, dtype, shape, lane=0):
        out = np.empty(shape, dtype)
        p, n = self.tensor(layer, name)
        share = n // max(1, self.cfg.lanes) if lane else n
        assert out.nbytes <= share, (name, out.nbytes, share)
        lib.check(self.l.sb_download(out.ctypes.data_as(_P), p + lane * share, out.nbytes, None))
        lib.stream_sync()
        return out

    def randomize(self, seed, committed):
        lib.check(self.l.sb_target_randomize(self.handle, seed, committed))

    def set_policy(self, min_p=0.0, top_k=0, top_p=1.0):
        self.l.sb_target_set_policy.argtypes = [_P, _F, _U, _F]
        lib.check(self.l.sb_target_set_policy(self.handle, min_p, top_k, top_p))

    def set_lane_policies(self, policies=None):
        """policies: a (temperature, min_p, top_k, top_p) per lane, or None to go back to the step's temperature."""
        self.l.sb_target_set_lane_policies.argtypes = [_P, _P]
        if policies is None:
            return lib.check(self.l.sb_target_set_lane_policies(self.handle, None))
        arr = (lib.SbLanePolicy * len(policies))(*[lib.SbLanePolicy(*p) for p in policies])
        assert len(policies) == max(1, self.cfg.lanes)
        lib.check(self.l.sb_target_set_lane_policies(self.handle, ctypes.cast(arr, _P)))

    def set_stop_tokens(self, tokens=()):
        e = np.ascontiguousarray(tokens, np.uint32)
        self.l.sb_target_set_stop_tokens.argtypes = [_P, _P, _U]
        lib.check(self.l.sb_target_set_stop_tokens(self.handle, e.ctypes.data_as(_P) if e.size else None, e.size))

    def set_admission(self, constrained=False, excluded=()):
        """The rows' admission: with `constrained` the step reads every row's constraint mask from the `constraint_masks` tensor;
        `excluded` are token ids no row selects."""
        e = np.ascontiguousarray(excluded, np.uint32)
        self.l.sb_target_set_admission.argtypes = [_P, ctypes.c_int, _P, _U]
        lib.check(self.l.sb_target_set_admission(self.handle, int(bool(constrained)), e.ctypes.data_as(_P) if e.size else None, e.size))

    def set_penalties(self, repetition=1.0, presence=0.0, frequency=0.0):
        lib.check(self.l.sb_target_set_penalties(self.handle, repetition, presence, frequency))

    def set_router_scores(self, scores):
        """Synthetic routing for measurements: every MoE block routes by `scores` (fp32 [rows of all lanes, experts]); None: by its own router."""
        if scores is None:
            lib.check(self.l.sb_target_set_router_scores(self.handle, 0))
            return
        self.upload(-1, "moe_scores", np.ascontiguousarray(scores, np.float32))
        lib.check(self.l.sb_target_set_router_scores(self.handle, 1))

    def reset(self, committed):
        lib.check(self.l.sb_target_reset(self.handle, committed))

    def reset_lanes(self, committed):
        c = np.ascontiguousarray(committed, np.uint32)
        assert len(c) == max(1, self.cfg.lanes)
        lib.check(self.l.sb_target_reset_lanes(self.handle, c.ctypes.data_as(_P)))

    def verify_lanes(self, tokens, uniforms=None, temperature=0.0, flags=0, stream=None, trees=None):
        """One step of every lane from host buffers: tokens [lanes, rows]; uniforms [lanes, 80] for a sampled policy; trees
        (uint32 [lanes, rows, 2]: ancestors, parent | depth << 16) makes every lane's block a tree.
        Returns per lane (retained tokens, retained, accepted, retained_rows mask)."""
        tokens = np.ascontiguousarray(tokens, np.uint32)
        lanes, rows = tokens.shape
        assert lanes == max(1, self.cfg.lanes)
        slots = np.zeros((lanes, 16), np.uint32)
        slots[:, :rows] = tokens
        u = None if uniforms is None else np.ascontiguousarray(uniforms, np.float32)
        assert u is None or u.shape == (lanes, 80)
        out_t, out_r = np.zeros((lanes, 16), np.uint32), np.zeros((lanes, 4), np.uint32)
        if trees is not None:
            tr = np.zeros((lanes, 16, 2), np.uint32)
            tr[:, :rows] = np.asarray(trees, np.uint32)
            self.upload(-1, "tree", tr)
            flags |= TREE
        lib.check(self.l.sb_target_verify_lanes(self.handle, stream, slots.ctypes.data_as(_P), None if u is None else u.ctypes.data_as(_P),
                                                rows, temperature, flags, out_t.ctypes.data_as(_P), out_r.ctypes.data_as(_P)))
        return [(out_t[l, :out_r[l, 0]].copy(), int(out_r[l, 0]), int(out_r[l, 1]), int(out_r[l, 2])) for l in range(lanes)]

    def verify_lanes_ragged(self, blocks, uniforms=None, temperature=0.0, flags=0, stream=None):
        """One step of lanes whose blocks differ in length: blocks is a list of token arrays (0..16 tokens each, an empty one
        for a lane that sits the step out). Returns per lane (retained tokens, retained, accepted, retained_rows mask)."""
        lanes = max(1, self.cfg.lanes)
        assert len(blocks) == lanes
        slots, rows = np.zeros((lanes, 16), np.uint32), np.zeros(lanes, np.uint32)
        for i, b in enumerate(blocks):
            b = np.asarray(b, np.uint32)
            slots[i, :len(b)], rows[i] = b, len(b)
        u = None if uniforms is None else np.ascontiguousarray(uniforms, np.float32)
        out_t, out_r = np.zeros((lanes, 16), np.uint32), np.zeros((lanes, 4), np.uint32)
        self.l.sb_target_verify_lanes_ragged.argtypes = [_P, _P, _P, _P, _P, _F, _U, _P, _P]
        lib.check(self.l.sb_target_verify_lanes_ragged(self.handle, stream, slots.ctypes.data_as(_P), None if u is None else u.ctypes.data_as(_P),
                                                       rows.ctypes.data_as(_P), temperature, flags, out_t.ctypes.data_as(_P), out_r.ctypes.data_as(_P)))
        return [(out_t[l, :out_r[l, 0]].copy(), int(out_r[l, 0]), int(out_r[l, 1]), int(out_r[l, 2])) for l in range(lanes)]

    def step(self, rows=16, temperature=0.0, flags=GRAPH, stream=None):
        lib.check(self.l.sb_target_step(self.handle, stream, rows, temperature, flags))

    def verify(self, tokens, uniforms=None, temperature=0.0, flags=0, stream=None, tree=None):
        """One step from host buffers; `tree` (uint32 [rows, 2]: ancestors, parent | depth << 16) makes the block a tree.
        Returns (retained tokens, retained, accepted, retained_rows mask)."""
        tokens = np.ascontiguousarray(tokens, np.uint32)
        rows = len(tokens)
        out_t, out_r = np.zeros(16, np.uint32), np.zeros(4, np.uint32)
        u = None if uniforms is None else np.ascontiguousarray(uniforms, np.float32)
        if tree is not None:
            tr = np.ascontiguousarray(tree, np.uint32)
            assert tr.shape == (rows, 2)
            lib.check(self.l.sb_target_verify_tree(self.handle, stream, tokens.ctypes.data_as(_P), tr.ctypes.data_as(_P),
                                                   None if u is None else u.ctypes.data_as(_P), rows, temperature, flags,
                                                   out_t.ctypes.data_as(_P), out_r.ctypes.data_as(_P)))
            return out_t[:out_r[0]].copy(), int(out_r[0]), int(out_r[1]), int(out_r[2])
        lib.check(self.l.sb_target_verify(self.handle, stream, tokens.ctypes.data_as(_P), None if u is None else u.ctypes.data_as(_P),
                                          rows, temperature, flags, out_t.ctypes.data_as(_P), out_r.ctypes.data_as(_P)))
        return out_t[:out_r[0]].copy(), int(out_r[0]), int(out_r[1]), int(out_r[2])

    def stats(self, rows=16):
        n, w, k, s = _U(), ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        lib.check(self.l.sb_target_stats(self.handle, rows, ctypes.byref(n), ctypes.byref(w), ctypes.byref(k), ctypes.byref(s)))
        return dict(launches=n.value, weight_bytes=w.value, kv_bytes=k.value, state_bytes=s.value)
