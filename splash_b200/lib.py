"""ctypes binding of libsplash_b200.so. There is no fallback: if the library is missing or a call
fails, an exception says so."""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# The library built in-tree; SPLASH_B200_LIBRARY names another build of it (a diagnostic build, say).
_PATH = os.environ.get("SPLASH_B200_LIBRARY") or os.path.join(_HERE, "libsplash_b200.so")

FMT_Q4K, FMT_Q6K, FMT_Q80, FMT_NVFP4, FMT_BF16, FMT_F16, FMT_F32 = 0, 4, 6, 37, 41, 42, 64
EP_NONE, EP_RESIDUAL, EP_UP_WITH_GATE, EP_GATE_UP, EP_PARTIALS, EP_GATE_UP_PARTIALS = 0, 1, 2, 3, 4, 5
LINEAR_PDL = 1
LINEAR_TCGEN05 = 2
LINEAR_WIDE_IMAGE = 4


class SbError(RuntimeError):
    pass


class SbLinearArgs(ctypes.Structure):
    _fields_ = [
        ("weights", ctypes.c_void_p), ("weights2", ctypes.c_void_p), ("x", ctypes.c_void_p),
        ("prepared", ctypes.c_void_p), ("aux", ctypes.c_void_p), ("out", ctypes.c_void_p), ("norm_weight", ctypes.c_void_p),
        ("format", ctypes.c_uint32), ("n", ctypes.c_uint32), ("k", ctypes.c_uint32), ("rows", ctypes.c_uint32),
        ("x_stride", ctypes.c_uint32), ("aux_stride", ctypes.c_uint32), ("out_stride", ctypes.c_uint32),
        ("epilogue", ctypes.c_uint32), ("out_f32", ctypes.c_uint32), ("flags", ctypes.c_uint32),
    ]


class SbLinearPlan(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint32) for n in
                ("slices", "ctas", "tile_rows", "stages", "smem_bytes", "stage_blocks", "slice_blocks_max", "tiles")]


_lib = None


def load():
    """The shared library; raises if it has not been built (python -c 'import __graft_entry__ as g; g.build()')."""
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            raise SbError(f"{_PATH} is missing: build it with `make -C splash_b200/csrc`; there is no CPU fallback")
        _lib = ctypes.CDLL(_PATH)
        _lib.sb_last_error.restype = ctypes.c_char_p
        _lib.sb_row_bytes.restype = ctypes.c_uint64
        _lib.sb_row_bytes.argtypes = [ctypes.c_uint32, ctypes.c_uint32]
        for name in ("sb_alloc", "sb_host_alloc"):
            getattr(_lib, name).argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]
        _lib.sb_free.argtypes = [ctypes.c_void_p]
        _lib.sb_host_free.argtypes = [ctypes.c_void_p]
        _lib.sb_memset.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p]
        _lib.sb_upload.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        _lib.sb_download.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        _lib.sb_stream_sync.argtypes = [ctypes.c_void_p]
        _lib.sb_stream_destroy.argtypes = [ctypes.c_void_p]
        _lib.sb_event_record.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        _lib.sb_event_sync.argtypes = [ctypes.c_void_p]
        _lib.sb_event_destroy.argtypes = [ctypes.c_void_p]
        _lib.sb_event_elapsed_ms.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
        _lib.sb_graph_begin.argtypes = [ctypes.c_void_p]
        _lib.sb_graph_end.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]
        _lib.sb_graph_launch.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        _lib.sb_graph_destroy.argtypes = [ctypes.c_void_p]
        _lib.sb_linear.argtypes = [ctypes.c_void_p, ctypes.POINTER(SbLinearArgs)]
        _lib.sb_linear_prepare.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                           ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32]
        _lib.sb_linear_prepared_bytes.restype = ctypes.c_uint64
        _lib.sb_linear_wide_prepared_bytes.restype = ctypes.c_uint64
        _lib.sb_linear_wide_image_bytes.restype = ctypes.c_uint64
        _lib.sb_linear_wide_image_bytes.argtypes = [ctypes.c_uint32] * 3
        _lib.sb_linear_wide_image.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]
        _lib.sb_linear_wide_prepared_bytes.argtypes = [ctypes.c_uint32, ctypes.c_uint32]
        _lib.sb_linear_wide_prepare.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p,
                                                ctypes.c_void_p, ctypes.c_uint32]
        _lib.sb_linear_prepare_sum.argtypes = ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32,
                                                ctypes.c_void_p] + [ctypes.c_uint32] * 3 + [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p,
                                                                                            ctypes.c_uint32])
        _lib.sb_dequant.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32,
                                    ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32]
    return _lib


def check(status):
    if status != 0:
        raise SbError(f"splash_b200 status {status}: {load().sb_last_error().decode(errors='replace')}")


def device_count():
    return load().sb_device_count()


def init(device=0):
    check(load().sb_init(device))


def device_status():
    s = ctypes.c_uint32(0)
    check(load().sb_device_status(ctypes.byref(s)))
    return s.value


class DeviceBuffer:
    """Owns one device allocation (sb_alloc / sb_free)."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)
        p = ctypes.c_void_p()
        check(load().sb_alloc(self.nbytes, ctypes.byref(p)))
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, a, slack=256):
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes + slack)
        check(load().sb_upload(b.ptr, a.ctypes.data_as(ctypes.c_void_p), a.nbytes, None))
        check(load().sb_stream_sync(None))
        return b

    def upload(self, a, stream=None, offset=0):
        a = np.ascontiguousarray(a)
        assert offset + a.nbytes <= self.nbytes
        check(load().sb_upload(self.ptr + offset, a.ctypes.data_as(ctypes.c_void_p), a.nbytes, stream))
        if stream is None:
            check(load().sb_stream_sync(None))

    def to_numpy(self, dtype, shape, offset=0):
        out = np.empty(shape, dtype)
        assert offset + out.nbytes <= self.nbytes
        check(load().sb_download(out.ctypes.data_as(ctypes.c_void_p), self.ptr + offset, out.nbytes, None))
        check(load().sb_stream_sync(None))
        return out

    def fill(self, byte):
        check(load().sb_memset(self.ptr, byte, self.nbytes, None))

    def free(self):
        if self.ptr:
            load().sb_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Event:
    def __init__(self):
        p = ctypes.c_void_p()
        check(load().sb_event_create(ctypes.byref(p)))
        self.ptr = p.value

    def record(self, stream=None):
        check(load().sb_event_record(self.ptr, stream))

    def sync(self):
        check(load().sb_event_sync(self.ptr))

    def elapsed_ms(self, stop):
        ms = ctypes.c_float()
        check(load().sb_event_elapsed_ms(self.ptr, stop.ptr, ctypes.byref(ms)))
        return ms.value


def stream_create():
    p = ctypes.c_void_p()
    check(load().sb_stream_create(ctypes.byref(p)))
    return p.value


def stream_sync(stream=None):
    check(load().sb_stream_sync(stream))


def linear(weights, x, out, fmt, n, k, rows, *, weights2=None, aux=None, norm_weight=None, prepared=None, epilogue=EP_NONE,
           out_f32=False, x_stride=None, aux_stride=None, out_stride=None, flags=0, stream=None):
    """sb_linear over device pointers (ints)."""
    a = SbLinearArgs(weights, weights2, x, prepared, aux, out, norm_weight, fmt, n, k, rows,
                     x_stride or k, (aux_stride or n) if aux else 0, out_stride or n, epilogue, int(out_f32), flags)
    check(load().sb_linear(stream, ctypes.byref(a)))


# ---- the remaining operators ----
_P, _U, _F = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_float


class SbKvLayer(ctypes.Structure):
    _fields_ = [("k", _P), ("v", _P), ("k_scale", _P), ("v_scale", _P),
                ("kv_heads", _U), ("head_dim", _U), ("page_tokens", _U), ("scale_f16", _U)]


class SbAttnStoreArgs(ctypes.Structure):
    _fields_ = [("qkv", _P), ("q_norm", _P), ("k_norm", _P), ("cos_tab", _P), ("sin_tab", _P), ("page_table", _P),
                ("queries", _P), ("cache", SbKvLayer), ("committed_dev", _P),
                ("rows", _U), ("q_heads", _U), ("gated", _U), ("pairs", _U), ("qkv_stride", _U), ("committed", _U),
                ("lanes", _U), ("page_table_stride", _U)]


class SbAttnArgs(ctypes.Structure):
    _fields_ = [("queries", _P), ("qkv", _P), ("page_table", _P), ("tree", _P), ("out", _P), ("cache", SbKvLayer), ("committed_dev", _P),
                ("rows", _U), ("q_heads", _U), ("gated", _U), ("qkv_stride", _U), ("out_stride", _U), ("committed", _U),
                ("lanes", _U), ("page_table_stride", _U)]


class SbGdnTape(ctypes.Structure):
    _fields_ = [("inputs", _P), ("k", _P), ("v", _P), ("beta", _P), ("decay", _P)]


class SbGdnArgs(ctypes.Structure):
    _fields_ = [("qkvz", _P), ("b", _P), ("a", _P), ("conv_w", _P), ("a_scale", _P), ("dt_bias", _P), ("norm_w", _P),
                ("conv_state_in", _P), ("conv_state_out", _P), ("state_in", _P), ("state_out", _P),
                ("pending", SbGdnTape), ("step", SbGdnTape), ("hidden", _P), ("pending_rows_dev", _P),
                ("rows", _U), ("pending_rows", _U), ("key_heads", _U), ("value_heads", _U), ("qkvz_stride", _U),
                ("ab_stride", _U), ("hidden_stride", _U), ("tiled", _U),
                ("gate_weight", _P), ("gate_input", _P), ("gate_k", _U), ("gate_input_stride", _U),
                ("tree", _P), ("pending_path_dev", _P), ("pending_path", _U), ("flags", _U), ("lanes", _U), ("reserved", _U)]


class SbSampleArgs(ctypes.Structure):
    _fields_ = [("logits", _P), ("input_tokens", _P), ("uniforms", _P), ("selected", _P), ("workspace", _P),
                ("rows", _U), ("vocab", _U), ("logit_stride", _U), ("temperature", _F),
                ("min_p", _F), ("top_k", _U), ("top_p", _F), ("cut_out", _P),
                ("candidate_ids", _P), ("candidate_q", _P), ("draws", _P), ("lanes", _U), ("reserved", _U), ("lane_policies", _P)]


class SbLanePolicy(ctypes.Structure):
    _fields_ = [("temperature", _F), ("min_p", _F), ("top_k", _U), ("top_p", _F)]


class SbPenaltyArgs(ctypes.Structure):
    _fields_ = [("logits", ctypes.c_void_p), ("words", ctypes.c_void_p), ("input_tokens", ctypes.c_void_p), ("tree", ctypes.c_void_p),
                ("rows", ctypes.c_uint32), ("vocab", ctypes.c_uint32), ("logit_stride", ctypes.c_uint32),
                ("repetition", ctypes.c_float), ("presence", ctypes.c_float), ("frequency", ctypes.c_float),
                ("lanes", ctypes.c_uint32), ("reserved", ctypes.c_uint32)]


class SbMoeRouteArgs(ctypes.Structure):
    _fields_ = [("scores", ctypes.c_void_p), ("input", ctypes.c_void_p), ("shared_gate", ctypes.c_void_p), ("selected", ctypes.c_void_p),
                ("weights", ctypes.c_void_p), ("rows", ctypes.c_uint32), ("experts", ctypes.c_uint32), ("slots", ctypes.c_uint32),
                ("top_k", ctypes.c_uint32), ("input_size", ctypes.c_uint32), ("sigmoid_normalized", ctypes.c_uint32)]


class SbMoeExpertArgs(ctypes.Structure):
    _fields_ = [("input", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("selected", ctypes.c_void_p), ("weights", ctypes.c_void_p),
                ("gate", ctypes.c_void_p), ("up", ctypes.c_void_p), ("down", ctypes.c_void_p), ("scratch", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("rows", ctypes.c_uint32), ("routes", ctypes.c_uint32), ("hidden", ctypes.c_uint32), ("inter", ctypes.c_uint32),
                ("format", ctypes.c_uint32), ("experts_total", ctypes.c_uint32)]


class SbAcceptArgs(ctypes.Structure):
    _fields_ = [("input_tokens", _P), ("tree", _P), ("tokens", _P), ("results", _P), ("stop_tokens", _P),
                ("rows", _U), ("remaining", _U), ("n_stop", _U), ("lanes", _U)]


class SbAdmitArgs(ctypes.Structure):
    _fields_ = [("logits", _P), ("masks", _P), ("excluded", _P), ("rows", _U), ("vocab", _U), ("logit_stride", _U), ("mask_words", _U),
                ("n_excluded", _U), ("lanes", _U)]


class SbSelectAcceptArgs(ctypes.Structure):
    _fields_ = [("sample", SbSampleArgs), ("accept", SbAcceptArgs), ("tickets", _P), ("committed", _P), ("pending_rows", _P),
                ("pending_path", _P), ("advance", _U), ("reserved", _U), ("lane_rows", _P), ("lane_remaining", _P)]


def _bind_ops():
    l = load()
    if getattr(l, "_ops_bound", False):
        return l
    l.sb_rmsnorm.argtypes = [_P, _P, _U, _U, _U, _P, _P, _U]
    l.sb_embed.argtypes = [_P, _U, _P, _U, _U, _P, _U, _P, _U]
    l.sb_rope_tables.argtypes = [_P, _P, _U, _P, _U, _F, _P, _P]
    l.sb_linear_f32.argtypes = [_P, _P, _P, _U, _U, _U, _U, _P, _U, _U, _P]
    l.sb_attn_store.argtypes = [_P, ctypes.POINTER(SbAttnStoreArgs)]
    l.sb_attn_verify.argtypes = [_P, ctypes.POINTER(SbAttnArgs)]
    l.sb_set_attention_kernel.argtypes = [ctypes.c_int]
    l.sb_kv_path_commit.argtypes = [_P, ctypes.POINTER(SbKvLayer), _P, _U, _P]
    l.sb_gdn_verify.argtypes = [_P, ctypes.POINTER(SbGdnArgs)]
    l.sb_gdn_verify_static.argtypes = [_P, ctypes.POINTER(SbGdnArgs)]
    l.sb_sample_workspace_bytes.restype = ctypes.c_uint64
    l.sb_sample_workspace_bytes.argtypes = [_U, _U]
    l.sb_sample_verify.argtypes = [_P, ctypes.POINTER(SbSampleArgs)]
    l.sb_accept.argtypes = [_P, ctypes.POINTER(SbAcceptArgs)]
    l.sb_select_accept.argtypes = [_P, ctypes.POINTER(SbSelectAcceptArgs)]
    l.sb_sample_admit.argtypes = [_P, ctypes.POINTER(SbAdmitArgs)]
    l.sb_moe_route.argtypes = [_P, ctypes.POINTER(SbMoeRouteArgs)]
    l.sb_moe_experts.argtypes = [_P, ctypes.POINTER(SbMoeExpertArgs)]
    l.sb_moe_scratch_bytes.restype = ctypes.c_uint64
    l.sb_moe_scratch_bytes.argtypes = [_U, _U, _U, _U]
    l.sb_sample_penalize.argtypes = [_P, ctypes.POINTER(SbPenaltyArgs)]
    l._ops_bound = True
    return l


def ops():
    """The library with every operator's signature bound."""
    return _bind_ops()


def chain_tree(rows):
    """SplashTreeRow records of a chain: ancestors, parent | depth << 16 (row 0's parent is itself)."""
    t = np.zeros((rows, 2), np.uint32)
    for r in range(rows):
        t[r, 0] = (1 << (r + 1)) - 1
        t[r, 1] = (max(r - 1, 0) & 0xFFFF) | (r << 16)
    return t
