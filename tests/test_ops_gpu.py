"""Parity of the glue operators, the KV store, attention, GDN, selection and acceptance (CUDA, through
the C ABI) with the oracle on the same seeded inputs."""
import ctypes

import numpy as np
import pytest

import oracle_lib as ol
import quant_fixtures as qf

pytestmark = pytest.mark.gpu
P = ol.ptr


def _setup():
    from splash_b200 import lib
    lib.init(0)
    return lib, lib.ops(), ol.bind_ops(ol.load())


def bf16_randn(rng, shape, scale=1.0):
    return ol.f2bf((rng.standard_normal(shape) * scale).astype(np.float32))


def ulp_bf16(x):
    e = np.floor(np.log2(np.maximum(np.abs(x), 2.0 ** -126)))
    return 2.0 ** (e - 7)


def test_rmsnorm_and_fused_float_projection():
    lib, l, o = _setup()
    rng = np.random.default_rng(1)
    rows, width = 16, 5120
    x = bf16_randn(rng, (rows, width), 3.0)
    w = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    want = np.zeros((rows, width), np.uint16)
    o.so_rmsnorm(P(x), rows, width, width, P(w), P(want), width)
    xd, wd = lib.DeviceBuffer.from_numpy(x), lib.DeviceBuffer.from_numpy(w)
    od = lib.DeviceBuffer(rows * width * 2)
    lib.check(l.sb_rmsnorm(None, xd.ptr, rows, width, width, wd.ptr, od.ptr, width))
    got = od.to_numpy(np.uint16, (rows, width))
    d = np.abs(ol.bf2f(got).astype(np.float64) - ol.bf2f(want))
    assert (d <= ulp_bf16(ol.bf2f(want))).all() and (got != want).mean() < 0.01
    # fp32 projection of fp32 rows over the normalised input (the GDN alpha/beta rows)
    n = 96
    wf = (rng.standard_normal((n, width)) * 0.02).astype(np.float32)
    wfd = lib.DeviceBuffer.from_numpy(wf)
    pd = lib.DeviceBuffer(rows * n * 4)
    lib.check(l.sb_linear_f32(None, wfd.ptr, xd.ptr, rows, n, width, width, pd.ptr, n, 1, wd.ptr))
    proj = pd.to_numpy(np.float32, (rows, n))
    ref = ol.bf2f(want).astype(np.float64) @ wf.astype(np.float64).T
    assert np.abs(proj - ref).max() <= 2e-3 * np.abs(ref).max()


@pytest.mark.parametrize("fmt", [4, 0, 6])
def test_embedding_gather(fmt):
    lib, l, o = _setup()
    vocab, width, rows = 1000, 1024, 16
    table = qf.realistic(fmt, vocab, width, seed=5)
    tokens = np.array([0, 999, 5, 1000, 4000000000, 17, 3, 3, 9, 100, 200, 300, 400, 500, 600, 700], np.uint32)
    want = np.zeros((rows, width), np.uint16)
    assert o.so_embed(fmt, P(table), vocab, width, P(tokens), rows, P(want), width) == 0
    td, kd = lib.DeviceBuffer.from_numpy(table), lib.DeviceBuffer.from_numpy(tokens)
    od = lib.DeviceBuffer(rows * width * 2)
    lib.check(l.sb_embed(None, fmt, td.ptr, vocab, width, kd.ptr, rows, od.ptr, width))
    assert np.array_equal(od.to_numpy(np.uint16, (rows, width)), want)


def test_rope_tables():
    lib, l, o = _setup()
    rows, pairs = 16, 32
    pos = (32768 + np.arange(rows)).astype(np.uint32)
    inv = (1e6 ** (-np.arange(pairs) / pairs)).astype(np.float32)
    c, s = np.zeros((rows, pairs), np.float32), np.zeros((rows, pairs), np.float32)
    o.so_rope_tables(P(pos), rows, P(inv), pairs, 1.0, P(c), P(s))
    pd, fd = lib.DeviceBuffer.from_numpy(pos), lib.DeviceBuffer.from_numpy(inv)
    cd, sd = lib.DeviceBuffer(c.nbytes), lib.DeviceBuffer(s.nbytes)
    lib.check(l.sb_rope_tables(None, pd.ptr, rows, fd.ptr, pairs, 1.0, cd.ptr, sd.ptr))
    assert np.abs(cd.to_numpy(np.float32, c.shape) - c).max() < 2e-6
    assert np.abs(sd.to_numpy(np.float32, s.shape) - s).max() < 2e-6


class DevKv:
    def __init__(self, lib, host):
        self.host = host
        self.k, self.v = lib.DeviceBuffer.from_numpy(host.k), lib.DeviceBuffer.from_numpy(host.v)
        self.ks, self.vs = lib.DeviceBuffer.from_numpy(host.ks), lib.DeviceBuffer.from_numpy(host.vs)

    def desc(self, lib):
        return lib.SbKvLayer(self.k.ptr, self.v.ptr, self.ks.ptr, self.vs.ptr, *self.host.geom)

    def download(self):
        h = self.host
        return (self.k.to_numpy(np.int8, h.k.shape), self.v.to_numpy(np.int8, h.v.shape),
                self.ks.to_numpy(h.ks.dtype, h.ks.shape), self.vs.to_numpy(h.vs.dtype, h.vs.shape))


def attention_case(lib, l, o, *, q_heads, kv_heads, D, page_tokens, scale_f16, committed, rows, gated, seed, kernel=0):
    lib.check(l.sb_set_attention_kernel(kernel))  # 0: tcgen05 (S and O in tensor memory), 1: warp-level MMA
    rng = np.random.default_rng(seed)
    pairs = 32 if D == 256 else 16
    pages = (committed + rows + page_tokens - 1) // page_tokens + 1
    host = ol.HostKv(pages, kv_heads, D, page_tokens, scale_f16)
    host.fill_random(rng)
    table = rng.permutation(pages).astype(np.uint32)
    qs = 2 * D if gated else D
    stride = q_heads * qs + 2 * kv_heads * D
    qkv = bf16_randn(rng, (rows, stride), 1.5)
    qn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    pos = (committed + np.arange(rows)).astype(np.uint32)
    inv = (1e6 ** (-np.arange(pairs) / pairs)).astype(np.float32)
    c, s = np.zeros((rows, pairs), np.float32), np.zeros((rows, pairs), np.float32)
    o.so_rope_tables(P(pos), rows, P(inv), pairs, 1.0, P(c), P(s))
    dev = DevKv(lib, host)  # upload before the oracle writes its rows
    # oracle
    queries = np.zeros((rows, q_heads, D), np.uint16)
    desc = host.desc()
    o.so_attn_store(P(qkv), stride, rows, q_heads, int(gated), P(qn), P(kn), P(c), P(s), pairs, ctypes.byref(desc),
                    P(table), committed, P(queries))
    want = np.zeros((rows, q_heads * D), np.uint16)
    want64 = np.zeros((rows, q_heads, D), np.float64)
    o.so_attention(P(queries), P(qkv), stride, rows, q_heads, int(gated), ctypes.byref(desc), P(table), committed, None,
                   P(want), q_heads * D, P(want64))
    # device
    bufs = {n: lib.DeviceBuffer.from_numpy(a) for n, a in dict(qkv=qkv, qn=qn, kn=kn, c=c, s=s, table=table).items()}
    qd = lib.DeviceBuffer(queries.nbytes)
    sa = lib.SbAttnStoreArgs(bufs["qkv"].ptr, bufs["qn"].ptr, bufs["kn"].ptr, bufs["c"].ptr, bufs["s"].ptr, bufs["table"].ptr,
                             qd.ptr, dev.desc(lib), None, rows, q_heads, int(gated), pairs, stride, committed)
    lib.check(l.sb_attn_store(None, ctypes.byref(sa)))
    od = lib.DeviceBuffer(want.nbytes)
    od.fill(0xFF)
    aa = lib.SbAttnArgs(qd.ptr, bufs["qkv"].ptr, bufs["table"].ptr, None, od.ptr, dev.desc(lib), None, rows, q_heads, int(gated),
                        stride, q_heads * D, committed)
    lib.check(l.sb_attn_verify(None, ctypes.byref(aa)))
    lib.stream_sync()
    assert lib.device_status() == 0
    got_q = qd.to_numpy(np.uint16, queries.shape)
    k, v, ks, vs = dev.download()
    return dict(host=host, got_q=got_q, want_q=queries, k=k, v=v, ks=ks, vs=vs,
                got=od.to_numpy(np.uint16, want.shape), want=want, want64=want64.reshape(rows, -1))


@pytest.mark.parametrize("cfg", [
    dict(q_heads=24, kv_heads=4, D=256, page_tokens=256, scale_f16=True, committed=2048, rows=16, gated=True, seed=1),
    dict(q_heads=8, kv_heads=2, D=128, page_tokens=256, scale_f16=True, committed=2048, rows=16, gated=False, seed=2),
    dict(q_heads=24, kv_heads=4, D=256, page_tokens=32, scale_f16=False, committed=1000, rows=5, gated=True, seed=3),
    dict(q_heads=16, kv_heads=2, D=256, page_tokens=64, scale_f16=False, committed=7, rows=16, gated=True, seed=4),
    dict(q_heads=8, kv_heads=2, D=128, page_tokens=32, scale_f16=True, committed=0, rows=1, gated=False, seed=5),
    dict(q_heads=24, kv_heads=4, D=256, page_tokens=32, scale_f16=True, committed=4999, rows=16, gated=True, seed=6),
])
@pytest.mark.parametrize("kernel", [0, 1])
def test_kv_store_bit_exact_and_attention_within_gates(cfg, kernel):
    lib, l, o = _setup()
    r = attention_case(lib, l, o, kernel=kernel, **cfg)
    # staged queries and the quantized rows: bit-exact
    assert np.array_equal(r["got_q"], r["want_q"])
    h = r["host"]
    assert np.array_equal(r["k"], h.k) and np.array_equal(r["v"], h.v)
    assert np.array_equal(r["ks"], h.ks) and np.array_equal(r["vs"], h.vs)
    # attention: the reference's gates (cosine > 0.9995, max-abs < 0.02) and 2e-3 of the output's scale
    got, want64 = ol.bf2f(r["got"]).astype(np.float64), r["want64"]
    cos = (got * want64).sum() / np.sqrt((got * got).sum() * (want64 * want64).sum())
    assert cos > 0.9995
    scale = np.abs(want64).max()
    assert np.abs(got - want64).max() < max(0.02, 4e-3 * scale)
    rel = np.abs(got - want64) / np.maximum(np.abs(want64), np.sqrt((want64 ** 2).mean()))
    assert np.median(rel) < 2e-3 and rel.max() < 2e-2


@pytest.mark.parametrize("kernel", [0, 1])
def test_attention_long_context_32k(kernel):
    lib, l, o = _setup()
    r = attention_case(lib, l, o, q_heads=24, kv_heads=4, D=256, page_tokens=256, scale_f16=True, committed=32768 - 16,
                       rows=16, gated=True, seed=9, kernel=kernel)
    got, want64 = ol.bf2f(r["got"]).astype(np.float64), r["want64"]
    cos = (got * want64).sum() / np.sqrt((got * got).sum() * (want64 * want64).sum())
    assert cos > 0.9995 and np.abs(got - want64).max() < 0.02


def gdn_case(lib, l, o, *, key_heads, value_heads, rows, pending_rows, tiled, seed, fused_gates=0, tree=None, pending_path=0):
    """fused_gates = k > 0: b and a are projections of a bf16 input [16, k] by fp32 rows [2 * value_heads, k]; the
    kernel computes them itself (gate_weight / gate_input) and the oracle gets what sb_linear_f32 gives for them."""
    rng = np.random.default_rng(seed)
    D = 128
    KW, VW = key_heads * D, value_heads * D
    C = 2 * KW + VW
    stride = C + VW
    qkvz = bf16_randn(rng, (16, stride), 1.0)
    b = bf16_randn(rng, (16, value_heads), 1.0)
    a = bf16_randn(rng, (16, value_heads), 1.0)
    gate = None
    if fused_gates:
        gk = fused_gates
        gw = (rng.standard_normal((2 * value_heads, gk)) / np.sqrt(gk)).astype(np.float32)
        gx = bf16_randn(rng, (16, gk), 1.0)
        gate = dict(w=lib.DeviceBuffer.from_numpy(gw), x=lib.DeviceBuffer.from_numpy(gx), k=gk)
        gd = lib.DeviceBuffer(16 * 2 * value_heads * 2)
        lib.check(l.sb_linear_f32(None, gate["w"].ptr, gate["x"].ptr, 16, 2 * value_heads, gk, gk, gd.ptr, 2 * value_heads, 0, None))
        gates = gd.to_numpy(np.uint16, (16, 2 * value_heads))
        b, a = np.ascontiguousarray(gates[:, :value_heads]), np.ascontiguousarray(gates[:, value_heads:])
    conv_w = bf16_randn(rng, (C, 4), 0.4)
    a_scale = (-np.exp(rng.uniform(-3, 0.5, value_heads))).astype(np.float32)
    dt_bias = bf16_randn(rng, (value_heads,), 0.5)
    norm_w = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    cs_in = bf16_randn(rng, (3, C), 1.0)
    state = (rng.standard_normal((value_heads, D, D)) * 0.05).astype(np.float32)
    pend = dict(inputs=bf16_randn(rng, (16, C), 1.0), k=bf16_randn(rng, (16, KW), 0.09), v=bf16_randn(rng, (16, VW), 0.5),
                beta=ol.f2bf(rng.uniform(0.1, 0.9, (16, value_heads)).astype(np.float32)),
                decay=rng.uniform(0.5, 1.0, (16, value_heads)).astype(np.float32))
    step = dict(inputs=np.zeros((16, C), np.uint16), k=np.zeros((16, KW), np.uint16), v=np.zeros((16, VW), np.uint16),
                beta=np.zeros((16, value_heads), np.uint16), decay=np.zeros((16, value_heads), np.float32))
    cs_out, state_out = np.zeros_like(cs_in), np.zeros_like(state)
    hidden = np.zeros((16, VW), np.uint16)
    tape = lambda t: ol.SoGdnTape(P(t["inputs"]), P(t["k"]), P(t["v"]), P(t["beta"]), P(t["decay"]))
    args = ol.SoGdnArgs(P(qkvz), P(b), P(a), P(conv_w), P(a_scale), P(dt_bias), P(norm_w), P(cs_in), P(cs_out), P(state),
                        P(state_out), tape(pend), tape(step), P(hidden), rows, pending_rows, key_heads, value_heads,
                        stride, value_heads, VW, int(tiled), P(tree) if tree is not None else None, pending_path)
    o.so_gdn_verify(ctypes.byref(args))
    up = lib.DeviceBuffer.from_numpy
    d = {n: up(x) for n, x in dict(qkvz=qkvz, b=b, a=a, conv_w=conv_w, a_scale=a_scale, dt_bias=dt_bias, norm_w=norm_w,
                                   cs_in=cs_in, state=state).items()}
    dp = {n: up(x) for n, x in pend.items()}
    ds = {n: lib.DeviceBuffer(x.nbytes) for n, x in step.items()}
    dcs, dst, dh = lib.DeviceBuffer(cs_out.nbytes), lib.DeviceBuffer(state.nbytes), lib.DeviceBuffer(hidden.nbytes)
    dtape = lambda t: lib.SbGdnTape(t["inputs"].ptr, t["k"].ptr, t["v"].ptr, t["beta"].ptr, t["decay"].ptr)
    ga = lib.SbGdnArgs(d["qkvz"].ptr, d["b"].ptr, d["a"].ptr, d["conv_w"].ptr, d["a_scale"].ptr, d["dt_bias"].ptr,
                       d["norm_w"].ptr, d["cs_in"].ptr, dcs.ptr, d["state"].ptr, dst.ptr, dtape(dp), dtape(ds), dh.ptr, None,
                       rows, pending_rows, key_heads, value_heads, stride, value_heads, VW, int(tiled))
    if tree is not None:
        tree_dev = up(tree)
        ga.tree = tree_dev.ptr
    ga.pending_path = pending_path
    if gate:
        ga.b = ga.a = None
        ga.gate_weight, ga.gate_input, ga.gate_k, ga.gate_input_stride = gate["w"].ptr, gate["x"].ptr, gate["k"], gate["k"]
    lib.check(l.sb_gdn_verify(None, ctypes.byref(ga)))
    lib.stream_sync()
    assert lib.device_status() == 0
    got = dict(cs=dcs.to_numpy(np.uint16, cs_out.shape), state=dst.to_numpy(np.float32, state.shape),
               hidden=dh.to_numpy(np.uint16, hidden.shape))
    got.update({n: ds[n].to_numpy(step[n].dtype, step[n].shape) for n in step})
    return got, dict(cs=cs_out, state=state_out, hidden=hidden, **step), rows


@pytest.mark.parametrize("cfg", [
    dict(key_heads=16, value_heads=48, rows=16, pending_rows=7, tiled=True, seed=1),
    dict(key_heads=8, value_heads=8, rows=16, pending_rows=16, tiled=False, seed=2),
    dict(key_heads=2, value_heads=6, rows=5, pending_rows=0, tiled=False, seed=3),
    dict(key_heads=2, value_heads=4, rows=1, pending_rows=2, tiled=True, seed=4),
])
def test_gdn_verify_within_reference_gates(cfg):
    lib, l, o = _setup()
    got, want, rows = gdn_case(lib, l, o, **cfg)
    assert np.array_equal(got["cs"], want["cs"])
    assert np.array_equal(got["inputs"][:rows], want["inputs"][:rows])
    # tape k / v and gates within 3 bf16 ulp (the reference's gate); state 1e-4 relative
    for n in ("k", "v", "beta"):
        g, w = ol.bf2f(got[n][:rows]).astype(np.float64), ol.bf2f(want[n][:rows]).astype(np.float64)
        assert (np.abs(g - w) <= 3 * ulp_bf16(w)).all(), n
    assert np.allclose(got["decay"][:rows], want["decay"][:rows], rtol=1e-5)
    s_scale = np.abs(want["state"]).max()
    assert np.abs(got["state"] - want["state"]).max() <= 1e-4 * s_scale
    g, w = ol.bf2f(got["hidden"][:rows]).astype(np.float64), ol.bf2f(want["hidden"][:rows]).astype(np.float64)
    bad = np.abs(g - w) > 3 * ulp_bf16(w) + 2e-3 * np.abs(w).mean()
    assert bad.mean() <= 0.01


def _tree_rows(parent):
    tree = np.zeros((len(parent), 2), np.uint32)
    for r in range(len(parent)):
        tree[r, 0] = (1 << r) | (tree[parent[r], 0] if r else 0)
        tree[r, 1] = parent[r] | ((bin(int(tree[r, 0])).count("1") - 1) << 16)
    return tree


@pytest.mark.parametrize("cfg", [
    dict(key_heads=16, value_heads=48, tiled=True, seed=31, parent=[0, 0, 1, 2, 3, 4, 5, 6, 3, 8, 9, 10, 1, 12, 13, 0], pending_path=0b1000100101),
    dict(key_heads=2, value_heads=6, tiled=False, seed=32, parent=[0, 0, 0, 0, 1, 1, 2, 4, 7], pending_path=0),
    dict(key_heads=2, value_heads=4, tiled=False, seed=33, parent=[0, 0, 1, 2, 3, 4], pending_path=0b111),   # a chain given as a tree
])
def test_gdn_tree_paths_within_reference_gates(cfg):
    """Tree rows: convolution taps along each row's path, outputs from the committed state along the path (the kernel by
    the transformed query, the oracle by definition), the previous step's accepted path as a row mask of its tape."""
    lib, l, o = _setup()
    parent = cfg.pop("parent")
    rows = len(parent)
    got, want, _ = gdn_case(lib, l, o, rows=rows, pending_rows=0, tree=_tree_rows(parent), **cfg)
    assert np.array_equal(got["cs"], want["cs"])
    assert np.array_equal(got["inputs"][:rows], want["inputs"][:rows])
    for n in ("k", "v", "beta"):
        g, w = ol.bf2f(got[n][:rows]).astype(np.float64), ol.bf2f(want[n][:rows]).astype(np.float64)
        assert (np.abs(g - w) <= 3 * ulp_bf16(w)).all(), n
    assert np.abs(got["state"] - want["state"]).max() <= 1e-4 * np.abs(want["state"]).max()
    g, w = ol.bf2f(got["hidden"][:rows]).astype(np.float64), ol.bf2f(want["hidden"][:rows]).astype(np.float64)
    bad = np.abs(g - w) > 3 * ulp_bf16(w) + 2e-3 * np.abs(w).mean()
    assert bad.mean() <= 0.01
    # every row on its own: a branch's rows differ from what the chain order would give
    for r in range(rows):
        gr, wr = g[r], w[r]
        assert np.abs(gr - wr).max() <= 0.02 * max(1e-6, np.abs(wr).max()), r


def test_gdn_fused_gate_projection_equals_separate_projection():
    """The kernel's own alpha / beta projection gives the bits of sb_linear_f32 followed by the plain kernel."""
    lib, l, o = _setup()
    cfg = dict(key_heads=4, value_heads=12, rows=16, pending_rows=5, tiled=True, seed=21)
    fused, want, rows = gdn_case(lib, l, o, fused_gates=5120, **cfg)
    assert np.array_equal(fused["beta"][:rows], want["beta"][:rows]) or \
        (np.abs(ol.bf2f(fused["beta"][:rows]).astype(np.float64) - ol.bf2f(want["beta"][:rows])) <= 3 * ulp_bf16(ol.bf2f(want["beta"][:rows]))).all()
    assert np.allclose(fused["decay"][:rows], want["decay"][:rows], rtol=1e-5)
    assert np.abs(fused["state"] - want["state"]).max() <= 1e-4 * np.abs(want["state"]).max()
    # and odd shapes: 5 rows, k = 1024
    fused2, want2, rows2 = gdn_case(lib, l, o, key_heads=2, value_heads=6, rows=5, pending_rows=0, tiled=False, seed=22, fused_gates=1024)
    assert np.allclose(fused2["decay"][:rows2], want2["decay"][:rows2], rtol=1e-5)
    assert np.abs(fused2["state"] - want2["state"]).max() <= 1e-4 * np.abs(want2["state"]).max()


def _gdn_inputs(rng, key_heads, value_heads):
    D = 128
    KW, VW = key_heads * D, value_heads * D
    C = 2 * KW + VW
    return dict(
        C=C, KW=KW, VW=VW, stride=C + VW, key_heads=key_heads, value_heads=value_heads,
        qkvz=bf16_randn(rng, (16, C + VW), 1.0), b=bf16_randn(rng, (16, value_heads), 1.0), a=bf16_randn(rng, (16, value_heads), 1.0),
        conv_w=bf16_randn(rng, (C, 4), 0.4), a_scale=(-np.exp(rng.uniform(-3, 0.5, value_heads))).astype(np.float32),
        dt_bias=bf16_randn(rng, (value_heads,), 0.5), norm_w=(1 + 0.1 * rng.standard_normal(D)).astype(np.float32),
        cs=bf16_randn(rng, (3, C), 1.0), state=(rng.standard_normal((value_heads, D, D)) * 0.05).astype(np.float32),
        pend=dict(inputs=bf16_randn(rng, (16, C), 1.0), k=bf16_randn(rng, (16, KW), 0.09), v=bf16_randn(rng, (16, VW), 0.5),
                  beta=ol.f2bf(rng.uniform(0.1, 0.9, (16, value_heads)).astype(np.float32)),
                  decay=rng.uniform(0.5, 1.0, (16, value_heads)).astype(np.float32)))


def _gdn_oracle(o, x, cs, state, rows, pending_rows):
    """One oracle call from the cell (cs, state): returns (cs_out, state_out, hidden, step tape)."""
    VH, VW, C, KW = x["value_heads"], x["VW"], x["C"], x["KW"]
    step = dict(inputs=np.zeros((16, C), np.uint16), k=np.zeros((16, KW), np.uint16), v=np.zeros((16, VW), np.uint16),
                beta=np.zeros((16, VH), np.uint16), decay=np.zeros((16, VH), np.float32))
    cs_out, state_out, hidden = np.zeros_like(cs), np.zeros_like(state), np.zeros((16, VW), np.uint16)
    tape = lambda t: ol.SoGdnTape(P(t["inputs"]), P(t["k"]), P(t["v"]), P(t["beta"]), P(t["decay"]))
    args = ol.SoGdnArgs(P(x["qkvz"]), P(x["b"]), P(x["a"]), P(x["conv_w"]), P(x["a_scale"]), P(x["dt_bias"]), P(x["norm_w"]), P(cs), P(cs_out),
                        P(state), P(state_out), tape(x["pend"]), tape(step), P(hidden), rows, pending_rows, x["key_heads"], VH, x["stride"], VH,
                        VW, 0, None, 0)
    o.so_gdn_verify(ctypes.byref(args))
    return cs_out, state_out, hidden, step


def test_gdn_fold_call_then_step_on_the_swapped_cells():
    """ops::GDN::addFold (the step with no rows of its own) followed at once by a step whose current cell is the fold's
    next cell, both launched with programmatic dependent launch and nothing between them: the step must read the cell
    the fold has just written (it does not carry SB_GDN_STATE_SETTLED). Checked against the oracle making the same two
    calls, and against one call that folds and steps at once: folding r accepted rows first and then stepping gives the
    bits of doing both in one launch (the reference tests the same: fold(first r rows) == the state the next step
    commits, dev/tests/engine/gdn_decode_metal_test.mm:12-20)."""
    lib, l, o = _setup()
    rng = np.random.default_rng(11)
    x = _gdn_inputs(rng, 2, 4)
    VH, VW, C, KW, pending = 4, x["VW"], x["C"], x["KW"], 5
    # oracle: fold, then step from the folded cell
    cs1, st1, _, _ = _gdn_oracle(o, x, x["cs"], x["state"], 0, pending)
    cs2, st2, hid2, tape2 = _gdn_oracle(o, x, cs1, st1, 16, 0)
    # device: the same two calls back to back on one stream, then the fused call
    up = lib.DeviceBuffer.from_numpy
    d = {n: up(x[n]) for n in ("qkvz", "b", "a", "conv_w", "a_scale", "dt_bias", "norm_w", "cs", "state")}
    dp = {n: up(v) for n, v in x["pend"].items()}
    sizes = dict(inputs=16 * C * 2, k=16 * KW * 2, v=16 * VW * 2, beta=16 * VH * 2, decay=16 * VH * 4)
    dtape = lambda t: lib.SbGdnTape(t["inputs"].ptr, t["k"].ptr, t["v"].ptr, t["beta"].ptr, t["decay"].ptr)

    def cell():
        return lib.DeviceBuffer(x["cs"].nbytes), lib.DeviceBuffer(x["state"].nbytes)

    def call(cs_in, st_in, cs_out, st_out, step, hidden, rows, pend_rows):
        ga = lib.SbGdnArgs(d["qkvz"].ptr, d["b"].ptr, d["a"].ptr, d["conv_w"].ptr, d["a_scale"].ptr, d["dt_bias"].ptr, d["norm_w"].ptr,
                           cs_in.ptr, cs_out.ptr, st_in.ptr, st_out.ptr, dtape(dp), dtape(step), hidden.ptr, None,
                           rows, pend_rows, 2, VH, x["stride"], VH, VW, 0)
        lib.check(l.sb_gdn_verify(None, ctypes.byref(ga)))

    results = {}
    for name in ("two calls", "one call"):
        (csa, sta), (csb, stb) = cell(), cell()
        step = {n: lib.DeviceBuffer(b) for n, b in sizes.items()}
        hidden = lib.DeviceBuffer(16 * VW * 2)
        for b in (csa, sta, csb, stb, hidden, *step.values()):
            b.fill(0)
        if name == "two calls":
            call(d["cs"], d["state"], csa, sta, step, hidden, 0, pending)   # addFold: the folded cell
            call(csa, sta, csb, stb, step, hidden, 16, 0)                  # addDecode on the swapped cells
        else:
            call(d["cs"], d["state"], csb, stb, step, hidden, 16, pending)
        lib.stream_sync()
        assert lib.device_status() == 0
        results[name] = dict(cs=csb.to_numpy(np.uint16, x["cs"].shape), state=stb.to_numpy(np.float32, x["state"].shape),
                             hidden=hidden.to_numpy(np.uint16, (16, VW)), k=step["k"].to_numpy(np.uint16, (16, KW)),
                             folded=sta.to_numpy(np.float32, x["state"].shape) if name == "two calls" else None)
    two, one = results["two calls"], results["one call"]
    # the fold alone, against the oracle's
    assert np.abs(two["folded"] - st1).max() <= 1e-4 * np.abs(st1).max()
    assert np.array_equal(two["cs"], cs2)
    assert np.abs(two["state"] - st2).max() <= 1e-4 * np.abs(st2).max()
    g, w = ol.bf2f(two["hidden"]).astype(np.float64), ol.bf2f(hid2).astype(np.float64)
    assert (np.abs(g - w) > 3 * ulp_bf16(w) + 2e-3 * np.abs(w).mean()).mean() <= 0.01
    assert np.abs(g).max() > 0
    # and fold-then-step is the one-launch step, bit for bit
    for n in ("cs", "state", "hidden", "k"):
        assert np.array_equal(two[n], one[n]), n


def test_greedy_selection_and_acceptance():
    lib, l, o = _setup()
    rng = np.random.default_rng(4)
    rows, vocab = 16, 151936
    logits = rng.standard_normal((rows, vocab)).astype(np.float32)
    logits[3, 77] = logits[3, 99000] = 50.0      # a tie: the lowest id wins
    logits[5, :] = np.nan                         # nothing selectable: the sentinel
    logits[6, 10] = np.inf
    logits[7, :] = -np.inf
    logits[7, 123] = -5.0
    want = np.zeros(rows, np.uint32)
    inputs = np.zeros(rows, np.uint32)
    o.so_sample_verify(P(logits), vocab, vocab, rows, P(inputs), 0.0, None, P(want), None)
    ld, idd = lib.DeviceBuffer.from_numpy(logits), lib.DeviceBuffer.from_numpy(inputs)
    sd = lib.DeviceBuffer(rows * 4)
    sa = lib.SbSampleArgs(ld.ptr, idd.ptr, None, sd.ptr, None, rows, vocab, vocab, 0.0)
    lib.check(l.sb_sample_verify(None, ctypes.byref(sa)))
    got = sd.to_numpy(np.uint32, (rows,))
    assert np.array_equal(got, want)
    assert got[3] == 77 and got[5] == 0xFFFFFFFF and got[6] == 10 and got[7] == 123
    # acceptance: the draft matched the first 4 selections
    inputs = np.concatenate([[1], got[:4], [5, 5, 5, 5, 5, 5, 5, 5, 5, 5, 5]]).astype(np.uint32)[:rows]
    tree = lib.chain_tree(rows)
    tokens = got.copy()
    res = np.zeros(3, np.uint32)
    o.so_accept(P(inputs), P(tree), P(tokens), rows, 100, None, 0, P(res[0:1]), P(res[1:2]), P(res[2:3]))
    idd.upload(inputs)
    td, kd, rd = lib.DeviceBuffer.from_numpy(tree), lib.DeviceBuffer.from_numpy(got), lib.DeviceBuffer(16)
    aa = lib.SbAcceptArgs(idd.ptr, td.ptr, kd.ptr, rd.ptr, None, rows, 100, 0)
    lib.check(l.sb_accept(None, ctypes.byref(aa)))
    dres = rd.to_numpy(np.uint32, (4,))
    assert dres[0] == res[0] == 5 and dres[1] == res[1] == 4 and dres[2] == res[2] == 0b11111
    assert np.array_equal(kd.to_numpy(np.uint32, (rows,))[:5], tokens[:5])


def test_stochastic_selection_with_supplied_uniforms():
    lib, l, o = _setup()
    rng = np.random.default_rng(8)
    rows, vocab = 16, 32000
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    greedy = logits.argmax(axis=1).astype(np.uint32)
    # the draft proposes the argmax with p = 0.7, else a random token
    inputs = np.zeros(rows, np.uint32)
    for r in range(1, rows):
        inputs[r] = greedy[r - 1] if rng.random() < 0.7 else rng.integers(0, vocab)
    uniforms = rng.random(80).astype(np.float32)
    want, margin = np.zeros(rows, np.uint32), np.zeros(rows, np.float64)
    o.so_sample_verify(P(logits), vocab, vocab, rows, P(inputs), 0.7, P(uniforms), P(want), P(margin))
    ld, idd, ud = (lib.DeviceBuffer.from_numpy(x) for x in (logits, inputs, uniforms))
    sd = lib.DeviceBuffer(rows * 4)
    wd = lib.DeviceBuffer(int(l.sb_sample_workspace_bytes(rows, vocab)))
    sa = lib.SbSampleArgs(ld.ptr, idd.ptr, ud.ptr, sd.ptr, wd.ptr, rows, vocab, vocab, 0.7)
    lib.check(l.sb_sample_verify(None, ctypes.byref(sa)))
    got = sd.to_numpy(np.uint32, (rows,))
    # bit-exact wherever the accept test is not within rounding of its threshold
    clear = margin > 1e-5
    assert clear.sum() >= rows - 2
    assert np.array_equal(got[clear], want[clear])


def test_recursive_rejection_over_drafted_children_matches_the_oracle():
    """Sampled rows with the draft's candidates, probabilities and up to four drawn children a row: the kernel's recursive
    rejection sampling against the oracle's, exact wherever no test sat within rounding of its threshold; with and without
    an end of the distribution (top-k / top-p)."""
    import ctypes as ct
    lib, l, o = _setup()
    o.so_sample_verify_draws.argtypes = ([ct.c_void_p, ct.c_uint32, ct.c_uint32, ct.c_uint32, ct.c_float, ct.c_float, ct.c_uint32, ct.c_float] +
                                         [ct.c_void_p] * 6)
    rows, vocab, T = 16, 32000, 0.7
    total_clear = taken = 0
    for seed, (min_p, top_k, top_p) in enumerate([(0.0, 0, 1.0), (0.0, 50, 0.9), (0.02, 0, 1.0)]):
        rng = np.random.default_rng(40 + seed)
        logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
        draft = logits + (rng.standard_normal((rows, vocab)) * 1.5).astype(np.float32)
        ids = np.argsort(-draft, axis=1)[:, :16].astype(np.uint32).copy()
        dq = np.exp((np.take_along_axis(draft, ids.astype(np.int64), 1) - draft.max(axis=1, keepdims=True)) / T)
        q = (dq / dq.sum(axis=1, keepdims=True)).astype(np.float32)
        draws = np.full((rows, 4), 255, np.uint8)
        for r in range(rows):
            n = int(rng.integers(0, 5))                      # 0 .. 4 children, drawn without replacement from q
            if n:
                draws[r, :n] = rng.choice(16, size=n, replace=False, p=q[r].astype(np.float64) / q[r].astype(np.float64).sum())
        ids[3, 12:] = 0xFFFFFFFF                              # a draft that listed fewer candidates
        q[3, 12:] = 0
        draws[3] = [1, 0, 255, 255]
        uniforms = rng.random(80).astype(np.float32)
        want, margin = np.zeros(rows, np.uint32), np.zeros(rows, np.float64)
        o.so_sample_verify_draws(P(logits), vocab, vocab, rows, T, min_p, top_k, top_p, P(uniforms), P(ids), P(q), P(draws), P(want), P(margin))
        up = lib.DeviceBuffer.from_numpy
        ld, ud, cd, qd, dd = up(logits), up(uniforms), up(ids), up(q), up(draws)
        inp = up(np.zeros(rows, np.uint32))
        sd = lib.DeviceBuffer(rows * 4)
        wd = lib.DeviceBuffer(int(l.sb_sample_workspace_bytes(rows, vocab)))
        sa = lib.SbSampleArgs(ld.ptr, inp.ptr, ud.ptr, sd.ptr, wd.ptr, rows, vocab, vocab, T, min_p, top_k, top_p, None, cd.ptr, qd.ptr, dd.ptr)
        lib.check(l.sb_sample_verify(None, ctypes.byref(sa)))
        got = sd.to_numpy(np.uint32, (rows,))
        assert lib.device_status() == 0
        clear = margin > 1e-5
        assert clear.sum() >= rows - 3
        assert np.array_equal(got[clear], want[clear]), (seed, got, want)
        total_clear += int(clear.sum())
        taken += sum(int(want[r]) in ids[r, draws[r][draws[r] < 16]].tolist() for r in range(rows))
    assert total_clear >= 40 and taken >= 5    # children were taken in a fair share of the rows


@pytest.mark.parametrize("min_p,top_k,top_p", [(0.05, 0, 1.0), (0.0, 40, 1.0), (0.0, 0, 0.9), (0.02, 50, 0.8), (0.0, 1, 1.0)])
def test_filtered_selection_matches_the_oracle(min_p, top_k, top_p):
    """min-p, top-k and top-p ends of the distribution and the selections under them."""
    lib, l, o = _setup()
    rng = np.random.default_rng(12)
    rows, vocab, T = 16, 32000, 0.7
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    logits[3, 500:520] = logits[3].max()        # ties at the top
    logits[5, ::5] = np.float32(-np.inf)
    greedy = logits.argmax(axis=1).astype(np.uint32)
    inputs = np.zeros(rows, np.uint32)
    for r in range(1, rows):
        inputs[r] = greedy[r - 1] if rng.random() < 0.7 else rng.integers(0, vocab)
    uniforms = rng.random(80).astype(np.float32)
    want, margin, wcut = np.zeros(rows, np.uint32), np.zeros(rows, np.float64), np.zeros((rows, 2), np.uint32)
    o.so_sample_verify_filtered(P(logits), vocab, vocab, rows, P(inputs), T, min_p, top_k, top_p, P(uniforms), P(want), P(margin), P(wcut))
    ld, idd, ud = (lib.DeviceBuffer.from_numpy(x) for x in (logits, inputs, uniforms))
    sd, cd = lib.DeviceBuffer(rows * 4), lib.DeviceBuffer(rows * 8)
    wd = lib.DeviceBuffer(int(l.sb_sample_workspace_bytes(rows, vocab)))
    sa = lib.SbSampleArgs(ld.ptr, idd.ptr, ud.ptr, sd.ptr, wd.ptr, rows, vocab, vocab, T, min_p, top_k, top_p, cd.ptr)
    lib.check(l.sb_sample_verify(None, ctypes.byref(sa)))
    got, gcut = sd.to_numpy(np.uint32, (rows,)), cd.to_numpy(np.uint32, (rows, 2))
    assert lib.device_status() == 0
    # the ends agree except where a mass sits within rounding of its nucleus (the device's expf is not the host's)
    same_cut = (gcut == wcut).all(axis=1)
    assert same_cut.sum() >= rows - 1
    clear = same_cut & (margin > 1e-5)
    assert clear.sum() >= rows - 3
    assert np.array_equal(got[clear], want[clear])
    if top_k == 1:
        assert np.array_equal(got, greedy)


@pytest.mark.parametrize("policy", [(1.3, 0.0, 0.0), (1.0, 0.6, 0.2), (0.85, 0.4, 0.1)])
def test_sampling_penalties_match_oracle_bitwise(policy):
    """sb_sample_penalize against the oracle's statement of decode_sample_penalize on a branching tree: every logit
    bit for bit (single IEEE operations in the reference's order), unselectable logits and saturation included."""
    lib, l, o = _setup()
    rng = np.random.default_rng(9)
    rows, vocab = 16, 151936
    logits = (rng.standard_normal((rows, vocab)) * 6).astype(np.float32)
    logits[2, 100] = np.nan
    logits[3, 101] = -np.inf
    logits[4, 102] = np.inf
    logits[5, 103] = 3.0e38
    logits[6, 104] = -3.0e38
    words = np.zeros(vocab, np.uint32)
    held = rng.choice(vocab, 4000, replace=False)
    words[held] = rng.integers(1, 40, 4000).astype(np.uint32)
    words[rng.choice(vocab, 3000, replace=False)] |= 0x80000000
    words[100:105] = 7 | 0x80000000
    inputs = rng.integers(0, vocab, rows).astype(np.uint32)
    inputs[5] = inputs[2]                 # the same draft token twice on one path
    inputs[9] = int(held[0])              # a draft token the output already holds
    # a tree: rows 1..7 a chain, rows 8..15 a second branch under row 3
    tree = np.zeros((rows, 2), np.uint32)
    parent = [0, 0, 1, 2, 3, 4, 5, 6, 3, 8, 9, 10, 11, 12, 13, 14]
    for r in range(rows):
        tree[r, 0] = (1 << r) | (tree[parent[r], 0] if r else 0)
        depth = bin(int(tree[r, 0])).count("1") - 1
        tree[r, 1] = parent[r] | (depth << 16)
    want = logits.copy()
    o.so_sample_penalize(P(want), vocab, vocab, rows, P(words), P(inputs), P(tree), *policy)
    ld, wd = lib.DeviceBuffer.from_numpy(logits), lib.DeviceBuffer.from_numpy(words)
    idd, td = lib.DeviceBuffer.from_numpy(inputs), lib.DeviceBuffer.from_numpy(tree)
    pa = lib.SbPenaltyArgs(ld.ptr, wd.ptr, idd.ptr, td.ptr, rows, vocab, vocab, *policy)
    lib.check(l.sb_sample_penalize(None, ctypes.byref(pa)))
    got = ld.to_numpy(np.float32, (rows, vocab))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert (got != logits).sum() > 10000 and np.isnan(got[2, 100]) and got[3, 101] == -np.inf
    assert got[4, 102] == np.float32(3.402823466e38)   # +inf saturates, as in the reference
    # arguments outside the contract are refused
    bad = lib.SbPenaltyArgs(ld.ptr, wd.ptr, idd.ptr, td.ptr, rows, vocab, vocab, 0.0, 0.0, 0.0)
    assert l.sb_sample_penalize(None, ctypes.byref(bad)) == -1


def test_kv_path_commit_moves_the_path_rows():
    """sb_kv_path_commit and sb_kv_path_commit_at against the oracle, bit for bit: the accepted path's rows (codes and
    scales) move from slot committed + row to slot committed + depth, across a page boundary."""
    lib, l, o = _setup()
    rng = np.random.default_rng(12)
    for scale_f16 in (1, 0):
        kv = ol.HostKv(6, 2, 128, 32, scale_f16)
        kv.fill_random(rng)
        table = rng.permutation(6).astype(np.uint32)
        committed, mask = 57, 0b1011001000110001   # rows 0, 4, 5, 9, 12, 13, 15 -> depths 0..6, slots 57.. cross into the next page
        dk, dv, dks, dvs = (lib.DeviceBuffer.from_numpy(x) for x in (kv.k, kv.v, kv.ks, kv.vs))
        dt, dm, dc = lib.DeviceBuffer.from_numpy(table), lib.DeviceBuffer.from_numpy(np.array([mask], np.uint32)), lib.DeviceBuffer.from_numpy(np.array([committed], np.uint32))
        cache = lib.SbKvLayer(dk.ptr, dv.ptr, dks.ptr, dvs.ptr, 2, 128, 32, scale_f16)
        l.sb_kv_path_commit_at.argtypes = [ctypes.c_void_p, ctypes.POINTER(lib.SbKvLayer), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        if scale_f16:
            lib.check(l.sb_kv_path_commit(None, ctypes.byref(cache), dt.ptr, committed, dm.ptr))
        else:
            lib.check(l.sb_kv_path_commit_at(None, ctypes.byref(cache), dt.ptr, dc.ptr, dm.ptr))
        lib.stream_sync()
        before = kv.k.copy()
        desc = kv.desc()
        o.so_kv_path_commit(ctypes.byref(desc), P(table), committed, mask)
        assert not np.array_equal(before, kv.k)
        assert np.array_equal(dk.to_numpy(np.int8, kv.k.shape), kv.k) and np.array_equal(dv.to_numpy(np.int8, kv.v.shape), kv.v)
        assert np.array_equal(dks.to_numpy(kv.ks.dtype, kv.ks.shape), kv.ks) and np.array_equal(dvs.to_numpy(kv.vs.dtype, kv.vs.shape), kv.vs)


@pytest.mark.parametrize("mode,shared", [(0, True), (1, False), (0, False)])
def test_moe_route_matches_oracle(mode, shared):
    """sb_moe_route against the oracle: the chosen experts exact (ties by id), the weights to rounding of exp2."""
    lib, l, o = _setup()
    rng = np.random.default_rng(6)
    rows, experts, slots, top_k, H = 16, 256, 256, 8, 2048
    scores = rng.standard_normal((rows, slots)).astype(np.float32)
    scores[2, 40] = scores[2, 7] = scores[2, 255] = 9.0
    scores[5, :] = -np.inf
    scores[6, ::2] = scores[6, 1::2]            # every score twice
    x = ol.f2bf(rng.standard_normal((rows, H)).astype(np.float32))
    gate = (rng.standard_normal(H) * 0.05).astype(np.float32)
    routes = top_k + (1 if shared else 0)
    want_s, want_w = np.zeros((rows, routes), np.uint32), np.zeros((rows, routes), np.float32)
    o.so_moe_route(P(scores), rows, experts, slots, top_k, mode, P(x), H, P(gate) if shared else None, P(want_s), P(want_w))
    sd, xd, gd = lib.DeviceBuffer.from_numpy(scores), lib.DeviceBuffer.from_numpy(x), lib.DeviceBuffer.from_numpy(gate)
    sel, wts = lib.DeviceBuffer(rows * routes * 4), lib.DeviceBuffer(rows * routes * 4)
    a = lib.SbMoeRouteArgs(sd.ptr, xd.ptr, gd.ptr if shared else None, sel.ptr, wts.ptr, rows, experts, slots, top_k, H, mode)
    lib.check(l.sb_moe_route(None, ctypes.byref(a)))
    lib.stream_sync()
    assert np.array_equal(sel.to_numpy(np.uint32, (rows, routes)), want_s)
    assert np.allclose(wts.to_numpy(np.float32, (rows, routes)), want_w, rtol=1e-5, atol=1e-7, equal_nan=True)  # (a row without a finite score has no weights: NaN on both sides)
    bad = lib.SbMoeRouteArgs(sd.ptr, None, None, sel.ptr, wts.ptr, rows, 300, 300, top_k, 0, 0)
    assert l.sb_moe_route(None, ctypes.byref(bad)) == -1


@pytest.mark.parametrize("shape", [
    dict(rows=13, experts=24, slots=32, top_k=8, H=1024, I=512),       # a small block, a ragged row count
    dict(rows=16, experts=256, slots=256, top_k=8, H=2048, I=512),     # the 35B-A3B block: 256 experts + the shared one
])
def test_moe_experts_match_oracle(shape):
    """sb_moe_route + sb_moe_experts on a MoE block (the experts + the shared one, 8 + 1 routes a row) against the oracle's
    fp64 statement: the per-route sums within 2e-3 of their scale, the combined rows within bf16 rounding of the
    oracle's."""
    lib, l, o = _setup()
    rng = np.random.default_rng(17)
    rows, experts, slots, top_k, H, I = (shape[n] for n in ("rows", "experts", "slots", "top_k", "H", "I"))
    total, routes = experts + 1, top_k + 1
    gate = np.concatenate([qf.realistic(0, I, H, seed=100 + e) for e in range(total)])
    up = np.concatenate([qf.realistic(0, I, H, seed=200 + e) for e in range(total)])
    down = np.concatenate([qf.realistic(0, H, I, seed=300 + e) for e in range(total)])
    x = ol.f2bf(rng.standard_normal((rows, H)).astype(np.float32))
    res = ol.f2bf(rng.standard_normal((rows, H)).astype(np.float32))
    scores = rng.standard_normal((rows, slots)).astype(np.float32)
    sgate = (rng.standard_normal(H) * 0.05).astype(np.float32)
    up_dev = lib.DeviceBuffer.from_numpy
    sd, xd, rd, gd = up_dev(scores), up_dev(x), up_dev(res), up_dev(sgate)
    sel, wts = lib.DeviceBuffer(rows * routes * 4), lib.DeviceBuffer(rows * routes * 4)
    ra = lib.SbMoeRouteArgs(sd.ptr, xd.ptr, gd.ptr, sel.ptr, wts.ptr, rows, experts, slots, top_k, H, 0)
    lib.check(l.sb_moe_route(None, ctypes.byref(ra)))
    wg, wu, wd = up_dev(gate), up_dev(up), up_dev(down)
    scratch = lib.DeviceBuffer(int(l.sb_moe_scratch_bytes(rows, routes, H, I)))
    out = lib.DeviceBuffer(rows * H * 2 + 256)
    ea = lib.SbMoeExpertArgs(xd.ptr, rd.ptr, sel.ptr, wts.ptr, wg.ptr, wu.ptr, wd.ptr, scratch.ptr, out.ptr, rows, routes, H, I, lib.FMT_Q4K, total)
    lib.check(l.sb_moe_experts(None, ctypes.byref(ea)))
    lib.stream_sync()
    assert lib.device_status() == 0
    selected, weights = sel.to_numpy(np.uint32, (rows, routes)), wts.to_numpy(np.float32, (rows, routes))
    assert (selected[:, top_k] == experts).all() and len(np.unique(selected[:, :top_k])) > 8
    want = np.zeros((rows, H), np.uint16)
    y64 = np.zeros((rows * routes, H), np.float64)
    assert o.so_moe_experts(P(x), P(res), P(selected), P(weights), P(gate), P(up), P(down), rows, routes, H, I, total, P(want), P(y64)) == 0
    y = ol.bf2f(scratch.to_numpy(np.uint16, (rows * routes * (I + H),))[rows * routes * I:].reshape(rows * routes, H)).astype(np.float64)
    # y is bf16: its rounding, and 2e-3 of the route's scale (a sum that cancels is judged against its row, not itself)
    ratio = np.abs(y - y64) / (ulp_bf16(y64) + 2e-3 * np.abs(y64).mean(axis=1, keepdims=True))
    # (an intermediate value that rounds to the neighbouring bf16 on one side moves a few sums a little further)
    assert (ratio > 1.0).mean() <= 1e-3 and ratio.max() <= 4.0, (float(ratio.max()), float((ratio > 1).mean()))
    g, w = ol.bf2f(out.to_numpy(np.uint16, (rows, H))).astype(np.float64), ol.bf2f(want).astype(np.float64)
    assert (np.abs(g - w) <= 2 * ulp_bf16(w) + 2e-3 * np.abs(w).mean()).all()
    assert np.abs(g - ol.bf2f(res)).max() > 1e-3     # the experts did contribute
    bad = lib.SbMoeExpertArgs(xd.ptr, rd.ptr, sel.ptr, wts.ptr, wg.ptr, wu.ptr, wd.ptr, scratch.ptr, out.ptr, rows, 33, H, I, lib.FMT_Q4K, total)
    assert l.sb_moe_experts(None, ctypes.byref(bad)) == -1
