"""Steps of several lanes (concurrent requests stepped together, the reference's StepRows / SplashLaneRows:
runtime/ops/LaneRows.hpp:36-62, runtime/metal/abi/VerifyTree.h:38-45): lane l's rows at 16 l of every row-indexed buffer,
per-lane state buffers arrays over the lanes. The operators with `lanes` against the same operator called a lane at a
time, and whole steps of a 4-lane target against 4 independent oracle lanes."""
import ctypes

import numpy as np
import pytest

import model_oracle as mo
import oracle_lib as ol
from test_ops_gpu import DevKv, bf16_randn, ulp_bf16

pytestmark = pytest.mark.gpu
P = ol.ptr


def _setup():
    from splash_b200 import lib
    lib.init(0)
    return lib, lib.ops(), ol.bind_ops(ol.load())


def test_gdn_lanes_equal_the_lanes_one_at_a_time():
    """3 lanes with their own cells, tapes, pending rows and row counts' worth of inputs: bit-equal to three one-lane calls."""
    lib, l, o = _setup()
    rng = np.random.default_rng(11)
    L, KH, VH, D, rows = 3, 4, 8, 128, 13
    KW, VW = KH * D, VH * D
    C = 2 * KW + VW
    stride = C + VW
    up = lib.DeviceBuffer.from_numpy
    qkvz, b, a = bf16_randn(rng, (16 * L, stride)), bf16_randn(rng, (16 * L, VH)), bf16_randn(rng, (16 * L, VH))
    conv_w, dt_bias = bf16_randn(rng, (C, 4), 0.4), bf16_randn(rng, (VH,), 0.5)
    a_scale = (-np.exp(rng.uniform(-3, 0.5, VH))).astype(np.float32)
    norm_w = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    cs_in = bf16_randn(rng, (L, 3, C))
    state = (rng.standard_normal((L, VH, D, D)) * 0.05).astype(np.float32)
    pend = dict(inputs=bf16_randn(rng, (16 * L, C)), k=bf16_randn(rng, (16 * L, KW), 0.09), v=bf16_randn(rng, (16 * L, VW), 0.5),
                beta=ol.f2bf(rng.uniform(0.1, 0.9, (16 * L, VH)).astype(np.float32)),
                decay=rng.uniform(0.5, 1.0, (16 * L, VH)).astype(np.float32))
    pending_rows = np.array([5, 0, 16], np.uint32)
    pending_path = np.zeros(L, np.uint32)
    d = {n: up(x) for n, x in dict(qkvz=qkvz, b=b, a=a, conv_w=conv_w, a_scale=a_scale, dt_bias=dt_bias, norm_w=norm_w, cs_in=cs_in,
                                   state=state, pr=pending_rows, pp=pending_path).items()}
    dp = {n: up(x) for n, x in pend.items()}
    step_shapes = dict(inputs=((16 * L, C), np.uint16), k=((16 * L, KW), np.uint16), v=((16 * L, VW), np.uint16),
                       beta=((16 * L, VH), np.uint16), decay=((16 * L, VH), np.float32))

    def run(lanes):
        ds = {n: lib.DeviceBuffer(int(np.prod(s)) * np.dtype(t).itemsize) for n, (s, t) in step_shapes.items()}
        dcs, dst, dh = lib.DeviceBuffer(cs_in.nbytes), lib.DeviceBuffer(state.nbytes), lib.DeviceBuffer(16 * L * VW * 2)
        for x in (dcs, dst, dh, *ds.values()):
            x.fill(0)

        def call(lane, n):
            off = lambda buf, per: buf.ptr + lane * per
            row = lambda buf, w, size: buf.ptr + lane * 16 * w * size
            tape = lambda t: lib.SbGdnTape(row(t["inputs"], C, 2), row(t["k"], KW, 2), row(t["v"], VW, 2), row(t["beta"], VH, 2),
                                           row(t["decay"], VH, 4))
            ga = lib.SbGdnArgs(row(d["qkvz"], stride, 2), row(d["b"], VH, 2), row(d["a"], VH, 2), d["conv_w"].ptr, d["a_scale"].ptr,
                               d["dt_bias"].ptr, d["norm_w"].ptr, off(d["cs_in"], 3 * C * 2), off(dcs, 3 * C * 2),
                               off(d["state"], VH * D * D * 4), off(dst, VH * D * D * 4), tape(dp), tape(ds), row(dh, VW, 2),
                               d["pr"].ptr + 4 * lane, rows, 0, KH, VH, stride, VH, VW, 0)
            ga.pending_path_dev = d["pp"].ptr + 4 * lane
            ga.lanes = n
            lib.check(l.sb_gdn_verify(None, ctypes.byref(ga)))

        if lanes:
            call(0, L)
        else:
            for lane in range(L):
                call(lane, 1)
        lib.stream_sync()
        assert lib.device_status() == 0
        out = dict(cs=dcs.to_numpy(np.uint16, cs_in.shape), state=dst.to_numpy(np.float32, state.shape),
                   hidden=dh.to_numpy(np.uint16, (16 * L, VW)))
        out.update({n: ds[n].to_numpy(t, s) for n, (s, t) in step_shapes.items()})
        return out

    one, many = run(False), run(True)
    for n in one:
        assert np.array_equal(one[n].view(np.uint8), many[n].view(np.uint8)), n
    assert np.abs(many["state"][1]).max() > 0 and many["hidden"][16 * 2: 16 * 2 + rows].any()


@pytest.mark.parametrize("kernel", [0, 1])
def test_attention_lanes_match_the_oracle_lane_by_lane(kernel):
    """4 lanes at positions 3000 / 17 / 1024 / 0 with their own page tables over one pool: the store bit-exact, the outputs
    within the one-lane gates, for each lane against the oracle run on that lane alone."""
    lib, l, o = _setup()
    lib.check(l.sb_set_attention_kernel(kernel))
    rng = np.random.default_rng(21)
    L, QH, KVH, D, PT, rows, pairs = 4, 8, 2, 128, 64, 16, 16
    committed = np.array([3000, 17, 1024, 0], np.uint32)
    per_lane = (int(committed.max()) + rows + PT - 1) // PT + 1
    pages = per_lane * L
    host = ol.HostKv(pages, KVH, D, PT, True)
    host.fill_random(rng)
    table = rng.permutation(pages).astype(np.uint32).reshape(L, per_lane)   # lanes' pages interleaved in the pool
    stride = QH * 2 * D + 2 * KVH * D
    qkv = bf16_randn(rng, (16 * L, stride), 1.5)
    qn, kn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32), (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    inv = (1e6 ** (-np.arange(pairs) / pairs)).astype(np.float32)
    pos = (committed[:, None] + np.arange(16)[None, :]).astype(np.uint32).reshape(-1)
    c, s = np.zeros((16 * L, pairs), np.float32), np.zeros((16 * L, pairs), np.float32)
    o.so_rope_tables(P(pos), 16 * L, P(inv), pairs, 1.0, P(c), P(s))
    dev = DevKv(lib, host)
    want_q = np.zeros((16 * L, QH, D), np.uint16)
    want = np.zeros((16 * L, QH * D), np.float64)
    desc = host.desc()
    for lane in range(L):
        r0 = 16 * lane
        q1 = np.zeros((rows, QH, D), np.uint16)
        o.so_attn_store(P(qkv[r0:]), stride, rows, QH, 1, P(qn), P(kn), P(c[r0:]), P(s[r0:]), pairs, ctypes.byref(desc),
                        P(table[lane]), int(committed[lane]), P(q1))
        w16, w64 = np.zeros((rows, QH * D), np.uint16), np.zeros((rows, QH, D), np.float64)
        o.so_attention(P(q1), P(qkv[r0:]), stride, rows, QH, 1, ctypes.byref(desc), P(table[lane]), int(committed[lane]), None,
                       P(w16), QH * D, P(w64))
        want_q[r0:r0 + rows], want[r0:r0 + rows] = q1, w64.reshape(rows, -1)
    b = {n: lib.DeviceBuffer.from_numpy(x) for n, x in dict(qkv=qkv, qn=qn, kn=kn, c=c, s=s, table=table, committed=committed).items()}
    qd, od = lib.DeviceBuffer(want_q.nbytes), lib.DeviceBuffer(16 * L * QH * D * 2)
    sa = lib.SbAttnStoreArgs(b["qkv"].ptr, b["qn"].ptr, b["kn"].ptr, b["c"].ptr, b["s"].ptr, b["table"].ptr, qd.ptr, dev.desc(lib),
                             b["committed"].ptr, rows, QH, 1, pairs, stride, int(committed.max()), L, per_lane)
    lib.check(l.sb_attn_store(None, ctypes.byref(sa)))
    aa = lib.SbAttnArgs(qd.ptr, b["qkv"].ptr, b["table"].ptr, None, od.ptr, dev.desc(lib), b["committed"].ptr, rows, QH, 1, stride,
                        QH * D, int(committed.max()), L, per_lane)
    lib.check(l.sb_attn_verify(None, ctypes.byref(aa)))
    lib.stream_sync()
    assert lib.device_status() == 0
    lib.check(l.sb_set_attention_kernel(0))
    assert np.array_equal(qd.to_numpy(np.uint16, want_q.shape), want_q)
    k, v, ks, vs = dev.download()
    assert np.array_equal(k, host.k) and np.array_equal(v, host.v) and np.array_equal(ks, host.ks) and np.array_equal(vs, host.vs)
    got = ol.bf2f(od.to_numpy(np.uint16, (16 * L, QH * D))).astype(np.float64)
    for lane in range(L):
        g, w = got[16 * lane:16 * lane + rows], want[16 * lane:16 * lane + rows]
        cos = (g * w).sum() / np.sqrt((g * g).sum() * (w * w).sum())
        assert cos > 0.9995 and np.abs(g - w).max() < max(0.02, 4e-3 * np.abs(w).max()), lane


def test_selection_penalties_and_acceptance_of_lanes_equal_the_lanes_one_at_a_time():
    lib, l, o = _setup()
    rng = np.random.default_rng(31)
    L, rows, V = 5, 9, 6000
    logits = (rng.standard_normal((16 * L, V)) * 3).astype(np.float32)
    tokens = rng.integers(0, V, 16 * L).astype(np.uint32)
    for lane in range(L):                      # lane `lane` accepts `lane` draft tokens when greedy
        for r in range(min(lane, rows - 1)):
            tokens[16 * lane + r + 1] = np.argmax(logits[16 * lane + r])
    uniforms = rng.random(80 * L).astype(np.float32)
    words = rng.integers(0, 3, (L, V)).astype(np.uint32) * (rng.random((L, V)) < 0.05)
    tree = np.tile(lib.chain_tree(16), (L, 1))
    up = lib.DeviceBuffer.from_numpy

    def run(lanes, temperature):
        dl, dt, du, dw, dtree = up(logits), up(tokens), up(uniforms), up(words), up(tree)
        sel, res = lib.DeviceBuffer(16 * L * 4), lib.DeviceBuffer(16 * L)
        ws = lib.DeviceBuffer(int(l.sb_sample_workspace_bytes(16 * L, V)))
        sel.fill(0), res.fill(0)

        def call(lane, n):
            r4 = 16 * lane * 4
            pa = lib.SbPenaltyArgs(dl.ptr + r4 * V, dw.ptr + lane * V * 4, dt.ptr + r4, dtree.ptr + 16 * lane * 8, rows, V, V, 1.2, 0.3, 0.1)
            pa.lanes = n
            lib.check(l.sb_sample_penalize(None, ctypes.byref(pa)))
            sa = lib.SbSampleArgs(dl.ptr + r4 * V, dt.ptr + r4, du.ptr + 80 * lane * 4 if temperature else None, sel.ptr + r4, ws.ptr,
                                  rows, V, V, temperature, 0.0, 0, 1.0)
            sa.lanes = n
            lib.check(l.sb_sample_verify(None, ctypes.byref(sa)))
            aa = lib.SbAcceptArgs(dt.ptr + r4, dtree.ptr + 16 * lane * 8, sel.ptr + r4, res.ptr + 16 * lane, None, rows, 16, 0)
            aa.lanes = n
            lib.check(l.sb_accept(None, ctypes.byref(aa)))

        if lanes:
            call(0, L)
        else:
            for lane in range(L):
                call(lane, 1)
        lib.stream_sync()
        assert lib.device_status() == 0
        return dl.to_numpy(np.float32, logits.shape), sel.to_numpy(np.uint32, (L, 16)), res.to_numpy(np.uint32, (L, 4))

    for temperature in (0.0, 0.8):
        one, many = run(False, temperature), run(True, temperature)
        for x, y in zip(one, many):
            assert np.array_equal(x.view(np.uint32), y.view(np.uint32))
    greedy = run(True, 0.0)[2]
    assert len(set(greedy[:, 0].tolist())) >= 3          # the lanes did accept different lengths


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_selection_and_acceptance_in_one_launch_equal_the_two_calls(temperature):
    """sb_select_accept against sb_sample_verify followed by sb_accept on the same lanes, bit for bit, over repeated launches
    (the ticket words return to zero), and the lanes' commit in each of its modes."""
    lib, l, o = _setup()
    rng = np.random.default_rng(41)
    L, rows, V = 5, 9, 6000
    logits = (rng.standard_normal((16 * L, V)) * 3).astype(np.float32)
    tokens = rng.integers(0, V, 16 * L).astype(np.uint32)
    for lane in range(L):
        for r in range(min(lane, rows - 1)):
            tokens[16 * lane + r + 1] = np.argmax(logits[16 * lane + r])
    uniforms = rng.random(80 * L).astype(np.float32)
    tree = np.tile(lib.chain_tree(16), (L, 1))
    up = lib.DeviceBuffer.from_numpy
    dl, dt, du, dtree = up(logits), up(tokens), up(uniforms), up(tree)
    ws = lib.DeviceBuffer(int(l.sb_sample_workspace_bytes(16 * L, V)))

    def args(sel, res):
        sa = lib.SbSampleArgs(dl.ptr, dt.ptr, du.ptr if temperature else None, sel.ptr, ws.ptr, rows, V, V, temperature, 0.0, 0, 1.0)
        sa.lanes = L
        aa = lib.SbAcceptArgs(dt.ptr, dtree.ptr, sel.ptr, res.ptr, None, rows, 16, 0)
        aa.lanes = L
        return sa, aa

    sel, res = lib.DeviceBuffer(16 * L * 4), lib.DeviceBuffer(16 * L)
    sel.fill(0), res.fill(0)
    sa, aa = args(sel, res)
    lib.check(l.sb_sample_verify(None, ctypes.byref(sa)))
    lib.check(l.sb_accept(None, ctypes.byref(aa)))
    lib.stream_sync()
    want_sel, want_res = sel.to_numpy(np.uint32, (L, 16)), res.to_numpy(np.uint32, (L, 4))

    tickets = lib.DeviceBuffer(4 * L)
    tickets.fill(0)
    committed0 = np.array([100, 200, 300, 400, 500], np.uint32)
    for advance in (None, 1, 0, 2, 3 | rows << 8):
        sel2, res2 = lib.DeviceBuffer(16 * L * 4), lib.DeviceBuffer(16 * L)
        sel2.fill(0), res2.fill(0)
        committed, pending_rows, pending_path = up(committed0), up(np.full(L, 7, np.uint32)), up(np.full(L, 0x55, np.uint32))
        c = lib.SbSelectAcceptArgs()
        c.sample, c.accept = args(sel2, res2)
        c.tickets = tickets.ptr
        if advance is not None:
            c.committed, c.pending_rows, c.pending_path, c.advance = committed.ptr, pending_rows.ptr, pending_path.ptr, advance
        for repeat in range(3):
            if repeat and advance is not None:
                break                                         # (a commit moves the lane: once)
            lib.check(l.sb_select_accept(None, ctypes.byref(c)))
        lib.stream_sync()
        assert lib.device_status() == 0
        assert not tickets.to_numpy(np.uint32, (L,)).any()
        got_sel, got_res = sel2.to_numpy(np.uint32, (L, 16)), res2.to_numpy(np.uint32, (L, 4))
        got = committed.to_numpy(np.uint32, (L,)), pending_rows.to_numpy(np.uint32, (L,)), pending_path.to_numpy(np.uint32, (L,))
        if advance == (3 | rows << 8):
            assert np.array_equal(got_res, np.tile(np.array([rows, rows - 1, (1 << rows) - 1, 0], np.uint32), (L, 1)))
            assert np.array_equal(got[0], committed0 + rows) and (got[1] == rows).all() and (got[2] == 0).all()
            continue
        assert np.array_equal(got_sel, want_sel) and np.array_equal(got_res, want_res)
        if advance is None or advance == 2:
            assert np.array_equal(got[0], committed0) and (got[1] == 7).all() and (got[2] == 0x55).all()
        elif advance == 1:
            assert np.array_equal(got[0], committed0 + want_res[:, 0]) and np.array_equal(got[1], want_res[:, 0]) and np.array_equal(got[2], want_res[:, 2])
        else:
            assert np.array_equal(got[0], committed0) and not got[1].any() and not got[2].any()
    # what the call refuses: acceptance over other rows than the selection's, no tickets
    c = lib.SbSelectAcceptArgs()
    c.sample, c.accept = args(sel, res)
    assert l.sb_select_accept(None, ctypes.byref(c)) == -1
    c.tickets = tickets.ptr
    c.accept.rows = rows - 1
    assert l.sb_select_accept(None, ctypes.byref(c)) == -1


@pytest.mark.parametrize("rows,n,k", [(200, 256, 2048), (512, 64, 1024), (17, 48, 512), (40, 32, 384)])
def test_float_projection_of_many_rows_keeps_fp32_accuracy(rows, n, k):
    """sb_linear_f32 over more than 16 rows runs on the tensor cores with the fp32 weights split into three bf16 terms:
    against fp64 it stays at fp32 accuracy (the router's scores decide routes)."""
    lib, l, o = _setup()
    rng = np.random.default_rng(rows)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = bf16_randn(rng, (rows, k), 2.0)
    wd, xd, od = lib.DeviceBuffer.from_numpy(w), lib.DeviceBuffer.from_numpy(x), lib.DeviceBuffer(rows * n * 4)
    lib.check(l.sb_linear_f32(None, wd.ptr, xd.ptr, rows, n, k, k, od.ptr, n, 1, None))
    lib.stream_sync()
    got = od.to_numpy(np.float32, (rows, n)).astype(np.float64)
    xf = ol.bf2f(x).astype(np.float64)
    want = xf @ w.astype(np.float64).T
    bound = 2.0 ** -20 * (np.abs(xf) @ np.abs(w.astype(np.float64)).T)      # fp32 sums of exact products (the tensor cores' additions truncate)
    assert (np.abs(got - want) <= bound + 1e-30).all(), float((np.abs(got - want) / bound).max())


@pytest.mark.parametrize("shape", [
    dict(rows=200, experts=24, slots=32, top_k=8, H=1024, I=512),     # about 67 routes an expert; the shared expert's 200 rows are two groups
    dict(rows=128, experts=256, slots=256, top_k=8, H=2048, I=512),   # the 35B-A3B block at 8 lanes: about 4 routes an expert
    dict(rows=40, experts=8, slots=8, top_k=2, H=512, I=256),         # ragged groups, experts that may stay empty
])
def test_moe_experts_of_many_rows_grouped_by_expert_match_oracle(shape):
    """sb_moe_experts with more than 16 rows: routes grouped by expert, each group's rows gathered and multiplied on the
    many-row kernel, combined in slot order. Against the oracle's statement of the block, the bound as for 16 rows with the
    weights rounded to half on top."""
    lib, l, o = _setup()
    rng = np.random.default_rng(23)
    rows, experts, slots, top_k, H, I = (shape[n] for n in ("rows", "experts", "slots", "top_k", "H", "I"))
    total, routes = experts + 1, top_k + 1
    import quant_fixtures as qf
    gate = np.concatenate([qf.realistic(0, I, H, seed=100 + e) for e in range(total)])
    up = np.concatenate([qf.realistic(0, I, H, seed=200 + e) for e in range(total)])
    down = np.concatenate([qf.realistic(0, H, I, seed=300 + e) for e in range(total)])
    x = ol.f2bf(rng.standard_normal((rows, H)).astype(np.float32))
    res = ol.f2bf(rng.standard_normal((rows, H)).astype(np.float32))
    scores = rng.standard_normal((rows, slots)).astype(np.float32)
    sgate = (rng.standard_normal(H) * 0.05).astype(np.float32)
    selected, weights = np.zeros((rows, routes), np.uint32), np.zeros((rows, routes), np.float32)
    o.so_moe_route(P(scores), rows, experts, slots, top_k, 0, P(x), H, P(sgate), P(selected), P(weights))
    up_dev = lib.DeviceBuffer.from_numpy
    xd, rd, sel, wts = up_dev(x), up_dev(res), up_dev(selected), up_dev(weights)
    wg, wu, wd = up_dev(gate), up_dev(up), up_dev(down)
    scratch = lib.DeviceBuffer(int(l.sb_moe_scratch_bytes(rows, routes, H, I)))
    out = lib.DeviceBuffer(rows * H * 2 + 256)
    out.fill(0xFF)
    ea = lib.SbMoeExpertArgs(xd.ptr, rd.ptr, sel.ptr, wts.ptr, wg.ptr, wu.ptr, wd.ptr, scratch.ptr, out.ptr, rows, routes, H, I, lib.FMT_Q4K, total)
    for _ in range(2):   # (a second call over the same scratch gives the same rows)
        lib.check(l.sb_moe_experts(None, ctypes.byref(ea)))
    lib.stream_sync()
    assert lib.device_status() == 0
    want = np.zeros((rows, H), np.uint16)
    assert o.so_moe_experts(P(x), P(res), P(selected), P(weights), P(gate), P(up), P(down), rows, routes, H, I, total, P(want), None) == 0
    g, w = ol.bf2f(out.to_numpy(np.uint16, (rows, H))).astype(np.float64), ol.bf2f(want).astype(np.float64)
    err = np.abs(g - w)
    assert (err <= 3 * ulp_bf16(w) + 4e-3 * np.abs(w).mean()).all(), float((err / (ulp_bf16(w) + 1e-3 * np.abs(w).mean())).max())
    assert np.median(err) <= 2e-3 * np.abs(w).mean()
    assert np.abs(g - ol.bf2f(res)).max() > 1e-3     # the experts did contribute


def build_lanes(lanes, positions, seed=0, **more):
    from splash_b200 import lib, target
    lib.init(0)
    cfg = dict(target.TINY, lanes=lanes, **more)     # (Q4_K projections, Q6_K head: the head runs from its image)
    t = target.Target(**cfg)
    w = mo.make_weights(cfg, seed)
    states = [mo.make_state(cfg, int(positions[i]), seed + 1 + i) for i in range(lanes)]
    for i, s in enumerate(states):
        mo.upload(t, w if i == 0 else {}, s, lane=i)
    t.reset_lanes(positions)
    return lib, target, t, cfg, w, states


@pytest.mark.parametrize("flags_name", ["eager", "graph"])
def test_tiny_model_of_four_lanes_matches_four_oracle_lanes(flags_name):
    """4 lanes at different positions, drafts of different quality (so unequal accept lengths), 3 committed steps. Per
    lane: logits within the many-row kernel's distance of the oracle's (weights and inputs rounded to half there), and the
    retained tokens, accept length and path equal wherever the top-2 gap of the retained rows exceeds that distance."""
    positions = np.array([2048, 300, 1537, 1000], np.uint32)
    lib, target, t, cfg, w, states = build_lanes(4, positions)
    flags = target.ADVANCE | (target.GRAPH if flags_name == "graph" else 0)
    match = [0.95, 0.3, 0.7, 0.0]
    first = [17, 400, 9000, 31999]
    compared, lengths = 0, []
    for step in range(3):
        blocks = np.stack([mo.draft_chain(cfg, w, states[i], first[i], rows=16, p_match=match[i], seed=10 * step + i) for i in range(4)])
        wants = [mo.verify_step(cfg, w, states[i], blocks[i], advance=True) for i in range(4)]
        got = t.verify_lanes(blocks, flags=flags)
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (64, cfg["vocab"]))
        for i in range(4):
            want, (tokens, retained, accepted, mask) = wants[i], got[i]
            mine = logits[16 * i:16 * i + 16]
            scale = np.abs(want["logits"]).max()
            err = np.abs(mine - want["logits"])
            assert err.max() <= 2e-2 * scale and np.median(err) <= 2e-3 * scale, (step, i)
            top2 = np.sort(want["logits"], axis=1)[:, -2:]
            clear = (top2[:, 1] - top2[:, 0]) > 2.5 * err.max(axis=1)
            if clear[:want["retained"]].all():
                assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"]), (step, i)
                assert np.array_equal(tokens, want["tokens"]), (step, i)
                compared += 1
                lengths.append(retained)
            else:  # follow the device where the oracle's own choice was a near tie
                states[i]["committed"] += retained - want["retained"]
                states[i]["pending_rows"] = retained
            first[i] = int(tokens[-1])
    assert compared >= 9 and len(set(lengths)) >= 3, (compared, lengths)


def test_tiny_moe_model_of_three_lanes_matches_three_oracle_lanes():
    """MoE feed-forward blocks (16 experts + the shared one, top 4, expert width 256) under several lanes: the 48 rows' routes
    grouped by expert inside whole steps."""
    positions = np.array([2048, 700, 1300], np.uint32)
    lib, target, t, cfg, w, states = build_lanes(3, positions, seed=5, moe_experts=16, moe_top_k=4, moe_intermediate=256)
    first, compared = [31, 77, 4000], 0
    for step in range(2):
        blocks = np.stack([mo.draft_chain(cfg, w, states[i], first[i], rows=16, p_match=0.6, seed=10 * step + i) for i in range(3)])
        wants = [mo.verify_step(cfg, w, states[i], blocks[i], advance=True) for i in range(3)]
        got = t.verify_lanes(blocks, flags=target.ADVANCE | target.GRAPH)
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (48, cfg["vocab"]))
        for i in range(3):
            want, (tokens, retained, accepted, mask) = wants[i], got[i]
            err = np.abs(logits[16 * i:16 * i + 16] - want["logits"])
            scale = np.abs(want["logits"]).max()
            assert err.max() <= 3e-2 * scale and np.median(err) <= 2e-3 * scale, (step, i)
            top2 = np.sort(want["logits"], axis=1)[:, -2:]
            if ((top2[:, 1] - top2[:, 0]) > 2.5 * err.max(axis=1))[:want["retained"]].all():
                assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"]), (step, i)
                assert np.array_equal(tokens, want["tokens"]), (step, i)
                compared += 1
            else:
                states[i]["committed"] += retained - want["retained"]
                states[i]["pending_rows"] = retained
            first[i] = int(tokens[-1])
    assert compared >= 4, compared


def test_prompt_blocks_of_two_lanes_match_two_oracle_lanes():
    """Two lanes take prompt blocks (every row committed) from different positions, then one verify step."""
    positions = np.array([0, 700], np.uint32)
    lib, target, t, cfg, w, states = build_lanes(2, positions, seed=6)
    rng = np.random.default_rng(12)

    def close(i, want, logits):
        mine = logits[16 * i:16 * i + len(want["logits"])]
        scale = np.abs(want["logits"]).max()
        err = np.abs(mine - want["logits"])
        assert err.max() <= 2e-2 * scale and np.median(err) <= 2e-3 * scale, i

    last = [0, 0]
    for rows in (16, 16, 5):
        blocks = rng.integers(0, cfg["vocab"], (2, rows)).astype(np.uint32)
        wants = [mo.verify_step(cfg, w, states[i], blocks[i], advance=True, prompt=True) for i in range(2)]
        got = t.verify_lanes(blocks, flags=target.ADVANCE | target.PROMPT)
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (32, cfg["vocab"]))
        for i in range(2):
            assert got[i][1:] == (rows, rows - 1, (1 << rows) - 1)
            close(i, wants[i], logits)
            last[i] = int(got[i][0][rows - 1])
    assert np.array_equal(t.download(-1, "committed", np.uint32, (2,)), positions + 37)
    blocks = np.stack([mo.draft_chain(cfg, w, states[i], last[i], rows=16, p_match=0.6, seed=i) for i in range(2)])
    wants = [mo.verify_step(cfg, w, states[i], blocks[i], advance=True) for i in range(2)]
    t.verify_lanes(blocks, flags=target.ADVANCE)
    logits = t.download(-1, "logits", np.float32, (32, cfg["vocab"]))
    for i in range(2):
        close(i, wants[i], logits)


def _tree_rows(parent):
    t = np.zeros((len(parent), 2), np.uint32)
    for r in range(len(parent)):
        t[r, 0] = (1 << r) | (t[parent[r], 0] if r else 0)
        t[r, 1] = parent[r] | ((bin(int(t[r, 0])).count("1") - 1) << 16)
    return t


def test_tiny_model_tree_blocks_of_two_lanes_match_two_oracle_lanes():
    """Every lane its own tree of draft tokens, two committed steps: positions by depth, attention and GDN along each row's
    path, the accepted path's KV rows moved to their depths per lane, the next step folding each lane's accepted path."""
    positions = np.array([2048, 900], np.uint32)
    lib, target, t, cfg, w, states = build_lanes(2, positions, seed=9)
    parents = [[0, 0, 1, 2, 0, 4, 5, 6, 6, 8, 9, 10, 9, 12, 0, 14], [0, 0, 0, 1, 1, 2, 3, 3, 5, 5, 8, 8, 10, 11, 12, 13]]
    goods = [[4, 5, 6, 8, 9, 12, 13], [2, 5, 9]]      # rows along which the draft matches the target (a path of each tree)
    first, compared = [17, 4000], 0
    for step in range(2):
        blocks, trees = [], []
        for i in range(2):
            good = goods[i]
            greedy = mo.draft_chain(cfg, w, states[i], first[i], rows=len(good) + 1, p_match=1.0, seed=step)
            tokens = np.random.default_rng(8 + i + 2 * step).integers(0, cfg["vocab"], 16).astype(np.uint32)
            tokens[0] = first[i]
            tokens[good] = greedy[1:]
            blocks.append(tokens), trees.append(_tree_rows(parents[i]))
        wants = [mo.verify_step(cfg, w, states[i], blocks[i], advance=True, tree=trees[i]) for i in range(2)]
        got = t.verify_lanes(np.stack(blocks), flags=target.ADVANCE | target.GRAPH, trees=np.stack(trees))
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (32, cfg["vocab"]))
        for i in range(2):
            want, (tokens, retained, accepted, mask) = wants[i], got[i]
            err = np.abs(logits[16 * i:16 * i + 16] - want["logits"])
            scale = np.abs(want["logits"]).max()
            assert err.max() <= 3e-2 * scale and np.median(err) <= 2e-3 * scale, (step, i)
            top2 = np.sort(want["logits"], axis=1)[:, -2:]
            on_path = [r for r in range(16) if want["mask"] >> r & 1]
            assert ((top2[:, 1] - top2[:, 0]) > 2.5 * err.max(axis=1))[on_path].all(), "a near tie on the accepted path: pick another seed"
            assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"]), (step, i)
            assert np.array_equal(tokens, want["tokens"]), (step, i)
            compared += 1
            first[i] = int(tokens[-1])
    assert compared == 4 and wants[0]["accepted"] >= 3


def test_lane_of_a_four_lane_step_does_not_depend_on_the_other_lanes():
    """The same lane 2 next to different neighbours: its logits and results are bit-equal."""
    positions = np.array([2048, 300, 1537, 1000], np.uint32)
    lib, target, t, cfg, w, states = build_lanes(4, positions, seed=3)
    rng = np.random.default_rng(5)
    blocks = rng.integers(0, cfg["vocab"], (4, 16)).astype(np.uint32)
    a = t.verify_lanes(blocks)
    la = t.download(-1, "logits", np.float32, (64, cfg["vocab"]))[32:48].copy()
    blocks2 = rng.integers(0, cfg["vocab"], (4, 16)).astype(np.uint32)
    blocks2[2] = blocks[2]
    t.reset_lanes(np.array([100, 2048, 1537, 5], np.uint32))   # (the furthest lane as before: the same split plan)
    b = t.verify_lanes(blocks2)
    lb = t.download(-1, "logits", np.float32, (64, cfg["vocab"]))[32:48]
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    assert a[2][1:] == b[2][1:] and np.array_equal(a[2][0], b[2][0])


def test_tiny_nvfp4_model_steps_match_oracle():
    """One lane with NVFP4 projections (Q6_K embedding): every projection runs on the many-row kernel from its image."""
    from splash_b200 import lib, target
    lib.init(0)
    cfg = dict(target.TINY, fmt_proj=lib.FMT_NVFP4, fmt_down=lib.FMT_NVFP4, fmt_head=lib.FMT_NVFP4)
    t = target.Target(**cfg)
    w = mo.make_weights(cfg, 2)
    s = mo.make_state(cfg, 2048, 3)
    mo.upload(t, w, s)
    t.reset(2048)
    token, compared = 5, 0
    for step in range(3):
        tokens = mo.draft_chain(cfg, w, s, token, rows=16, seed=step)
        want = mo.verify_step(cfg, w, s, tokens, advance=True)
        got_tokens, retained, accepted, mask = t.verify(tokens, flags=target.ADVANCE | target.GRAPH)
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
        scale = np.abs(want["logits"]).max()
        err = np.abs(logits - want["logits"])
        assert err.max() <= 3e-2 * scale and np.median(err) <= 2e-3 * scale, step
        top2 = np.sort(want["logits"], axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 2.5 * err.max(axis=1)
        if clear[:want["retained"]].all():
            assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"]), step
            assert np.array_equal(got_tokens, want["tokens"]), step
            compared += 1
        else:
            s["committed"] += retained - want["retained"]
            s["pending_rows"] = retained
        token = int(got_tokens[-1])
    assert compared >= 2


def test_lanes_reject_what_they_do_not_step():
    from splash_b200 import lib, target
    lib.init(0)
    with pytest.raises(lib.SbError):
        target.Target(**dict(target.TINY, fmt_down=lib.FMT_BF16, lanes=4))    # plain rows are not a projection format
    with pytest.raises(lib.SbError):
        target.Target(**dict(target.TINY, lanes=33))
    t = target.Target(**dict(target.TINY, lanes=2))
    with pytest.raises(lib.SbError):
        t.verify(np.arange(16, dtype=np.uint32))                             # the one-lane entry


def test_admission_of_lanes_equals_the_oracles():
    """sb_sample_admit on the rows of several lanes in one launch: the logits bit for bit what the oracle's pass leaves lane by lane
    (constraint masks with and without excluded tokens), then greedy selections that respect them."""
    lib, l, o = _setup()
    o.so_sample_admit.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32,
                                  ctypes.c_void_p, ctypes.c_uint32]
    rng = np.random.default_rng(51)
    L, rows, V = 3, 11, 5003
    words = (V + 31) // 32
    logits = rng.standard_normal((16 * L, V)).astype(np.float32)
    masks = rng.integers(0, 2 ** 32, (16 * L, words), dtype=np.uint64).astype(np.uint32)
    masks[16 + 2] = 0                                     # a row of lane 1 that admits nothing
    excluded = np.array([7, int(np.argmax(logits[0])), V - 1], np.uint32)
    up = lib.DeviceBuffer.from_numpy
    for use_masks, use_excluded in ((True, True), (True, False), (False, True)):
        dl, dm, de = up(logits), up(masks), up(excluded)
        a = lib.SbAdmitArgs(dl.ptr, dm.ptr if use_masks else None, de.ptr if use_excluded else None, rows, V, V, words, 3 if use_excluded else 0, L)
        lib.check(l.sb_sample_admit(None, ctypes.byref(a)))
        lib.stream_sync()
        got = dl.to_numpy(np.float32, logits.shape)
        want = logits.copy()
        for lane in range(L):
            block = want[16 * lane:16 * lane + rows]
            o.so_sample_admit(P(block), V, V, rows, P(np.ascontiguousarray(masks[16 * lane:16 * lane + rows])) if use_masks else None, words,
                              P(excluded) if use_excluded else None, 3 if use_excluded else 0)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        assert np.array_equal(got[rows:16], logits[rows:16])          # the slots past the lane's rows stay as they were
        sel = lib.DeviceBuffer(16 * L * 4)
        sel.fill(0)
        sa = lib.SbSampleArgs(dl.ptr, up(np.zeros(16 * L, np.uint32)).ptr, None, sel.ptr, None, rows, V, V, 0.0, 0.0, 0, 1.0)
        sa.lanes = L
        lib.check(l.sb_sample_verify(None, ctypes.byref(sa)))
        lib.stream_sync()
        chosen = sel.to_numpy(np.uint32, (L, 16))
        for lane in range(L):
            for r in range(rows):
                t = int(chosen[lane, r])
                if use_masks and lane == 1 and r == 2:
                    assert t == 0xffffffff
                    continue
                assert not use_masks or (masks[16 * lane + r, t // 32] >> (t % 32)) & 1
                assert not use_excluded or t not in excluded
    bad = lib.SbAdmitArgs(dl.ptr, None, None, rows, V, V, words, 0, L)
    assert l.sb_sample_admit(None, ctypes.byref(bad)) == -1               # neither masks nor excluded tokens
    bad = lib.SbAdmitArgs(dl.ptr, dm.ptr, None, rows, V, V, words - 1, 0, L)
    assert l.sb_sample_admit(None, ctypes.byref(bad)) == -1               # mask rows too short for the vocabulary


@pytest.mark.parametrize("flags_name", ["eager", "graph"])
def test_lanes_select_each_by_its_own_policy(flags_name):
    """A greedy lane beside two sampled ones with different temperatures and ends of the distribution, in one step; then other
    policies without a new capture (the values are read on the device). Each lane against the oracle's lane with its policy,
    wherever no test or cut sat within rounding of its threshold."""
    positions = np.array([900, 40, 1500], np.uint32)
    lib, target, t, cfg, w, states = build_lanes(3, positions, seed=8)
    flags = target.GRAPH if flags_name == "graph" else 0
    rng = np.random.default_rng(77)
    compared = 0
    for policies in ([(0.0, 0.0, 0, 1.0), (0.8, 0.0, 10, 1.0), (1.2, 0.05, 0, 1.0)], [(1.0, 0.0, 20, 0.95), (0.0, 0.0, 0, 1.0), (0.6, 0.0, 0, 0.9)]):
        t.set_lane_policies(policies)
        for trial in range(3):
            blocks = np.stack([mo.draft_chain(cfg, w, states[i], 5 + i, rows=16, p_match=0.8, seed=10 * trial + i) for i in range(3)])
            uniforms = rng.random((3, 80)).astype(np.float32)
            wants = [mo.verify_step(cfg, w, states[i], blocks[i], temperature=policies[i][0], uniforms=uniforms[i], mutate=False,
                                    policy=policies[i][1:]) for i in range(3)]
            got = t.verify_lanes(blocks, uniforms=uniforms, flags=flags)
            assert lib.device_status() == 0
            logits = t.download(-1, "logits", np.float32, (48, cfg["vocab"]))
            for i in range(3):
                want, (tokens, retained, accepted, mask) = wants[i], got[i]
                if policies[i][0] == 0.0:
                    err = np.abs(logits[16 * i:16 * i + 16] - want["logits"]).max(axis=1)
                    top2 = np.sort(want["logits"], axis=1)[:, -2:]
                    clear = ((top2[:, 1] - top2[:, 0]) > 2.5 * err)[:want["retained"]].all()
                else:
                    clear = (want["margin"][:want["retained"]] > 1e-3).all()
                if not clear:
                    continue
                compared += 1
                assert (retained, accepted) == (want["retained"], want["accepted"]), (policies[i], trial, i)
                assert np.array_equal(tokens, want["tokens"]), (policies[i], trial, i)
    assert compared >= 12, compared
    t.set_lane_policies(None)
    with pytest.raises(lib.SbError):
        t.set_lane_policies([(1.0, 0.0, 0, 1.0), (1.0, 2.0, 0, 1.0), (1.0, 0.0, 0, 1.0)])     # min_p above 1


@pytest.mark.parametrize("flags_name", ["eager", "graph"])
def test_lanes_step_together_with_blocks_of_different_lengths(flags_name):
    """Blocks of 16, 5 and 0 rows in one step, then of 3, 16 and 9: every lane selects, accepts and commits among its own rows
    (the slots past them hold tokens that would have been accepted had they counted), a lane without rows sits the step out
    with its position and state intact. Each lane against the oracle's lane stepped with its own block."""
    positions = np.array([1200, 64, 500], np.uint32)
    lib, target, t, cfg, w, states = build_lanes(3, positions, seed=10)
    flags = target.ADVANCE | (target.GRAPH if flags_name == "graph" else 0)
    first = [17, 400, 9000]
    compared = 0
    for step, lengths in enumerate(([16, 5, 0], [3, 16, 9], [16, 16, 16])):
        full = [mo.draft_chain(cfg, w, states[i], first[i], rows=16, p_match=1.0, seed=7 * step + i) for i in range(3)]   # all would be accepted
        blocks = [full[i][:lengths[i]] for i in range(3)]
        wants = []
        for i in range(3):
            if lengths[i]:
                wants.append(mo.verify_step(cfg, w, states[i], blocks[i], advance=True))
            else:   # a lane that sits out: its pending rows are folded, nothing is committed (a held step in the oracle)
                wants.append(mo.verify_step(cfg, w, states[i], full[i], advance=False))
        # the device's slots past a lane's rows hold the rest of the chain: tokens that match the target's own selections
        slots = np.stack(full)
        got = t.verify_lanes_ragged([slots[i][:lengths[i]] for i in range(3)], flags=flags) if step != 1 else None
        if got is None:   # (the same through explicit slots: the tokens past the lanes' rows are there, and ignored)
            out_t, out_r = np.zeros((3, 16), np.uint32), np.zeros((3, 4), np.uint32)
            rows = np.array(lengths, np.uint32)
            P_ = ctypes.c_void_p
            t.l.sb_target_verify_lanes_ragged.argtypes = [P_, P_, P_, P_, P_, ctypes.c_float, ctypes.c_uint32, P_, P_]
            lib.check(t.l.sb_target_verify_lanes_ragged(t.handle, None, slots.ctypes.data_as(P_), None, rows.ctypes.data_as(P_), 0.0, flags,
                                                        out_t.ctypes.data_as(P_), out_r.ctypes.data_as(P_)))
            got = [(out_t[l, :out_r[l, 0]].copy(), int(out_r[l, 0]), int(out_r[l, 1]), int(out_r[l, 2])) for l in range(3)]
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (48, cfg["vocab"]))
        for i in range(3):
            tokens, retained, accepted, mask = got[i]
            if not lengths[i]:
                assert (retained, accepted, mask) == (0, 0, 0) and len(tokens) == 0
                continue
            want = wants[i]
            assert retained <= lengths[i]
            mine = logits[16 * i:16 * i + lengths[i]]
            scale = np.abs(want["logits"]).max()
            err = np.abs(mine - want["logits"])
            assert err.max() <= 2e-2 * scale and np.median(err) <= 2e-3 * scale, (step, i)
            top2 = np.sort(want["logits"], axis=1)[:, -2:]
            if ((top2[:, 1] - top2[:, 0]) > 2.5 * err.max(axis=1))[:want["retained"]].all():
                assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"]), (step, i)
                assert np.array_equal(tokens, want["tokens"]), (step, i)
                compared += 1
            else:
                states[i]["committed"] += retained - want["retained"]
                states[i]["pending_rows"] = retained
            first[i] = int(tokens[-1])
        committed = t.download(-1, "committed", np.uint32, (3,))
        assert [int(c) for c in committed] == [states[i]["committed"] for i in range(3)], step
    assert compared >= 6, compared
    # a request that may take two more tokens retains two, however many its block would give
    t.upload(-1, "remaining", np.array([2, 0xffffffff, 1], np.uint32))
    full = [mo.draft_chain(cfg, w, states[i], first[i], rows=16, p_match=1.0, seed=90 + i) for i in range(3)]
    got = t.verify_lanes(np.stack(full), flags=flags)
    assert got[0][1] <= 2 and got[2][1] == 1 and got[1][1] >= got[0][1]
    t.upload(-1, "remaining", np.full(3, 0xffffffff, np.uint32))
