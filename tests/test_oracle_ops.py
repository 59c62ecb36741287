"""CPU checks of the oracle itself: the INT8 KV quantizer against the reference's own CPU code (where the
reference shim was built), the acceptance rule on hand-made chains and trees, selection invariants, and
the oracle's linear port against its own fp64 dot products within the reference's bound."""
import ctypes

import numpy as np
import pytest

import oracle_lib as ol
import quant_fixtures as qf

P = ol.ptr


def test_kv_quantizer_matches_reference_code():
    ref = ol.load_ref()
    if ref is None:
        pytest.skip("reference shim not built (reference tree absent)")
    o = ol.bind_ops(ol.load())
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * 3, [0.0, 1e-30, -2.5, 127.0, 0.5, 1.5, 2.5]])
    for m in [0.0, 1.0, 3.7, 127.0, 1e-20, 1e20]:
        assert o.so_kv_scale(m) == ref.ref_kv_scale(m)
        for v in vals[:500]:
            v = float(np.clip(v, -m, m)) if m else float(v)
            assert o.so_kv_code(v, m) == ref.ref_kv_code(v, m)


def chain(rows):
    t = np.zeros((rows, 2), np.uint32)
    for r in range(rows):
        t[r, 0] = (1 << (r + 1)) - 1
        t[r, 1] = max(r - 1, 0) | (r << 16)
    return t


def accept(o, inputs, tree, tokens, remaining=100, stops=()):
    inputs, tokens = np.array(inputs, np.uint32), np.array(tokens, np.uint32)
    stops = np.array(stops, np.uint32)
    res = np.zeros(3, np.uint32)
    o.so_accept(P(inputs), P(tree), P(tokens), len(tokens), remaining, P(stops) if len(stops) else None, len(stops),
                P(res[0:1]), P(res[1:2]), P(res[2:3]))
    return tokens, res


def test_accept_longest_matching_prefix_of_a_chain():
    o = ol.load()
    # row r's input is the draft of position r; the target selected 10, 11, 12, 99 ...
    tokens, res = accept(o, [1, 10, 11, 12, 13, 14], chain(6), [10, 11, 12, 99, 50, 60])
    assert res[0] == 4 and res[1] == 3 and res[2] == 0b1111
    assert list(tokens[:4]) == [10, 11, 12, 99]
    # nothing matches: only the bonus token of row 0 is kept
    tokens, res = accept(o, [1, 2, 3], chain(3), [7, 8, 9])
    assert res[0] == 1 and res[1] == 0 and tokens[0] == 7
    # the lane's cap and a stop token truncate
    tokens, res = accept(o, [1, 10, 11, 12], chain(4), [10, 11, 12, 13], remaining=2)
    assert res[0] == 2 and res[1] == 2
    tokens, res = accept(o, [1, 10, 11, 12], chain(4), [10, 11, 12, 13], stops=[11])
    assert res[0] == 2 and res[1] == 2


def test_accept_follows_a_tree():
    o = ol.load()
    # rows: 0 root; 1, 2 children of 0; 3 child of 2; 4 child of 3
    tree = np.array([[0b00001, 0 | (0 << 16)], [0b00011, 0 | (1 << 16)], [0b00101, 0 | (1 << 16)],
                     [0b01101, 2 | (2 << 16)], [0b11101, 3 | (3 << 16)]], np.uint32)
    tokens, res = accept(o, [1, 20, 30, 31, 32], tree, [30, 0, 31, 32, 77])
    assert res[0] == 4 and res[1] == 3 and res[2] == 0b11101
    assert list(tokens[:4]) == [30, 31, 32, 77]


def test_selection_greedy_equals_numpy_argmax_and_rejection_sampling_statistics():
    o = ol.bind_ops(ol.load())
    rng = np.random.default_rng(2)
    rows, vocab = 8, 1000
    logits = rng.standard_normal((rows, vocab)).astype(np.float32)
    sel = np.zeros(rows, np.uint32)
    inputs = np.zeros(rows, np.uint32)
    o.so_sample_verify(P(logits), vocab, vocab, rows, P(inputs), 0.0, None, P(sel), None)
    assert np.array_equal(sel, logits.argmax(axis=1))
    # sampled: the marginal of the selected token of the last row follows softmax(l / T)
    T = 0.7
    p = np.exp((logits[-1] - logits[-1].max()) / T)
    p /= p.sum()
    counts = np.zeros(vocab)
    for i in range(3000):
        u = rng.random(80).astype(np.float32)
        o.so_sample_verify(P(logits), vocab, vocab, rows, P(inputs), T, P(u), P(sel), None)
        counts[sel[-1]] += 1
    top = np.argsort(-p)[:5]
    assert np.abs(counts[top] / 3000 - p[top]).max() < 0.03


def test_rejection_rule_keeps_the_target_distribution():
    """With a deterministic draft d: P(select d) = p(d), and P(select v != d) = p(v): rejection sampling is
    exact (sampling.metal:778-800 with q = 1)."""
    o = ol.bind_ops(ol.load())
    rng = np.random.default_rng(3)
    vocab = 50
    logits = np.tile(rng.standard_normal(vocab).astype(np.float32) * 2, (2, 1))
    p = np.exp((logits[0] - logits[0].max()) / 0.7)
    p /= p.sum()
    inputs = np.array([0, int(np.argsort(-p)[1])], np.uint32)
    sel = np.zeros(2, np.uint32)
    counts = np.zeros(vocab)
    n = 20000
    for i in range(n):
        u = rng.random(80).astype(np.float32)
        o.so_sample_verify(P(logits), vocab, vocab, 2, P(inputs), 0.7, P(u), P(sel), None)
        counts[sel[0]] += 1
    assert np.abs(counts / n - p).max() < 0.015


def _kept_set_by_sorting(l, T, min_p, top_k, top_p):
    """The distribution's end stated with a sort (order: logit descending, id ascending) and fp64 masses."""
    order = np.lexsort((np.arange(l.size), -l.astype(np.float64)))
    w = np.exp((l.astype(np.float64) - l.max()) / T)
    keep = order
    if min_p > 0:
        keep = keep[l[keep] >= np.float32(l.max() + np.float32(T) * np.float32(np.log(np.float32(min_p))))]
    if 0 < top_k < keep.size:
        keep = keep[:top_k]
    if 0 < top_p < 1:
        c = np.cumsum(w[keep])
        over = np.nonzero(c > top_p * c[-1])[0]
        if over.size:
            keep = keep[:over[0] + 1]
    return set(int(v) for v in keep)


@pytest.mark.parametrize("min_p,top_k,top_p", [(0.05, 0, 1.0), (0.0, 40, 1.0), (0.0, 0, 0.9), (0.02, 50, 0.8), (0.0, 3, 0.5)])
def test_distribution_end_equals_a_sorted_statement(min_p, top_k, top_p):
    o = ol.bind_ops(ol.load())
    rng = np.random.default_rng(11)
    rows, vocab, T = 4, 3000, 0.8
    logits = (rng.standard_normal((rows, vocab)) * 2.5).astype(np.float32)
    logits[1, 100:110] = logits[1].max()          # ties at the top, resolved by id
    logits[2, ::7] = np.float32(-np.inf)          # unselectable tokens never stay
    inputs = np.zeros(rows, np.uint32)
    u = rng.random(80).astype(np.float32)
    sel, cut = np.zeros(rows, np.uint32), np.zeros((rows, 2), np.uint32)
    o.so_sample_verify_filtered(P(logits), vocab, vocab, rows, P(inputs), T, min_p, top_k, top_p, P(u), P(sel), None, P(cut))
    for r in range(rows):
        l = logits[r]
        key = l.copy()
        key[key == 0] = 0.0
        bits = key.view(np.uint32).astype(np.uint64)
        keys = np.where(bits & 0x80000000, (~bits) & 0xFFFFFFFF, bits | 0x80000000)
        finite = np.isfinite(l) | (l == np.inf)
        kept = {int(v) for v in np.nonzero(finite & ((keys > cut[r, 0]) | ((keys == cut[r, 0]) & (np.arange(vocab) <= cut[r, 1]))))[0]}
        want = _kept_set_by_sorting(np.where(finite, l, -np.inf).astype(np.float32), T, min_p, top_k, top_p)
        want = {v for v in want if finite[v]}
        # fp32 shard sums against fp64 sums may move a nucleus by a token at most
        assert len(kept ^ want) <= (1 if 0 < top_p < 1 else 0), (r, len(kept), len(want))
        assert int(sel[r]) in kept


@pytest.mark.parametrize("fmt", [0, 4, 6])
def test_linear_port_within_projection_bound(fmt):
    o = ol.load()
    n, k, rows = 64, 1024, 4
    W = qf.realistic(fmt, n, k)
    X = qf.activations(rows, k)
    v = np.zeros((rows, n))
    be, bs = np.zeros_like(v), np.zeros_like(v)
    assert o.so_linear_f64(fmt, P(W), n, k, P(X), rows, P(v), P(be), P(bs)) == 0
    out = np.zeros((rows, n), np.float32)
    assert o.so_linear(fmt, P(W), n, k, P(X), rows, 0, None, 0, P(out), n, 1, 0) == 0
    assert (np.abs(out - v) <= be).all()
    out16 = np.zeros((rows, n), np.float32)
    assert o.so_linear(fmt, P(W), n, k, P(X), rows, 0, None, 0, P(out16), n, 1, 1) == 0
    assert (np.abs(out16 - v) <= bs).all()
    ref = ol.load_ref()
    if ref is not None:  # the bound itself against the reference's projectionBound
        w = ol.dequant(o, fmt, W, n, k)
        x = ol.bf2f(X)
        val, ex, st = ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
        ref.ref_projection(P(x[1]), P(w[5]), k, ctypes.byref(val), ctypes.byref(ex), ctypes.byref(st))
        assert np.isclose(val.value, v[1, 5]) and np.isclose(ex.value, be[1, 5]) and np.isclose(st.value, bs[1, 5])


def test_penalty_arithmetic_matches_the_reference_vectors():
    """The oracle's penalize_logit against vectors written from the reference's own host statement
    (tests/golden/make_penalty_goldens.py), bit for bit, and against that code itself where the shim is built."""
    import json
    import os
    import struct
    o = ol.bind_ops(ol.load())
    gold = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "penalty_goldens.json")))
    f = lambda b: struct.unpack("<f", struct.pack("<I", b))[0]
    bits = lambda v: struct.unpack("<I", struct.pack("<f", v))[0]
    ref = ol.load_ref()
    if ref is not None:
        ref.ref_penalty.restype = ctypes.c_float
        ref.ref_penalty.argtypes = [ctypes.c_float, ctypes.c_uint32, ctypes.c_int] + [ctypes.c_float] * 3
    assert len(gold["cases"]) >= 1000
    for vb, count, prompt, rb, pb, fb, want in gold["cases"]:
        v, rep, pres, freq = f(vb), f(rb), f(pb), f(fb)
        with np.errstate(over="ignore"):
            inverse = float(np.minimum(np.float32(1.0) / np.float32(rep), np.float32(3.402823466e38)))
        got = v if not count and not prompt else o.so_penalize_logit(v, count, rep, inverse, pres, freq)
        assert bits(got) == want or (got != got and f(want) != f(want)), (v, count, prompt, rep, pres, freq)
        if ref is not None:
            assert bits(ref.ref_penalty(v, count, prompt, rep, pres, freq)) == want or got != got


def test_penalty_pass_counts_the_path():
    """so_sample_penalize on a small tree: a row's count is the table's plus the draft tokens on its own path."""
    o = ol.bind_ops(ol.load())
    vocab, rows = 64, 4
    logits = np.ones((rows, vocab), np.float32)
    words = np.zeros(vocab, np.uint32)
    words[5] = 2                      # the output holds token 5 twice
    words[9] = 0x80000000             # the prompt holds token 9
    inputs = np.array([1, 7, 7, 5], np.uint32)
    # rows 1 and 2 are siblings under the anchor, row 3 is a child of row 1
    tree = np.array([[0b0001, 0], [0b0011, 0 | 1 << 16], [0b0101, 0 | 1 << 16], [0b1011, 1 | 2 << 16]], np.uint32)
    o.so_sample_penalize(P(logits), vocab, vocab, rows, P(words), P(inputs), P(tree), 2.0, 0.5, 0.25)
    want = np.ones((rows, vocab), np.float32)
    want[:, 9] = 0.5                                  # prompt only: repetition
    want[:, 5] = 0.5 - (0.25 * 2 + 0.5)               # the table's count
    want[3, 5] = 0.5 - (0.25 * 3 + 0.5)               # row 3 holds token 5 itself
    want[1, 7] = want[3, 7] = 0.5 - (0.25 * 1 + 0.5)  # row 1 and its child hold the first 7
    want[2, 7] = 0.5 - (0.25 * 1 + 0.5)               # row 2 holds its own 7 only
    assert np.array_equal(logits, want)


def _gdn_oracle(o, rng_seed, rows, tree=None, pending_rows=0, pending_path=0, order=None, KH=1, VH=2):
    """so_gdn_verify on seeded inputs; `order` permutes the block's rows (inputs and gates) before the call."""
    rng = np.random.default_rng(rng_seed)
    D = 128
    KW, VW = KH * D, VH * D
    C = 2 * KW + VW
    stride = C + VW
    bf = lambda shape, scale: ol.f2bf((rng.standard_normal(shape) * scale).astype(np.float32))
    qkvz, b, a = bf((16, stride), 1.0), bf((16, VH), 1.0), bf((16, VH), 1.0)
    conv_w = bf((C, 4), 0.4)
    a_scale = (-np.exp(rng.uniform(-3, 0.5, VH))).astype(np.float32)
    dt_bias, norm_w = bf((VH,), 0.5), (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    cs_in = bf((3, C), 1.0)
    state = (rng.standard_normal((VH, D, D)) * 0.05).astype(np.float32)
    pend = dict(inputs=bf((16, C), 1.0), k=bf((16, KW), 0.09), v=bf((16, VW), 0.5),
                beta=ol.f2bf(rng.uniform(0.1, 0.9, (16, VH)).astype(np.float32)), decay=rng.uniform(0.5, 1.0, (16, VH)).astype(np.float32))
    if order is not None:
        qkvz[:len(order)], b[:len(order)], a[:len(order)] = qkvz[order].copy(), b[order].copy(), a[order].copy()
    step = dict(inputs=np.zeros((16, C), np.uint16), k=np.zeros((16, KW), np.uint16), v=np.zeros((16, VW), np.uint16),
                beta=np.zeros((16, VH), np.uint16), decay=np.zeros((16, VH), np.float32))
    cs_out, state_out, hidden = np.zeros_like(cs_in), np.zeros_like(state), np.zeros((16, VW), np.uint16)
    tape = lambda t: ol.SoGdnTape(P(t["inputs"]), P(t["k"]), P(t["v"]), P(t["beta"]), P(t["decay"]))
    args = ol.SoGdnArgs(P(qkvz), P(b), P(a), P(conv_w), P(a_scale), P(dt_bias), P(norm_w), P(cs_in), P(cs_out), P(state), P(state_out),
                        tape(pend), tape(step), P(hidden), rows, pending_rows, KH, VH, stride, VH, VW, 0,
                        P(tree) if tree is not None else None, pending_path)
    o.so_gdn_verify(ctypes.byref(args))
    return dict(hidden=hidden, cs=cs_out, state=state_out, step=step)


def test_gdn_tree_rows_equal_their_paths_run_as_chains():
    """A row of a tree gives what the same row gives at the end of a chain made of its path: anchor 0, a branch
    1-2-3 and a branch 4-5 under row 1. The pending path in the tape is a row mask, folded in depth order."""
    o = ol.bind_ops(ol.load())
    parent = [0, 0, 1, 2, 1, 4]
    rows = len(parent)
    tree = np.zeros((rows, 2), np.uint32)
    for r in range(rows):
        tree[r, 0] = (1 << r) | (tree[parent[r], 0] if r else 0)
        tree[r, 1] = parent[r] | ((bin(int(tree[r, 0])).count("1") - 1) << 16)
    pending_path = 0b101001   # tape rows 0, 3, 5 of the previous step
    got = _gdn_oracle(o, 3, rows, tree=tree, pending_path=pending_path)
    for leaf in (3, 5):
        path = [r for r in range(rows) if tree[leaf, 0] >> r & 1]
        chain = _gdn_oracle(o, 3, len(path), pending_path=pending_path, order=path)
        for depth, r in enumerate(path):
            assert np.array_equal(got["hidden"][r], chain["hidden"][depth]), (leaf, r)
            assert np.array_equal(got["step"]["k"][r], chain["step"]["k"][depth])
        assert np.array_equal(got["state"], chain["state"]) and np.array_equal(got["cs"], chain["cs"])
    # a pending path that is the tape's first rows equals pending_rows
    a = _gdn_oracle(o, 5, 4, pending_rows=3)
    b = _gdn_oracle(o, 5, 4, pending_path=0b111)
    assert np.array_equal(a["hidden"], b["hidden"]) and np.array_equal(a["state"], b["state"])


def test_moe_route_is_a_stable_top_k_with_softmax_weights():
    """so_moe_route against a sorted statement: experts by descending score then ascending id, weights the softmax of
    the top_k scores (or their normalised sigmoids), the shared expert's route last."""
    o = ol.bind_ops(ol.load())
    rng = np.random.default_rng(2)
    rows, experts, slots, top_k, H = 16, 250, 256, 8, 512
    scores = rng.standard_normal((rows, slots)).astype(np.float32)
    scores[3, 10] = scores[3, 200] = scores[3, 5] = 7.0          # a three-way tie: ids 5, 10, 200 in that order
    scores[4, :] = -np.inf                                         # nothing to choose: id 0 every time
    x = ol.f2bf(rng.standard_normal((rows, H)).astype(np.float32))
    gate = (rng.standard_normal(H) * 0.1).astype(np.float32)
    for mode in (0, 1):
        sel, wts = np.zeros((rows, top_k + 1), np.uint32), np.zeros((rows, top_k + 1), np.float32)
        o.so_moe_route(P(scores), rows, experts, slots, top_k, mode, P(x), H, P(gate), P(sel), P(wts))
        for r in range(rows):
            if r == 4:
                assert (sel[r, :top_k] == 0).all()
                continue
            order = sorted(range(experts), key=lambda e: (-scores[r, e], e))[:top_k]
            assert sel[r, :top_k].tolist() == order
            s = scores[r, order].astype(np.float64)
            want = np.exp(s - s[0]) / np.exp(s - s[0]).sum() if mode == 0 else (1 / (1 + np.exp(-s))) / (1 / (1 + np.exp(-s))).sum()
            assert np.allclose(wts[r, :top_k], want, rtol=2e-6)
            assert sel[r, top_k] == experts
            assert np.isclose(wts[r, top_k], 1 / (1 + np.exp(-float(ol.bf2f(x[r]).astype(np.float64) @ gate))), rtol=1e-5)
        assert sel[3, :3].tolist() == [5, 10, 200]


def _draws_setup(o):
    import ctypes
    o.so_sample_verify_draws.argtypes = ([ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_float, ctypes.c_float,
                                          ctypes.c_uint32, ctypes.c_float] + [ctypes.c_void_p] * 6)
    return o


def test_recursive_rejection_sampling_draws_from_the_target_distribution():
    """The property the reference states for its sampled verify rows (runtime/metal/abi/Sampling.h:17-28): whatever the
    children the draft drew and whatever its probabilities q, a row's selection is a draw from the target's distribution.
    60,000 rows with fresh uniforms and fresh draws (up to 3 children drawn without replacement from q over the 16
    candidates): the selections' frequencies match softmax(logits / T) within five standard deviations."""
    o = _draws_setup(ol.bind_ops(ol.load()))
    rng = np.random.default_rng(0)
    vocab, T, N = 600, 0.7, 60000
    logits = (rng.standard_normal((1, vocab)) * 2).astype(np.float32)
    w = np.exp((logits[0].astype(np.float64) - logits[0].max()) / T)
    p = w / w.sum()
    draft = logits[0] + rng.standard_normal(vocab).astype(np.float32)          # a draft that disagrees with the target
    ids = np.argsort(-draft)[:16].astype(np.uint32)[None, :].copy()
    q = rng.dirichlet(np.ones(16)).astype(np.float32)[None, :]
    counts = np.zeros(vocab)
    sel = np.zeros(1, np.uint32)
    taken_child = 0
    for t in range(N):
        u = rng.random(80).astype(np.float32)
        order = rng.choice(16, size=3, replace=False, p=q[0].astype(np.float64) / q[0].astype(np.float64).sum())
        draws = np.full((1, 4), 255, np.uint8)
        draws[0, :3] = order
        o.so_sample_verify_draws(P(logits), vocab, vocab, 1, T, 0.0, 0, 1.0, P(u), P(ids), P(q), P(draws), P(sel), None)
        counts[sel[0]] += 1
        taken_child += int(sel[0]) in ids[0, order].tolist()
    emp = counts / N
    sigma = np.sqrt(np.maximum(p * (1 - p), 1e-12) / N)
    assert (np.abs(emp - p) <= 5 * sigma + 1e-4).all()
    assert 0.1 * N < taken_child < 0.95 * N        # children were taken often, and rejected often


def test_rejection_sampling_with_one_certain_child_is_the_chain_rule():
    """One candidate drawn with q = 1 is the chain from a deterministic draft: the row keeps the child iff u < p(child) and
    otherwise draws from the distribution without it, which is what so_sample_verify does with the next row's token."""
    o = _draws_setup(ol.bind_ops(ol.load()))
    rng = np.random.default_rng(3)
    rows, vocab, T = 16, 3000, 0.7
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    inputs = np.zeros(rows, np.uint32)
    inputs[1:] = [int(logits[r].argmax()) if rng.random() < 0.7 else int(rng.integers(0, vocab)) for r in range(rows - 1)]
    uniforms = rng.random(80).astype(np.float32)
    chain, m1 = np.zeros(rows, np.uint32), np.zeros(rows, np.float64)
    o.so_sample_verify(P(logits), vocab, vocab, rows, P(inputs), T, P(uniforms), P(chain), P(m1))
    ids = np.full((rows, 16), 0xFFFFFFFF, np.uint32)
    q = np.zeros((rows, 16), np.float32)
    draws = np.full((rows, 4), 255, np.uint8)
    ids[:-1, 0], q[:-1, 0], draws[:-1, 0] = inputs[1:], 1.0, 0
    got, m2 = np.zeros(rows, np.uint32), np.zeros(rows, np.float64)
    o.so_sample_verify_draws(P(logits), vocab, vocab, rows, T, 0.0, 0, 1.0, P(uniforms), P(ids), P(q), P(draws), P(got), P(m2))
    clear = (m1 > 1e-5) & (m2 > 1e-5)
    assert clear.sum() >= rows - 3 and np.array_equal(got[clear], chain[clear])
