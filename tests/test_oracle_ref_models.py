"""The oracle's attention, GDN and sampled-selection restatements against the reference's own fp64 CPU models
(dev/tests/engine/q8_flash_attention_metal_test.mm cpuReference, dev/tests/engine/gdn_decode_metal_test.mm
convolutionSilu / normalizedHead / recurrence, dev/tests/engine/target_sampling_metal_test.mm
referenceDistribution / referenceSelection), compiled from the reference tree into
oracle/_ref/libsplash_ref_models.so by `make -C oracle ref`. Skipped where that library was not built.
The tolerances are the ones the reference's tests give their kernels against these models."""
import ctypes
import os

import numpy as np
import pytest

import oracle_lib as ol

P = ol.ptr
_U, _V = ctypes.c_uint32, ctypes.c_void_p


def _models():
    path = os.path.join(ol.ORACLE_DIR, "_ref", "libsplash_ref_models.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libsplash_ref_models.so was not built (no reference tree here)")
    lib = ctypes.CDLL(path)
    lib.ref_attention.argtypes = [_V, _V, _V, _V, _V, _V, _U, _U, _U, _U, _V, _V]
    lib.ref_gdn_rows.argtypes = [_V, _V, _U, _V, _U, _U, _U, _V, _V, _V]
    lib.ref_gdn_recurrence.argtypes = [_V, _V, _V, _V, _U, _U, _U, _V, _V, _U, _V, _V, _V, _V]
    return lib


def _bf16_ulp(x):
    """One bf16 unit in the last place at |x| (the reference tests' bfloatUlp)."""
    _, e = np.frexp(np.abs(x))
    return np.ldexp(1.0, e - 8)


def _tree(parent):
    t = np.zeros((len(parent), 2), np.uint32)
    for r, p in enumerate(parent):
        t[r, 0] = (1 << r) | (int(t[p, 0]) if r else 0)
        t[r, 1] = p | ((bin(int(t[r, 0])).count("1") - 1) << 16)
    return t


@pytest.mark.parametrize("kv_heads,group,committed,rows,parent", [
    (2, 4, 0, 16, None),
    (2, 6, 5, 16, None),
    (1, 8, 100, 7, None),
    (4, 2, 1000, 16, None),
    (2, 4, 37, 9, [0, 0, 1, 2, 1, 4, 0, 6, 7]),
])
def test_attention_matches_the_reference_model(kv_heads, group, committed, rows, parent):
    ref = _models()
    o = ol.bind_ops(ol.load())
    D, T = int(ref.ref_attention_head_dim()), int(ref.ref_attention_page_tokens())
    rng = np.random.default_rng(committed + rows)
    pages = (committed + rows + T - 1) // T
    kv = ol.HostKv(pages + 3, kv_heads, D, T, scale_f16=False)
    kv.fill_random(rng)
    table = rng.permutation(pages + 3)[:pages].astype(np.uint32)
    heads = kv_heads * group
    q = ol.f2bf(rng.standard_normal((rows, heads, D)).astype(np.float32))
    tree = _tree(parent) if parent else None
    want = np.zeros((rows, heads, D), np.uint16)
    assert ref.ref_attention(P(q), P(kv.k), P(kv.v), P(kv.ks), P(kv.vs), P(table), kv_heads, group, committed, rows, P(tree), P(want)) == 0
    got = np.zeros((rows, heads * D), np.uint16)
    desc = kv.desc()
    o.so_attention(P(q), None, 0, rows, heads, 0, ctypes.byref(desc), P(table), committed, P(tree), P(got), heads * D, None)
    got, want = ol.bf2f(got).reshape(-1).astype(np.float64), ol.bf2f(want).reshape(-1).astype(np.float64)
    # Both sum in fp64 and round once; the model multiplies code and scale in fp32 first, so a value on a
    # rounding boundary may land on the neighbouring bf16.
    assert np.all(np.abs(got - want) <= _bf16_ulp(want) + 1e-30)
    assert np.mean(got != want) < 1e-3


def _gdn_step(o, seed, rows, KH, VH, pending=None, state=None, cs=None):
    """One so_gdn_verify call on seeded inputs; `pending` (a step's tape and its row count) is folded first."""
    rng = np.random.default_rng(seed)
    D = 128
    KW, VW = KH * D, VH * D
    C = 2 * KW + VW
    stride = C + VW
    bf = lambda shape, scale: ol.f2bf((rng.standard_normal(shape) * scale).astype(np.float32))
    qkvz, b, a = bf((16, stride), 1.0), bf((16, VH), 1.0), bf((16, VH), 1.0)
    conv_w = bf((C, 4), 0.4)
    a_scale = (-np.exp(rng.uniform(-3, 0.5, VH))).astype(np.float32)
    dt_bias, norm_w = bf((VH,), 0.5), (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    cs_in = bf((3, C), 1.0) if cs is None else cs
    state_in = (rng.standard_normal((VH, D, D)) * 0.05).astype(np.float32) if state is None else state
    blank = lambda: dict(inputs=np.zeros((16, C), np.uint16), k=np.zeros((16, KW), np.uint16), v=np.zeros((16, VW), np.uint16),
                         beta=np.zeros((16, VH), np.uint16), decay=np.zeros((16, VH), np.float32))
    pend, pending_rows = (blank(), 0) if pending is None else pending
    step = blank()
    cs_out, state_out, hidden = np.zeros_like(cs_in), np.zeros_like(state_in), np.zeros((16, VW), np.uint16)
    tape = lambda t: ol.SoGdnTape(P(t["inputs"]), P(t["k"]), P(t["v"]), P(t["beta"]), P(t["decay"]))
    args = ol.SoGdnArgs(P(qkvz), P(b), P(a), P(conv_w), P(a_scale), P(dt_bias), P(norm_w), P(cs_in), P(cs_out), P(state_in), P(state_out),
                        tape(pend), tape(step), P(hidden), rows, pending_rows, KH, VH, stride, VH, VW, 0, None, 0)
    o.so_gdn_verify(ctypes.byref(args))
    return dict(qkvz=qkvz, b=b, a=a, conv_w=conv_w, a_scale=a_scale, dt_bias=dt_bias, norm_w=norm_w, cs_in=cs_in, cs=cs_out,
                state_in=state_in, state=state_out, hidden=hidden, step=step, stride=stride, C=C)


@pytest.mark.parametrize("KH,VH,rows", [(1, 2, 16), (2, 4, 16), (2, 6, 5)])
def test_gdn_matches_the_reference_model(KH, VH, rows):
    ref = _models()
    o = ol.bind_ops(ol.load())
    D, KW, VW = 128, KH * 128, VH * 128
    s = _gdn_step(o, 11 + VH, rows, KH, VH)
    # The step's tape rows: k per key head, v per value head (3 bf16 units, as the reference's checkTapeRows).
    q64, k64, v64 = np.zeros((rows, KW)), np.zeros((rows, KW)), np.zeros((rows, VW))
    assert ref.ref_gdn_rows(P(s["cs_in"]), P(s["qkvz"]), s["stride"], P(s["conv_w"]), rows, KH, VH, P(q64), P(k64), P(v64)) == 0
    for got, want in ((s["step"]["k"][:rows], k64), (s["step"]["v"][:rows], v64)):
        got = ol.bf2f(got).astype(np.float64)
        assert np.all(np.abs(got - want) <= 3.0 * _bf16_ulp(want) + 1e-6)
        assert np.mean(got != ol.bf2f(ol.f2bf(want.astype(np.float32)))) < 0.01
    # Gates (the reference's checkGates): beta = sigmoid(b) within 2 units; decay = exp(a_scale * softplus), softplus
    # rounded to bf16, one step either way allowed.
    b = ol.bf2f(s["b"][:rows]).astype(np.float64)
    beta = ol.bf2f(s["step"]["beta"][:rows]).astype(np.float64)
    assert np.all(np.abs(beta - 1 / (1 + np.exp(-b))) <= 2.0 * _bf16_ulp(1 / (1 + np.exp(-b))) + 1e-6)
    x = ol.bf2f(ol.f2bf((ol.bf2f(s["a"][:rows]) + ol.bf2f(s["dt_bias"])[None, :]).astype(np.float32))).astype(np.float64)
    softplus = np.maximum(x, 0) + np.log1p(np.exp(-np.abs(x)))
    rounded = ol.f2bf(softplus.astype(np.float32)).astype(np.int32)
    decay = s["step"]["decay"][:rows].astype(np.float64)
    matched = np.zeros(decay.shape, bool)
    for step in (-1, 0, 1):
        cand = np.exp(s["a_scale"].astype(np.float64)[None, :] * ol.bf2f((rounded + step).astype(np.uint16)))
        matched |= np.abs(decay - cand) <= 1e-4 * (1 + np.abs(cand))
    assert matched.all()

    # The state the rows leave: the oracle folds them in the next step; the model runs its delta rule over the tape.
    tape_kv = np.concatenate([s["step"]["k"][:rows], s["step"]["v"][:rows]], axis=1).copy()
    state64, rows64, mag64 = np.zeros((VH, D, D)), np.zeros((rows, VW)), np.zeros((rows, VW))
    assert ref.ref_gdn_recurrence(P(s["state_in"]), P(tape_kv), P(s["step"]["decay"]), P(s["step"]["beta"]), rows, KH, VH,
                                  P(s["cs_in"]), P(s["qkvz"]), s["stride"], P(s["conv_w"]), P(state64), P(rows64), P(mag64)) == 0
    nxt = _gdn_step(o, 99, 4, KH, VH, pending=(s["step"], rows), state=s["state_in"], cs=s["cs"])
    assert np.all(np.abs(nxt["state"].astype(np.float64) - state64) <= 1e-4 * (1 + np.abs(state64)))   # checkState's gate
    assert np.all(np.abs(nxt["state"].astype(np.float64) - state64) <= 2e-6 * (1 + np.abs(state64)))   # what fp32 sums give
    # The carried convolution inputs: the last three rows before the next block.
    assert np.array_equal(nxt["cs"], np.concatenate([s["cs_in"], s["qkvz"][:rows, :s["C"]]])[-3:])

    # Hidden rows: the gated RMSNorm of the model's recurrent rows, as the reference's checkStep states it.
    z = ol.bf2f(s["qkvz"][:rows, s["C"]:]).astype(np.float64).reshape(rows, VH, D)
    rec = ol.bf2f(ol.f2bf(rows64.astype(np.float32))).astype(np.float64).reshape(rows, VH, D)
    inverse = 1.0 / np.sqrt((rec * rec).mean(axis=2, keepdims=True) + 1e-6)
    w = s["norm_w"].astype(np.float64)[None, None, :]
    normalized = ol.bf2f(ol.f2bf((rec * inverse * w).astype(np.float32))).astype(np.float64)
    gate = z / (1 + np.exp(-z))
    want = normalized * gate
    allowed = 3.0 * _bf16_ulp(want) + 1e-6 + inverse * np.abs(w * gate) * np.ldexp(mag64.reshape(rows, VH, D), -7)
    got = ol.bf2f(s["hidden"][:rows]).astype(np.float64).reshape(rows, VH, D)
    assert np.all(np.abs(got - want) <= allowed)
    assert np.mean(got != ol.bf2f(ol.f2bf(want.astype(np.float32)))) <= 0.01


@pytest.mark.parametrize("policy", [(20, 1.0, 0.95, 0.0), (20, 0.7, 0.8, 0.0), (0, 1.0, 1.0, 0.0), (40, 1.3, 0.9, 0.0), (0, 0.7, 1.0, 0.05)])
def test_sampled_selection_matches_the_reference_model(policy):
    """Rows that test the children a draft drew, then draw from the last residual: the oracle's fp32 restatement of the
    kernel against the reference's fp64 recursion (referenceDistribution, referenceSelection), row by row except where
    the model itself says a comparison is within float rounding of its threshold or a policy cut is ambiguous, as the
    reference's childTests does; nine rows in ten must remain."""
    ref = _models()
    F, U8 = ctypes.c_float, ctypes.c_void_p
    ref.ref_sample_row.argtypes = [_V, _U, F, F, _U, F, _V, _V, _V, _V, F, _V, _V, _V, _V]
    o = ol.load()
    o.so_sample_verify_draws.argtypes = [_V, _U, _U, _U, F, F, _U, F, _V, _V, _V, _V, _V, _V]
    top_k, temperature, top_p, min_p = policy
    C, vocab, rows = int(ref.ref_sampling_candidates()), 1003, 16
    rng = np.random.default_rng(int(temperature * 100) + top_k)
    checked = drawn = 0
    for round_ in range(12):
        logits = (rng.standard_normal((rows, vocab)) * 0.3).astype(np.float32)
        for r in range(rows):
            spikes = rng.choice(vocab, 40, replace=False)
            logits[r, spikes] = (1.0 + 0.25 * np.arange(40) * rng.uniform(0.2, 1.0) + 0.1 * rng.standard_normal(40)).astype(np.float32)
        uniforms = rng.uniform(0, 1, 80).astype(np.float32)
        ids = np.zeros((rows, C), np.uint32)
        q = np.zeros((rows, C), np.float32)
        draws = np.full((rows, 4), 0xff, np.uint8)
        for r in range(rows):
            best = list(np.lexsort((np.arange(vocab), -logits[r]))[:6])
            while len(best) < C:
                t = int(rng.integers(vocab))
                if t not in best:
                    best.append(t)
            ids[r] = rng.permutation(np.array(best, np.uint32))
            if r == round_ % rows:
                ids[r, C - 1] = 0xffffffff       # a candidate past the vocabulary, never drawn
            qq = np.where(rng.integers(0, 4, C) > 0, rng.uniform(0, 1, C) ** 3, 0.0)
            if ids[r, C - 1] == 0xffffffff:
                qq[C - 1] = 0.0
            if qq.sum() == 0:
                qq[0] = 1.0
            qq /= qq.sum()
            q[r] = qq.astype(np.float32)
            count = (round_ + r) % 5
            keys = [(np.log(qq[i]) - np.log(-np.log(rng.uniform(1e-300, 1))), i) for i in range(C) if qq[i] > 0]
            keys.sort(reverse=True)
            for c, (_, i) in enumerate(keys[:count]):
                draws[r, c] = i
        got = np.zeros(rows, np.uint32)
        o.so_sample_verify_draws(P(logits), vocab, vocab, rows, temperature, min_p, top_k, top_p, P(uniforms), P(ids), P(q), P(draws), P(got), None)
        for r in range(rows):
            token, close, amb = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_double()
            tests = uniforms[16 + 4 * r:20 + 4 * r].copy()
            assert ref.ref_sample_row(P(logits[r]), vocab, temperature, min_p, top_k, top_p, P(ids[r]), P(q[r]), P(draws[r]), P(tests),
                                      float(uniforms[r]), ctypes.byref(token), ctypes.byref(close), ctypes.byref(amb), None) == 0
            drawn += 1
            if close.value or amb.value > 0.0:
                continue
            checked += 1
            assert got[r] == token.value, (round_, r, int(got[r]), token.value)
    assert checked * 10 >= drawn * 9, (checked, drawn)


def test_greedy_selection_matches_the_reference_order():
    """Temperature 0: the oracle's selection is the first token of the reference's order (value descending, id ascending),
    ties and all; the order itself is what numpy's stable sort gives."""
    ref = _models()
    ref.ref_argmax.argtypes = [_V, _U]
    ref.ref_best.argtypes = [_V, _U, _U, _V]
    o = ol.bind_ops(ol.load())
    rng = np.random.default_rng(17)
    rows, vocab = 16, 5003
    logits = rng.standard_normal((rows, vocab)).astype(np.float32)
    logits[1, [7, 4000, 300]] = 9.0                      # a three-way tie for the maximum: the lowest id
    logits[2, :] = 0.25                                  # every token ties
    logits[3, vocab - 1] = 11.0                          # the last id
    logits[4, 100] = np.nextafter(np.float32(30.0), np.float32(31.0))   # one unit in the last place apart
    logits[4, 50] = np.float32(30.0)
    logits[5, :] = -np.inf                               # no comparable logit ...
    logits[5, 4321] = -1e30                              # ... but one
    tokens = np.zeros(rows, np.uint32)
    selected = np.zeros(rows, np.uint32)
    o.so_sample_verify(P(logits), vocab, vocab, rows, P(tokens), 0.0, None, P(selected), None)
    for r in range(rows):
        assert selected[r] == ref.ref_argmax(P(logits[r]), vocab), r
        best = np.zeros(8, np.uint32)
        assert ref.ref_best(P(logits[r]), vocab, 8, P(best)) == 8
        assert np.array_equal(best, np.lexsort((np.arange(vocab), -logits[r]))[:8])
    assert selected[1] == 7 and selected[2] == 0 and selected[3] == vocab - 1 and selected[4] == 100 and selected[5] == 4321


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_admission_matches_the_reference_model(temperature):
    """Rows that admit only the tokens of a constraint mask, less the excluded ones: the oracle's in-place -inf followed by its
    selection against the reference's selections under the same admission (referenceArgmax / referenceDistribution with an
    Admission, dev/tests/engine/target_sampling_metal_test.mm:269-300,333-403)."""
    ref = _models()
    F = ctypes.c_float
    ref.ref_select_admitted.argtypes = [_V, _U, _V, _V, _U, F, F, _U, F, F, _V, _V, _V]
    o = ol.bind_ops(ol.load())
    o.so_sample_admit.argtypes = [_V, _U, _U, _U, _V, _U, _V, _U]
    rng = np.random.default_rng(23)
    rows, vocab = 16, 3001
    words = (vocab + 31) // 32
    logits = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
    masks = rng.integers(0, 2 ** 32, (rows, words), dtype=np.uint64).astype(np.uint32)
    masks[3] = 0                                          # a row that admits nothing
    masks[4] = 0
    masks[4, 40] = 1 << 7                                 # a row that admits one token, 40 * 32 + 7
    excluded = np.array([int(np.argmax(logits[0])), int(np.argmax(logits[1])), 5], np.uint32)
    masks[0, excluded[0] // 32] |= np.uint32(1 << (excluded[0] % 32))   # admitted by the mask, excluded all the same
    uniforms = rng.uniform(0, 1, 80).astype(np.float32)
    for use_mask, use_excluded in ((True, True), (True, False), (False, True)):
        mine = logits.copy()
        ex = excluded if use_excluded else np.zeros(0, np.uint32)
        o.so_sample_admit(P(mine), vocab, vocab, rows, P(masks) if use_mask else None, words, P(ex) if len(ex) else None, len(ex))
        selected = np.zeros(rows, np.uint32)
        o.so_sample_verify(P(mine), vocab, vocab, 1, P(np.zeros(rows, np.uint32)), temperature, P(uniforms), P(selected), None)
        for r in range(rows):
            # one row at a time: a row alone has no drafted child to test
            one = np.zeros(1, np.uint32)
            u = uniforms.copy()
            u[0] = uniforms[r]
            o.so_sample_verify(P(mine[r]), vocab, vocab, 1, P(np.zeros(1, np.uint32)), temperature, P(u), P(one), None)
            token, close, amb = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_double()
            ref.ref_select_admitted(P(logits[r]), vocab, P(masks[r]) if use_mask else None, P(ex) if len(ex) else None, len(ex), temperature,
                                    0.0, 0, 1.0, float(uniforms[r]), ctypes.byref(token), ctypes.byref(close), ctypes.byref(amb))
            if close.value or amb.value > 0:
                continue
            assert one[0] == token.value, (use_mask, use_excluded, r)
            if token.value != 0xffffffff:
                assert not use_mask or (masks[r, token.value // 32] >> (token.value % 32)) & 1
                assert not use_excluded or token.value not in excluded
        if use_mask:
            o.so_sample_verify(P(mine[3]), vocab, vocab, 1, P(np.zeros(1, np.uint32)), temperature, P(uniforms), P(one), None)
            assert one[0] == 0xffffffff
            o.so_sample_verify(P(mine[4]), vocab, vocab, 1, P(np.zeros(1, np.uint32)), temperature, P(uniforms), P(one), None)
            assert one[0] == 40 * 32 + 7


def test_rmsnorm_matches_the_reference_model():
    """so_rmsnorm against the reference's fp64 norm (dev/tests/engine/NormReference.hpp rmsNorm): every value the exact one
    rounded once to bf16 by the reference's own criterion (roundedOnceToBf16), rows of small and large magnitudes."""
    ref = _models()
    ref.ref_rmsnorm.argtypes = [_V, _U, _U, _V, _V, _V, _V]
    o = ol.bind_ops(ol.load())
    o.so_rmsnorm.argtypes = [_V, _U, _U, _U, _V, _V, _U]
    rng = np.random.default_rng(29)
    rows, size = 16, 5120
    x = (rng.standard_normal((rows, size)) * np.exp(rng.uniform(-6, 6, (rows, 1)))).astype(np.float32)
    x[3] = 0.0                                            # a row of zeros: the epsilon alone
    xb = ol.f2bf(x)
    w = (1 + 0.1 * rng.standard_normal(size)).astype(np.float32)
    got = np.zeros((rows, size), np.uint16)
    o.so_rmsnorm(P(xb), rows, size, size, P(w), P(got), size)
    exact, once = np.zeros((rows, size)), np.zeros((rows, size), np.uint8)
    ref.ref_rmsnorm(P(xb), rows, size, P(w), P(exact), P(got), P(once))
    assert once.all(), int((once == 0).sum())
    assert np.mean(ol.bf2f(got) != ol.bf2f(ol.f2bf(exact.astype(np.float32)))) < 2e-3   # (fp32 sums move a value on a rounding boundary)
