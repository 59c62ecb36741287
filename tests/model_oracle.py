"""The tiny hybrid model's verify step on the CPU oracle (test infrastructure): the same layer loop as
splash_b200/csrc/model/QwenTarget.hpp, every operator an oracle call, for parity of whole steps."""
import ctypes

import numpy as np

import oracle_lib as ol
import quant_fixtures as qf

P = ol.ptr


def make_weights(cfg, seed=0):
    """Seeded synthetic tensors of the tiny configuration, keyed (layer, name) like sb_target_tensor."""
    rng = np.random.default_rng(seed)
    H, D, I = cfg["hidden"], cfg["head_dim"], cfg["intermediate"]
    KH, VH = cfg["gdn_key_heads"], cfg["gdn_value_heads"]
    conv = (2 * KH + VH) * 128
    attn_in = cfg["q_heads"] * (2 * D if cfg["gated_attention"] else D) + 2 * cfg["kv_heads"] * D
    gdn_in = conv + VH * 128
    w = {}
    norm = lambda n: (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    rows = lambda fmt, n, k: qf.realistic(fmt, n, k, seed=int(rng.integers(1 << 30)))
    for l in range(cfg["layers"]):
        attention = (l + 1) % cfg["attention_interval"] == 0
        w[l, "attn_norm"], w[l, "ffn_norm"] = norm(H), norm(H)
        if attention:
            w[l, "in_proj"] = rows(cfg["fmt_proj"], attn_in, H)
            w[l, "out_proj"] = rows(cfg["fmt_proj"], H, cfg["q_heads"] * D)
            w[l, "q_norm"], w[l, "k_norm"] = norm(D), norm(D)
        else:
            w[l, "in_proj"] = rows(cfg["fmt_proj"], gdn_in, H)
            w[l, "out_proj"] = rows(cfg["fmt_proj"], H, VH * 128)
            w[l, "ssm_ab"] = (rng.standard_normal((2 * VH, H)) * 0.02).astype(np.float32)
            w[l, "ssm_conv"] = ol.f2bf((rng.standard_normal((conv, 4)) * 0.4).astype(np.float32))
            w[l, "ssm_a"] = (-np.exp(rng.uniform(-3, 0.5, VH))).astype(np.float32)
            w[l, "ssm_dt_bias"] = ol.f2bf((rng.standard_normal(VH) * 0.5).astype(np.float32))
            w[l, "ssm_norm"] = norm(128)
        if cfg.get("moe_experts"):
            E, Ie = cfg["moe_experts"] + 1, cfg["moe_intermediate"]
            w[l, "ffn_router"] = (rng.standard_normal((cfg["moe_experts"], H)) * 0.05).astype(np.float32)
            w[l, "ffn_shared_gate"] = (rng.standard_normal(H) * 0.02).astype(np.float32)
            w[l, "ffn_gate_exps"] = np.concatenate([rows(cfg["fmt_proj"], Ie, H) for _ in range(E)])
            w[l, "ffn_up_exps"] = np.concatenate([rows(cfg["fmt_proj"], Ie, H) for _ in range(E)])
            w[l, "ffn_down_exps"] = np.concatenate([rows(cfg["fmt_proj"], H, Ie) for _ in range(E)])
            continue
        w[l, "ffn_gate"] = rows(cfg["fmt_proj"], I, H)
        w[l, "ffn_up"] = rows(cfg["fmt_proj"], I, H)
        w[l, "ffn_down"] = rows(cfg["fmt_down"], H, I)
    w[-1, "token_embd"] = rows(cfg["fmt_embed"], cfg["vocab"], H)
    w[-1, "output_norm"] = norm(H)
    w[-1, "output"] = rows(cfg["fmt_head"], cfg["vocab"], H)
    return w


def make_state(cfg, committed, seed=1):
    """A prefilled INT8 cache of `committed` random tokens per attention layer and random GDN cells."""
    rng = np.random.default_rng(seed)
    KH, VH = cfg["gdn_key_heads"], cfg["gdn_value_heads"]
    conv = (2 * KH + VH) * 128
    pages = (cfg["max_context"] + 16 + cfg["page_tokens"] - 1) // cfg["page_tokens"]
    s = {"committed": committed, "pending_rows": 0, "step": 0}
    for l in range(cfg["layers"]):
        if (l + 1) % cfg["attention_interval"] == 0:
            kv = ol.HostKv(pages, cfg["kv_heads"], cfg["head_dim"], cfg["page_tokens"], cfg["kv_scale_f16"])
            kv.fill_random(rng)
            s[l, "kv"] = kv
        else:
            for i in range(2):
                s[l, f"state{i}"] = (rng.standard_normal((VH, 128, 128)) * 0.05).astype(np.float32)
                s[l, f"conv{i}"] = ol.f2bf(rng.standard_normal((3, conv)).astype(np.float32))
                s[l, f"tape{i}"] = dict(inputs=np.zeros((16, conv), np.uint16), k=np.zeros((16, KH * 128), np.uint16),
                                        v=np.zeros((16, VH * 128), np.uint16), beta=np.zeros((16, VH), np.uint16),
                                        decay=np.zeros((16, VH), np.float32))
    return s


def upload(t, w, s, cut=lambda layer, name, array: array, lane=0):
    """Uploads weights `w` and state `s` into the device target `t`; `cut` takes a rank's share of each array. With `lane`
    the state goes into that lane's share of every state tensor (w may be empty for the lanes after the first)."""
    for (layer, name), arr in w.items():
        t.upload(layer, name, cut(layer, name, arr))
    _up = t.upload
    if lane:
        class _Lane:
            @staticmethod
            def upload(layer, name, array):
                _up(layer, name, array, lane=lane)
        t = _Lane
    for key, val in s.items():
        if not isinstance(key, tuple):
            continue
        layer, name = key
        if name == "kv":
            for tn, arr in (("kv_k", val.k), ("kv_v", val.v), ("kv_ks", val.ks), ("kv_vs", val.vs)):
                t.upload(layer, tn, cut(layer, tn, arr))
        elif name.startswith("tape"):
            i = name[-1]
            for f, tn in (("inputs", "tape_inputs"), ("k", "tape_k"), ("v", "tape_v"), ("beta", "tape_beta"), ("decay", "tape_decay")):
                t.upload(layer, tn + i, cut(layer, tn + i, val[f]))
        else:
            t.upload(layer, name, cut(layer, name, val))


def input_projection(o, cfg, w, l, n, k, X, rows):
    """A layer's fused input projection: one tensor `in_proj` of the configuration's format, or `in_parts`, a list of
    (format, rows array) tensors of different formats whose outputs lie side by side."""
    if (l, "in_parts") not in w:
        return linear(o, cfg["fmt_proj"], w[l, "in_proj"], n, k, X, rows)
    outs = [linear(o, fmt, part, len(part), k, X, rows) for fmt, part in w[l, "in_parts"]]
    out = np.concatenate(outs, axis=1)
    assert out.shape[1] == n
    return np.ascontiguousarray(out)


def linear(o, fmt, W, n, k, X, rows, epilogue=0, aux=None, out_f32=False, W2=None):
    out = np.zeros((rows, n), np.float32 if out_f32 else np.uint16)
    Wfull = W if W2 is None else np.concatenate([W, W2], axis=0)
    assert o.so_linear(fmt, P(np.ascontiguousarray(Wfull)), n, k, P(X), rows, epilogue, P(aux) if aux is not None else None, n,
                       P(out), n, int(out_f32), 0) == 0
    return out


def verify_step(cfg, w, s, tokens, temperature=0.0, uniforms=None, advance=True, mutate=True, tree=None, penalties=None, penalty_words=None,
                draws=None, prompt=False, admission=None, policy=(0.0, 0, 1.0), stop_tokens=()):
    """One verify step of a chain, or of the tree whose rows `tree` holds (uint32 [rows, 2]: ancestors, parent | depth << 16).
    draws = (candidate ids u32 [rows, 16], draft probabilities f32 [rows, 16], drawn children u8 [rows, 4]): sampled rows
    select by recursive rejection sampling over these children. prompt: the rows are prompt tokens, all committed whatever
    was selected. admission = (masks u32 [rows, words] or None, excluded token ids): what the rows may select. policy = (min_p,
    top_k, top_p): the end of a sampled row's distribution. Returns dict(logits, selected, retained, accepted, mask, tokens)."""
    o = ol.bind_ops(ol.load())
    rows = len(tokens)
    H, D, I, V = cfg["hidden"], cfg["head_dim"], cfg["intermediate"], cfg["vocab"]
    KH, VH, QH, KVH = cfg["gdn_key_heads"], cfg["gdn_value_heads"], cfg["q_heads"], cfg["kv_heads"]
    conv = (2 * KH + VH) * 128
    pairs = cfg["rotary_pairs"]
    committed, parity = s["committed"], s["step"] & 1
    tokens = np.ascontiguousarray(tokens, np.uint32)
    chain_rows = np.zeros((rows, 2), np.uint32)
    for r in range(rows):
        chain_rows[r] = ((2 << r) - 1, max(r - 1, 0) | (r << 16))
    rows_tree = chain_rows if tree is None else np.ascontiguousarray(tree, np.uint32)
    pos = (committed + (rows_tree[:, 1] >> 16)).astype(np.uint32)
    inv = (np.float32(cfg["rope_theta"]) ** (-np.arange(pairs, dtype=np.float32) / np.float32(pairs))).astype(np.float32)
    cos, sin = np.zeros((rows, pairs), np.float32), np.zeros((rows, pairs), np.float32)
    o.so_rope_tables(P(pos), rows, P(inv), pairs, 1.0, P(cos), P(sin))
    h = np.zeros((rows, H), np.uint16)
    assert o.so_embed(cfg["fmt_embed"], P(w[-1, "token_embd"]), V, H, P(tokens), rows, P(h), H) == 0
    page_table = np.arange((cfg["max_context"] + 16 + cfg["page_tokens"] - 1) // cfg["page_tokens"], dtype=np.uint32)
    new_state = {}
    for l in range(cfg["layers"]):
        attention = (l + 1) % cfg["attention_interval"] == 0
        n1 = np.zeros_like(h)
        o.so_rmsnorm(P(h), rows, H, H, P(w[l, "attn_norm"]), P(n1), H)
        if attention:
            attn_in = QH * (2 * D if cfg["gated_attention"] else D) + 2 * KVH * D
            packed = input_projection(o, cfg, w, l, attn_in, H, n1, rows)
            kv = s[l, "kv"]
            if not mutate:
                import copy
                kv = copy.deepcopy(kv)
            desc = kv.desc()
            queries = np.zeros((rows, QH, D), np.uint16)
            o.so_attn_store(P(packed), attn_in, rows, QH, cfg["gated_attention"], P(w[l, "q_norm"]), P(w[l, "k_norm"]), P(cos), P(sin),
                            pairs, ctypes.byref(desc), P(page_table), committed, P(queries))
            mixed = np.zeros((rows, QH * D), np.uint16)
            o.so_attention(P(queries), P(packed), attn_in, rows, QH, cfg["gated_attention"], ctypes.byref(desc), P(page_table),
                           committed, P(rows_tree) if tree is not None else None, P(mixed), QH * D, None)
            mixed_w = QH * D
        else:
            gdn_in = conv + VH * 128
            packed = input_projection(o, cfg, w, l, gdn_in, H, n1, rows)
            ab = ol.f2bf((ol.bf2f(n1).astype(np.float32) @ w[l, "ssm_ab"].T.astype(np.float32)).astype(np.float32))
            b, a = np.ascontiguousarray(ab[:, :VH]), np.ascontiguousarray(ab[:, VH:])
            cur, nxt = parity, parity ^ 1
            pend, step = s[l, f"tape{nxt}"], s[l, f"tape{cur}"]
            if not mutate:
                step = {k: v.copy() for k, v in step.items()}
            cs_out, st_out = np.zeros_like(s[l, f"conv{cur}"]), np.zeros_like(s[l, f"state{cur}"])
            mixed = np.zeros((rows, VH * 128), np.uint16)
            tape = lambda t: ol.SoGdnTape(P(t["inputs"]), P(t["k"]), P(t["v"]), P(t["beta"]), P(t["decay"]))
            args = ol.SoGdnArgs(P(packed), P(b), P(a), P(w[l, "ssm_conv"]), P(w[l, "ssm_a"]), P(w[l, "ssm_dt_bias"]), P(w[l, "ssm_norm"]),
                                P(s[l, f"conv{cur}"]), P(cs_out), P(s[l, f"state{cur}"]), P(st_out), tape(pend), tape(step), P(mixed),
                                rows, s["pending_rows"], KH, VH, gdn_in, VH, VH * 128, cfg["tiled_heads"],
                                P(rows_tree) if tree is not None else None, s.get("pending_path", 0))
            o.so_gdn_verify(ctypes.byref(args))
            new_state[l, f"conv{nxt}"], new_state[l, f"state{nxt}"] = cs_out, st_out
            mixed_w = VH * 128
        h = linear(o, w.get((l, "out_proj_fmt"), cfg["fmt_proj"]), w[l, "out_proj"], H, mixed_w, mixed, rows, epilogue=1, aux=h)
        n2 = np.zeros_like(h)
        o.so_rmsnorm(P(h), rows, H, H, P(w[l, "ffn_norm"]), P(n2), H)
        if cfg.get("moe_experts"):
            E, K, Ie = cfg["moe_experts"], cfg["moe_top_k"], cfg["moe_intermediate"]
            scores = np.ascontiguousarray((ol.bf2f(n2).astype(np.float32) @ w[l, "ffn_router"].T).astype(np.float32))
            sel, wts = np.zeros((rows, K + 1), np.uint32), np.zeros((rows, K + 1), np.float32)
            o.so_moe_route(P(scores), rows, E, E, K, 0, P(n2), H, P(w[l, "ffn_shared_gate"]), P(sel), P(wts))
            out = np.zeros_like(h)
            assert o.so_moe_experts(P(n2), P(h), P(sel), P(wts), P(w[l, "ffn_gate_exps"]), P(w[l, "ffn_up_exps"]), P(w[l, "ffn_down_exps"]),
                                    rows, K + 1, H, Ie, E + 1, P(out), None) == 0
            h = out
            continue
        act = linear(o, cfg["fmt_proj"], w[l, "ffn_gate"], I, H, n2, rows, epilogue=3, W2=w[l, "ffn_up"])
        h = linear(o, w.get((l, "ffn_down_fmt"), cfg["fmt_down"]), w[l, "ffn_down"], H, I, act, rows, epilogue=1, aux=h)
    nf = np.zeros_like(h)
    o.so_rmsnorm(P(h), rows, H, H, P(w[-1, "output_norm"]), P(nf), H)
    logits = linear(o, cfg["fmt_head"], w[-1, "output"], V, H, nf, rows, out_f32=True)
    if admission is not None:
        masks, excluded = admission
        excluded = np.ascontiguousarray(excluded, np.uint32)
        o.so_sample_admit.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32,
                                      ctypes.c_void_p, ctypes.c_uint32]
        o.so_sample_admit(P(logits), V, V, rows, P(np.ascontiguousarray(masks[:rows], np.uint32)) if masks is not None else None,
                          (V + 31) // 32, P(excluded) if len(excluded) else None, len(excluded))
    if penalties is not None:  # (repetition, presence, frequency) over the table and each row's path
        o.so_sample_penalize(P(logits), V, V, rows, P(np.ascontiguousarray(penalty_words, np.uint32)), P(tokens), P(rows_tree), *penalties)
    selected = np.zeros(rows, np.uint32)
    margin = np.zeros(rows, np.float64)
    if draws is not None and temperature > 0:
        o.so_sample_verify_draws.argtypes = ([ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_float, ctypes.c_float,
                                              ctypes.c_uint32, ctypes.c_float] + [ctypes.c_void_p] * 6)
        ids, q, dr = (np.ascontiguousarray(a) for a in draws)
        o.so_sample_verify_draws(P(logits), V, V, rows, float(temperature), float(policy[0]), int(policy[1]), float(policy[2]), P(uniforms), P(ids), P(q), P(dr),
                                 P(selected), P(margin))
    else:
        o.so_sample_verify_filtered.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_float,
                                                ctypes.c_float, ctypes.c_uint32, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        o.so_sample_verify_filtered(P(logits), V, V, rows, P(tokens), float(temperature), float(policy[0]), int(policy[1]), float(policy[2]),
                                    P(uniforms) if uniforms is not None else None, P(selected), P(margin), None)
    out_tokens = selected.copy()
    res = np.zeros(3, np.uint32)
    stops = np.ascontiguousarray(stop_tokens, np.uint32)
    o.so_accept(P(tokens), P(rows_tree), P(out_tokens), rows, 16, P(stops) if len(stops) else None, len(stops), P(res[0:1]), P(res[1:2]), P(res[2:3]))
    if prompt:
        assert advance and tree is None
        res[:] = (rows, rows - 1, (2 << (rows - 1)) - 1)
        out_tokens = selected.copy()
    if mutate:
        s.update(new_state)
        s["step"] += 1
        if advance:
            if tree is not None:  # the accepted path's KV rows move to their depths
                for l in range(cfg["layers"]):
                    if (l + 1) % cfg["attention_interval"] == 0:
                        desc = s[l, "kv"].desc()
                        o.so_kv_path_commit(ctypes.byref(desc), P(page_table), committed, int(res[2]))
            s["committed"] += int(res[0])
            s["pending_rows"] = int(res[0])
            s["pending_path"] = int(res[2]) if tree is not None else 0
            if prompt:
                s["pending_path"] = 0
        else:
            s["pending_rows"] = 0
            s["pending_path"] = 0
    return dict(logits=logits, selected=selected, retained=int(res[0]), accepted=int(res[1]), mask=int(res[2]),
                tokens=out_tokens[:res[0]].copy(), margin=margin, hidden=h)


def draft_chain(cfg, w, s, first_token, rows=16, p_match=0.7, seed=5):
    """A draft block for the current state: token r + 1 equals the target's greedy choice after row r with
    probability p_match, else a uniform token (the benchmark configuration's draft model stand-in)."""
    rng = np.random.default_rng(seed)
    tokens = [int(first_token)]
    for r in range(rows - 1):
        out = verify_step(cfg, w, s, tokens, mutate=False)
        target = int(out["selected"][r])
        tokens.append(target if rng.random() < p_match else int(rng.integers(0, cfg["vocab"])))
    return np.array(tokens, np.uint32)
