"""The GGUF reader (host code: runs without a GPU) and the loader that fills a target from a GGUF of the Qwen3.5 hybrid
family. The files are written by tests/gguf_writer.py from the tiny model's synthetic tensors, with the names, shapes and
llama.cpp's tiled value-head order the reference's loader expects (runtime/model/GgufImage.cpp:477-556)."""
import ctypes
import os

import numpy as np
import pytest

import gguf_writer as gw
import model_oracle as mo
import oracle_lib as ol

FMT_TO_GGML = {0: gw.GGML["Q4_K"], 4: gw.GGML["Q6_K"], 6: gw.GGML["Q8_0"]}


def tiny_config():
    from splash_b200 import target
    return dict(target.TINY, gdn_key_heads=4, gdn_value_heads=8, tiled_heads=1)   # (two value heads a key head: the head order matters)


def ungroup(rows, start, head_rows, key_heads, per_key):
    """Rows in grouped head order (as the target holds them) back into llama.cpp's tiled order from row `start` on."""
    out = rows.copy()
    heads = (len(rows) - start) // head_rows
    for h in range(heads):
        src = (h % per_key) * key_heads + h // per_key
        out[start + src * head_rows:start + (src + 1) * head_rows] = rows[start + h * head_rows:start + (h + 1) * head_rows]
    return out


def model_to_gguf(path, cfg, w, arch="qwen35", drop=(), replace=None):
    """Writes the model's tensors `w` (keyed as sb_target_tensor names them) as a GGUF of architecture `arch`."""
    H, D = cfg["hidden"], cfg["head_dim"]
    KH, VH = cfg["gdn_key_heads"], cfg["gdn_value_heads"]
    per_key, KW, VW = VH // KH, KH * 128, VH * 128
    conv = 2 * KW + VW
    a = arch + "."
    meta = [("general.architecture", gw.STRING, arch), ("general.name", gw.STRING, "tiny synthetic"), ("general.alignment", gw.U32, 32),
            (a + "block_count", gw.U32, cfg["layers"]), (a + "embedding_length", gw.U32, H), (a + "feed_forward_length", gw.U32, cfg["intermediate"]),
            (a + "attention.head_count", gw.U32, cfg["q_heads"]), (a + "attention.head_count_kv", gw.U32, cfg["kv_heads"]),
            (a + "attention.key_length", gw.U32, D), (a + "attention.value_length", gw.U32, D),
            (a + "rope.dimension_count", gw.U32, 2 * cfg["rotary_pairs"]), (a + "rope.freq_base", gw.F32, cfg["rope_theta"]),
            (a + "attention.layer_norm_rms_epsilon", gw.F32, 1e-6), (a + "full_attention_interval", gw.U32, cfg["attention_interval"]),
            (a + "ssm.conv_kernel", gw.U32, 4), (a + "ssm.group_count", gw.U32, KH), (a + "ssm.time_step_rank", gw.U32, VH),
            (a + "ssm.state_size", gw.U32, 128), (a + "ssm.inner_size", gw.U32, VW),
            ("tokenizer.ggml.tokens", gw.ARRAY, (gw.STRING, ["<a>", "<b>", "<c>"])), ("tokenizer.ggml.scores", gw.ARRAY, (gw.F32, [0.5, -1.0, 2.0])),
            ("some.negative", gw.I32, -7), ("some.flag", gw.BOOL, 1)]
    if cfg.get("moe_experts"):
        meta += [(a + "expert_count", gw.U32, cfg["moe_experts"]), (a + "expert_used_count", gw.U32, cfg["moe_top_k"]),
                 (a + "expert_feed_forward_length", gw.U32, cfg["moe_intermediate"])]
    tensors = []

    def quantized(name, fmt, rows, k):
        tensors.append((name, FMT_TO_GGML[fmt], [k, len(rows)], rows))

    def floats(name, values, dims=None):
        values = np.ascontiguousarray(values, np.float32)
        tensors.append((name, gw.GGML["F32"], dims or [values.size], values))

    quantized("token_embd.weight", cfg["fmt_embed"], w[-1, "token_embd"], H)
    floats("output_norm.weight", w[-1, "output_norm"])
    quantized("output.weight", cfg["fmt_head"], w[-1, "output"], H)
    for l in range(cfg["layers"]):
        p = f"blk.{l}."
        floats(p + "attn_norm.weight", w[l, "attn_norm"])
        floats(p + "post_attention_norm.weight", w[l, "ffn_norm"])
        if (l + 1) % cfg["attention_interval"] == 0:
            q, kv = cfg["q_heads"] * D * (2 if cfg["gated_attention"] else 1), cfg["kv_heads"] * D
            if (l, "in_parts") in w:
                for stem, (fmt, part) in zip(("attn_q", "attn_k", "attn_v"), w[l, "in_parts"]):
                    quantized(p + stem + ".weight", fmt, part, H)
            else:
                rows = w[l, "in_proj"]
                quantized(p + "attn_q.weight", cfg["fmt_proj"], rows[:q], H)
                quantized(p + "attn_k.weight", cfg["fmt_proj"], rows[q:q + kv], H)
                quantized(p + "attn_v.weight", cfg["fmt_proj"], rows[q + kv:], H)
            floats(p + "attn_q_norm.weight", w[l, "q_norm"])
            floats(p + "attn_k_norm.weight", w[l, "k_norm"])
            quantized(p + "attn_output.weight", w.get((l, "out_proj_fmt"), cfg["fmt_proj"]), w[l, "out_proj"], cfg["q_heads"] * D)
        else:
            if (l, "in_parts") in w:
                (f0, qkv), (f1, gate) = w[l, "in_parts"]
            else:
                (f0, qkv), (f1, gate) = (cfg["fmt_proj"], w[l, "in_proj"][:conv]), (cfg["fmt_proj"], w[l, "in_proj"][conv:])
            quantized(p + "attn_qkv.weight", f0, ungroup(qkv, 2 * KW, 128, KH, per_key), H)
            quantized(p + "attn_gate.weight", f1, ungroup(gate, 0, 128, KH, per_key), H)
            ab = w[l, "ssm_ab"]
            floats(p + "ssm_beta.weight", ungroup(ab[:VH], 0, 1, KH, per_key), [H, VH])
            floats(p + "ssm_alpha.weight", ungroup(ab[VH:], 0, 1, KH, per_key), [H, VH])
            floats(p + "ssm_conv1d.weight", ungroup(ol.bf2f(w[l, "ssm_conv"]), 2 * KW, 128, KH, per_key), [4, conv])
            floats(p + "ssm_a", ungroup(w[l, "ssm_a"], 0, 1, KH, per_key))
            floats(p + "ssm_dt.bias", ungroup(ol.bf2f(w[l, "ssm_dt_bias"]), 0, 1, KH, per_key))
            floats(p + "ssm_norm.weight", w[l, "ssm_norm"])
            quantized(p + "ssm_out.weight", w.get((l, "out_proj_fmt"), cfg["fmt_proj"]), w[l, "out_proj"], VW)
        if cfg.get("moe_experts"):
            E, I = cfg["moe_experts"], cfg["moe_intermediate"]
            floats(p + "ffn_gate_inp.weight", w[l, "ffn_router"], [H, E])
            floats(p + "ffn_gate_inp_shexp.weight", w[l, "ffn_shared_gate"])
            kind = FMT_TO_GGML[cfg["fmt_proj"]]
            for part, rows_, k in (("gate", I, H), ("up", I, H), ("down", H, I)):
                stacked = w[l, f"ffn_{part}_exps"]
                tensors.append((p + f"ffn_{part}_exps.weight", kind, [k, rows_, E], stacked[:E * rows_]))
                quantized(p + f"ffn_{part}_shexp.weight", cfg["fmt_proj"], stacked[E * rows_:], k)
            continue
        quantized(p + "ffn_gate.weight", cfg["fmt_proj"], w[l, "ffn_gate"], H)
        quantized(p + "ffn_up.weight", cfg["fmt_proj"], w[l, "ffn_up"], H)
        quantized(p + "ffn_down.weight", w.get((l, "ffn_down_fmt"), cfg["fmt_down"]), w[l, "ffn_down"], cfg["intermediate"])
    tensors = [t for t in tensors if t[0] not in drop]
    if replace:                                  # name -> (ggml type, dims, data)
        tensors = [(n,) + tuple(replace[n]) if n in replace else (n, k, d, x) for n, k, d, x in tensors]
    return gw.write(path, meta, tensors)


@pytest.fixture(scope="module")
def tiny_file(tmp_path_factory):
    cfg = tiny_config()
    w = mo.make_weights(cfg, 3)
    path = str(tmp_path_factory.mktemp("gguf") / "tiny.gguf")
    start = model_to_gguf(path, cfg, w)
    return path, cfg, w, start


def test_reader_lists_the_files_tensors_and_metadata(tiny_file):
    from splash_b200 import gguf
    path, cfg, w, start = tiny_file
    f = gguf.GgufFile(path)
    tensors = {t["name"]: t for t in f.tensors()}
    assert len(tensors) == 3 + sum(11 if (l + 1) % 4 == 0 else 14 for l in range(cfg["layers"]))
    t = tensors["blk.3.attn_k.weight"]
    q = cfg["q_heads"] * cfg["head_dim"] * 2
    assert t["type"] == 12 and t["dims"] == [cfg["hidden"], cfg["kv_heads"] * cfg["head_dim"]]
    assert np.array_equal(t["data"].reshape(-1), w[3, "in_proj"][q:q + cfg["kv_heads"] * cfg["head_dim"]].reshape(-1))
    t = f.find("blk.0.ssm_conv1d.weight")
    assert t["type"] == 0 and t["dims"] == [4, (2 * 4 + 8) * 128] and len(t["data"]) == 4 * 4 * 2048
    assert f.find("blk.0.nothing") is None
    # every tensor starts on the file's alignment, inside the file
    raw = open(path, "rb").read()
    for t in tensors.values():
        at = t["data"].ctypes.data - tensors["token_embd.weight"]["data"].ctypes.data
        assert at % 32 == 0 and raw[start + at:start + at + 16] == bytes(t["data"][:16])
    assert f.meta("general.architecture") == "qwen35" and f.meta("qwen35.block_count") == 4
    assert f.meta("qwen35.rope.freq_base") == 1e6 and f.meta("general.alignment") == 32
    assert f.meta("some.negative") == 2 ** 64 - 7 and f.meta("some.flag") == 1 and f.meta("no.such.key") is None
    f.close()


def test_reader_makes_the_targets_configuration(tiny_file):
    from splash_b200 import gguf
    path, cfg, w, _ = tiny_file
    got = gguf.GgufFile(path).target_config(page_tokens=cfg["page_tokens"], kv_scale_f16=cfg["kv_scale_f16"], max_context=cfg["max_context"])
    for key, value in cfg.items():
        assert got[key] == value, key
    assert got["moe_experts"] == 0 and got["lanes"] == 0


def test_reader_refuses_what_is_not_a_readable_gguf(tmp_path):
    from splash_b200 import gguf, lib
    one = [("t", 0, [4], np.arange(4, dtype=np.float32))]
    meta = [("general.architecture", gw.STRING, "llama")]
    cases = {}
    gw.write(tmp_path / "magic.gguf", meta, one, magic=b"GGML")
    cases["magic.gguf"] = "magic"
    gw.write(tmp_path / "version.gguf", meta, one, version=2)
    cases["version.gguf"] = "version 2"
    gw.write(tmp_path / "type.gguf", meta, [("t", 99, [4], np.arange(4, dtype=np.float32))])
    cases["type.gguf"] = "cannot size"
    gw.write(tmp_path / "blocks.gguf", meta, [("t", 12, [100, 2], np.zeros(288, np.uint8))])
    cases["blocks.gguf"] = "whole Q4_K blocks"
    gw.write(tmp_path / "twice.gguf", meta, one + one)
    cases["twice.gguf"] = "two tensors named t"
    gw.write(tmp_path / "whole.gguf", meta, [("t", 0, [1024], np.zeros(1024, np.float32))])
    raw = open(tmp_path / "whole.gguf", "rb").read()
    open(tmp_path / "cut.gguf", "wb").write(raw[:-64])
    cases["cut.gguf"] = "past the end"
    open(tmp_path / "header.gguf", "wb").write(raw[:40])
    cases["header.gguf"] = "past the end"
    open(tmp_path / "short.gguf", "wb").write(b"GGUF")
    cases["short.gguf"] = "too short"
    for name, words in cases.items():
        with pytest.raises(lib.SbError, match=words):
            gguf.GgufFile(tmp_path / name)
    with pytest.raises(lib.SbError, match="cannot open"):
        gguf.GgufFile(tmp_path / "absent.gguf")
    # a readable file of another architecture gives no target configuration
    with pytest.raises(lib.SbError, match="architecture is 'llama'"):
        gguf.GgufFile(tmp_path / "whole.gguf").target_config()


def test_reader_takes_the_parts_of_a_split_file(tiny_file, tmp_path):
    """The tiny model's tensors dealt over three parts as gguf-split writes them (every part a GGUF with split.no, split.count
    and split.tensors.count; the model's metadata in the first): read together they are the whole file; alone, out of order or
    short of a part they are refused."""
    from splash_b200 import gguf, lib
    path, cfg, w, _ = tiny_file
    whole = gguf.GgufFile(path)
    tensors = whole.tensors()
    model_meta = [("general.architecture", gw.STRING, "qwen35"), ("qwen35.block_count", gw.U32, 4), ("some.array", gw.ARRAY, (gw.I32, [3, -1, 4]))]
    cuts = [0, 20, 41, len(tensors)]
    parts = []
    for i in range(3):
        meta = (model_meta if i == 0 else []) + [("split.no", gw.U16, i), ("split.count", gw.U16, 3), ("split.tensors.count", gw.I32, len(tensors))]
        part = str(tmp_path / f"tiny-{i + 1:05d}-of-00003.gguf")
        gw.write(part, meta, [(t["name"], t["type"], t["dims"], t["data"]) for t in tensors[cuts[i]:cuts[i + 1]]])
        parts.append(part)
    split = gguf.GgufFile(parts)
    got = split.tensors()
    assert [t["name"] for t in got] == [t["name"] for t in tensors]
    for a, b in zip(got, tensors):
        assert a["type"] == b["type"] and a["dims"] == b["dims"] and np.array_equal(a["data"], b["data"])
    assert split.meta("qwen35.block_count") == 4 and split.meta("split.count") == 3
    assert np.array_equal(split.array("some.array"), [3.0, -1.0, 4.0]) and split.array("no.such") is None
    assert split.find("blk.3.attn_v.weight") is not None
    for wrong, words in (([parts[1]], "part 2 of 3"), ([parts[0], parts[2], parts[1]], "given as part 2"), (parts[:2], "of 3 of a split"),
                         ([parts[0], parts[1], parts[1]], "two tensors named")):
        with pytest.raises(lib.SbError, match=words):
            gguf.GgufFile(wrong)


@pytest.mark.gpu
def test_loader_fills_a_target_that_steps_like_the_oracle(tiny_file):
    from splash_b200 import gguf, lib
    lib.init(0)
    path, cfg, w, _ = tiny_file
    t, f = gguf.load_target(path, page_tokens=cfg["page_tokens"], kv_scale_f16=cfg["kv_scale_f16"], max_context=cfg["max_context"])
    for (layer, name), want in w.items():
        got = t.download(layer, name, want.dtype, want.shape)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (layer, name)
    s = mo.make_state(cfg, 1000, 5)
    mo.upload(t, {}, s)
    t.reset(1000)
    tokens = mo.draft_chain(cfg, w, s, 17, rows=16, seed=0)
    want = mo.verify_step(cfg, w, s, tokens, advance=True)
    t.verify(tokens, flags=1)
    assert lib.device_status() == 0
    logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
    scale = np.abs(want["logits"]).max()
    assert np.abs(logits - want["logits"]).max() <= 2e-2 * scale and np.median(np.abs(logits - want["logits"])) <= 2e-3 * scale


@pytest.mark.gpu
def test_loader_refuses_files_that_do_not_fit_the_target(tiny_file, tmp_path):
    from splash_b200 import gguf, lib, target
    lib.init(0)
    path, cfg, w, _ = tiny_file
    runtime = dict(page_tokens=cfg["page_tokens"], kv_scale_f16=cfg["kv_scale_f16"], max_context=cfg["max_context"])
    f = gguf.GgufFile(path)
    # another model's target
    other = target.Target(**dict(cfg, q_heads=4))
    assert f.l.sb_target_load_gguf(other.handle, f.handle) == -1 and b"query heads" in f.l.sb_last_error()
    other.close()
    # a tensor missing
    missing = str(tmp_path / "missing.gguf")
    model_to_gguf(missing, cfg, w, drop=("blk.1.ssm_a",))
    with pytest.raises(lib.SbError, match="no tensor blk.1.ssm_a"):
        gguf.load_target(missing, **runtime)
    # a tensor of another format than a target of one format a kind holds (the target made for the file takes it: below)
    import quant_fixtures as qf
    mixed = str(tmp_path / "mixed.gguf")
    v_rows = cfg["kv_heads"] * cfg["head_dim"]
    model_to_gguf(mixed, cfg, w, replace={"blk.3.attn_v.weight": (gw.GGML["Q6_K"], [cfg["hidden"], v_rows], qf.realistic(4, v_rows, cfg["hidden"], seed=1))})
    uniform = target.Target(**cfg)
    with pytest.raises(lib.SbError, match="blk.3.attn_v.weight is Q6_K"):
        gguf.load_into(uniform, gguf.GgufFile(mixed))
    uniform.close()
    # a type that no kernel here reads
    q5 = str(tmp_path / "q5.gguf")
    model_to_gguf(q5, cfg, w, replace={"blk.0.attn_qkv.weight": (gw.GGML["Q5_K"], [cfg["hidden"], 2048], np.zeros(2048 * 4 * 176, np.uint8))})
    with pytest.raises(lib.SbError, match="Q5_K, which no kernel"):
        gguf.load_target(q5, **runtime)


@pytest.mark.gpu
def test_loader_fills_a_moe_target_that_steps_like_the_oracle(tmp_path):
    """A qwen35moe file: router, stacked routed experts (one tensor of three extents each) and the shared expert."""
    from splash_b200 import gguf, lib
    lib.init(0)
    cfg = dict(tiny_config(), moe_experts=16, moe_top_k=4, moe_intermediate=256)
    w = mo.make_weights(cfg, 6)
    path = str(tmp_path / "moe.gguf")
    model_to_gguf(path, cfg, w, arch="qwen35moe")
    t, f = gguf.load_target(path, page_tokens=cfg["page_tokens"], kv_scale_f16=cfg["kv_scale_f16"], max_context=cfg["max_context"])
    assert t.config["moe_experts"] == 16 and t.config["moe_top_k"] == 4 and t.config["moe_intermediate"] == 256
    for (layer, name), want in w.items():
        got = t.download(layer, name, want.dtype, want.shape)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (layer, name)
    s = mo.make_state(cfg, 500, 5)
    mo.upload(t, {}, s)
    t.reset(500)
    tokens = mo.draft_chain(cfg, w, s, 17, rows=16, seed=0)
    want = mo.verify_step(cfg, w, s, tokens, advance=True)
    t.verify(tokens, flags=1)
    assert lib.device_status() == 0
    logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
    scale = np.abs(want["logits"]).max()
    assert np.abs(logits - want["logits"]).max() <= 2e-2 * scale and np.median(np.abs(logits - want["logits"])) <= 2e-3 * scale


@pytest.mark.gpu
@pytest.mark.parametrize("lanes", [1, 2])
def test_a_file_of_mixed_formats_loads_and_steps_like_the_oracle(tmp_path, lanes):
    """The mix of llama.cpp's Q4_K_M: attn_v, a GDN layer's attn_gate, an out projection and some ffn_down tensors in Q6_K
    (one more in Q8_0) among Q4_K ones. The target made for the file holds each tensor in its format; the layers' fused input
    projections run as one launch a tensor. One lane (the 16-row kernel, two fragment layouts of the input) and two lanes
    (the many-row kernel from images)."""
    import quant_fixtures as qf
    from splash_b200 import gguf, lib
    lib.init(0)
    cfg = tiny_config()
    w = mo.make_weights(cfg, 9)
    H, D = cfg["hidden"], cfg["head_dim"]
    q, kv = cfg["q_heads"] * D * 2, cfg["kv_heads"] * D
    conv, VW = (2 * 4 + 8) * 128, 8 * 128
    rows = w.pop((3, "in_proj"))
    w[3, "in_parts"] = [(0, rows[:q]), (0, rows[q:q + kv]), (4, qf.realistic(4, kv, H, seed=21))]
    rows = w.pop((1, "in_proj"))
    w[1, "in_parts"] = [(0, rows[:conv]), (4, qf.realistic(4, VW, H, seed=22))]
    rows = w.pop((2, "in_proj"))
    w[2, "in_parts"] = [(6, qf.realistic(6, conv, H, seed=23)), (0, rows[conv:])]
    w[0, "ffn_down"], w[0, "ffn_down_fmt"] = qf.realistic(4, H, cfg["intermediate"], seed=24), 4
    w[2, "ffn_down"], w[2, "ffn_down_fmt"] = qf.realistic(6, H, cfg["intermediate"], seed=25), 6
    w[1, "out_proj"], w[1, "out_proj_fmt"] = qf.realistic(4, H, VW, seed=26), 4
    path = str(tmp_path / "mixed.gguf")
    model_to_gguf(path, cfg, w)
    t, f = gguf.load_target(path, page_tokens=cfg["page_tokens"], kv_scale_f16=cfg["kv_scale_f16"], max_context=cfg["max_context"], lanes=lanes)
    assert [t.tensor_format(3, n) for n in ("attn_q", "attn_k", "attn_v")] == [0, 0, 4]
    assert [t.tensor_format(2, n) for n in ("attn_qkv", "attn_gate", "ffn_down")] == [6, 0, 6] and t.tensor_format(1, "out_proj") == 4
    assert t.tensor_format(0, "in_proj") == 0
    with pytest.raises(lib.SbError):
        t.tensor(3, "in_proj")                            # (held tensor by tensor)
    for layer, stems in ((3, ("attn_q", "attn_k", "attn_v")), (1, ("attn_qkv", "attn_gate")), (2, ("attn_qkv", "attn_gate"))):
        for stem, (fmt, part) in zip(stems, w[layer, "in_parts"]):
            assert np.array_equal(t.download(layer, stem, np.uint8, part.shape), part), (layer, stem)
    positions = [700, 33][:lanes]
    states = [mo.make_state(cfg, positions[i], 5 + i) for i in range(lanes)]
    for i, s in enumerate(states):
        mo.upload(t, {}, s, lane=i)
    t.reset_lanes(np.array(positions, np.uint32)) if lanes > 1 else t.reset(positions[0])
    for step in range(2):
        blocks = np.stack([mo.draft_chain(cfg, w, states[i], 17 + i, rows=16, seed=step) for i in range(lanes)])
        wants = [mo.verify_step(cfg, w, states[i], blocks[i], advance=True) for i in range(lanes)]
        got = t.verify_lanes(blocks, flags=1) if lanes > 1 else [t.verify(blocks[0], flags=1)]
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (16 * lanes, cfg["vocab"]))
        for i in range(lanes):
            want = wants[i]
            scale = np.abs(want["logits"]).max()
            err = np.abs(logits[16 * i:16 * i + 16] - want["logits"])
            assert err.max() <= 2e-2 * scale and np.median(err) <= 2e-3 * scale, (step, i)
            states[i]["committed"] += got[i][1] - want["retained"]     # follow the device's own choice at near ties
            states[i]["pending_rows"] = got[i][1]


def test_reader_survives_damaged_files(tmp_path):
    """Truncations and flipped bytes of a small valid file: the reader opens what is still a GGUF and refuses the rest with an
    error; it never reads outside the mapping (a fault would end the test run)."""
    from splash_b200 import gguf, lib
    meta = [("general.architecture", gw.STRING, "qwen35"), ("a.count", gw.U32, 7), ("a.list", gw.ARRAY, (gw.F32, [1.0, 2.0, 3.0])),
            ("a.names", gw.ARRAY, (gw.STRING, ["x", "yy", "zzz"])), ("a.flag", gw.BOOL, 1), ("a.big", gw.U64, 2 ** 40)]
    tensors = [("t0", 0, [8, 4], np.arange(32, dtype=np.float32)), ("t1", 12, [256, 2], np.zeros(288, np.uint8)),
               ("t2", 30, [16], np.zeros(16, np.uint16))]
    good = tmp_path / "good.gguf"
    gw.write(good, meta, tensors)
    raw = bytearray(open(good, "rb").read())
    rng = np.random.default_rng(1)
    opened = refused = 0
    for trial in range(400):
        data = bytearray(raw)
        kind = trial % 4
        if kind == 0:
            data = data[:int(rng.integers(0, len(data)))]
        elif kind == 1:
            for _ in range(int(rng.integers(1, 4))):
                data[int(rng.integers(0, min(len(data), 400)))] = int(rng.integers(0, 256))      # in the header
        elif kind == 2:
            at = int(rng.integers(0, min(len(data), 400) - 8))
            data[at:at + 8] = (2 ** 64 - 1 - int(rng.integers(0, 1000))).to_bytes(8, "little")    # a huge count, length or offset
        else:
            at = int(rng.integers(0, min(len(data), 400) - 4))
            data[at:at + 4] = int(rng.integers(0, 2 ** 32)).to_bytes(4, "little")
        path = tmp_path / "damaged.gguf"
        open(path, "wb").write(bytes(data))
        try:
            f = gguf.GgufFile(path)
            for t in f.tensors():
                assert len(t["data"]) == 0 or int(t["data"][0]) >= 0 and int(t["data"][-1]) >= 0   # the tensor's bytes are inside the mapping
            f.meta("a.count"), f.array("a.list")
            f.close()
            opened += 1
        except lib.SbError:
            refused += 1
    assert opened + refused == 400 and refused >= 150 and opened >= 20, (opened, refused)
