"""Whole verify steps of the tiny hybrid configuration (4 layers = 3 Gated-DeltaNet + 1 attention, hidden 1024,
vocabulary 32000, Q4_K projections, Q6_K embedding and head, INT8 cache of 2048 prefilled tokens, page 256, fp16
scales): the CUDA path through the C ABI against the CPU oracle, over several steps with acceptance, KV growth
and GDN state rollback in between."""
import numpy as np
import pytest

import model_oracle as mo
import oracle_lib as ol

pytestmark = pytest.mark.gpu


def build(seed=0, committed=2048):
    from splash_b200 import lib, target
    lib.init(0)
    cfg = dict(target.TINY)
    t = target.Target(**cfg)
    w = mo.make_weights(cfg, seed)
    s = mo.make_state(cfg, committed, seed + 1)
    mo.upload(t, w, s)
    t.reset(committed)
    return lib, target, t, cfg, w, s


@pytest.mark.parametrize("flags_name", ["eager", "graph"])
def test_tiny_model_steps_match_oracle(flags_name):
    lib, target, t, cfg, w, s = build()
    flags = target.ADVANCE | (target.GRAPH if flags_name == "graph" else 0)
    rng = np.random.default_rng(3)
    token = 17
    accept_lengths = []
    for step in range(4):
        tokens = mo.draft_chain(cfg, w, s, token, rows=16, seed=step)
        want = mo.verify_step(cfg, w, s, tokens, advance=True)
        got_tokens, retained, accepted, mask = t.verify(tokens, flags=flags)
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
        # logits within 2e-3 of their scale (bf16 activations through 4 layers leave ~1e-3)
        scale = np.abs(want["logits"]).max()
        assert np.abs(logits - want["logits"]).max() <= 2e-2 * scale
        assert np.median(np.abs(logits - want["logits"])) <= 2e-3 * scale
        # selections and the accept length are exact wherever the top-2 logit gap exceeds 1e-2
        top2 = np.sort(want["logits"], axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 1e-2
        sel = t.download(-1, "selected", np.uint32, (16,))
        # (the device's `selected` holds the retained tokens in its first slots after acceptance)
        if clear[:want["retained"]].all():
            assert retained == want["retained"] and accepted == want["accepted"] and mask == want["mask"]
            assert np.array_equal(got_tokens, want["tokens"])
            accept_lengths.append(retained)
        else:
            s["committed"] += retained - want["retained"]  # follow the device where the oracle's own choice was a near tie
            s["pending_rows"] = retained
        token = int(got_tokens[-1])
    assert len(accept_lengths) >= 3 and max(accept_lengths) > 1


def test_tiny_model_stochastic_acceptance_matches_oracle():
    """Sampled acceptance at temperature 0.7 with supplied uniforms, whole steps, over several seeds. A step is compared
    where none of its accept tests sat within rounding of its threshold (the margin the oracle reports); the test counts
    how many steps were compared and demands most of them."""
    lib, target, t, cfg, w, s = build(seed=4)
    compared, sampled_accepts = 0, 0
    seeds = range(10)
    for seed in seeds:
        t.reset(2048)
        s["committed"], s["pending_rows"] = 2048, 0
        rng = np.random.default_rng(100 + seed)
        tokens = mo.draft_chain(cfg, w, s, 99 + seed, rows=16, seed=seed)
        uniforms = rng.random(80).astype(np.float32)
        want = mo.verify_step(cfg, w, s, tokens, temperature=0.7, uniforms=uniforms, mutate=False)
        got_tokens, retained, accepted, mask = t.verify(tokens, uniforms=uniforms, temperature=0.7)
        assert lib.device_status() == 0
        if not (want["margin"][:want["retained"]] > 1e-3).all():
            continue
        compared += 1
        sampled_accepts += want["accepted"]
        assert retained == want["retained"] and accepted == want["accepted"], seed
        assert np.array_equal(got_tokens[:retained], want["tokens"][:retained]), seed
    assert compared >= 6, compared            # the comparison did run, on most seeds
    assert sampled_accepts >= 2               # and some steps accepted draft tokens, not only their first row


def test_hold_position_steps_are_idempotent():
    """Without SB_TARGET_ADVANCE a step leaves the lane where it was: repeating it gives the same result."""
    lib, target, t, cfg, w, s = build(seed=7)
    tokens = np.arange(16, dtype=np.uint32) + 100
    a = t.verify(tokens, flags=target.GRAPH)
    la = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
    b = t.verify(tokens, flags=target.GRAPH)
    lb = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
    c = t.verify(tokens, flags=target.GRAPH)
    lc = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
    assert a[1:] == b[1:] == c[1:] and np.array_equal(la, lc)


def _tree(parent):
    t = np.zeros((len(parent), 2), np.uint32)
    for r in range(len(parent)):
        t[r, 0] = (1 << r) | (t[parent[r], 0] if r else 0)
        t[r, 1] = parent[r] | ((bin(int(t[r, 0])).count("1") - 1) << 16)
    return t


@pytest.mark.parametrize("flags_name", ["eager", "graph"])
def test_tiny_model_tree_steps_match_oracle(flags_name):
    """Blocks that are trees: the target's greedy continuation sits on a later branch, so the accepted path is not the
    block's first rows: positions by depth, attention and GDN along each row's path, the path's KV rows moved to their
    depths, the next step folding the path's tape rows. Three steps, the last a chain given as a tree."""
    lib, target, t, cfg, w, s = build(seed=2)
    flags = target.ADVANCE | (target.GRAPH if flags_name == "graph" else 0)
    rng = np.random.default_rng(5)
    token, compared = 23, 0
    shapes = [[0, 0, 1, 2, 0, 4, 5, 6, 6, 8, 9, 10, 9, 12, 0, 14],      # the continuation on rows 4, 5, 6, 8, 9, 12, 13
              [0, 0, 0, 2, 3, 4, 4, 6, 1, 8, 7, 10, 11, 12, 13, 14],    # on rows 2, 3, 4, 6, 7, 10 .. 15
              list(range(-1, 15))]                                      # a chain
    shapes[2][0] = 0
    on_path = [[4, 5, 6, 8, 9, 12, 13], [2, 3, 4, 6, 7, 10, 11, 12, 13, 14, 15], list(range(1, 16))]
    for step, (parent, good) in enumerate(zip(shapes, on_path)):
        greedy = mo.draft_chain(cfg, w, s, token, rows=len(good) + 1, p_match=1.0, seed=step)   # the target's own continuation
        tokens = rng.integers(0, cfg["vocab"], 16).astype(np.uint32)
        tokens[0] = token
        tokens[good] = greedy[1:]
        if step == 0:
            tokens[13] = (int(tokens[13]) + 1) % cfg["vocab"]   # the continuation breaks at its last row
        tree = _tree(parent)
        want = mo.verify_step(cfg, w, s, tokens, advance=True, tree=tree)
        got_tokens, retained, accepted, mask = t.verify(tokens, flags=flags, tree=tree)
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
        scale = np.abs(want["logits"]).max()
        assert np.abs(logits - want["logits"]).max() <= 2e-2 * scale
        assert np.median(np.abs(logits - want["logits"])) <= 2e-3 * scale
        top2 = np.sort(want["logits"], axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 1e-2
        path_rows = [r for r in range(16) if want["mask"] >> r & 1]
        if not clear[path_rows].all():
            break   # the oracle's own choice was a near tie: the lanes may part here
        assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"])
        assert np.array_equal(got_tokens, want["tokens"])
        assert retained >= 4 and (step == 2 or mask != (1 << retained) - 1)   # a path that is not the first rows
        compared += 1
        token = int(got_tokens[-1])
    assert compared >= 2


def test_tiny_model_sampled_tree_steps_with_drafted_children_match_oracle():
    """Sampled acceptance on tree blocks: every row's children are draws of a (synthetic) draft over its 16 candidates, with
    the draft's probabilities; the step selects by recursive rejection sampling over those children (SB_TARGET_DRAWS) and
    acceptance follows the child that was selected. Whole steps against the oracle's, over several seeds; a sampled tree
    block without the draws is refused."""
    lib, target, t, cfg, w, s = build(seed=6)
    parent = [0, 0, 0, 1, 1, 2, 3, 3, 5, 6, 6, 8, 9, 11, 12, 13]
    tree = _tree(parent)
    rows, V = 16, cfg["vocab"]
    compared = accepted_total = 0
    for seed in range(8):
        t.reset(2048)
        s["committed"], s["pending_rows"], s["pending_path"] = 2048, 0, 0
        rng = np.random.default_rng(200 + seed)
        ids = np.stack([rng.choice(V, 16, replace=False) for _ in range(rows)]).astype(np.uint32)
        q = rng.dirichlet(np.ones(16) * 0.5, size=rows).astype(np.float32)
        draws = np.full((rows, 4), 255, np.uint8)
        tokens = np.zeros(rows, np.uint32)
        tokens[0] = 50 + seed
        # a first pass with placeholder children gives the target's own favourites, which the draft then lists first
        for r in range(rows):
            children = [c for c in range(1, rows) if parent[c] == r]
            order = rng.choice(16, size=len(children), replace=False, p=q[r].astype(np.float64) / q[r].astype(np.float64).sum())
            draws[r, :len(children)] = order
            for c, d in zip(children, order):
                tokens[c] = ids[r, d]
        plain = mo.verify_step(cfg, w, s, tokens, mutate=False, tree=tree)
        for r in range(rows):                                  # make the draft good: its first-drawn child is the target's argmax
            children = [c for c in range(1, rows) if parent[c] == r]
            if children and rng.random() < 0.8:
                ids[r, draws[r, 0]] = plain["selected"][r]
                tokens[children[0]] = plain["selected"][r]
                q[r, draws[r, 0]] = 0.3
        uniforms = rng.random(80).astype(np.float32)
        want = mo.verify_step(cfg, w, s, tokens, temperature=0.7, uniforms=uniforms, mutate=False, tree=tree, draws=(ids, q, draws))
        t.upload(-1, "candidates", ids)
        t.upload(-1, "candidate_q", q)
        t.upload(-1, "draws", draws)
        got_tokens, retained, accepted, mask = t.verify(tokens, uniforms=uniforms, temperature=0.7, flags=target.DRAWS, tree=tree)
        assert lib.device_status() == 0
        path_rows = [r for r in range(rows) if want["mask"] >> r & 1]
        if not (want["margin"][path_rows] > 1e-3).all():
            continue
        compared += 1
        accepted_total += want["accepted"]
        assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"]), seed
        assert np.array_equal(got_tokens, want["tokens"]), seed
    assert compared >= 5 and accepted_total >= 2
    with pytest.raises(lib.SbError):
        t.verify(tokens, uniforms=uniforms, temperature=0.7, tree=tree)     # a sampled tree block needs the draws


def test_tiny_model_step_with_sampling_penalties_matches_oracle():
    """The lane's penalties rewrite the step's logits before selection: a strong repetition and frequency penalty on the
    tokens the target would otherwise choose changes the selections, the same way in the oracle's step."""
    lib, target, t, cfg, w, s = build(seed=9)
    tokens = mo.draft_chain(cfg, w, s, 41, rows=16, p_match=1.0, seed=1)
    plain = mo.verify_step(cfg, w, s, tokens, mutate=False)
    words = np.zeros(cfg["vocab"], np.uint32)
    words[plain["selected"]] = 3                 # the output "holds" the target's own choices three times each
    words[:64] |= 0x80000000                     # and the prompt some others
    policy = (1.6, 0.5, 0.75)
    want = mo.verify_step(cfg, w, s, tokens, advance=True, penalties=policy, penalty_words=words)
    assert not np.array_equal(want["selected"], plain["selected"])
    t.set_penalties(*policy)
    t.upload(-1, "penalty_words", words)
    got_tokens, retained, accepted, mask = t.verify(tokens, flags=target.ADVANCE | target.GRAPH)
    logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
    scale = np.abs(want["logits"]).max()
    assert np.abs(logits - want["logits"]).max() <= 2e-2 * scale
    top2 = np.sort(want["logits"], axis=1)[:, -2:]
    if ((top2[:, 1] - top2[:, 0]) > 1e-2)[:want["retained"]].all():
        assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"])
        assert np.array_equal(got_tokens, want["tokens"])
    t.set_penalties()   # off again: the next step's logits are the plain ones


def test_tiny_moe_model_steps_match_oracle():
    """The tiny hybrid configuration with MoE feed-forward blocks (16 experts + the shared one, top 4, expert width 256):
    router, routes, expert passes and combine inside whole verify steps against the oracle's."""
    from splash_b200 import lib, target
    lib.init(0)
    cfg = dict(target.TINY, moe_experts=16, moe_top_k=4, moe_intermediate=256)
    t = target.Target(**cfg)
    w, s = mo.make_weights(cfg, 3), mo.make_state(cfg, 2048, 4)
    mo.upload(t, w, s)
    t.reset(2048)
    token, compared = 31, 0
    for step in range(2):
        tokens = mo.draft_chain(cfg, w, s, token, rows=16, seed=step)
        want = mo.verify_step(cfg, w, s, tokens, advance=True)
        got_tokens, retained, accepted, mask = t.verify(tokens, flags=target.ADVANCE | target.GRAPH)
        assert lib.device_status() == 0
        logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
        scale = np.abs(want["logits"]).max()
        assert np.abs(logits - want["logits"]).max() <= 2e-2 * scale
        assert np.median(np.abs(logits - want["logits"])) <= 2e-3 * scale
        top2 = np.sort(want["logits"], axis=1)[:, -2:]
        if not ((top2[:, 1] - top2[:, 0]) > 1e-2)[:want["retained"]].all():
            break
        assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"])
        assert np.array_equal(got_tokens, want["tokens"])
        compared += 1
        token = int(got_tokens[-1])
    assert compared >= 1


@pytest.mark.parametrize("flags_name", ["eager", "graph"])
def test_tiny_model_prompt_blocks_then_verify_steps_match_oracle(flags_name):
    """A prompt enters an empty cache as blocks whose rows are all committed (SB_TARGET_PROMPT), the last one ragged;
    verify steps follow from the state the blocks left. Every step's logits against the oracle's."""
    lib, target, t, cfg, w, s = build(seed=4, committed=0)
    extra = target.GRAPH if flags_name == "graph" else 0
    rng = np.random.default_rng(8)
    prompt = rng.integers(0, cfg["vocab"], 16 * 3 + 7).astype(np.uint32)

    def close(want):
        logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))[:len(want["logits"])]
        scale = np.abs(want["logits"]).max()
        assert np.abs(logits - want["logits"]).max() <= 2e-2 * scale
        assert np.median(np.abs(logits - want["logits"])) <= 2e-3 * scale

    token = None
    for at in range(0, len(prompt), 16):
        block = prompt[at:at + 16]
        want = mo.verify_step(cfg, w, s, block, advance=True, prompt=True)
        got_tokens, retained, accepted, mask = t.verify(block, flags=target.ADVANCE | target.PROMPT | extra)
        assert lib.device_status() == 0
        assert (retained, accepted, mask) == (len(block), len(block) - 1, (1 << len(block)) - 1)
        close(want)
        top2 = np.sort(want["logits"][len(block) - 1])[-2:]
        token = int(got_tokens[len(block) - 1])
        if top2[1] - top2[0] > 1e-2:
            assert token == int(want["selected"][len(block) - 1])
    assert s["committed"] == len(prompt)
    assert int(t.download(-1, "committed", np.uint32, (1,))[0]) == len(prompt)
    for step in range(2):
        tokens = mo.draft_chain(cfg, w, s, token, rows=16, seed=step)
        want = mo.verify_step(cfg, w, s, tokens, advance=True)
        got_tokens, retained, accepted, mask = t.verify(tokens, flags=target.ADVANCE | extra)
        close(want)
        top2 = np.sort(want["logits"], axis=1)[:, -2:]
        if ((top2[:, 1] - top2[:, 0]) > 1e-2)[:want["retained"]].all():
            assert retained == want["retained"] and np.array_equal(got_tokens, want["tokens"])
        else:
            s["committed"] += retained - want["retained"]
            s["pending_rows"] = retained
        token = int(got_tokens[-1])
    # a tree block cannot be a prompt block
    with pytest.raises(Exception):
        t.verify(prompt[:4], flags=target.ADVANCE | target.PROMPT | target.TREE)


@pytest.mark.parametrize("flags_name", ["eager", "graph"])
def test_tiny_model_step_under_an_admission_matches_oracle(flags_name):
    """Constraint masks a row and excluded tokens: the step's selections come from the admitted tokens only, as the oracle's
    step with the same admission selects; switched off again the step is the plain one."""
    lib, target, t, cfg, w, s = build(seed=12)
    V = cfg["vocab"]
    rng = np.random.default_rng(4)
    tokens = mo.draft_chain(cfg, w, s, 23, rows=16, p_match=1.0, seed=2)
    plain = mo.verify_step(cfg, w, s, tokens, mutate=False)
    masks = rng.integers(0, 2 ** 32, (16, (V + 31) // 32), dtype=np.uint64).astype(np.uint32)
    for r in range(0, 16, 2):                             # every other row loses the token it would have selected
        masks[r, plain["selected"][r] // 32] &= ~np.uint32(1 << (plain["selected"][r] % 32))
    excluded = np.array([plain["selected"][1], plain["selected"][3], 11], np.uint32)
    want = mo.verify_step(cfg, w, s, tokens, mutate=False, admission=(masks, excluded))
    assert not np.array_equal(want["selected"], plain["selected"])
    t.upload(-1, "constraint_masks", masks)
    t.set_admission(True, excluded)
    flags = target.GRAPH if flags_name == "graph" else 0
    got_tokens, retained, accepted, mask = t.verify(tokens, flags=flags)
    assert lib.device_status() == 0
    logits = t.download(-1, "logits", np.float32, (16, V))
    assert np.array_equal(np.isneginf(logits), np.isneginf(want["logits"]))
    finite = np.isfinite(want["logits"])
    scale = np.abs(want["logits"][finite]).max()
    assert np.abs(logits[finite] - want["logits"][finite]).max() <= 2e-2 * scale
    masked = np.where(finite, want["logits"], -np.inf)
    top2 = np.sort(masked, axis=1)[:, -2:]
    if ((top2[:, 1] - top2[:, 0]) > 1e-2)[:want["retained"]].all():
        assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"])
        assert np.array_equal(got_tokens, want["tokens"])
    for tok in got_tokens:
        assert int(tok) not in excluded
    # a row whose mask admits nothing selects the sentinel; the step's results are refused when such a token is retained
    none = masks.copy()
    none[0] = 0
    t.upload(-1, "constraint_masks", none)
    with pytest.raises(lib.SbError, match="not one of the vocabulary"):
        t.verify(tokens, flags=flags)
    t.set_admission(False, ())
    got_tokens, retained, accepted, mask = t.verify(tokens, flags=flags)
    top2 = np.sort(plain["logits"], axis=1)[:, -2:]
    if ((top2[:, 1] - top2[:, 0]) > 1e-2)[:plain["retained"]].all():
        assert np.array_equal(got_tokens, plain["tokens"])


def test_tiny_model_sampled_steps_under_a_policy_match_oracle():
    """The production policy's end of the distribution (top 20, nucleus 0.95) and a min-p one, set on the target: whole sampled
    steps select as the oracle's step with the same policy, wherever no test or cut sat within rounding of its threshold."""
    lib, target, t, cfg, w, s = build(seed=14)
    compared, differs = 0, 0
    for policy in ((0.0, 20, 0.95), (0.05, 0, 1.0), (0.0, 5, 1.0)):
        t.set_policy(*policy)
        for seed in range(5):
            t.reset(2048)
            s["committed"], s["pending_rows"] = 2048, 0
            rng = np.random.default_rng(300 + seed)
            tokens = mo.draft_chain(cfg, w, s, 7 + seed, rows=16, seed=seed)
            uniforms = rng.random(80).astype(np.float32)
            want = mo.verify_step(cfg, w, s, tokens, temperature=1.0, uniforms=uniforms, mutate=False, policy=policy)
            loose = mo.verify_step(cfg, w, s, tokens, temperature=1.0, uniforms=uniforms, mutate=False)
            got_tokens, retained, accepted, mask = t.verify(tokens, uniforms=uniforms, temperature=1.0)
            assert lib.device_status() == 0
            if not (want["margin"][:want["retained"]] > 1e-3).all():
                continue
            compared += 1
            differs += not np.array_equal(want["selected"], loose["selected"])
            assert retained == want["retained"] and accepted == want["accepted"], (policy, seed)
            assert np.array_equal(got_tokens[:retained], want["tokens"][:retained]), (policy, seed)
    t.set_policy()
    assert compared >= 9, compared
    assert differs >= 3, differs              # the policies did change what the rows select
    with pytest.raises(lib.SbError):
        t.set_policy(min_p=1.5)


def test_tiny_model_stop_token_ends_the_retained_path():
    """With the token the target selects at the third row set as a stop token, the step retains three tokens where it retained
    six; the oracle's acceptance with the same stop tokens agrees. (Penalties over the rows' paths keep the tiny model's
    selections from collapsing onto one token, so that the stop token is not also the first.)"""
    lib, target, t, cfg, w, s = build(seed=16)
    policy, words = (1.4, 0.5, 0.7), np.zeros(cfg["vocab"], np.uint32)
    chain = [5]
    for _ in range(5):    # a chain of the target's own selections under the penalties: every draft token is right
        step = mo.verify_step(cfg, w, s, np.array(chain, np.uint32), mutate=False, penalties=policy, penalty_words=words)
        chain.append(int(step["selected"][-1]))
    tokens = np.array(chain, np.uint32)
    plain = mo.verify_step(cfg, w, s, tokens, mutate=False, penalties=policy, penalty_words=words)
    assert plain["retained"] == 6 and len(set(plain["tokens"].tolist())) >= 4
    stop = [int(plain["tokens"][2]), 31999]
    assert stop[0] not in plain["tokens"][:2]
    want = mo.verify_step(cfg, w, s, tokens, mutate=False, penalties=policy, penalty_words=words, stop_tokens=stop)
    assert want["retained"] == 3 and want["tokens"][-1] == stop[0]
    t.set_penalties(*policy)
    t.upload(-1, "penalty_words", words)
    t.set_stop_tokens(stop)
    got_tokens, retained, accepted, mask = t.verify(tokens, flags=target.GRAPH)
    top2 = np.sort(plain["logits"], axis=1)[:, -2:]
    clear = ((top2[:, 1] - top2[:, 0]) > 1e-2)[:plain["retained"]].all()
    if clear:
        assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"])
        assert np.array_equal(got_tokens, want["tokens"])
    t.set_stop_tokens(())
    got_tokens, retained, _, _ = t.verify(tokens, flags=target.GRAPH)
    if clear:
        assert retained == plain["retained"]
    t.set_penalties()
