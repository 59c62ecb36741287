"""A closed decode loop on the tiny model: a prompt enters the cache as prompt blocks, then every cycle proposes the
request's own lookup chain (prompt lookup), verifies it as the block's chain and keeps what the target accepted. Greedy
speculative decoding selects what plain decoding selects, whatever the proposals, sampling penalties over the output
included: the loop's tokens are held against the same model stepped one row at a time."""
import numpy as np
import pytest

import model_oracle as mo

pytestmark = pytest.mark.gpu


_weights = {}


def _model(seed):
    """The tiny model with the test oracle's synthetic tensors (their logits do not collapse onto one token) and an empty cache."""
    from splash_b200 import lib, target
    lib.init(0)
    cfg = dict(target.TINY)
    t = target.Target(**cfg)
    if seed not in _weights:
        _weights[seed] = (mo.make_weights(cfg, seed), mo.make_state(cfg, 0, seed + 1))
    mo.upload(t, *_weights[seed])
    t.reset(0)
    return lib, target, t, cfg


def _prefill(target, t, prompt):
    token = None
    for at in range(0, len(prompt), 16):
        block = prompt[at:at + 16]
        tokens, retained, _, _ = t.verify(block, flags=target.ADVANCE | target.PROMPT)
        assert retained == len(block)
        token = int(tokens[len(block) - 1])
    return token


def _generate(seed, prompt, count, speculate, history=None):
    """`history`: tokens the index holds before the prompt (text seen earlier): a source of proposals, not of context."""
    from splash_b200 import lookup
    lib, target, t, cfg = _model(seed)
    # Greedy decoding of a model with random weights settles on one token; penalties on what the output already holds keep it
    # moving. The host keeps the table current: every output token counted, the latest included, the prompt's tokens marked.
    t.set_penalties(1.3, 0.4, 0.6)
    words = np.zeros(cfg["vocab"], np.uint32)
    words[prompt] |= 0x80000000
    t.upload(-1, "penalty_words", words)
    first = _prefill(target, t, prompt)
    words[first] += 1
    out, index = [first], lookup.LookupIndex()
    if history is not None:
        index.append(history)
    index.append(prompt)
    index.append([first])
    proposed = accepted = cycles = 0
    while len(out) < count:
        chain = index.proposals(15) if speculate else np.zeros(0, np.uint32)
        block = np.concatenate([[out[-1]], chain]).astype(np.uint32)
        t.upload(-1, "penalty_words", words)
        tokens, retained, took, _ = t.verify(block, flags=target.ADVANCE)
        np.add.at(words, tokens[:retained], 1)
        assert lib.device_status() == 0 and retained == took + 1 and 1 <= retained <= len(block)
        assert np.array_equal(tokens[:took], chain[:took])        # the accepted proposals are the chain's first ones
        out += [int(x) for x in tokens[:retained]]
        index.append(tokens[:retained])
        proposed, accepted, cycles = proposed + len(chain), accepted + took, cycles + 1
    position = int(t.download(-1, "committed", np.uint32, (1,))[0])
    assert position == len(prompt) + len(out) - 1                  # everything but the latest token is in the cache
    t.close()
    return out[:count], proposed, accepted, cycles


def test_lookup_speculation_selects_what_plain_decoding_selects():
    rng = np.random.default_rng(1)
    unit = rng.integers(0, 32000, 23).astype(np.uint32)
    prompt = np.concatenate([unit, unit, unit, unit[:11]])        # 80 tokens whose suffix occurred before
    plain, _, _, plain_cycles = _generate(7, prompt, 64, speculate=False)
    fast, proposed, accepted, cycles = _generate(7, prompt, 64, speculate=True)
    assert plain_cycles == 63
    assert fast == plain, (fast, plain)
    assert cycles <= plain_cycles
    # With the plain run's own continuation in the index as text seen earlier, the proposals are right from the third
    # generated token on: the same tokens in a fraction of the cycles.
    known, proposed2, accepted2, cycles2 = _generate(7, prompt, 64, speculate=True, history=np.array(plain, np.uint32))
    assert known == plain
    assert accepted2 >= 48 and cycles2 <= 12, (accepted2, cycles2)


def _serve(prompts, counts, speculate, histories=None):
    """Three requests on a target of three lanes: ragged prompt blocks until every prompt is in, then decode cycles in which
    every lane verifies its own lookup chain (or just its last token), bounded by what its request may still take; a lane
    that is done sits the steps out. Returns the requests' tokens and the number of decode cycles."""
    from splash_b200 import lib, lookup, target
    lib.init(0)
    lanes = len(prompts)
    cfg = dict(target.TINY, lanes=lanes)
    t = target.Target(**cfg)
    if "serve" not in _weights:
        _weights["serve"] = (mo.make_weights(cfg, 21), [mo.make_state(cfg, 0, 30 + i) for i in range(lanes)])
    w, states = _weights["serve"]
    for i, s in enumerate(states):
        mo.upload(t, w if i == 0 else {}, s, lane=i)
    t.reset_lanes(np.zeros(lanes, np.uint32))
    t.set_penalties(1.3, 0.4, 0.6)
    words = np.zeros((lanes, cfg["vocab"]), np.uint32)
    for i, p in enumerate(prompts):
        words[i, p] |= 0x80000000
    t.upload(-1, "penalty_words", words)
    indexes = [lookup.LookupIndex() for _ in range(lanes)]
    for i in range(lanes):
        if histories is not None:
            indexes[i].append(histories[i])
        indexes[i].append(prompts[i])
    # prompts, 16 tokens a lane and step; a lane whose prompt is in sits out until the others' are
    at, out = [0] * lanes, [[] for _ in range(lanes)]
    while any(at[i] < len(prompts[i]) for i in range(lanes)):
        blocks = [prompts[i][at[i]:at[i] + 16] for i in range(lanes)]
        got = t.verify_lanes_ragged(blocks, flags=target.ADVANCE | target.PROMPT)
        for i in range(lanes):
            assert got[i][1] == len(blocks[i])
            at[i] += len(blocks[i])
            if len(blocks[i]) and at[i] == len(prompts[i]):
                out[i].append(int(got[i][0][len(blocks[i]) - 1]))      # the request's first token
    for i in range(lanes):
        words[i, out[i][0]] += 1
        indexes[i].append(out[i])
    cycles = 0
    while any(len(out[i]) < counts[i] for i in range(lanes)):
        blocks = []
        for i in range(lanes):
            if len(out[i]) >= counts[i]:
                blocks.append(np.zeros(0, np.uint32))                   # done: the lane sits out
                continue
            chain = indexes[i].proposals(15) if speculate else np.zeros(0, np.uint32)
            blocks.append(np.concatenate([[out[i][-1]], chain]).astype(np.uint32))
        t.upload(-1, "penalty_words", words)
        t.upload(-1, "remaining", np.array([max(1, counts[i] - len(out[i])) for i in range(lanes)], np.uint32))
        got = t.verify_lanes_ragged(blocks, flags=target.ADVANCE)
        assert lib.device_status() == 0
        for i in range(lanes):
            tokens, retained, took, _ = got[i]
            if not len(blocks[i]):
                assert retained == 0
                continue
            assert 1 <= retained <= min(len(blocks[i]), counts[i] - len(out[i]))
            out[i] += [int(x) for x in tokens]
            np.add.at(words[i], tokens, 1)
            indexes[i].append(tokens)
        cycles += 1
    positions = t.download(-1, "committed", np.uint32, (lanes,))
    for i in range(lanes):
        assert len(out[i]) == counts[i] and int(positions[i]) == len(prompts[i]) + counts[i] - 1
    t.close()
    return out, cycles


def test_three_requests_of_different_lengths_served_together():
    """Prompts of 40, 23 and 61 tokens, replies of 24, 40 and 9 tokens: with lookup chains (right ones, from the plain run's
    replies held as text seen earlier) the requests produce the tokens of plain one-row decoding in fewer cycles."""
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, 32000, n).astype(np.uint32) for n in (40, 23, 61)]
    counts = [24, 40, 9]
    plain, plain_cycles = _serve(prompts, counts, speculate=False)
    assert plain_cycles == max(counts) - 1
    for reply in plain:
        assert len(set(reply)) > len(reply) // 2          # (the penalties keep the replies from collapsing)
    fast, cycles = _serve(prompts, counts, speculate=True, histories=[np.array(r, np.uint32) for r in plain])
    assert fast == plain
    assert cycles <= plain_cycles // 3, (cycles, plain_cycles)
