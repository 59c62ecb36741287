"""A closed decode loop on the tiny model: a prompt enters the cache as prompt blocks, then every cycle proposes the
request's own lookup chain (prompt lookup), verifies it as the block's chain and keeps what the target accepted. Greedy
speculative decoding selects what plain decoding selects, whatever the proposals: the loop's tokens are held against the
same model stepped one row at a time."""
import numpy as np
import pytest

import model_oracle as mo

pytestmark = pytest.mark.gpu


def _model(seed):
    from splash_b200 import lib, target
    lib.init(0)
    cfg = dict(target.TINY)
    t = target.Target(**cfg)
    t.randomize(seed, 0)
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
    first = _prefill(target, t, prompt)
    out, index = [first], lookup.LookupIndex()
    if history is not None:
        index.append(history)
    index.append(prompt)
    index.append([first])
    proposed = accepted = cycles = 0
    while len(out) < count:
        chain = index.proposals(15) if speculate else np.zeros(0, np.uint32)
        block = np.concatenate([[out[-1]], chain]).astype(np.uint32)
        tokens, retained, took, _ = t.verify(block, flags=target.ADVANCE)
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
    assert proposed > 0 and cycles <= plain_cycles
    # With the plain run's own continuation in the index as text seen earlier, the proposals are right from the third
    # generated token on: the same tokens in a fraction of the cycles.
    known, proposed2, accepted2, cycles2 = _generate(7, prompt, 64, speculate=True, history=np.array(plain, np.uint32))
    assert known == plain
    assert accepted2 >= 48 and cycles2 <= 12, (accepted2, cycles2)
