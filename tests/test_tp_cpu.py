"""Host logic of tensor parallelism, no GPU: the ranks' shares tile the model, the cut of whole tensors into shares
loses and duplicates nothing, and two gloo ranks pass each other their handles in rank order."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import quant_fixtures as qf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shares_tile_the_27b_model(world):
    from splash_b200 import target, tp
    c = target.QWEN27B
    shares = [tp.share(c, world, r) for r in range(world)]
    for field, total in (("intermediate", c["intermediate"]), ("vocab", c["vocab"]), ("q_heads", c["q_heads"]),
                         ("gdn_key_heads", c["gdn_key_heads"]), ("gdn_value_heads", c["gdn_value_heads"])):
        first = field.replace("heads", "head") + "0"
        at = 0
        for s in shares:
            assert s[first] == at and s[field] > 0
            at += s[field]
        assert at == total
    assert all(s["intermediate"] % 256 == 0 and s["vocab0"] % 64 == 0 for s in shares)
    # every rank's query heads read the KV heads it holds, and its value heads the key heads it holds
    group, per_key = c["q_heads"] // c["kv_heads"], c["gdn_value_heads"] // c["gdn_key_heads"]
    for s in shares:
        for h in range(s["q_head0"], s["q_head0"] + s["q_heads"]):
            assert s["kv_head0"] <= h // group < s["kv_head0"] + s["kv_heads"]
        for h in range(s["gdn_value_head0"], s["gdn_value_head0"] + s["gdn_value_heads"]):
            assert s["gdn_key_head0"] <= h // per_key < s["gdn_key_head0"] + s["gdn_key_heads"]
    if world == 8:
        assert [s["intermediate"] // 256 for s in shares] == [9, 9, 9, 9, 8, 8, 8, 8]


def test_shares_that_do_not_divide_are_refused():
    from splash_b200 import lib, target, tp
    with pytest.raises(lib.SbError):
        tp.share(target.TINY, 3, 0)       # 8 heads over 3 ranks
    with pytest.raises(lib.SbError):
        tp.share(target.QWEN27B, 2, 2)    # rank outside the group


@pytest.mark.parametrize("world", [2, 4])
def test_cut_tensors_reassemble(world):
    from splash_b200 import lib, target, tp
    c = dict(target.TINY)
    H, D, I = c["hidden"], c["head_dim"], c["intermediate"]
    KH, VH, Q, K = c["gdn_key_heads"], c["gdn_value_heads"], c["q_heads"], c["kv_heads"]
    shares = [tp.share(c, world, r) for r in range(world)]
    gdn, attn = 0, c["attention_interval"] - 1
    # column splits: tag every row with its index; the shares hold each row exactly once (KV rows once per holder)
    for layer, rows, name in ((gdn, (2 * KH + 2 * VH) * 128, "in_proj"), (gdn, 2 * VH, "ssm_ab"), (gdn, (2 * KH + VH) * 128, "ssm_conv"),
                              (gdn, I, "ffn_gate"), (-1, c["vocab"], "output")):
        tags = np.arange(rows, dtype=np.int64).reshape(rows, 1)
        got = np.concatenate([tp.shard(c, s, layer, name, tags) for s in shares]).ravel()
        assert sorted(got.tolist()) == list(range(rows)), name
    tags = np.arange(Q * 2 * D + 2 * K * D, dtype=np.int64).reshape(-1, 1)
    got = np.concatenate([tp.shard(c, s, attn, "in_proj", tags) for s in shares]).ravel()
    holders = max(1, world // K)
    counts = np.bincount(got, minlength=len(tags))
    assert (counts[:Q * 2 * D] == 1).all() and (counts[Q * 2 * D:] == holders).all()
    # splits of the reduction dimension: whole blocks, in order, nothing lost
    for layer, name, fmt, n, k in ((gdn, "ffn_down", c["fmt_down"], H, I), (gdn, "out_proj", c["fmt_proj"], H, VH * 128),
                                   (attn, "out_proj", c["fmt_proj"], H, Q * D)):
        w = qf.realistic(fmt, 64, k, seed=5)
        parts = [tp.shard(c, s, layer, name, w) for s in shares]
        assert np.array_equal(np.concatenate(parts, axis=1), w), name
    # state follows its heads
    state = np.arange(VH * 4, dtype=np.float32).reshape(VH, 2, 2)
    assert np.array_equal(np.concatenate([tp.shard(c, s, gdn, "state0", state) for s in shares]), state)
    kv = np.arange(3 * K * 2 * 2, dtype=np.int8).reshape(3, K, 2, 2)
    for s in shares:
        assert np.array_equal(tp.shard(c, s, attn, "kv_k", kv), kv[:, s["kv_head0"]:s["kv_head0"] + s["kv_heads"]])


def test_tiled_value_heads_keep_their_columns():
    """With tiled heads, value head h writes column block (h % per_key) * KH + h / per_key; a rank's local rule on its own
    heads must pick the whole model's columns of exactly those heads."""
    from splash_b200 import target, tp
    c = dict(target.QWEN27B)
    KH, VH = c["gdn_key_heads"], c["gdn_value_heads"]
    per_key = VH // KH
    # a "weight" whose input column j carries the tag j / 128 (the column block), as one Q8_0-like block per 128 columns
    blocks = np.arange(VH, dtype=np.uint8).reshape(1, VH, 1).repeat(4 * 34, axis=2).reshape(1, -1)  # 4 Q8_0 blocks per head
    c["fmt_proj"] = 6
    for world in (2, 4, 8):
        for r in range(world):
            s = tp.share(c, world, r)
            part = tp.shard(c, s, 0, "out_proj", blocks).reshape(-1, 4 * 34)[:, 0]
            kl = s["gdn_key_heads"]
            for p, block in enumerate(part):   # local column block p belongs to local head hl
                hl = (p % kl) * per_key + p // kl
                h = s["gdn_value_head0"] + hl
                assert block == (h % per_key) * KH + h // per_key


def test_two_gloo_ranks_exchange_handles_in_rank_order():
    code = textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        from splash_b200.dist import Group
        from splash_b200 import target, tp
        g = Group(backend="gloo")
        mine = bytes([g.rank + 1]) * tp.HANDLE_BYTES
        got = g.all_gather_bytes(mine)
        assert got == [bytes([1]) * tp.HANDLE_BYTES, bytes([2]) * tp.HANDLE_BYTES], got
        s = tp.share(target.QWEN27B, g.world, g.rank)
        assert g.reduce_sum(s["intermediate"]) == target.QWEN27B["intermediate"]
        assert g.reduce_sum(s["vocab"]) == target.QWEN27B["vocab"]
        g.barrier()
        g.close()
        print("rank", g.rank, "ok")
    """ % ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29733", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, "-c", code], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "rank 0 ok" in outs[0] and "rank 1 ok" in outs[1]
