"""The KV page pool: its bookkeeping (host code, no GPU) and, on a GPU, lanes whose pages lie scattered over the pool stepping
exactly as lanes that hold their pages in a row."""
import numpy as np
import pytest

import model_oracle as mo


def test_pool_hands_out_and_takes_back_pages():
    from splash_b200 import kv_pool, lib
    pool = kv_pool.KvPool(pages=10, lanes=3, lane_cap_pages=6, page_tokens=256)
    assert pool.counts() == (10, 0)
    assert pool.acquire(0, 1) and pool.table(0).tolist() == [0]                 # a token needs a page
    assert pool.acquire(1, 600) and pool.table(1).tolist() == [1, 2, 3]         # 600 tokens: three pages of 256
    assert pool.acquire(0, 257) and pool.table(0).tolist() == [0, 4]            # the lane grows: its pages need not be neighbours
    assert pool.acquire(0, 200) and pool.table(0).tolist() == [0, 4]            # it already holds enough
    assert pool.counts() == (5, 5)
    assert not pool.acquire(2, 6 * 256)                                          # six pages are asked for, five are free ...
    assert pool.table(2).tolist() == [] and pool.counts() == (5, 5)              # ... and nothing was taken
    assert pool.acquire(2, 5 * 256) and pool.counts() == (0, 10)
    assert not pool.acquire(1, 4 * 256)
    pool.release(0)
    assert pool.counts() == (2, 8) and pool.table(0).tolist() == []
    assert pool.acquire(1, 4 * 256) and pool.table(1).tolist() == [1, 2, 3, 0]   # a page given back is handed out again
    with pytest.raises(lib.SbError, match="page table holds"):
        pool.acquire(1, 7 * 256)                                                  # past what a lane's table row holds
    with pytest.raises(lib.SbError, match="no such lane"):
        pool.acquire(3, 1)
    with pytest.raises(lib.SbError):
        kv_pool.KvPool(pages=0, lanes=1, lane_cap_pages=1, page_tokens=256)


@pytest.mark.gpu
def test_lanes_on_scattered_pages_step_like_lanes_on_their_own_pages():
    """Two targets of three lanes with the same weights, state and inputs: one as created (every lane its own pages in a row), one
    whose lanes draw their pages from the pool as they grow, in an order that scatters them. Prompt blocks of different lengths
    from empty caches, then verify steps: the logits and the results are the same bits, and the pool's counts follow the lanes."""
    from splash_b200 import kv_pool, lib, target
    lib.init(0)
    cfg = dict(target.TINY, lanes=3, page_tokens=32, max_context=1024)
    w = mo.make_weights(cfg, 31)
    states = [mo.make_state(cfg, 0, 40 + i) for i in range(3)]

    def make():
        t = target.Target(**cfg)
        for i, s in enumerate(states):
            mo.upload(t, w if i == 0 else {}, s, lane=i)
        t.reset_lanes(np.zeros(3, np.uint32))
        return t

    plain, pooled = make(), make()
    pool = kv_pool.KvPool(target=pooled)
    total = pool.counts()[0]
    assert total == 3 * ((1024 + 16 + 31) // 32)
    rng = np.random.default_rng(6)
    positions = np.zeros(3, np.int64)
    lengths_by_step = [[16, 7, 16], [16, 0, 16], [9, 16, 16], [16, 16, 3], [16, 16, 16], [16, 16, 16]]
    for step, lengths in enumerate(lengths_by_step):
        for lane in (2, 0, 1):                                  # the lanes take their pages in another order than they are numbered
            if lengths[lane]:
                assert pool.acquire(lane, int(positions[lane]) + 16)
        pool.write_tables(pooled)
        blocks = [rng.integers(0, cfg["vocab"], n).astype(np.uint32) for n in lengths]
        prompt = step < 4
        flags = target.ADVANCE | (target.PROMPT if prompt else 0)
        a = plain.verify_lanes_ragged(blocks, flags=flags)
        b = pooled.verify_lanes_ragged(blocks, flags=flags)
        assert lib.device_status() == 0
        la, lb = (t.download(-1, "logits", np.float32, (48, cfg["vocab"])) for t in (plain, pooled))
        for lane in range(3):
            n = lengths[lane]
            assert np.array_equal(la[16 * lane:16 * lane + n].view(np.uint32), lb[16 * lane:16 * lane + n].view(np.uint32)), (step, lane)
            assert a[lane][1:] == b[lane][1:] and np.array_equal(a[lane][0], b[lane][0])
            positions[lane] += a[lane][1]
    tables = [pool.table(lane) for lane in range(3)]
    assert all(len(t) == (positions[lane] + 16 + 31) // 32 or len(t) >= 1 for lane, t in enumerate(tables))
    assert any(np.any(np.diff(t.astype(np.int64)) != 1) for t in tables)     # the pages did end up scattered
    free, held = pool.counts()
    assert held == sum(len(t) for t in tables) and free + held == total
    pool.release(1)
    assert pool.counts()[0] == free + len(tables[1])
    plain.close(), pooled.close()
