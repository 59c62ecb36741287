"""Tensor-parallel verify steps of the tiny hybrid configuration on two and on four GPUs, one process per GPU: each rank holds its
share of the same seeded model (splash_b200.tp.shard), the ranks exchange through each other's memory, and the
results are held against the CPU oracle's whole-model step and against each other (every rank must hold the same
logits bit for bit). Skipped where the machine has fewer GPUs."""
import ctypes
import multiprocessing as mp

import numpy as np
import pytest

import model_oracle as mo

pytestmark = pytest.mark.gpu
COMMITTED = 2048


def _worker(rank, world, shots, barrier, handles, results, step_tokens):
    try:
        from splash_b200 import lib, target, tp
        lib.init(rank)
        lib.check(lib.load().sb_tp_set_exchange(shots))
        cfg = dict(target.TINY)
        t = target.Target(**cfg, tp_world=world, tp_rank=rank)
        sh = tp.share(cfg, world, rank)
        w, s = mo.make_weights(cfg, 0), mo.make_state(cfg, COMMITTED, 1)
        mo.upload(t, w, s, cut=lambda layer, name, arr: tp.shard(cfg, sh, layer, name, arr))
        t.reset(COMMITTED)

        def all_gather(mine):
            ctypes.memmove(ctypes.addressof(handles) + rank * tp.HANDLE_BYTES, mine, tp.HANDLE_BYTES)
            barrier.wait(timeout=120)
            return [bytes(handles[i * tp.HANDLE_BYTES:(i + 1) * tp.HANDLE_BYTES]) for i in range(world)]

        tp.connect(t, all_gather)
        for step, (tokens, tree) in enumerate(step_tokens):
            barrier.wait(timeout=120)
            got = t.verify(tokens, flags=target.ADVANCE | target.GRAPH, tree=tree)
            logits = t.download(-1, "logits", np.float32, (16, cfg["vocab"]))
            results.put((rank, step, got, lib.device_status(), logits))
        barrier.wait(timeout=120)  # nobody unmaps its window while a peer may still write to it
        t.close()
    except Exception as e:  # the parent turns this into a failure instead of waiting for a result
        results.put((rank, -1, repr(e), 1, None))
        try:
            barrier.abort()
        except Exception:
            pass


@pytest.mark.parametrize("world,shots", [(2, 0), (2, 2), (4, 0), (4, 1)])
def test_ranks_match_the_whole_model_oracle(world, shots):
    """Two ranks: every rank its own KV head. Four ranks: each KV head and its pages are held by two ranks, and the
    11 super-blocks of the intermediate width fall 3, 3, 3, 2. shots: how the shares travel (0: one shot with two ranks, two
    shots with more; 1, 2: forced), so both ways run on two and on four ranks."""
    from splash_b200 import lib, target
    if lib.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    steps = 4   # three chains, then a tree whose accepted path is not its first rows
    cfg = dict(target.TINY)
    w, s = mo.make_weights(cfg, 0), mo.make_state(cfg, COMMITTED, 1)
    step_tokens, wants, token = [], [], 17
    for step in range(steps):
        tree = None
        if step < 3:
            tokens = mo.draft_chain(cfg, w, s, token, rows=16, seed=step)
        else:
            parent, good = [0, 0, 1, 2, 0, 4, 5, 6, 6, 8, 9, 10, 9, 12, 0, 14], [4, 5, 6, 8, 9, 12, 13]
            greedy = mo.draft_chain(cfg, w, s, token, rows=len(good) + 1, p_match=1.0, seed=step)
            tokens = np.random.default_rng(8).integers(0, cfg["vocab"], 16).astype(np.uint32)
            tokens[0] = token
            tokens[good] = greedy[1:]
            tree = np.zeros((16, 2), np.uint32)
            for r in range(16):
                tree[r, 0] = (1 << r) | (tree[parent[r], 0] if r else 0)
                tree[r, 1] = parent[r] | ((bin(int(tree[r, 0])).count("1") - 1) << 16)
        want = mo.verify_step(cfg, w, s, tokens, advance=True, tree=tree)
        step_tokens.append((tokens, tree)), wants.append(want)
        token = int(want["tokens"][-1])
    ctx = mp.get_context("spawn")
    barrier, results = ctx.Barrier(world), ctx.Queue()
    handles = ctx.RawArray(ctypes.c_ubyte, world * 64)
    procs = [ctx.Process(target=_worker, args=(r, world, shots, barrier, handles, results, step_tokens)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(world * steps):
            rank, step, out, status, logits = results.get(timeout=600)
            assert step >= 0, f"rank {rank} failed: {out}"
            assert status == 0, f"rank {rank} step {step}: device status {status}"
            got[rank, step] = (out, logits)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    compared = 0
    for step in range(steps):
        out0, logits0 = got[0, step]
        for r in range(1, world):
            out1, logits1 = got[r, step]
            assert np.array_equal(logits0, logits1), "the ranks hold different logits"
            assert out0[1:] == out1[1:] and np.array_equal(out0[0], out1[0])
        want = wants[step]
        scale = np.abs(want["logits"]).max()
        assert np.abs(logits0 - want["logits"]).max() <= 2e-2 * scale
        assert np.median(np.abs(logits0 - want["logits"])) <= 2e-3 * scale
        top2 = np.sort(want["logits"], axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 1e-2
        if not clear[[r for r in range(16) if want["mask"] >> r & 1]].all():
            break  # the oracle's own choice was a near tie: later steps start from another position
        tokens, retained, accepted, mask = out0
        assert retained == want["retained"] and accepted == want["accepted"] and mask == want["mask"]
        assert np.array_equal(tokens, want["tokens"])
        compared += 1
    assert compared >= 1


def _op_worker(rank, world, shots, barrier, handles, results):
    try:
        import ctypes as C
        from splash_b200 import lib, tp
        import oracle_lib as ol
        lib.init(rank)
        L = lib.load()
        lib.check(L.sb_tp_set_exchange(shots))
        H, S, V, rows = 2048, 3, 4096, 13

        def all_gather(mine):
            C.memmove(C.addressof(handles) + rank * tp.HANDLE_BYTES, mine, tp.HANDLE_BYTES)
            barrier.wait(timeout=120)
            return [bytes(handles[i * tp.HANDLE_BYTES:(i + 1) * tp.HANDLE_BYTES]) for i in range(world)]

        g = tp.Group(world, rank, H, V, all_gather)
        rng = np.random.default_rng(100 + rank)
        parts = rng.standard_normal((S, 16, H)).astype(np.float32)
        res = ol.f2bf(np.random.default_rng(7).standard_normal((16, H)).astype(np.float32))   # the same on every rank
        pd, rd = lib.DeviceBuffer.from_numpy(parts), lib.DeviceBuffer.from_numpy(res)
        out = lib.DeviceBuffer(16 * H * 2 + 256)
        prep = lib.DeviceBuffer(int(L.sb_linear_prepared_bytes(H)))
        outs = []
        for index in range(3):       # three exchanges of one step: both inbox slots, then the first again
            barrier.wait(timeout=120)
            g.prepare_sum(None, index, pd.ptr, S, H, rd.ptr, out.ptr, rows, H, None, lib.FMT_Q4K, prep.ptr, 0)
            lib.stream_sync()
            outs.append(out.to_numpy(np.uint16, (16, H))[:rows].copy())
        # this rank's columns of the gather matrix, then the gather
        cols = V // world
        mine = rng.standard_normal((16, cols)).astype(np.float32)
        full = np.zeros((16, V), np.float32)
        full[:, rank * cols:(rank + 1) * cols] = mine
        lib.check(L.sb_upload(g.gather_ptr, full.ctypes.data_as(C.c_void_p), full.nbytes, None))
        lib.stream_sync()
        barrier.wait(timeout=120)
        g.all_gather(None, 3, rows, rank * cols, cols)
        g.advance(None, 4)
        lib.stream_sync()
        gathered = np.empty((16, V), np.float32)
        lib.check(L.sb_download(gathered.ctypes.data_as(C.c_void_p), g.gather_ptr, gathered.nbytes, None))
        lib.stream_sync()
        results.put((rank, parts, outs, mine, gathered[:rows].copy(), lib.device_status()))
        barrier.wait(timeout=120)
        g.close()
    except Exception as e:
        results.put((rank, None, repr(e), None, None, 1))
        try:
            barrier.abort()
        except Exception:
            pass


@pytest.mark.parametrize("shots", [1, 2])
def test_exchange_operators_against_numpy(shots):
    """sb_tp_prepare_sum and sb_tp_all_gather on two ranks against numpy: the new hidden state is
    bf16(residual + the ranks' shares added in rank order, each the rank's slices added in slice order), the same bits on
    both ranks, over three exchanges; the gathered matrix holds every rank's columns."""
    from splash_b200 import lib
    import oracle_lib as ol
    if lib.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    barrier, results = ctx.Barrier(world), ctx.Queue()
    handles = ctx.RawArray(ctypes.c_ubyte, world * 64)
    procs = [ctx.Process(target=_op_worker, args=(r, world, shots, barrier, handles, results)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(world):
            rank, parts, outs, mine, gathered, status = results.get(timeout=300)
            assert parts is not None, f"rank {rank} failed: {outs}"
            assert status == 0
            got[rank] = (parts, outs, mine, gathered)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    H, rows = 2048, 13
    shares = []
    for r in range(world):
        s = np.zeros((16, H), np.float32)
        for sl in range(3):
            s = s + got[r][0][sl]
        shares.append(s)
    total = np.zeros((16, H), np.float32)
    for s in shares:
        total = total + s
    res = ol.bf2f(ol.f2bf(np.random.default_rng(7).standard_normal((16, H)).astype(np.float32)))
    want = ol.f2bf((total + res).astype(np.float32))[:rows]
    for r in range(world):
        for o in got[r][1]:
            assert np.array_equal(o, want)
        cols = 4096 // world
        for src in range(world):
            assert np.array_equal(got[r][3][:, src * cols:(src + 1) * cols], got[src][2][:rows])
