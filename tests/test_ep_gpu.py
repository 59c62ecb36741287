"""Expert-parallel verify steps of the tiny MoE configuration on two GPUs, one process per GPU: each rank steps two lanes of
its own and holds half of the routed experts and a copy of the shared one; a block's rows meet their experts through the
ranks' exchange windows (dispatch, then combine). Every lane is held against its own CPU oracle lane, which runs the whole
block with all experts. Skipped where the machine has fewer than two GPUs."""
import ctypes
import multiprocessing as mp

import numpy as np
import pytest

import model_oracle as mo

pytestmark = pytest.mark.gpu
WORLD, LANES, EXPERTS = 2, 2, 16
POSITIONS = np.array([2048, 700, 1300, 333], np.uint32)


def _config():
    from splash_b200 import target
    return dict(target.TINY, moe_experts=EXPERTS, moe_top_k=4, moe_intermediate=256)


def _cut(cfg, rank):
    """A rank's share of the whole model's tensors: its routed experts, then the shared one; everything else whole."""
    per = EXPERTS // WORLD

    def cut(layer, name, array):
        if name in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
            a = np.asarray(array)
            rows = a.shape[0] // (EXPERTS + 1)
            return np.ascontiguousarray(np.concatenate([a[rank * per * rows:(rank + 1) * per * rows], a[EXPERTS * rows:]]))
        return array
    return cut


def _worker(rank, barrier, handles, results, step_blocks):
    try:
        from splash_b200 import lib, target, tp
        lib.init(rank)
        cfg = _config()
        t = target.Target(**cfg, lanes=LANES, ep_world=WORLD, ep_rank=rank)
        w = mo.make_weights(cfg, 5)
        for i in range(LANES):
            s = mo.make_state(cfg, int(POSITIONS[LANES * rank + i]), 6 + LANES * rank + i)
            mo.upload(t, w if i == 0 else {}, s, cut=_cut(cfg, rank), lane=i)
        t.reset_lanes(POSITIONS[LANES * rank:LANES * rank + LANES])

        def all_gather(mine):
            ctypes.memmove(ctypes.addressof(handles) + rank * tp.HANDLE_BYTES, mine, tp.HANDLE_BYTES)
            barrier.wait(timeout=120)
            return [bytes(handles[i * tp.HANDLE_BYTES:(i + 1) * tp.HANDLE_BYTES]) for i in range(WORLD)]

        tp.connect(t, all_gather)
        for step, blocks in enumerate(step_blocks):
            barrier.wait(timeout=120)
            got = t.verify_lanes(blocks[LANES * rank:LANES * rank + LANES], flags=target.ADVANCE | target.GRAPH)
            logits = t.download(-1, "logits", np.float32, (16 * LANES, cfg["vocab"]))
            results.put((rank, step, got, lib.device_status(), logits))
        barrier.wait(timeout=120)  # nobody unmaps its window while a peer may still write to it
        t.close()
    except Exception as e:
        results.put((rank, -1, repr(e), 1, None))
        try:
            barrier.abort()
        except Exception:
            pass


def test_two_ranks_of_two_lanes_match_four_oracle_lanes():
    from splash_b200 import lib
    if lib.device_count() < WORLD:
        pytest.skip(f"needs {WORLD} GPUs")
    cfg = _config()
    w = mo.make_weights(cfg, 5)
    states = [mo.make_state(cfg, int(POSITIONS[i]), 6 + i) for i in range(WORLD * LANES)]
    first = [31, 77, 4000, 9]
    steps, step_blocks, wants = 2, [], []
    for step in range(steps):
        blocks = np.stack([mo.draft_chain(cfg, w, states[i], first[i], rows=16, p_match=0.6, seed=10 * step + i) for i in range(len(states))])
        want = [mo.verify_step(cfg, w, states[i], blocks[i], advance=True) for i in range(len(states))]
        step_blocks.append(blocks), wants.append(want)
        first = [int(x["tokens"][-1]) for x in want]
    ctx = mp.get_context("spawn")
    barrier, results = ctx.Barrier(WORLD), ctx.Queue()
    handles = ctx.RawArray(ctypes.c_ubyte, WORLD * 64)
    procs = [ctx.Process(target=_worker, args=(r, barrier, handles, results, step_blocks)) for r in range(WORLD)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(WORLD * steps):
            rank, step, out, status, logits = results.get(timeout=600)
            assert step >= 0, f"rank {rank} failed: {out}"
            assert status == 0, f"rank {rank} step {step}: device status {status}"
            got[rank, step] = (out, logits)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    compared, diverged = 0, set()
    for step in range(steps):
        for lane in range(WORLD * LANES):
            if lane in diverged:
                continue
            rank, local = divmod(lane, LANES)
            out, logits = got[rank, step]
            tokens, retained, accepted, mask = out[local]
            want = wants[step][lane]
            err = np.abs(logits[16 * local:16 * local + 16] - want["logits"])
            scale = np.abs(want["logits"]).max()
            assert err.max() <= 3e-2 * scale and np.median(err) <= 2e-3 * scale, (step, lane)
            top2 = np.sort(want["logits"], axis=1)[:, -2:]
            if ((top2[:, 1] - top2[:, 0]) > 2.5 * err.max(axis=1))[:want["retained"]].all():
                assert (retained, accepted, mask) == (want["retained"], want["accepted"], want["mask"]), (step, lane)
                assert np.array_equal(tokens, want["tokens"]), (step, lane)
                compared += 1
            else:
                diverged.add(lane)   # the oracle's own choice was a near tie: the lane's later steps start elsewhere
    assert compared >= 4, compared


def _expiry_worker(rank, barrier, handles, results):
    try:
        import time
        from splash_b200 import lib, tp
        lib.init(rank)
        l = lib.load()
        P, U = ctypes.c_void_p, ctypes.c_uint32
        l.sb_ep_create.argtypes = [U, U, U, U, U, ctypes.POINTER(P)]
        l.sb_ep_export.argtypes = [P, P]
        l.sb_ep_connect.argtypes = [P, P]
        l.sb_ep_destroy.argtypes = [P]
        l.sb_ep_dispatch.argtypes = [P, P, P, P, P]
        l.sb_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
        rows, hidden, routes = 16, 256, 3
        g = P()
        lib.check(l.sb_ep_create(WORLD, rank, rows, hidden, routes, ctypes.byref(g)))
        mine = ctypes.create_string_buffer(tp.HANDLE_BYTES)
        lib.check(l.sb_ep_export(g, mine))
        ctypes.memmove(ctypes.addressof(handles) + rank * tp.HANDLE_BYTES, mine.raw, tp.HANDLE_BYTES)
        barrier.wait(timeout=120)
        lib.check(l.sb_ep_connect(g, bytes(handles[:WORLD * tp.HANDLE_BYTES])))
        out = None
        if rank == 0:   # the only rank that dispatches: its peer's flag never comes
            lib.check(l.sb_set_wait_limit_ns(5_000_000))   # 5 ms
            x = lib.DeviceBuffer(rows * hidden * 2)
            sel, wts = lib.DeviceBuffer(rows * routes * 4), lib.DeviceBuffer(rows * routes * 4)
            for b in (x, sel, wts):
                b.fill(0)
            t0 = time.time()
            lib.check(l.sb_ep_dispatch(None, g, x.ptr, sel.ptr, wts.ptr))
            lib.stream_sync()
            first = time.time() - t0
            status = lib.device_status()            # reads and clears the word
            # a kernel that finds the status word set does not wait: leave it set by a second expiry, then time a third call
            lib.check(l.sb_ep_dispatch(None, g, x.ptr, sel.ptr, wts.ptr))
            lib.stream_sync()
            again = lib.device_status()
            # the context is usable: a local operator runs and the status word stays clear
            y, w = lib.DeviceBuffer(rows * hidden * 2), lib.DeviceBuffer.from_numpy(np.ones(hidden, np.float32))
            lib.check(lib.ops().sb_rmsnorm(None, x.ptr, rows, hidden, hidden, w.ptr, y.ptr, hidden))   # (lib.ops() declares the argument types)
            lib.stream_sync()
            out = (first, status, again, lib.device_status())
            lib.check(l.sb_set_wait_limit_ns(0))
        barrier.wait(timeout=120)   # rank 1 keeps its window mapped until rank 0 is done
        results.put((rank, out, None))
        barrier.wait(timeout=120)
        l.sb_ep_destroy(g)
    except Exception as e:
        results.put((rank, None, repr(e)))
        try:
            barrier.abort()
        except Exception:
            pass


def test_a_wait_for_a_rank_that_never_joins_runs_out_and_says_so():
    """Failure made on the host: rank 1 connects its window and then never takes part. Rank 0's exchange waits for the flag
    that nothing sets, gives up after the limit set with sb_set_wait_limit_ns, records SB_DEV_WAIT_EXPIRED and returns; the
    context stays usable. No GPU faults or hangs: the wait is bounded by the clock."""
    from splash_b200 import lib
    if lib.device_count() < WORLD:
        pytest.skip(f"needs {WORLD} GPUs")
    ctx = mp.get_context("spawn")
    barrier, results = ctx.Barrier(WORLD), ctx.Queue()
    handles = ctx.RawArray(ctypes.c_ubyte, WORLD * 64)
    procs = [ctx.Process(target=_expiry_worker, args=(r, barrier, handles, results)) for r in range(WORLD)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(WORLD):
            rank, out, err = results.get(timeout=300)
            assert err is None, f"rank {rank} failed: {err}"
            got[rank] = out
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    first, status, again, after = got[0]
    assert status == 1 and again == 1          # SB_DEV_WAIT_EXPIRED, both times
    assert 0.004 < first < 2.0                 # it waited for the limit, not for the default 2 s
    assert after == 0                          # and the context carried on
