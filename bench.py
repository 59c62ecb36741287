#!/usr/bin/env python
"""Benchmark of the DFlash2 verify step on B200: verify tokens/s of a Qwen3.x-27B-shaped hybrid model
(64 layers at 3:1 Gated-DeltaNet : attention, Q4_K_M mix, batch 1, block 16, 32K-token INT8 paged KV
context, greedy acceptance) with seeded synthetic weights, cache and state written on the device.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--parallel tp|replicas]
    python bench.py --case linear|attention|gdn|moe|exchange ...   (one operator on one shape: bench_cases.py)

With N > 1 (one process per GPU under torchrun) the N GPUs run ONE lane tensor-parallel: every rank holds its share
of the model, the shares of out_proj / down meet through peer memory inside the next input conversion, the logits'
columns are gathered the same way (`scaling: "strong"`, value = the lane's tokens/s). `--parallel replicas` runs N
independent lanes instead (`scaling: "weak"`).

One JSON line on stdout (rank 0). `value` is device-resident steps; `e2e` goes through the host-facing call
sb_target_verify with pinned host buffers, copies and the result read-back inside the timed region;
`roofline` is the dominant kernel (the Q4_K gate/up projection) timed alone over the layers' weights;
`cpu_baseline` is the CPU oracle's port of the step's projections, attention and Gated-DeltaNet work on bounded samples;
`parity_check` is one checked step after the timed loops (finite logits, a sane accept length, equal logits on all ranks).
--impl reference times the reference's arithmetic for this path on the host cores: the oracle port
(the reference's own GPU kernels are Metal and cannot run here)."""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS = 16
CONTEXT = 32768
# Rows of the previous step's tape that every timed step folds into the Gated-DeltaNet state: the lane is held at its
# position (every step does the same work) but keeps this many pending rows, a typical accept length, so the fold a
# committing cycle performs stays inside the timed region.
FOLD_ROWS = 6
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from one ncu capture of that kernel
# at this bench's own shape (100,532,736 bytes read + 3,923,200 written), so no scaling. ncu cannot run inside a timed
# run; the figure is carried here and re-taken whenever the kernel changes.
DOMINANT_TRAFFIC_BYTES = 104455936


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_peak_tensor():
    """Dense bf16 TFLOP/s of a library GEMM timed alone (the burst figure: the projection launch is timed alone too)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi samples of one GPU's SM clock and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except Exception:
            self.proc.kill()
            out = ""
        clocks, mx, reasons = [], None, set()
        for line in out.splitlines():
            p = [x.strip() for x in line.split(",")]
            if len(p) < 6 or not p[0].isdigit():
                continue
            clocks.append(int(p[0]))
            mx = int(p[1])
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": mx, "reasons": sorted(reasons)}


def cpu_baseline(seconds_budget=20.0):
    """The oracle's port of the verify step's three kinds of work on the host cores, each on a bounded sample and scaled
    to a whole 27B-shaped step: the quantized projections (one FFN: gate/up in one pass, then down; scaled by weight
    bytes), INT8 paged attention (one KV head with its 6 query heads over the 32K context; scaled to 4 heads x 16 layers)
    and the Gated-DeltaNet step (one layer of 48 heads, folding 6 rows; x 48 layers). OpenMP over all host cores, the
    thread count set here (a launcher may export OMP_NUM_THREADS=1). Returns (tokens/s, threads, sample description)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    import quant_fixtures as qf
    o = ol.bind_ops(ol.load())
    o.so_threads.argtypes = [ctypes.c_int]
    threads = int(o.so_threads(os.cpu_count() or 1))
    H, I = 5120, 17408
    P = ol.ptr

    def best_of(run, budget, least=2, most=200):
        runs, spent = [], 0.0
        while len(runs) < least or (spent < budget and len(runs) < most):
            t0 = time.perf_counter()
            run()
            runs.append(time.perf_counter() - t0)
            spent += runs[-1]
        return min(runs), len(runs), spent

    # ---- projections: a slice of `n` of the FFN's 17408 intermediate columns, sized from a quick probe ----
    def ffn(n):
        wg, wu = qf.realistic(0, n, H, seed=1), qf.realistic(0, n, H, seed=2)
        w2 = np.ascontiguousarray(np.concatenate([wg, wu], axis=0))
        kd = max(256, n // 256 * 256)
        wd = qf.realistic(4, H, kd, seed=3)
        x, xa = qf.activations(ROWS, H), qf.activations(ROWS, kd, seed=1)
        act, out = np.zeros((ROWS, n), np.uint16), np.zeros((ROWS, H), np.uint16)

        def run():
            assert o.so_linear(0, P(w2), n, H, P(x), ROWS, 3, None, 0, P(act), n, 0, 0) == 0
            assert o.so_linear(4, P(wd), H, kd, P(xa), ROWS, 0, None, 0, P(out), H, 0, 0) == 0
        return run, w2.nbytes + wd.nbytes
    probe, _ = ffn(1024)
    dt, _, _ = best_of(probe, 0.0, least=1)
    n = int(min(I, max(1024, 1024 * seconds_budget / 6 / max(dt, 1e-3)))) // 256 * 256
    run, nbytes = ffn(n)
    ffn_s, ffn_runs, ffn_spent = best_of(run, seconds_budget / 3, least=3)
    proj_s = ffn_s * 15.89e9 / nbytes  # weight bytes of one 27B-shaped step

    # ---- attention: one KV head (6 query heads, D = 256) over 32K tokens of INT8 pages, 16 rows ----
    rng = np.random.default_rng(5)
    D, G, page = 256, 6, 256
    pages = (CONTEXT + page - 1) // page + 1
    kv = ol.HostKv(pages, 1, D, page, True)
    kv.fill_random(rng)
    table = np.arange(pages, dtype=np.uint32)
    queries = ol.f2bf(rng.standard_normal((ROWS, G, D)).astype(np.float32))
    qkv = ol.f2bf(rng.standard_normal((ROWS, G * 2 * D + 2 * D)).astype(np.float32))
    attn_out = np.zeros((ROWS, G * D), np.uint16)
    desc = kv.desc()
    o.so_attention.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_uint32] * 4 + [ctypes.c_void_p] * 2 + [ctypes.c_uint32] + [ctypes.c_void_p] * 2 + [ctypes.c_uint32, ctypes.c_void_p]
    attn_s, attn_runs, attn_spent = best_of(
        lambda: o.so_attention(P(queries), P(qkv), qkv.shape[1], ROWS, G, 1, ctypes.byref(desc), P(table), CONTEXT - ROWS, None, P(attn_out), G * D, None),
        seconds_budget / 3, least=1)
    attn_step_s = attn_s * 4 * 16

    # ---- Gated DeltaNet: one layer (16 key / 48 value heads), 16 rows, folding 6 pending rows ----
    KH, VH = 16, 48
    KW, VW = KH * 128, VH * 128
    C = 2 * KW + VW
    bf = lambda shape, sc: ol.f2bf((rng.standard_normal(shape) * sc).astype(np.float32))
    g = dict(qkvz=bf((ROWS, C + VW), 1.0), b=bf((ROWS, VH), 1.0), a=bf((ROWS, VH), 1.0), conv_w=bf((C, 4), 0.4),
             a_scale=(-np.exp(rng.uniform(-3, 0.5, VH))).astype(np.float32), dt_bias=bf((VH,), 0.5), norm_w=np.ones(128, np.float32),
             cs_in=bf((3, C), 1.0), cs_out=np.zeros((3, C), np.uint16), state=(rng.standard_normal((VH, 128, 128)) * 0.05).astype(np.float32),
             state_out=np.zeros((VH, 128, 128), np.float32), hidden=np.zeros((ROWS, VW), np.uint16))
    pend = dict(inputs=bf((ROWS, C), 1.0), k=bf((ROWS, KW), 0.09), v=bf((ROWS, VW), 0.5), beta=ol.f2bf(rng.uniform(0.1, 0.9, (ROWS, VH)).astype(np.float32)),
                decay=rng.uniform(0.5, 1.0, (ROWS, VH)).astype(np.float32))
    step = dict(inputs=np.zeros((ROWS, C), np.uint16), k=np.zeros((ROWS, KW), np.uint16), v=np.zeros((ROWS, VW), np.uint16),
                beta=np.zeros((ROWS, VH), np.uint16), decay=np.zeros((ROWS, VH), np.float32))
    tape = lambda t: ol.SoGdnTape(P(t["inputs"]), P(t["k"]), P(t["v"]), P(t["beta"]), P(t["decay"]))
    ga = ol.SoGdnArgs(P(g["qkvz"]), P(g["b"]), P(g["a"]), P(g["conv_w"]), P(g["a_scale"]), P(g["dt_bias"]), P(g["norm_w"]), P(g["cs_in"]), P(g["cs_out"]),
                      P(g["state"]), P(g["state_out"]), tape(pend), tape(step), P(g["hidden"]), ROWS, FOLD_ROWS, KH, VH, C + VW, VH, VW, 1, None, 0)
    gdn_s, gdn_runs, gdn_spent = best_of(lambda: o.so_gdn_verify(ctypes.byref(ga)), seconds_budget / 6, least=3)
    gdn_step_s = gdn_s * 48

    step_seconds = proj_s + attn_step_s + gdn_step_s
    sample = (f"oracle port on {threads} OpenMP threads: projections from an FFN slice of {n} of {I} columns ({nbytes / 1e6:.0f} MB of weights, best of "
              f"{ffn_runs} runs) scaled by weight bytes = {proj_s:.2f} s; attention of one KV head x 6 query heads over {CONTEXT} tokens (best of {attn_runs}) "
              f"x 4 heads x 16 layers = {attn_step_s:.2f} s; one Gated-DeltaNet layer of {VH} heads folding {FOLD_ROWS} rows (best of {gdn_runs}) x 48 layers = "
              f"{gdn_step_s:.2f} s; {ffn_spent + attn_spent + gdn_spent:.0f} s of CPU work in all")
    return ROWS / step_seconds, threads, sample


def main():
    if "--case" in sys.argv[1:]:  # one operator on one shape (bench_cases.py), not the benchmark
        import bench_cases
        argv = sys.argv[1:]
        argv.remove("--case")
        return bench_cases.main(argv)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--tiny", action="store_true", help="the 4-layer configuration (a smoke run, not the benchmark)")
    ap.add_argument("--moe", action="store_true", help="the 35B-A3B-shaped MoE model, one lane of 16 rows at an 8K context (an extra measurement, not the benchmark)")
    ap.add_argument("--tp-shots", type=int, default=0, choices=(0, 1, 2), help="how tensor-parallel shares travel (sb_tp_set_exchange); 0: by the number of ranks")
    ap.add_argument("--parallel", default="tp", choices=("tp", "replicas", "ep"), help="what N > 1 GPUs do: one lane tensor-parallel, N independent lanes, or (--moe --lanes L) the L lanes dealt to the ranks with the experts divided among them")
    ap.add_argument("--lanes", type=int, default=1, help="concurrent requests stepped together on each GPU, 16 rows each (an extra measurement, not the benchmark)")
    ap.add_argument("--nvfp4", action="store_true", help="NVFP4 projections (e2m1 codes, e4m3 scale per 16, fp32 scale) instead of the Q4_K_M mix (an extra measurement)")
    ap.add_argument("--context", type=int, default=0, help="tokens of context each lane holds (default: the workload's)")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    workload = "tiny hybrid verify" if args.tiny else "Qwen3.x-27B-shaped hybrid verify, Q4_K_M mix, batch 1, block 16, 32K INT8 paged KV, greedy"
    expert_parallel = args.parallel == "ep" and world > 1
    if expert_parallel and not (args.moe and args.lanes % world == 0 and args.lanes // world >= 2):
        raise SystemExit("--parallel ep needs --moe and --lanes a multiple of the ranks, two lanes a rank at least")
    if args.moe:
        workload = "35B-A3B-shaped MoE verify (256 experts + shared, top 8, router logits ~ N(0,1) given), Q4_K, batch 1, block 16, 8K INT8 paged KV, rejection sampling at temperature 0.7 with supplied uniforms"
        args.tiny = True  # (the extra legs of the benchmark are for the 27B workload only)
        if not expert_parallel:
            args.parallel = "replicas"
    L = max(1, args.lanes)
    total_lanes = L
    if expert_parallel:
        L //= world  # a rank's lanes
    if args.nvfp4:
        workload = workload.replace("Q4_K_M mix", "NVFP4 projections")
        args.parallel = "replicas"
    if args.context:
        workload = workload.replace("32K", f"{args.context // 1024}K")
    if total_lanes > 1:
        workload = f"{total_lanes} lanes stepped together: " + workload.replace("batch 1", f"batch {total_lanes}")
        if not expert_parallel:
            args.parallel = "replicas"

    if args.impl == "reference":
        if rank != 0:
            return
        tps, cores, sample = cpu_baseline(30.0)
        print(json.dumps({"impl": "reference", "metric": "verify_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": ROWS / tps * 1e3, "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                          "config": {"workload": workload},
                          "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
                          "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    from splash_b200 import lib, target
    from splash_b200.dist import Group
    group = Group("nccl")
    lib.init(local)
    lib.check(lib.load().sb_tp_set_exchange(args.tp_shots))
    cfg = dict(target.QWEN35B_A3B if args.moe else target.TINY if args.tiny else target.QWEN27B)
    context = args.context or (8192 if args.moe else 2048 if args.tiny else CONTEXT)
    cfg["max_context"] = max(cfg["max_context"], context + 1024)
    if args.nvfp4:
        cfg.update(fmt_proj=lib.FMT_NVFP4, fmt_down=lib.FMT_NVFP4, fmt_head=lib.FMT_NVFP4)
    stream = lib.stream_create()
    tensor_parallel = world > 1 and args.parallel == "tp"
    fell_back = None
    if tensor_parallel:
        # every rank its share of the same model: same seed (tensors held whole must agree), same input tokens
        from splash_b200 import tp
        t = target.Target(**cfg, tp_world=world, tp_rank=rank)
        t.randomize(1234, context)
        try:
            tp.connect(t, group.all_gather_bytes)
            bad = 0
        except lib.SbError as e:  # the peers' memory could not be mapped
            bad, fell_back = 1, f"tensor-parallel windows could not be mapped ({e}); measured as independent lanes"
        bad = int(group.reduce_max(bad))
        if not bad:
            t.upload(-1, "tokens", np.random.default_rng(0).integers(0, cfg["vocab"], ROWS).astype(np.uint32))
            group.barrier()
            # Two steps before anything is timed: an exchange that cannot reach a peer gives up after its bounded wait
            # and says so in the device status word. The run then measures independent lanes and reports why.
            for _ in range(2):
                t.step(ROWS, 0.0, target.GRAPH, stream)
            lib.stream_sync(stream)
            bad = int(group.reduce_max(lib.device_status()))
            if bad:
                fell_back = f"tensor-parallel exchange failed (device status {bad}); measured as independent lanes"
        if bad:
            fell_back = fell_back or "tensor parallelism failed on another rank; measured as independent lanes"
            group.barrier()
            t.close()
            tensor_parallel = False
    if not tensor_parallel:
        if L > 1:
            cfg.update(lanes=L)
        if expert_parallel:
            from splash_b200 import tp
            cfg.update(ep_world=world, ep_rank=rank)
        t = target.Target(**cfg)
        t.randomize(1234 + rank, context)
        if expert_parallel:
            tp.connect(t, group.all_gather_bytes)
            group.barrier()
    if args.moe:
        # Router logits ~ N(0, 1), as the benchmark's configuration states them: random weights do not make a router whose
        # routes spread over the experts as a trained one's do (its rows collapse onto a few experts, which flatters the step).
        t.set_router_scores(np.random.default_rng(77 + rank).standard_normal((ROWS * L, cfg["moe_experts"])).astype(np.float32))
    lanes = 1 if tensor_parallel else world * L
    warm = max(args.warmup, 3)
    # The lane is held at its context length, so every step does the same work, and keeps FOLD_ROWS pending rows, so
    # every step also folds that many rows of the previous step's tape into the Gated-DeltaNet state, as a committing
    # cycle with that accept length would.
    flags = target.GRAPH | target.KEEP_PENDING
    rng = np.random.default_rng(0 if tensor_parallel else rank)
    t.upload(-1, "tokens", rng.integers(0, cfg["vocab"], ROWS * L).astype(np.uint32))
    t.upload(-1, "pending_rows", np.full(L, FOLD_ROWS, np.uint32))
    # The MoE configuration verifies by rejection sampling at temperature 0.7 with supplied uniforms (80 a lane and step);
    # the others greedily.
    temperature = 0.7 if args.moe else 0.0
    uniforms = rng.random(80 * L).astype(np.float32)
    if temperature:
        t.upload(-1, "uniforms", uniforms)

    def barrier():
        lib.stream_sync(stream)
        group.barrier()

    reduce_max = group.reduce_max

    # ---- device-resident steps ----
    for _ in range(warm):
        t.step(ROWS, temperature, flags, stream)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = lib.Event(), lib.Event()
    e0.record(stream)
    for _ in range(args.steps):
        t.step(ROWS, temperature, flags, stream)
    e1.record(stream)
    e1.sync()
    barrier()
    ms = reduce_max(e0.elapsed_ms(e1)) / args.steps
    clocks = sampler.stop() if sampler else None
    status = lib.device_status()
    stats = t.stats(ROWS)
    if tensor_parallel:  # the job's bytes are all ranks' shares; a failed exchange on any rank fails the run
        for key in ("weight_bytes", "kv_bytes", "state_bytes"):
            stats[key] = int(group.reduce_sum(stats[key]))
        status = int(reduce_max(status))
    if expert_parallel:
        status = int(reduce_max(status))

    # ---- end to end through the host-facing call, pinned host buffers ----
    pinned = ctypes.c_void_p()
    lib.check(lib.load().sb_host_alloc(8 * 4096, ctypes.byref(pinned)))
    host = np.ctypeslib.as_array((ctypes.c_uint32 * 1024).from_address(pinned.value))
    host[:ROWS * L] = rng.integers(0, cfg["vocab"], ROWS * L)
    host_u = np.ctypeslib.as_array((ctypes.c_float * (80 * L)).from_address(pinned.value + 3 * 4096))
    host_u[:] = uniforms
    u_ptr = pinned.value + 3 * 4096 if temperature else None
    l = target._bind()
    out_t, out_r = pinned.value + 4096, pinned.value + 2 * 4096
    def verify_once():
        if L > 1:
            lib.check(l.sb_target_verify_lanes(t.handle, stream, pinned.value, u_ptr, ROWS, temperature, flags, out_t, out_r))
        else:
            lib.check(l.sb_target_verify(t.handle, stream, pinned.value, u_ptr, ROWS, temperature, flags, out_t, out_r))
    for _ in range(2):
        verify_once()
    barrier()
    e2, e3 = lib.Event(), lib.Event()
    e2.record(stream)
    for _ in range(args.steps):
        verify_once()
    e3.record(stream)
    e3.sync()
    barrier()
    e2e_ms = reduce_max(e2.elapsed_ms(e3)) / args.steps

    # ---- one checked step after the timed loops: the step computed something sane, and the same thing on every rank ----
    if L > 1:
        per_lane = t.verify_lanes(host[:ROWS * L].copy().reshape(L, ROWS), uniforms=uniforms.reshape(L, 80) if temperature else None,
                                  temperature=temperature, flags=flags, stream=stream)
        retained = min(r[1] for r in per_lane)  # (the bounds below then hold for every lane)
        if max(r[1] for r in per_lane) > ROWS:
            retained = 0
    else:
        _, retained, _, _ = t.verify(host[:ROWS].copy(), uniforms=uniforms if temperature else None, temperature=temperature, flags=flags, stream=stream)
    logits = t.download(-1, "logits", np.float32, (ROWS * L, cfg["vocab"]))
    finite = bool(np.isfinite(logits).all())
    bits = logits.view(np.uint32).astype(np.uint64)
    checksum = float(int((bits * (np.arange(bits.size, dtype=np.uint64).reshape(bits.shape) % 65521 + 1)).sum() % (1 << 52)))
    spread = 0.0
    if tensor_parallel:  # every rank selected from the same gathered logits: the ranks' checksums must be one value
        spread = reduce_max(checksum) + reduce_max(-checksum)
    finite = int(reduce_max(0 if finite else 1)) == 0  # on every rank
    parity_check = {"finite_logits": finite, "retained": int(retained),
                    "retained_ok": 1 <= int(retained) <= ROWS, "device_status": int(reduce_max(lib.device_status())),
                    "ranks_agree": (spread == 0.0) if tensor_parallel else None,
                    "what": "one verify step after the timed loops: logits finite, 1 <= retained <= 16, device status 0" +
                            ("; a position-weighted checksum of the logits' bits is equal on all ranks (max - min = 0)" if tensor_parallel else "")}

    if rank != 0:
        group.close()
        return

    # ---- the dominant kernel alone: the one-pass Q4_K gate/up projection over each layer's weights ----
    peak, peak_kind = measured_peak()
    roofline = None
    extra = L > 1 or args.nvfp4 or bool(args.context)
    fmt = lib.FMT_NVFP4 if args.nvfp4 else lib.FMT_Q4K
    if not args.tiny and (L > 1 or args.nvfp4):
        # the many-row projection on the tensor cores: the one-pass gate/up launch over 16 x lanes rows
        H, I, M = cfg["hidden"], cfg["intermediate"], ROWS * L
        x = lib.DeviceBuffer(M * H * 2 + 256)
        x.upload(rng.standard_normal((M, H)).astype(np.float16).view(np.uint16))
        prep = lib.DeviceBuffer(int(lib.load().sb_linear_wide_prepared_bytes(M, H)))
        lib.check(lib.load().sb_linear_wide_prepare(stream, x.ptr, M, H, H, None, prep.ptr, 0))
        out = lib.DeviceBuffer(M * I * 2 + 256)
        names = ("ffn_gate_image", "ffn_up_image") if args.nvfp4 else ("ffn_gate", "ffn_up")
        ptrs = [(t.tensor(layer, names[0])[0], t.tensor(layer, names[1])[0]) for layer in range(cfg["layers"])]
        def gate_up(i):
            g, u = ptrs[i % len(ptrs)]
            lib.linear(g, None, out.ptr, fmt, I, H, M, weights2=u, prepared=prep.ptr, epilogue=lib.EP_GATE_UP, stream=stream,
                       flags=lib.LINEAR_PDL | (lib.LINEAR_WIDE_IMAGE if args.nvfp4 else 0))
        for i in range(8):
            gate_up(i)
        lib.stream_sync(stream)
        n = 64
        k0, k1 = lib.Event(), lib.Event()
        k0.record(stream)
        for i in range(n):
            gate_up(i + 8)
        k1.record(stream)
        k1.sync()
        launch_ms = k0.elapsed_ms(k1) / n
        flops = 2.0 * M * 2 * I * H
        algo = 2 * I * (H // 256) * (160 if args.nvfp4 else 144) + M * H * 2 + M * I * 2
        tensor_peak = measured_peak_tensor()
        achieved = flops / launch_ms / 1e9
        roofline = {"bound": "tensor", "kernel": "linear_wide_kernel<%s> gate/up 2x[%dx%d], M=%d (weights dequantized to half, tcgen05, accumulators in tensor memory)" % ("NVFP4 image" if args.nvfp4 else "Q4_K", I, H, M),
                    "achieved": achieved, "peak": tensor_peak[0], "unit": "TFLOP/s", "frac": achieved / tensor_peak[0], "peak_kind": tensor_peak[1],
                    "algorithmic_bytes": algo, "hbm_gbs": algo / launch_ms / 1e6, "launch_us": launch_ms * 1e3, "traffic": None}
    elif not args.tiny:
        H, I = cfg["hidden"], cfg["intermediate"]
        if tensor_parallel:
            I = tp.share(cfg, world, rank)["intermediate"]  # the launch as this rank runs it
        x = lib.DeviceBuffer(ROWS * H * 2 + 256)
        x.upload(rng.standard_normal((ROWS, H)).astype(np.float16).view(np.uint16))  # any finite bf16 bits
        prep = lib.DeviceBuffer(int(lib.load().sb_linear_prepared_bytes(H)))
        lib.check(lib.load().sb_linear_prepare(stream, x.ptr, ROWS, H, H, None, lib.FMT_Q4K, prep.ptr, None, 0))
        out = lib.DeviceBuffer(ROWS * I * 2 + 256)
        ptrs = [(t.tensor(layer, "ffn_gate")[0], t.tensor(layer, "ffn_up")[0]) for layer in range(cfg["layers"])]
        def gate_up(i):
            g, u = ptrs[i % len(ptrs)]
            # launched as in the step: programmatic dependent launch, so a launch's ring fills while the one before drains
            lib.linear(g, None, out.ptr, lib.FMT_Q4K, I, H, ROWS, weights2=u, prepared=prep.ptr, epilogue=lib.EP_GATE_UP, stream=stream,
                       flags=lib.LINEAR_PDL)
        for i in range(8):
            gate_up(i)
        lib.stream_sync(stream)
        n = 64
        k0, k1 = lib.Event(), lib.Event()
        k0.record(stream)
        for i in range(n):
            gate_up(i + 8)
        k1.record(stream)
        k1.sync()
        launch_ms = k0.elapsed_ms(k1) / n
        algo = 2 * I * (H // 256) * 144 + ROWS * H * 2 + ROWS * I * 2
        achieved = algo / launch_ms / 1e6
        roofline = {"bound": "hbm", "kernel": "linear_kernel<Q4_K> gate/up 2x[%dx%d], M=16" % (I, H), "achieved": achieved, "peak": peak,
                    "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "algorithmic_bytes": algo,
                    "launch_us": launch_ms * 1e3, "traffic": None if tensor_parallel else DOMINANT_TRAFFIC_BYTES}
    step_bytes = stats["weight_bytes"] + stats["kv_bytes"] + stats["state_bytes"]
    step_gbs = step_bytes / ms / 1e6 / (world if tensor_parallel else 1)  # per GPU
    if args.tiny or extra:
        cpu_tps, cores, sample = None, os.cpu_count(), "skipped: not the benchmark's workload"
    elif world > 1:
        cpu_tps, cores, sample = None, os.cpu_count(), "timed at N = 1 only"
    else:
        cpu_tps, cores, sample = cpu_baseline(15.0)
    result = {
        "metric": "verify_tokens_per_s", "value": lanes * ROWS / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if tensor_parallel or expert_parallel else "weak", "vs_baseline": None,
        "dtype": "f16 operands (exact integer codes), f32 accumulate, bf16 activations", "data": "synthetic",
        "config": {"workload": workload, "context_tokens": context, "block": ROWS,
                   "fold": f"held lane that keeps {FOLD_ROWS} pending rows: every timed step folds {FOLD_ROWS} tape rows into the GDN state",
                   "parallelism": "tp1" if world == 1 else (f"tp{world}: one lane, shares exchanged through peer memory over NVLink in the input conversions" if tensor_parallel else f"ep{world}: {L} lanes and {cfg.get('moe_experts', 0) // world} of the routed experts a rank, rows dispatched and sums combined through peer memory over NVLink" if expert_parallel else f"{world} independent replicas (lanes)" + (f"; {fell_back}" if fell_back else "")),
                   "l2": "inputs exceed L2: one step streams %.1f GB of weights" % (stats["weight_bytes"] / 1e9), "cuda_graph": True, "pdl": True},
        "e2e": {"value": lanes * ROWS / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": (ROWS * 4 + (320 if temperature else 0)) * L, "d2h_bytes_per_step": (16 + ROWS * 4) * L},
        "gpu_launches": stats["launches"] * args.steps,
        "launches_per_step": stats["launches"],
        "step_roofline": {"bytes_per_step": step_bytes, "weight_bytes": stats["weight_bytes"], "kv_bytes": stats["kv_bytes"],
                          "state_bytes": stats["state_bytes"], "achieved_gbs": step_gbs, "frac_of_measured_peak": step_gbs / peak},
        "roofline": roofline,
        "cpu_baseline": {"value": cpu_tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "clocks": clocks, "device_status": status, "parity_check": parity_check,
    }
    print(json.dumps(result))
    group.close()


if __name__ == "__main__":
    main()
