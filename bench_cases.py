"""Single-operator cases of bench.py on seeded synthetic inputs, timed with CUDA events: the small commands that
single-kernel ncu captures are taken from, and a quick way to time one kernel on a shape.

    python bench.py --case linear --fmt q4k --n 17408 --k 5120 --epilogue gate_up [--iters 20]
    python bench.py --case attention --context 32768 [--q-heads 24 --kv-heads 4 --head-dim 256]
    python bench.py --case gdn [--key-heads 16 --value-heads 48]
    python bench.py --case moe
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 bench.py --case exchange
        (one rank per GPU: the tensor-parallel input conversion against the local one, replayed as CUDA graphs)

Weights are random native blocks with scale fields in the ranges the tests use (Q4_K / Q8_0 d, dmin in
U(5e-4, 4e-3); Q6_K d in U(2e-5, 1e-4)); several copies rotate so every launch streams from HBM, not L2."""
import argparse
import ctypes
import sys

import numpy as np

from splash_b200 import lib

FMT = {"q4k": lib.FMT_Q4K, "q6k": lib.FMT_Q6K, "q80": lib.FMT_Q80, "nvfp4": lib.FMT_NVFP4}
EPI = {"none": lib.EP_NONE, "residual": lib.EP_RESIDUAL, "gate_up": lib.EP_GATE_UP, "partials": lib.EP_PARTIALS}


def bf16_bits(x):
    v = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return (((v + 0x7FFF + ((v >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def native_rows(rng, fmt, n, k):
    """Random native rows with plausible half scales (other bytes uniform)."""
    if fmt == lib.FMT_Q4K:
        nb, bb = k // 256, 144
        blk = rng.integers(0, 256, (n, nb, bb), dtype=np.uint8)
        blk[..., 0:2] = rng.uniform(5e-4, 4e-3, (n, nb)).astype(np.float16).view(np.uint8).reshape(n, nb, 2)
        blk[..., 2:4] = rng.uniform(5e-4, 4e-3, (n, nb)).astype(np.float16).view(np.uint8).reshape(n, nb, 2)
    elif fmt == lib.FMT_Q6K:
        nb, bb = k // 256, 210
        blk = rng.integers(0, 256, (n, nb, bb), dtype=np.uint8)
        blk[..., 208:210] = rng.uniform(2e-5, 1e-4, (n, nb)).astype(np.float16).view(np.uint8).reshape(n, nb, 2)
    elif fmt == lib.FMT_NVFP4:
        nb, bb = k // 256, 148
        blk = rng.integers(0, 256, (n, nb, bb), dtype=np.uint8)
        blk[..., 0:16] = (rng.integers(0, 2, (n, nb, 16)) << 7) | (rng.integers(6, 9, (n, nb, 16)) << 3) | rng.integers(0, 8, (n, nb, 16))
        blk[..., 16:20] = np.full((n, nb), 1e-3, np.float32).view(np.uint8).reshape(n, nb, 4)
    else:
        nb, bb = k // 32, 34
        blk = rng.integers(0, 256, (n, nb, bb), dtype=np.uint8)
        blk[..., 0:2] = rng.uniform(5e-4, 4e-3, (n, nb)).astype(np.float16).view(np.uint8).reshape(n, nb, 2)
    return blk.reshape(n, nb * bb)


def timed(launch, iters, warm=3, graph=False):
    """Microseconds per launch. graph: the launches are captured into one CUDA graph and replayed, which takes the
    host's launch rate (several microseconds a call from Python) out of the figure."""
    if graph:
        l = lib.load()
        st = lib.stream_create()
        for i in range(warm):
            launch(i, st)
        lib.stream_sync(st)
        lib.check(l.sb_graph_begin(st))
        for i in range(iters):
            launch(i + warm, st)
        g = ctypes.c_void_p()
        lib.check(l.sb_graph_end(st, ctypes.byref(g)))
        lib.check(l.sb_graph_launch(g, st))
        lib.stream_sync(st)
        e0, e1 = lib.Event(), lib.Event()
        e0.record(st)
        for _ in range(5):
            lib.check(l.sb_graph_launch(g, st))
        e1.record(st)
        e1.sync()
        return e0.elapsed_ms(e1) / iters / 5 * 1e3
    for i in range(warm):
        launch(i)
    lib.stream_sync()
    e0, e1 = lib.Event(), lib.Event()
    e0.record()
    for i in range(iters):
        launch(i + warm)
    e1.record()
    e1.sync()
    return e0.elapsed_ms(e1) / iters * 1e3  # microseconds


def case_linear(a):
    rng = np.random.default_rng(0)
    fmt, n, k, ep = FMT[a.fmt], a.n, a.k, EPI[a.epilogue]
    rb = int(lib.load().sb_row_bytes(fmt, k))
    tensors = 2 if ep == lib.EP_GATE_UP else 1
    base = native_rows(rng, fmt, min(n, 2048), k)
    rows = np.tile(base, ((n + base.shape[0] - 1) // base.shape[0], 1))[:n]
    copies = max(2, int(a.resident_mb * 1e6 // (n * rb * tensors)) + 1)
    bufs = [lib.DeviceBuffer.from_numpy(rows) for _ in range(copies * tensors)]
    wide = a.rows > 16 or fmt == lib.FMT_NVFP4   # the many-row kernel
    image = wide and fmt in (lib.FMT_Q6K, lib.FMT_Q80, lib.FMT_NVFP4)
    if image:  # it reads Q6_K and NVFP4 rows as images made once
        natives, bufs = bufs, []
        for b in natives:
            img = lib.DeviceBuffer(int(lib.load().sb_linear_wide_image_bytes(fmt, n, k)))
            lib.check(lib.load().sb_linear_wide_image(None, fmt, b.ptr, n, k, img.ptr))
            bufs.append(img)
        lib.stream_sync()
        rb = int(lib.load().sb_linear_wide_image_bytes(fmt, n, k)) // n
    slots = max(16, a.rows)
    x = lib.DeviceBuffer.from_numpy(bf16_bits(rng.standard_normal((slots, k))))
    l = lib.load()
    if wide:  # its own conversion, once
        prep = lib.DeviceBuffer(int(l.sb_linear_wide_prepared_bytes(a.rows, k)))
        lib.check(l.sb_linear_wide_prepare(None, x.ptr, a.rows, k, k, None, prep.ptr, 0))
    else:
        prep = lib.DeviceBuffer(int(l.sb_linear_prepared_bytes(k)))
        lib.check(l.sb_linear_prepare(None, x.ptr, a.rows, k, k, None, fmt, prep.ptr, None, (lib.LINEAR_TCGEN05 if a.tcgen05 else 0)))
    splits = 1
    if ep == lib.EP_PARTIALS:
        l.sb_linear_wide_splits.argtypes = [ctypes.c_uint32] * 2
        splits = int(l.sb_linear_wide_splits(n, k)) if wide else 16
    out = lib.DeviceBuffer(splits * slots * n * 4 + 512)
    aux = lib.DeviceBuffer.from_numpy(np.zeros((slots, n), np.uint16))

    def launch(i, stream=None):
        kw = {}
        if ep == lib.EP_GATE_UP:
            kw = dict(weights2=bufs[(2 * i + 1) % len(bufs)].ptr)
            w = bufs[(2 * i) % len(bufs)].ptr
        else:
            w = bufs[i % len(bufs)].ptr
            if ep == lib.EP_RESIDUAL:
                kw = dict(aux=aux.ptr)
        flags = (lib.LINEAR_PDL if a.pdl else 0) | (lib.LINEAR_TCGEN05 if a.tcgen05 else 0) | (lib.LINEAR_WIDE_IMAGE if image else 0)
        lib.linear(w, None, out.ptr, fmt, n, k, a.rows, prepared=prep.ptr, epilogue=ep, out_f32=ep == lib.EP_PARTIALS, flags=flags, stream=stream, **kw)

    us = timed(launch, a.iters, graph=a.graph)
    algo = n * rb * tensors + a.rows * k * 2 + a.rows * n * 2
    flops = 2.0 * a.rows * n * tensors * k
    print(f"linear {a.fmt} n={n} k={k} rows={a.rows} epilogue={a.epilogue}: {us:.1f} us per launch, {algo / us / 1e3:.0f} GB/s "
          f"of {algo} algorithmic bytes, {flops / us / 1e6:.1f} TFLOP/s, device status {lib.device_status()}")


def case_attention(a):
    rng = np.random.default_rng(0)
    l = lib.ops()
    lib.check(l.sb_set_attention_kernel(1 if a.warp_mma else 0))
    QH, KH, D, PT, committed, rows = a.q_heads, a.kv_heads, a.head_dim, a.page_tokens, a.context, a.rows
    pages = (committed + rows + PT - 1) // PT + 1
    k = lib.DeviceBuffer.from_numpy(rng.integers(-127, 128, (pages, KH, PT, D), dtype=np.int8))
    v = lib.DeviceBuffer.from_numpy(rng.integers(-127, 128, (pages, KH, PT, D), dtype=np.int8))
    ks = lib.DeviceBuffer.from_numpy(rng.uniform(0.005, 0.03, (pages, KH, PT)).astype(np.float16))
    vs = lib.DeviceBuffer.from_numpy(rng.uniform(0.005, 0.03, (pages, KH, PT)).astype(np.float16))
    table = lib.DeviceBuffer.from_numpy(np.arange(pages, dtype=np.uint32))
    stride = QH * 2 * D + 2 * KH * D
    qkv = lib.DeviceBuffer.from_numpy(bf16_bits(rng.standard_normal((rows, stride))))
    q = lib.DeviceBuffer.from_numpy(bf16_bits(rng.standard_normal((rows, QH, D))))
    out = lib.DeviceBuffer(rows * QH * D * 2)
    cache = lib.SbKvLayer(k.ptr, v.ptr, ks.ptr, vs.ptr, KH, D, PT, 1)
    args = lib.SbAttnArgs(q.ptr, qkv.ptr, table.ptr, None, out.ptr, cache, None, rows, QH, 1, stride, QH * D, committed)
    us = timed(lambda i: lib.check(l.sb_attn_verify(None, ctypes.byref(args))), a.iters)
    algo = 2 * (committed + rows) * KH * (D + 2)
    print(f"attention ({'warp MMA' if a.warp_mma else 'tcgen05'}) q_heads={QH} kv_heads={KH} D={D} context={committed} rows={rows}: {us:.1f} us per launch, "
          f"{algo / us / 1e3:.0f} GB/s of {algo} algorithmic bytes, device status {lib.device_status()}")


def case_gdn(a):
    rng = np.random.default_rng(0)
    l = lib.ops()
    KH, VH, D = a.key_heads, a.value_heads, 128
    KW, VW = KH * D, VH * D
    C = 2 * KW + VW
    up = lambda x: lib.DeviceBuffer.from_numpy(x)
    bf = lambda shape, s: bf16_bits(rng.standard_normal(shape) * s)
    d = dict(qkvz=up(bf((16, C + VW), 1.0)), b=up(bf((16, VH), 1.0)), a=up(bf((16, VH), 1.0)), conv_w=up(bf((C, 4), 0.4)),
             a_scale=up((-np.exp(rng.uniform(-3, 0.5, VH))).astype(np.float32)), dt_bias=up(bf((VH,), 0.5)),
             norm_w=up(np.ones(D, np.float32)), cs_in=up(bf((3, C), 1.0)), state=up((rng.standard_normal((VH, D, D)) * 0.05).astype(np.float32)))
    tape = lambda: dict(inputs=lib.DeviceBuffer(16 * C * 2), k=lib.DeviceBuffer(16 * KW * 2), v=lib.DeviceBuffer(16 * VW * 2),
                        beta=lib.DeviceBuffer(16 * VH * 2), decay=lib.DeviceBuffer(16 * VH * 4))
    pend, step = tape(), tape()
    for t in (pend, step):
        for b in t.values():
            b.fill(0)
    cs_out, st_out, hid = lib.DeviceBuffer(3 * C * 2), lib.DeviceBuffer(VH * D * D * 4), lib.DeviceBuffer(16 * VW * 2)
    T = lambda t: lib.SbGdnTape(t["inputs"].ptr, t["k"].ptr, t["v"].ptr, t["beta"].ptr, t["decay"].ptr)
    args = lib.SbGdnArgs(d["qkvz"].ptr, d["b"].ptr, d["a"].ptr, d["conv_w"].ptr, d["a_scale"].ptr, d["dt_bias"].ptr, d["norm_w"].ptr,
                         d["cs_in"].ptr, cs_out.ptr, d["state"].ptr, st_out.ptr, T(pend), T(step), hid.ptr, None,
                         a.rows, a.pending, KH, VH, C + VW, VH, VW, 0)
    if a.fused_gates:  # the kernel projects b and a itself from a [16, k] input and fp32 rows [2 * value_heads, k]
        gk = a.fused_gates
        gw = up((rng.standard_normal((2 * VH, gk)) / np.sqrt(gk)).astype(np.float32))
        gx = up(bf(( 16, gk), 1.0))
        args.gate_weight, args.gate_input, args.gate_k, args.gate_input_stride = gw.ptr, gx.ptr, gk, gk
    us = timed(lambda i: lib.check(l.sb_gdn_verify(None, ctypes.byref(args))), a.iters)
    algo = 2 * VH * D * D * 4
    print(f"gdn key_heads={KH} value_heads={VH} rows={a.rows} pending={a.pending}: {us:.1f} us per launch, "
          f"{algo / us / 1e3:.0f} GB/s of {algo} state bytes, device status {lib.device_status()}")


def case_moe(a):
    """Routing and expert passes of one MoE layer for a lane's rows (35B-A3B shape by default: 256 experts + the shared one,
    top 8, hidden 2048, intermediate 512), random router scores so the routes spread over the experts."""
    rng = np.random.default_rng(0)
    l = lib.ops()
    rows, E, K, H, I = a.rows, a.experts, a.top_k, a.hidden, a.inter
    total, routes = E + 1, K + 1
    one = native_rows(rng, lib.FMT_Q4K, I, H)
    gate = lib.DeviceBuffer.from_numpy(np.tile(one, (total, 1)))
    up = lib.DeviceBuffer.from_numpy(np.tile(one[::-1], (total, 1)))
    down = lib.DeviceBuffer.from_numpy(np.tile(native_rows(rng, lib.FMT_Q4K, H, I), (total, 1)))
    x = lib.DeviceBuffer.from_numpy(bf16_bits(rng.standard_normal((rows, H))))
    scores = lib.DeviceBuffer.from_numpy(rng.standard_normal((rows, E)).astype(np.float32))
    sgate = lib.DeviceBuffer.from_numpy((rng.standard_normal(H) * 0.05).astype(np.float32))
    sel, wts = lib.DeviceBuffer(rows * routes * 4), lib.DeviceBuffer(rows * routes * 4)
    scratch = lib.DeviceBuffer(int(l.sb_moe_scratch_bytes(rows, routes, H, I)))
    out = lib.DeviceBuffer(rows * H * 2 + 256)
    ra = lib.SbMoeRouteArgs(scores.ptr, x.ptr, sgate.ptr, sel.ptr, wts.ptr, rows, E, E, K, H, 0)
    ea = lib.SbMoeExpertArgs(x.ptr, x.ptr, sel.ptr, wts.ptr, gate.ptr, up.ptr, down.ptr, scratch.ptr, out.ptr, rows, routes, H, I, lib.FMT_Q4K, total)

    def launch(i, stream=None):
        lib.check(l.sb_moe_route(stream, ctypes.byref(ra)))
        lib.check(l.sb_moe_experts(stream, ctypes.byref(ea)))

    us = timed(launch, a.iters, graph=a.graph)
    if rows > 16:  # grouped by expert: every expert that has a route streams once
        hit = len(np.unique(sel.to_numpy(np.uint32, (rows, routes))))
        algo = hit * 3 * I * (H // 256) * 144
        print(f"moe rows={rows} experts={E}+1 top_k={K} hidden={H} intermediate={I}: {us:.1f} us per layer (routing, grouping, 2 conversions, 2 grouped "
              f"expert launches, combine), {algo / us / 1e3:.0f} GB/s of {algo} bytes of the {hit} experts hit, "
              f"{2.0 * rows * routes * 3 * I * H / us / 1e6:.1f} TFLOP/s, device status {lib.device_status()}")
        return
    algo = rows * routes * 3 * I * (H // 256) * 144
    print(f"moe rows={rows} experts={E}+1 top_k={K} hidden={H} intermediate={I}: {us:.1f} us per layer (routing + 3 expert launches), "
          f"{algo / us / 1e3:.0f} GB/s of {algo} expert bytes (every route its own), device status {lib.device_status()}")


def case_exchange(a):
    """sb_tp_prepare_sum (push + conversion with the peers' shares) against sb_linear_prepare_sum, `launches` calls
    captured into one CUDA graph and replayed, so the host's launch rate does not enter."""
    from splash_b200 import tp
    from splash_b200.dist import Group
    d = Group("nccl")
    lib.init(d.local)
    l = lib.load()
    H, S, N = a.width, a.slices, a.launches
    g = tp.Group(d.world, d.rank, H, 1024, d.all_gather_bytes)
    P, U = ctypes.c_void_p, ctypes.c_uint32
    l.sb_linear_prepare_sum.argtypes = [P, P, U, U, P, U, P, U, U, U, P, U, P, P, U]
    rng = np.random.default_rng(d.rank)
    part = lib.DeviceBuffer.from_numpy(rng.standard_normal((S, 16, H)).astype(np.float32))
    res = lib.DeviceBuffer.from_numpy(np.zeros((16, H), np.uint16))
    out = lib.DeviceBuffer(16 * H * 2 + 256)
    norm = lib.DeviceBuffer.from_numpy(np.ones(H, np.float32))
    prep = lib.DeviceBuffer(int(l.sb_linear_prepared_bytes(H)))
    st = lib.stream_create()
    flags = lib.LINEAR_PDL if a.pdl else 0
    for mode in ("local", "exchange"):
        lib.check(l.sb_graph_begin(st))
        for i in range(N):
            if mode == "exchange":
                g.prepare_sum(st, i, part.ptr, S, H, res.ptr, out.ptr, 16, H, norm.ptr, lib.FMT_Q4K, prep.ptr, flags)
            else:
                lib.check(l.sb_linear_prepare_sum(st, part.ptr, S, H, res.ptr, H, out.ptr, H, 16, H, norm.ptr, lib.FMT_Q4K, prep.ptr, None, flags))
        if mode == "exchange":
            g.advance(st, N)
        graph = P()
        lib.check(l.sb_graph_end(st, ctypes.byref(graph)))
        for _ in range(3):
            lib.check(l.sb_graph_launch(graph, st))
        lib.stream_sync(st)
        d.barrier()
        e0, e1 = lib.Event(), lib.Event()
        e0.record(st)
        for _ in range(a.iters):
            lib.check(l.sb_graph_launch(graph, st))
        e1.record(st)
        e1.sync()
        us = d.reduce_max(e0.elapsed_ms(e1)) / N / a.iters * 1e3
        status = lib.device_status()
        d.barrier()
        if d.rank == 0:
            print(f"{mode} conversion, width {H}, {S} slices, {d.world} ranks, pdl={int(a.pdl)}: {us:.2f} us per exchange (max over ranks), "
                  f"device status {status}", flush=True)
    d.barrier()
    g.close()
    d.close()


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python bench.py --case")
    sub = ap.add_subparsers(dest="case", required=True)
    p = sub.add_parser("linear")
    p.add_argument("--fmt", choices=sorted(FMT), default="q4k")
    p.add_argument("--n", type=int, default=17408)
    p.add_argument("--k", type=int, default=5120)
    p.add_argument("--rows", type=int, default=16)
    p.add_argument("--epilogue", choices=sorted(EPI), default="none")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--pdl", action="store_true")
    p.add_argument("--graph", action="store_true", help="capture the launches into a CUDA graph and time its replay")
    p.add_argument("--tcgen05", action="store_true", help="Q4_K on the tensor-memory kernel (SB_LINEAR_TCGEN05)")
    p.add_argument("--resident-mb", type=float, default=400.0, help="rotate weight copies over at least this many MB")
    p = sub.add_parser("attention")
    p.add_argument("--context", type=int, default=32768)
    p.add_argument("--q-heads", type=int, default=24)
    p.add_argument("--kv-heads", type=int, default=4)
    p.add_argument("--head-dim", type=int, default=256)
    p.add_argument("--page-tokens", type=int, default=256)
    p.add_argument("--rows", type=int, default=16)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warp-mma", action="store_true", help="the mma.sync kernel instead of the tcgen05 one")
    p = sub.add_parser("gdn")
    p.add_argument("--key-heads", type=int, default=16)
    p.add_argument("--value-heads", type=int, default=48)
    p.add_argument("--rows", type=int, default=16)
    p.add_argument("--pending", type=int, default=8)
    p.add_argument("--fused-gates", type=int, default=0, help="k of the fused alpha / beta projection (0: b and a given)")
    p.add_argument("--iters", type=int, default=20)
    p = sub.add_parser("moe")
    p.add_argument("--rows", type=int, default=16)
    p.add_argument("--experts", type=int, default=256)
    p.add_argument("--top-k", type=int, default=8)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--inter", type=int, default=512)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--graph", action="store_true")
    p = sub.add_parser("exchange")
    p.add_argument("--width", type=int, default=5120)
    p.add_argument("--slices", type=int, default=3)
    p.add_argument("--launches", type=int, default=200)
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--pdl", action="store_true")
    a = ap.parse_args(argv)
    if a.case == "exchange":
        return case_exchange(a)
    lib.init(0)
    {"linear": case_linear, "attention": case_attention, "gdn": case_gdn, "moe": case_moe}[a.case](a)


if __name__ == "__main__":
    main(sys.argv[1:])
