"""Seeded synthetic GGUF tensors for the tests and the benchmark (numpy only).

`config0_q4k` follows the benchmark configuration's recipe: fp16 d and dmin = |N(0,1)| * 1e-3, 6-bit
scales and mins uniform 0..63, 4-bit codes uniform 0..15. `realistic` follows the scale ranges of
the reference's own kernel tests (dev/tests/engine/GgufFormatReference.hpp:292-324): Q4_K / Q8_0 d,
dmin in U(5e-4, 4e-3), Q6_K d in U(2e-5, 1e-4), every other byte random."""
import numpy as np


def pack_q4k_scales(sc, mn):
    """[..., 8] 6-bit scales and mins -> [..., 12] bytes in llama.cpp's get_scale_min_k4 packing."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    return out


def q4k_blocks(rng, n, k, d, dmin):
    """[n, k/256, 144] blocks with the given fp16 d, dmin arrays [n, k/256]."""
    nb = k // 256
    blk = np.zeros((n, nb, 144), np.uint8)
    blk[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(n, nb, 2)
    blk[..., 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(n, nb, 2)
    sc = rng.integers(0, 64, (n, nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, (n, nb, 8), dtype=np.uint8)
    blk[..., 4:16] = pack_q4k_scales(sc, mn)
    blk[..., 16:144] = rng.integers(0, 256, (n, nb, 128), dtype=np.uint8)
    return blk.reshape(n, nb * 144)


def config0_q4k(n, k, seed=0):
    rng = np.random.default_rng(seed)
    nb = k // 256
    d = np.abs(rng.standard_normal((n, nb))).astype(np.float32) * 1e-3
    dmin = np.abs(rng.standard_normal((n, nb))).astype(np.float32) * 1e-3
    return q4k_blocks(rng, n, k, d, dmin)


def realistic(fmt, n, k, seed=42):
    rng = np.random.default_rng(seed)
    if fmt == 0:
        nb = k // 256
        return q4k_blocks(rng, n, k, rng.uniform(5e-4, 4e-3, (n, nb)), rng.uniform(5e-4, 4e-3, (n, nb)))
    if fmt == 4:
        nb = k // 256
        blk = rng.integers(0, 256, (n, nb, 210), dtype=np.uint8)
        d = rng.uniform(2e-5, 1e-4, (n, nb)).astype(np.float16)
        blk[..., 208:210] = d.view(np.uint8).reshape(n, nb, 2)
        return blk.reshape(n, nb * 210)
    if fmt == 6:
        nb = k // 32
        blk = rng.integers(0, 256, (n, nb, 34), dtype=np.uint8)
        d = rng.uniform(5e-4, 4e-3, (n, nb)).astype(np.float16)
        blk[..., 0:2] = d.view(np.uint8).reshape(n, nb, 2)
        return blk.reshape(n, nb * 34)
    if fmt == 37:  # NVFP4: 16 e4m3 scales, an fp32 scale, 128 bytes of e2m1 codes
        nb = k // 256
        blk = rng.integers(0, 256, (n, nb, 148), dtype=np.uint8)
        blk[..., 0:16] = (rng.integers(0, 2, (n, nb, 16)) << 7) | (rng.integers(6, 9, (n, nb, 16)) << 3) | rng.integers(0, 8, (n, nb, 16))
        g = rng.uniform(2e-4, 2e-3, (n, 1)).astype(np.float32) * np.ones((1, nb), np.float32)  # one scale a tensor row here
        blk[..., 16:20] = g.view(np.uint8).reshape(n, nb, 4)
        return blk.reshape(n, nb * 148)
    raise ValueError(fmt)


def activations(rows, k, seed=0):
    """bf16 bit patterns of N(0,1) inputs."""
    rng = np.random.default_rng(seed + 1000)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    v = x.view(np.uint32).astype(np.uint64)
    return (((v + 0x7FFF + ((v >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)
