"""Shared test inputs: seeded weights in the three GGUF formats and a numpy model of the
repacked layouts (what each lane of the kernels decodes), used to check the layout
arithmetic on the CPU before anything runs on a GPU."""
from __future__ import annotations

import numpy as np

import oracle
from ojas_engine_b200 import Q4_K, Q6_K, Q8_0, encode, raw_bytes

TYPES = {"q4k": Q4_K, "q6k": Q6_K, "q80": Q8_0}


def gauss_weights(ggml_type: int, n: int, k: int, seed: int = 0, sigma: float = 0.02) -> np.ndarray:
    """N(0, sigma) weights quantized with the library's test-input encoder -> GGUF bytes."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(sigma)).astype(np.float32)
    return encode(ggml_type, w)


def synth_weights(ggml_type: int, n: int, k: int) -> np.ndarray:
    """The reference's own random-block generator (crates/ojas-formats/src/synth.rs:29)."""
    bb, bw = oracle.block_shape(ggml_type)
    return oracle.synth_blocks(ggml_type, n * k // bw)


def activations(m: int, k: int, seed: int = 1) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.standard_normal((m, k), dtype=np.float32)


def plane_offsets(ggml_type: int, n: int, k: int) -> list[int]:
    a = lambda v: (v + 255) & ~255
    nsb = k // 256
    if ggml_type == Q4_K:
        return [0, a(n * nsb * 128)]
    if ggml_type == Q6_K:
        o1 = a(n * nsb * 128)
        o2 = o1 + a(n * nsb * 64)
        o3 = o2 + a(n * nsb * 16)
        return [0, o1, o2, o3]
    return [0, a(n * k)]


def f16(u16: np.ndarray) -> np.ndarray:
    return u16.view(np.float16).astype(np.float32)


def model_dequant(ggml_type: int, packed: np.ndarray, n: int, k: int) -> np.ndarray:
    """Decode repacked planes the way the kernels' lanes do -> f32 [n, k] with the decoder's
    own arithmetic order, so it must equal the oracle's dequant exactly."""
    nsb = k // 256
    off = plane_offsets(ggml_type, n, k)
    nb = n * nsb
    if ggml_type == Q4_K:
        qs = packed[off[0]:off[0] + nb * 128].reshape(nb, 2, 4, 16)            # [blk][h][c][i]
        hdr = packed[off[1]:off[1] + nb * 16].reshape(nb, 16)
        d = f16(hdr[:, 0:2].copy().view(np.uint16).reshape(nb))
        dmin = f16(hdr[:, 2:4].copy().view(np.uint16).reshape(nb))
        sc = hdr[:, 4:16].astype(np.uint32)
        s = np.empty((nb, 8), np.float32)
        mn = np.empty((nb, 8), np.float32)
        for c in range(4):  # 24-bit group per chunk: s(2c) | s(2c+1)<<6 | m(2c)<<12 | m(2c+1)<<18
            g = sc[:, 3 * c] | (sc[:, 3 * c + 1] << 8) | (sc[:, 3 * c + 2] << 16)
            s[:, 2 * c], s[:, 2 * c + 1] = g & 63, (g >> 6) & 63
            mn[:, 2 * c], mn[:, 2 * c + 1] = (g >> 12) & 63, (g >> 18) & 63
        out = np.empty((nb, 256), np.float32)
        for c in range(4):
            for h in range(2):
                b = qs[:, h, c, :]
                lo, hi = (b & 0xF).astype(np.float32), (b >> 4).astype(np.float32)
                j0, j1 = 2 * c, 2 * c + 1
                out[:, 64 * c + 16 * h:64 * c + 16 * h + 16] = (d * s[:, j0])[:, None] * lo - (dmin * mn[:, j0])[:, None]
                out[:, 64 * c + 32 + 16 * h:64 * c + 32 + 16 * h + 16] = (d * s[:, j1])[:, None] * hi - (dmin * mn[:, j1])[:, None]
        return out.reshape(n, k)
    if ggml_type == Q6_K:
        lo = packed[off[0]:off[0] + nb * 128].reshape(nb, 2, 4, 16)
        hi = packed[off[1]:off[1] + nb * 64].reshape(nb, 4, 4, 4)               # [blk][c][k][i]
        sc = packed[off[2]:off[2] + nb * 16].view(np.int8).reshape(nb, 16).astype(np.float32)
        d = f16(packed[off[3]:off[3] + nb * 2].copy().view(np.uint16).reshape(nb))
        out = np.empty((nb, 256), np.float32)
        for c in range(4):
            for t in range(4):
                h = t & 1
                nibs = lo[:, h, c, :]
                nib = (nibs & 0xF) if t < 2 else (nibs >> 4)
                hb = ((hi[:, c, :, :] >> (2 * t)) & 3).reshape(nb, 16)
                q = (nib.astype(np.int32) | (hb.astype(np.int32) << 4)) - 32
                sidx = 4 * c + t
                out[:, 64 * c + 16 * t:64 * c + 16 * t + 16] = (d * sc[:, sidx])[:, None] * q.astype(np.float32)
        return out.reshape(n, k)
    q = packed[off[0]:off[0] + n * k].view(np.int8).reshape(n * k // 32, 32).astype(np.float32)
    d = f16(packed[off[1]:off[1] + n * k // 32 * 2].copy().view(np.uint16))
    return (d[:, None] * q).reshape(n, k)


__all__ = ["TYPES", "gauss_weights", "synth_weights", "activations", "model_dequant", "raw_bytes"]
