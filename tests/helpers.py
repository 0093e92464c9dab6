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


TILE_BYTES = {Q4_K: 1152, Q6_K: 1680, Q8_0: 2176}


def f16(u16: np.ndarray) -> np.ndarray:
    return u16.view(np.float16).astype(np.float32)


def _pieces(tiles: np.ndarray, first: int, count: int) -> np.ndarray:
    """Pieces first .. first+count-1 of every row of every tile: [tile, row, count, 16] bytes.
    A tile keeps piece p of row r at byte (p * 8 + r) * 16."""
    t = tiles[:, first * 128:(first + count) * 128].reshape(-1, count, 8, 16)
    return t.transpose(0, 2, 1, 3)


def model_dequant(ggml_type: int, packed: np.ndarray, n: int, k: int) -> np.ndarray:
    """Decode a repacked weight the way the kernels' lanes do -> f32 [n, k] with the decoder's
    own arithmetic order, so it must equal the oracle's dequant exactly."""
    nsb = k // 256
    units = (n + 7) // 8
    tb = TILE_BYTES[ggml_type]
    tiles = packed[:units * nsb * tb].reshape(units * nsb, tb)
    nb = units * nsb * 8                                     # (unit, super-block, row) in that order
    if ggml_type == Q4_K:
        qs = _pieces(tiles, 0, 8).reshape(nb, 128)           # GGUF order
        hdr = _pieces(tiles, 8, 1).reshape(nb, 16)
        d = f16(hdr[:, 0:2].copy().view(np.uint16).reshape(nb))
        dmin = f16(hdr[:, 2:4].copy().view(np.uint16).reshape(nb))
        sc = hdr[:, 4:16].astype(np.uint32)
        s = np.empty((nb, 8), np.float32)
        mn = np.empty((nb, 8), np.float32)
        for j in range(8):                                   # get_scale_min_k4
            if j < 4:
                s[:, j], mn[:, j] = sc[:, j] & 63, sc[:, j + 4] & 63
            else:
                s[:, j] = (sc[:, j + 4] & 0xF) | ((sc[:, j - 4] >> 6) << 4)
                mn[:, j] = (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)
        out = np.empty((nb, 256), np.float32)
        for c in range(4):
            b = qs[:, 32 * c:32 * c + 32]
            lo, hi = (b & 0xF).astype(np.float32), (b >> 4).astype(np.float32)
            j0, j1 = 2 * c, 2 * c + 1
            out[:, 64 * c:64 * c + 32] = (d * s[:, j0])[:, None] * lo - (dmin * mn[:, j0])[:, None]
            out[:, 64 * c + 32:64 * c + 64] = (d * s[:, j1])[:, None] * hi - (dmin * mn[:, j1])[:, None]
    elif ggml_type == Q6_K:
        lo = _pieces(tiles, 0, 8).reshape(nb, 2, 4, 16)      # [blk][h][c][i]
        hi = _pieces(tiles, 8, 4).reshape(nb, 4, 16)         # [blk][c][b]
        sc = _pieces(tiles, 12, 1).reshape(nb, 16).view(np.int8).astype(np.float32)
        d = f16(tiles[:, 13 * 128:13 * 128 + 16].copy().view(np.uint16).reshape(nb))
        out = np.empty((nb, 256), np.float32)
        for c in range(4):
            for t in range(4):
                h = t & 1
                nibs = lo[:, h, c, :]
                nib = (nibs & 0xF) if t < 2 else (nibs >> 4)
                hb = (hi[:, c, :] >> (2 * t)) & 3
                q = (nib.astype(np.int32) | (hb.astype(np.int32) << 4)) - 32
                sidx = 4 * c + t
                out[:, 64 * c + 16 * t:64 * c + 16 * t + 16] = (d * sc[:, sidx])[:, None] * q.astype(np.float32)
    else:
        q = _pieces(tiles, 0, 16).reshape(nb, 8, 32).view(np.int8).astype(np.float32)
        d = f16(_pieces(tiles, 16, 1).reshape(nb, 16).copy().view(np.uint16).reshape(nb, 8))
        out = (d[:, :, None] * q).reshape(nb, 256)
    # [unit, sb, row, 256] -> [unit * 8 + row, sb * 256 + i]
    full = out.reshape(units, nsb, 8, 256).transpose(0, 2, 1, 3).reshape(units * 8, k)
    return full[:n]


__all__ = ["TYPES", "gauss_weights", "synth_weights", "activations", "model_dequant", "raw_bytes"]
