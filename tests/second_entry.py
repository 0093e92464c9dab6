"""A second, independent entry of the reference's CPU quantized dot layer in numpy / Python scalars, written from the
Rust source (crates/ojas-cpu/src/cpu_math.rs) and not from the C oracle.  The reference has no unit test or golden
vector for quant_q8k / dot_q4k / dot_q6k / dot_q80, so the C oracle is checked against this transcription instead:
two entries of the same text that agree bit for bit on random and on the reference's synthetic blocks.

Every f32 operation is done in np.float32 in the order the Rust source performs it (Rust does not fuse
multiply-adds).  Small inputs only: the loops are plain Python."""
from __future__ import annotations

import numpy as np

F = np.float32


def _round_half_away(v: np.float32) -> np.float32:
    """f32::round: to nearest, ties away from zero (cpu_math.rs:557)."""
    t = np.trunc(v)
    return F(t + np.copysign(F(1.0), v)) if abs(F(v - t)) >= F(0.5) else F(t)


def quant_q8k(x: np.ndarray):
    """cpu_math.rs:545-563."""
    x = np.asarray(x, F)
    nsb = (x.size + 255) // 256
    scales = np.empty(nsb, F)
    q = np.zeros(nsb * 256, np.int8)
    bsums = np.zeros(nsb * 8, np.int32)
    for sb in range(nsb):
        seg = x[sb * 256:min(sb * 256 + 256, x.size)]
        m = F(0)
        for v in seg:                                   # fold(0, |a, v| a.max(v.abs())): NaN is ignored by f32::max
            a = F(abs(v))
            if a > m:
                m = a
        scale = F(m / F(127.0)) if m > 0 else F(1.0)
        inv = F(F(1.0) / scale)
        scales[sb] = scale
        for i, v in enumerate(seg):
            r = _round_half_away(F(v * inv))
            if np.isnan(r):
                qi = 0                                  # `as i8` of NaN
            else:
                qi = int(min(max(r, F(-127.0)), F(127.0)))
            q[sb * 256 + i] = qi
            bsums[sb * 8 + i // 32] += qi
    return scales, q, bsums


def _f16(b: np.ndarray, off: int) -> np.float32:
    return F(np.frombuffer(bytes(b[off:off + 2]), np.float16)[0])


def _scale_min_k4(j: int, s: np.ndarray):
    """cpu_math.rs:566-574."""
    if j < 4:
        return F(int(s[j]) & 63), F(int(s[j + 4]) & 63)
    d = (int(s[j + 4]) & 0xF) | ((int(s[j - 4]) >> 6) << 4)
    m = (int(s[j + 4]) >> 4) | ((int(s[j]) >> 6) << 4)
    return F(d), F(m)


def dot_q4k(row: np.ndarray, act):
    """cpu_math.rs:609-635.  Returns (value, the eight integer sub-block dots per super-block)."""
    scales, q, bsums = act
    total = F(0)
    idots = []
    for sb in range(row.size // 144):
        blk = row[sb * 144:(sb + 1) * 144]
        d, dmin = _f16(blk, 0), _f16(blk, 2)
        sc, qs = blk[4:16], blk[16:144]
        sx = F(scales[sb])
        xq = q[sb * 256:(sb + 1) * 256].astype(np.int32)
        bs = bsums[sb * 8:(sb + 1) * 8]
        sumd, summ = F(0), F(0)
        for c in range(4):
            qq = qs[c * 32:c * 32 + 32].astype(np.int32)
            lo, hi = qq & 0xF, qq >> 4
            s1, m1 = _scale_min_k4(c * 2, sc)
            s2, m2 = _scale_min_k4(c * 2 + 1, sc)
            i1 = int((lo * xq[c * 64:c * 64 + 32]).sum())
            i2 = int((hi * xq[c * 64 + 32:c * 64 + 64]).sum())
            idots += [i1, i2]
            sumd = F(sumd + F(s1 * F(i1)))
            sumd = F(sumd + F(s2 * F(i2)))
            summ = F(summ + F(F(m1 * F(int(bs[c * 2]))) + F(m2 * F(int(bs[c * 2 + 1])))))
        total = F(total + F(sx * F(F(d * sumd) - F(dmin * summ))))
    return total, np.array(idots, np.int32)


def dot_q5k(row: np.ndarray, act):
    """cpu_math.rs:637-671: as dot_q4k on five-bit values; bit j of qh[l] is the fifth bit of weight l of sub-block j."""
    scales, q, bsums = act
    total = F(0)
    idots = []
    for sb in range(scales.size):
        blk = row[sb * 176:(sb + 1) * 176]
        d, dmin = _f16(blk, 0), _f16(blk, 2)
        sc, qh, qs = blk[4:16], blk[16:48], blk[48:176]
        xq = q[sb * 256:(sb + 1) * 256].astype(np.int64)
        bs = bsums[sb * 8:(sb + 1) * 8]
        sumd, summ = F(0), F(0)
        for c in range(4):
            qq = qs[c * 32:(c + 1) * 32]
            lo = (qq & 0xF).astype(np.int64) + 16 * ((qh >> (2 * c)) & 1).astype(np.int64)
            hi = (qq >> 4).astype(np.int64) + 16 * ((qh >> (2 * c + 1)) & 1).astype(np.int64)
            s1, m1 = _scale_min_k4(2 * c, sc)
            s2, m2 = _scale_min_k4(2 * c + 1, sc)
            i1 = int((lo * xq[c * 64:c * 64 + 32]).sum())
            i2 = int((hi * xq[c * 64 + 32:c * 64 + 64]).sum())
            idots += [i1, i2]
            sumd = F(sumd + F(s1 * F(i1)))
            sumd = F(sumd + F(s2 * F(i2)))
            summ = F(summ + F(F(m1 * F(int(bs[2 * c]))) + F(m2 * F(int(bs[2 * c + 1])))))
        total = F(total + F(scales[sb] * F(F(d * sumd) - F(dmin * summ))))
    return total, np.asarray(idots, np.int32)


def dot_q6k(row: np.ndarray, act):
    """cpu_math.rs:674-722.  Returns (value, the sixteen integer dots of 16 weights per super-block, in weight order)."""
    scales, q, _ = act
    total = F(0)
    idots = []
    for sb in range(row.size // 210):
        blk = row[sb * 210:(sb + 1) * 210]
        d = _f16(blk, 208)
        sx = F(scales[sb])
        xq = q[sb * 256:(sb + 1) * 256].astype(np.int32)
        s_sum, s_sub = F(0), F(0)
        for half in range(2):
            ql = blk[half * 64:half * 64 + 64].astype(np.int32)
            qh = blk[128 + half * 32:128 + half * 32 + 32].astype(np.int32)
            sc = blk[192 + half * 8:192 + half * 8 + 8].view(np.int8)
            xh = xq[half * 128:half * 128 + 128]
            for quarter in range(4):
                if quarter == 0:
                    w = (ql[:32] & 0xF) | ((qh & 3) << 4)
                elif quarter == 1:
                    w = (ql[32:] & 0xF) | (((qh >> 2) & 3) << 4)
                elif quarter == 2:
                    w = (ql[:32] >> 4) | (((qh >> 4) & 3) << 4)
                else:
                    w = (ql[32:] >> 4) | (((qh >> 6) & 3) << 4)
                x32 = xh[quarter * 32:quarter * 32 + 32]
                s0, s1 = F(int(sc[quarter * 2])), F(int(sc[quarter * 2 + 1]))
                i0, i1 = int((w[:16] * x32[:16]).sum()), int((w[16:] * x32[16:]).sum())
                x0, x1 = int(x32[:16].sum()), int(x32[16:].sum())
                idots += [i0, i1]
                s_sum = F(s_sum + F(F(s0 * F(i0)) + F(s1 * F(i1))))
                s_sub = F(s_sub + F(F(s0 * F(x0)) + F(s1 * F(x1))))
        total = F(total + F(F(sx * d) * F(s_sum - F(F(32.0) * s_sub))))
    return total, np.array(idots, np.int32)


def dot_q80(row: np.ndarray, x: np.ndarray) -> np.float32:
    """cpu_math.rs:971-981."""
    x = np.asarray(x, F)
    s = F(0)
    for b in range(x.size // 32):
        blk = row[b * 34:(b + 1) * 34]
        d = _f16(blk, 0)
        acc = F(0)
        qv = blk[2:34].view(np.int8)
        for j in range(32):
            acc = F(acc + F(F(int(qv[j])) * x[b * 32 + j]))
        s = F(s + F(d * acc))
    return s


KVALUES_IQ4NL = (-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113)   # ggml's kvalues_iq4nl


def dot_iq4nl(row: np.ndarray, x: np.ndarray) -> np.float32:
    """cpu_math.rs:993-1010."""
    x = np.asarray(x, F)
    s = F(0)
    for b in range(x.size // 32):
        blk = row[b * 18:(b + 1) * 18]
        d = _f16(blk, 0)
        bsum = F(0)
        for j in range(16):
            qb = int(blk[2 + j])
            bsum = F(bsum + F(F(KVALUES_IQ4NL[qb & 0xF]) * x[b * 32 + j]))
            bsum = F(bsum + F(F(KVALUES_IQ4NL[qb >> 4]) * x[b * 32 + j + 16]))
        s = F(s + F(d * bsum))
    return s


def dot_iq4xs(row: np.ndarray, x: np.ndarray) -> np.float32:
    """cpu_math.rs:943-967: per group of 32 the codebook values times x (low nibble j, high nibble j + 16, alternating),
    times (ls - 32); the block's sum times d."""
    x = np.asarray(x, F)
    s = F(0)
    for b in range(x.size // 256):
        blk = row[b * 136:(b + 1) * 136]
        d = _f16(blk, 0)
        sh = int(blk[2]) | (int(blk[3]) << 8)
        sl, qs = blk[4:8], blk[8:136]
        bsum = F(0)
        for g in range(8):
            ls = ((int(sl[g // 2]) >> (4 * (g % 2))) & 0xF) | (((sh >> (2 * g)) & 3) << 4)
            gsum = F(0)
            for j in range(16):
                qb = int(qs[16 * g + j])
                gsum = F(gsum + F(F(KVALUES_IQ4NL[qb & 0xF]) * x[b * 256 + g * 32 + j]))
                gsum = F(gsum + F(F(KVALUES_IQ4NL[qb >> 4]) * x[b * 256 + g * 32 + j + 16]))
            bsum = F(bsum + F(F(ls - 32) * gsum))
        s = F(s + F(d * bsum))
    return s


def matvec_kq(raw: np.ndarray, t: int, n: int, k: int, x: np.ndarray) -> np.ndarray:
    """cpu_math.rs:1145-1189: activations quantized once (K-quants), one block dot per row."""
    rb = {12: 144 * (k // 256), 13: 176 * (k // 256), 14: 210 * (k // 256), 8: 34 * (k // 32), 20: 18 * (k // 32), 23: 136 * (k // 256)}[t]
    rows = np.asarray(raw, np.uint8).reshape(n, rb)
    out = np.empty(n, F)
    if t in (8, 20, 23):
        for r in range(n):
            out[r] = {8: dot_q80, 20: dot_iq4nl, 23: dot_iq4xs}[t](rows[r], x)
        return out
    act = quant_q8k(x)
    for r in range(n):
        out[r] = {12: dot_q4k, 13: dot_q5k, 14: dot_q6k}[t](rows[r], act)[0]
    return out


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """cpu_math.rs:456-460: the mean of squares summed in index order, inv = 1 / sqrt(mean + eps), (x * inv) * w."""
    x, w = np.asarray(x, F), np.asarray(w, F)
    ss = F(0)
    for v in x:
        ss = F(ss + F(v * v))
    ss = F(ss / F(x.size))
    inv = F(F(1) / np.sqrt(F(ss + F(eps)), dtype=F))
    return (x * inv).astype(F) * w


def silu_mul(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """cpu_math.rs:486 and cpu_glm.rs:556: act = (g / (1 + exp(-g))) * u."""
    g, u = np.asarray(g, F), np.asarray(u, F)
    with np.errstate(over="ignore"):                  # exp(-g) of a large negative g is inf: g / inf = -0, as in Rust
        return ((g / (F(1) + np.exp(-g, dtype=F))).astype(F) * u).astype(F)


def moe_topk(logits: np.ndarray, ksel: int):
    """crates/ojas-cuda/src/kernels/moe.rs:45-70: softmax over the logits, KSEL passes each taking the largest remaining
    probability (ties to the lowest index), the chosen weights renormalised to sum to 1."""
    lg = np.asarray(logits, F)
    p = np.exp(lg - lg.max(), dtype=F)
    total = F(p.sum(dtype=np.float64))
    idx, tw = [], []
    for _ in range(ksel):
        best = int(np.argmax(p))                      # numpy's argmax returns the first of equal maxima
        idx.append(best)
        tw.append(F(p[best] / total))
        p[best] = F(-1)
    wsum = F(0)
    for v in tw:
        wsum = F(wsum + v)
    return np.asarray(idx, np.uint32), np.asarray([F(v / wsum) for v in tw], F)


def moe_ffn(wg, wu, wd, t_gu: int, t_d: int, h: np.ndarray, idx: np.ndarray, wgt: np.ndarray, d: int, ffn: int) -> np.ndarray:
    """cpu_glm.rs:551-582: per token, per pick in order: gate and up of the expert over the token's row, SwiGLU, the
    expert's down projection, added with the pick's weight."""
    h = np.asarray(h, F).reshape(-1, d)
    rg, rd = {12: 144, 14: 210}[t_gu] * (d // 256) * ffn, {12: 144, 14: 210}[t_d] * (ffn // 256) * d
    wg, wu, wd = np.asarray(wg, np.uint8).reshape(-1), np.asarray(wu, np.uint8).reshape(-1), np.asarray(wd, np.uint8).reshape(-1)
    out = np.zeros((h.shape[0], d), F)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            gv = matvec_kq(wg[e * rg:(e + 1) * rg], t_gu, ffn, d, h[t])
            uv = matvec_kq(wu[e * rg:(e + 1) * rg], t_gu, ffn, d, h[t])
            dv = matvec_kq(wd[e * rd:(e + 1) * rd], t_d, d, ffn, silu_mul(gv, uv))
            out[t] = (out[t] + (F(wgt[t, j]) * dv).astype(F)).astype(F)
    return out
