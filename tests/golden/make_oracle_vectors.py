"""Writes tests/golden/oracle_vectors.npz: outputs of the CPU oracle (oracle/ojas_oracle.c) on fixed inputs, one small
case per format of the path.  The oracle itself is pinned elsewhere (the reference's digests and known answers, an
independent transcription of the Rust source); these vectors freeze its outputs bit for bit, so that a change of compiler
flags, of the oracle or of its build shows up as a test failure instead of as a silent shift of what the GPU is compared
with.  Run from the repository root:  python tests/golden/make_oracle_vectors.py"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402

CASES = [("q80", oracle.Q8_0), ("q4k", oracle.Q4_K), ("q5k", oracle.Q5_K), ("q6k", oracle.Q6_K), ("iq4nl", oracle.IQ4_NL), ("iq4xs", oracle.IQ4_XS)]
N, K = 12, 768


def inputs():
    x = np.random.default_rng(20260101).standard_normal(K).astype(np.float32)
    x[5], x[300] = 0.0, -3.75                                   # an exact zero and a value that is exact in every format
    return x


def compute():
    x = inputs()
    out = {"x": x}
    for tag, t in CASES:
        raw = oracle.synth_blocks(t, N * K // oracle.block_shape(t)[1])
        out[f"y_{tag}"] = oracle.matvec_kq(raw, t, N, K, x, threads=1)
    scales, q, bsums = oracle.quant_q8k(x)
    out.update(q8k_scales=scales, q8k_q=q, q8k_bsums=bsums)
    lg = np.random.default_rng(7).standard_normal((5, 8)).astype(np.float32)
    idx, wgt = oracle.moe_topk(lg, 2)
    out.update(topk_logits=lg, topk_idx=idx, topk_wgt=wgt)
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_vectors.npz")
    np.savez(path, **compute())
    print("wrote", path, os.path.getsize(path), "bytes")
