"""Host-side logic of the product library: exports, layouts, encoders (no GPU, no compute calls)."""
import ctypes as C

import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import lib as oblib

from helpers import TYPES, gauss_weights, model_dequant, synth_weights


def test_library_exports_every_declared_symbol():
    l = oblib.load()
    declared = oblib.header_symbols()
    assert len(declared) >= 30
    assert set(declared) == set(oblib.SIGNATURES)
    for name in declared:
        assert hasattr(l, name), name
    assert b"sm_100a" in l.ojas_b200_version()


def test_kernel_name_table():
    l = oblib.load()
    names = [l.ojas_b200_kernel_name(i).decode() for i in range(l.ojas_b200_kernel_count())]
    assert len(names) == len(set(names))
    # every native GEMV format carries its four forms (crates/ojas-cuda/tests/conformance.rs:85-202)
    for tag in ("q4k", "q5k", "q6k", "q80", "iq4xs", "iq4nl"):
        for suffix in ("", "_accum", "_bias", "_m"):
            assert f"gemv_nat_{tag}{suffix}" in names
            assert l.ojas_b200_has_kernel(f"gemv_nat_{tag}{suffix}".encode())
    # the engine's IQ expert entries (crates/ojas-cuda/src/kernels/moe_iq.rs:64-108) and the token-table gather (qwen35.rs:53)
    for name in ("moe_gu_iq4xs", "moe_down_iq4nl", "moe_gu_q80", "moe_down_q80_slots", "q35_embed_q4k", "moe_topk", "quant_q8k"):
        assert name in names
    assert not l.ojas_b200_has_kernel(b"gemv_nat_q2k")


@pytest.mark.parametrize("tag", ["q4k", "q5k", "q6k", "q80", "iq4xs", "iq4nl"])
def test_sizes(tag):
    t = {**TYPES, "q5k": ob.Q5_K, "iq4xs": ob.IQ4_XS, "iq4nl": ob.IQ4_NL}[tag]
    per256 = {"q4k": 144, "q5k": 176, "q6k": 210, "q80": 272, "iq4xs": 136, "iq4nl": 144}[tag]
    assert ob.raw_bytes(t, 4096, 4096) == 4096 * 16 * per256
    assert ob.raw_bytes(t, 3, 256) == oracle.row_bytes(t, 256) * 3
    rp = ob.repacked_bytes(t, 4096, 4096)
    assert ob.raw_bytes(t, 4096, 4096) <= rp <= ob.raw_bytes(t, 4096, 4096) + 4 * 256  # lossless, padding only
    assert ob.repacked_bytes(t, 8, 100) == 0  # K must be a multiple of 256
    assert ob.repacked_bytes(5, 8, 256) == 0  # unsupported type


@pytest.mark.parametrize("tag", ["q4k", "q6k", "q80"])
@pytest.mark.parametrize("source", ["synth", "gauss"])
def test_repack_is_lossless(tag, source):
    """Decoding the repacked planes the way the kernels' lanes do gives exactly the values the
    reference decoder gives for the GGUF blocks."""
    t = TYPES[tag]
    n, k = 5, 768
    raw = synth_weights(t, n, k) if source == "synth" else gauss_weights(t, n, k, seed=4)
    packed = ob.repack_host(t, raw, n, k)
    got = model_dequant(t, packed, n, k)
    want = oracle.dequant_f32(raw, t, n * k).reshape(n, k)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("tag,tol", [("q4k", 0.12), ("q6k", 0.03), ("q80", 0.01)])
def test_encoders_round_trip(tag, tol):
    t = TYPES[tag]
    n, k = 16, 1024
    w = (np.random.default_rng(0).standard_normal((n, k)) * 0.02).astype(np.float32)
    raw = ob.encode(t, w)
    assert raw.size == ob.raw_bytes(t, n, k)
    back = oracle.dequant_f32(raw, t, n * k).reshape(n, k)
    err = np.linalg.norm(back - w) / np.linalg.norm(w)
    assert err < tol, err
    assert np.isfinite(back).all()


def test_encoder_handles_zeros():
    for t in TYPES.values():
        raw = ob.encode(t, np.zeros((2, 256), np.float32))
        assert not oracle.dequant_f32(raw, t, 512).any()


def test_no_gpu_fails_loudly():
    l = oblib.load()
    ctx = C.c_void_p()
    rc = l.ojas_b200_create(9999, None, C.byref(ctx))
    assert rc != 0 and not ctx.value


def test_expert_lru_bookkeeping():
    """The expert cache's slot bookkeeping (host code): hits, misses, least-recently-used eviction, and the refusal of a
    request that names more distinct experts than there are slots (crates/ojas-cuda/src/expert_cache.rs:96-150)."""
    l = oblib.load()
    h = C.c_void_p()
    assert l.ojas_b200_expert_lru_create(3, C.byref(h)) == 0

    def plan(ids):
        ids = np.asarray(ids, np.uint32)
        slot, miss = np.zeros(ids.size, np.uint32), np.zeros(ids.size, np.uint8)
        rc = l.ojas_b200_expert_lru_plan(h, ids.ctypes.data_as(C.POINTER(C.c_uint32)), ids.size, slot.ctypes.data_as(C.POINTER(C.c_uint32)),
                                         miss.ctypes.data_as(C.POINTER(C.c_uint8)))
        return rc, list(slot), list(miss)

    def stats():
        out = (C.c_size_t * 3)()
        l.ojas_b200_expert_lru_stats(h, out)
        return tuple(out)

    assert plan([7, 9]) == (0, [0, 1], [1, 1])
    assert plan([9, 7, 9]) == (0, [1, 0, 1], [0, 0, 0])           # hits: an address, not a copy
    assert plan([4]) == (0, [2], [1])                              # the free slot
    assert plan([5]) == (0, [0], [1])                              # evicts 7 (used before 9 and 4)
    assert plan([9, 4]) == (0, [1, 2], [0, 0])
    assert plan([7]) == (0, [0], [1])                              # evicts 5: the least recently used now
    assert stats() == (5, 5, 2)
    rc, _, _ = plan([1, 2, 3, 4])                                  # four distinct experts, three slots
    assert rc == -6 and stats() == (5, 5, 2)                       # refused, nothing changed
    assert plan([1, 1, 2, 2, 3]) == (0, [1, 1, 2, 2, 0], [1, 0, 1, 0, 1])
    l.ojas_b200_expert_lru_destroy(h)
