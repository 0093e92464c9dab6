"""The loader entries on the host: the GGUF tensor directory and the cache file of repacked weights.  The GGUF files
are written here, field by field, from the published container layout (header, typed metadata, tensor infos, aligned
payload), as the reference's reader expects it (crates/ojas-formats/src/gguf.rs:298-455)."""
import os
import struct

import numpy as np
import pytest

import oracle
import ojas_engine_b200 as ob
from ojas_engine_b200 import Q4_K, Q6_K, Q8_0
from ojas_engine_b200.loader import GgufFile, LoaderError, WeightCache

from helpers import gauss_weights

F32 = 0


def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, tensors, version=3, alignment=64):
    """tensors: [(name, ggml_type, dims in GGUF order, payload bytes)]."""
    kv = [
        _s("general.architecture") + struct.pack("<I", 8) + _s("llama"),
        _s("general.alignment") + struct.pack("<II", 4, alignment),
        _s("llama.rope.freq_base") + struct.pack("<If", 6, 1e6),
        _s("flag") + struct.pack("<IB", 7, 1),
        _s("big") + struct.pack("<Iq", 11, -5),
        _s("tokenizer.ggml.tokens") + struct.pack("<IIQ", 9, 8, 3) + _s("a") + _s("bc") + _s(""),
        _s("tokenizer.ggml.scores") + struct.pack("<IIQ", 9, 6, 3) + struct.pack("<3f", 0.0, 1.0, 2.0),
    ]
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv)) + b"".join(kv)
    infos, rel, payload = b"", 0, b""
    for name, t, dims, data in tensors:
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", t, rel)
        payload += data + b"\0" * (-len(data) % alignment)
        rel = len(payload)
    body = head + infos
    body += b"\0" * (-len(body) % alignment)
    with open(path, "wb") as f:
        f.write(body + payload)


@pytest.fixture
def model(tmp_path):
    rng = np.random.default_rng(7)
    tensors = [
        ("token_embd.weight", F32, (64, 10), rng.standard_normal(640).astype(np.float32).tobytes()),
        ("blk.0.attn_q.weight", Q4_K, (512, 24), gauss_weights(Q4_K, 24, 512, 1).tobytes()),
        ("blk.0.attn_k.weight", Q4_K, (512, 13), gauss_weights(Q4_K, 13, 512, 2).tobytes()),      # ragged last unit
        ("blk.0.ffn_down.weight", Q6_K, (768, 16), gauss_weights(Q6_K, 16, 768, 3).tobytes()),
        ("output.weight", Q8_0, (256, 40), gauss_weights(Q8_0, 40, 256, 4).tobytes()),
        ("blk.0.ffn_gate_exps.weight", Q4_K, (256, 8, 3), gauss_weights(Q4_K, 24, 256, 5).tobytes()),  # 3 experts of 8 rows
        ("blk.0.attn_norm.weight", F32, (64,), rng.standard_normal(64).astype(np.float32).tobytes()),
        ("blk.0.attn_v.weight", ob.Q5_K, (512, 16), oracle.synth_blocks(ob.Q5_K, 16 * 2).tobytes()),
        ("blk.0.ffn_up_exps.weight", ob.IQ4_XS, (256, 8, 2), oracle.synth_blocks(ob.IQ4_XS, 16).tobytes()),
        ("blk.0.ffn_down_exps.weight", ob.IQ4_NL, (256, 8, 2), oracle.synth_blocks(ob.IQ4_NL, 16 * 8).tobytes()),
    ]
    path = tmp_path / "tiny.gguf"
    write_gguf(path, tensors)
    return path, tensors


def test_gguf_directory_and_payloads(model):
    path, tensors = model
    with GgufFile(path) as g:
        assert len(g) == len(tensors)
        for i, (name, t, dims, data) in enumerate(tensors):
            ti = g.info(i)
            assert (ti.name, ti.ggml_type, ti.dims, ti.nbytes) == (name, t, tuple(dims), len(data))
            assert ti.file_offset % 64 == 0                      # general.alignment of the file
            assert g.find(name) == i
            assert g.read_raw(i).tobytes() == data
        with pytest.raises(KeyError):
            g.find("missing")
        with pytest.raises(IndexError):
            g.info(len(tensors))


def test_gguf_version_2_and_default_alignment(tmp_path):
    raw = gauss_weights(Q4_K, 8, 256, 9).tobytes()
    path = tmp_path / "v2.gguf"
    head = b"GGUF" + struct.pack("<IQQ", 2, 1, 0)
    info = _s("w") + struct.pack("<IQQIQ", 2, 256, 8, Q4_K, 0)
    body = head + info
    body += b"\0" * (-len(body) % 32)                            # no general.alignment key: 32
    path.write_bytes(body + raw)
    with GgufFile(path) as g:
        assert g.info(0).file_offset == len(body) and g.read_raw(0).tobytes() == raw


@pytest.mark.parametrize("damage", ["magic", "version", "truncated_directory", "tensor_past_end", "ragged_k"])
def test_malformed_gguf_is_rejected(tmp_path, damage):
    raw = gauss_weights(Q4_K, 8, 256, 9).tobytes()
    path = tmp_path / "bad.gguf"
    write_gguf(path, [("w", Q4_K, (256, 8), raw)])
    blob = bytearray(path.read_bytes())
    if damage == "magic":
        blob[:4] = b"GGML"
    elif damage == "version":
        blob[4:8] = struct.pack("<I", 1)
    elif damage == "truncated_directory":
        blob = blob[:40]
    elif damage == "tensor_past_end":
        blob = blob[:-64]
    else:
        write_gguf(path, [("w", Q4_K, (255, 8), raw)])
        blob = bytearray(path.read_bytes())
    path.write_bytes(bytes(blob))
    with pytest.raises(LoaderError):
        GgufFile(path)


def test_weight_cache_holds_the_repacked_matrices_and_follows_its_source(model, tmp_path):
    path, tensors = model
    cache_path = tmp_path / "tiny.ojb2wc"
    with WeightCache.for_gguf(path, cache_path) as c:            # missing: built, then opened
        got = {e.name: e for e in c.entries()}
        want = [(n, t, d, raw) for n, t, d, raw in tensors if t != F32]
        assert list(got) == [n for n, *_ in want]                # file order, f32 tensors left out
        for name, t, dims, raw in want:
            e = got[name]
            k, n = dims[0], int(np.prod(dims[1:]))
            assert (e.ggml_type, e.N, e.K) == (t, n, k)
            assert e.data.ctypes.data % 256 == 0                 # the mapping is page aligned and entries sit on 256 B
            assert e.data.tobytes() == ob.repack_host(t, np.frombuffer(raw, np.uint8), n, k).tobytes()
    built = os.stat(cache_path).st_mtime_ns
    with WeightCache.for_gguf(path, cache_path):                 # valid: opened, not rebuilt
        assert os.stat(cache_path).st_mtime_ns == built
    st = os.stat(path)
    os.utime(path, (st.st_atime, st.st_mtime + 5))               # the source changed
    with pytest.raises(LoaderError, match="rebuild"):
        WeightCache(cache_path, path)
    with WeightCache(cache_path) as c:                           # without a source to compare with it still opens
        assert len(c) == 8
    with WeightCache.for_gguf(path, cache_path) as c:            # stale: rebuilt
        assert len(c) == 8 and os.stat(cache_path).st_mtime_ns != built


def test_corrupt_cache_is_rejected(model, tmp_path):
    path, _ = model
    cache_path = tmp_path / "c.bin"
    WeightCache.build(path, cache_path)
    blob = cache_path.read_bytes()
    (tmp_path / "short.bin").write_bytes(blob[:-10])
    with pytest.raises(LoaderError):
        WeightCache(tmp_path / "short.bin")
    (tmp_path / "magic.bin").write_bytes(b"X" + blob[1:])
    with pytest.raises(LoaderError):
        WeightCache(tmp_path / "magic.bin")


def test_fused_groups_are_concatenations_of_repacked_parts():
    """Q, K and V (or gate and up) become one matrix by writing their repacked units one after another when each part
    has a multiple of 8 rows: the fused buffer equals the repack of the row-wise concatenation."""
    parts = [gauss_weights(Q4_K, n, 512, s) for n, s in ((32, 1), (8, 2), (16, 3))]
    whole = ob.repack_host(Q4_K, np.concatenate([p.reshape(-1) for p in parts]), 56, 512)
    pieces = [ob.repack_host(Q4_K, p, n, 512) for p, n in zip(parts, (32, 8, 16))]
    assert np.concatenate(pieces).tobytes() == whole.tobytes()


@pytest.mark.gpu
def test_cache_entry_uploads_to_the_same_weight_as_the_device_repack(gpu, model, tmp_path):
    """An entry of the cache, uploaded as it is, gives the GEMV the same bits as the GGUF bytes repacked on the device."""
    from helpers import activations
    path, tensors = model
    with WeightCache.for_gguf(path, tmp_path / "w.bin") as c:
        for e in c.entries():
            raw = np.frombuffer(next(r for n, _, _, r in tensors if n == e.name), np.uint8)
            a, b = gpu.load_weight(raw, e.ggml_type, e.N, e.K), gpu.load_repacked(e.data, e.ggml_type, e.N, e.K)
            x = gpu.upload(activations(1, e.K, seed=3))
            ya, yb = gpu.alloc(e.N), gpu.alloc(e.N)
            gpu.gemv(a, x, ya)
            gpu.gemv(b, x, yb)
            assert gpu.read(ya, np.float32, e.N).tobytes() == gpu.read(yb, np.float32, e.N).tobytes()
            for buf in (a.buf, b.buf, x, ya, yb):
                gpu.free(buf)
