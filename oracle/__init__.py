"""ctypes front end of the CPU oracle (``ojas_oracle.c``).

Test infrastructure only: the tests, the smoke check and the CPU-baseline leg of
the benchmark import this module; the product package never does.  Every function
is a thin wrapper; the arithmetic and its reference citations live in the C file.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS = 8, 12, 13, 14, 20, 23


def _cpu_tag() -> str:
    """Short tag of this host's CPU feature flags: a -march=native build is only valid here."""
    import hashlib
    flags = ""
    try:
        with open("/proc/cpuinfo") as fh:
            for line in fh:
                if line.startswith(("flags", "model name")):
                    flags += line
                    if line.startswith("flags"):
                        break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:10]


def _lib_name(native: bool) -> str:
    return f"libojas_oracle_native_{_cpu_tag()}.so" if native else "libojas_oracle.so"


def build(native: bool = False) -> str:
    """Compile the oracle with make; returns the path of the shared object."""
    cmd = ["make", "-C", _HERE, "native", f"NATIVE_TAG={_cpu_tag()}"] if native else ["make", "-C", _HERE, "all"]
    subprocess.run(cmd, check=True, capture_output=True)
    return os.path.join(_HERE, _lib_name(native))


def _load(native: bool = False) -> C.CDLL:
    name = _lib_name(native)
    path = os.path.join(_HERE, name)
    src = os.path.join(_HERE, "ojas_oracle.c")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        build(native)
    lib = C.CDLL(path)
    u8p, f32p, i8p, i32p, u16p, u32p = (C.POINTER(t) for t in (C.c_uint8, C.c_float, C.c_int8, C.c_int32, C.c_uint16, C.c_uint32))
    sig = {
        "orc_f16_to_f32": (C.c_float, [C.c_uint16]),
        "orc_f32_to_f16": (C.c_uint16, [C.c_float]),
        "orc_synth_blocks": (C.c_int, [C.c_uint32, C.c_size_t, u8p]),
        "orc_dequant_f32": (C.c_int, [u8p, C.c_uint32, C.c_size_t, f32p]),
        "orc_dequant_f16": (C.c_int, [u8p, C.c_uint32, C.c_size_t, u16p]),
        "orc_digest_f16": (C.c_uint64, [u16p, C.c_size_t]),
        "orc_quant_q8k": (None, [f32p, C.c_size_t, f32p, i8p, i32p]),
        "orc_dot_q4k": (C.c_float, [u8p, C.c_size_t, f32p, i8p, i32p, i32p]),
        "orc_dot_q5k": (C.c_float, [u8p, C.c_size_t, f32p, i8p, i32p, i32p]),
        "orc_dot_q6k": (C.c_float, [u8p, C.c_size_t, f32p, i8p, i32p]),
        "orc_dot_q80": (C.c_float, [u8p, f32p, C.c_size_t]),
        "orc_dot_iq4xs": (C.c_float, [u8p, f32p, C.c_size_t]),
        "orc_dot_iq4nl": (C.c_float, [u8p, f32p, C.c_size_t]),
        "orc_row_bytes": (C.c_size_t, [C.c_uint32, C.c_size_t]),
        "orc_matvec_kq": (C.c_int, [u8p, C.c_uint32, C.c_size_t, C.c_size_t, f32p, C.c_int, f32p]),
        "orc_matmul_kq": (C.c_int, [u8p, C.c_uint32, C.c_size_t, C.c_size_t, f32p, C.c_size_t, C.c_int, f32p]),
        "orc_moe_topk": (None, [f32p, C.c_int, C.c_int, u32p, f32p]),
        "orc_moe_ffn": (C.c_int, [u8p, u8p, u8p, C.c_uint32, C.c_uint32, f32p, u32p, f32p, C.c_size_t, C.c_int,
                                  C.c_size_t, C.c_size_t, C.c_int, f32p]),
        "orc_tvec": (None, [C.c_size_t, C.c_uint32, f32p]),
        "orc_rmsnorm": (None, [f32p, f32p, C.c_size_t, C.c_float, f32p]),
        "orc_silu_mul": (None, [f32p, f32p, C.c_size_t, f32p]),
    }
    for name_, (res, args) in sig.items():
        fn = getattr(lib, name_)
        fn.restype, fn.argtypes = res, args
    return lib


_libs: dict[bool, C.CDLL] = {}


def lib(native: bool = False) -> C.CDLL:
    if native not in _libs:
        _libs[native] = _load(native)
    return _libs[native]


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(C.POINTER(t))


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def block_shape(t: int) -> tuple[int, int]:
    return {Q8_0: (34, 32), Q4_K: (144, 256), Q5_K: (176, 256), Q6_K: (210, 256), IQ4_NL: (18, 32), IQ4_XS: (136, 256)}[t]


def row_bytes(t: int, k: int) -> int:
    return int(lib().orc_row_bytes(t, k))


def synth_blocks(t: int, nb: int) -> np.ndarray:
    bb, _ = block_shape(t)
    out = np.empty(nb * bb, np.uint8)
    assert lib().orc_synth_blocks(t, nb, _p(out, C.c_uint8)) == 0
    return out


def dequant_f32(raw, t: int, n: int) -> np.ndarray:
    raw = _u8(raw)
    out = np.empty(n, np.float32)
    assert lib().orc_dequant_f32(_p(raw, C.c_uint8), t, n, _p(out, C.c_float)) == 0
    return out


def dequant_f16(raw, t: int, n: int) -> np.ndarray:
    raw = _u8(raw)
    out = np.empty(n, np.uint16)
    assert lib().orc_dequant_f16(_p(raw, C.c_uint8), t, n, _p(out, C.c_uint16)) == 0
    return out


def digest_f16(vals: np.ndarray) -> int:
    vals = np.ascontiguousarray(vals, np.uint16)
    return int(lib().orc_digest_f16(_p(vals, C.c_uint16), vals.size))


def quant_q8k(x) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(scales f32[K/256], q i8[K], bsums i32[K/32]) of one activation row."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    k = x.size
    assert k % 256 == 0
    scales = np.empty(k // 256, np.float32)
    q = np.empty(k, np.int8)
    bsums = np.empty(k // 32, np.int32)
    lib().orc_quant_q8k(_p(x, C.c_float), k, _p(scales, C.c_float), _p(q, C.c_int8), _p(bsums, C.c_int32))
    return scales, q, bsums


def dot_q4k(row, act, want_idots: bool = False):
    row = _u8(row)
    scales, q, bsums = act
    nsb = scales.size
    idots = np.empty(nsb * 8, np.int32) if want_idots else None
    v = lib().orc_dot_q4k(_p(row, C.c_uint8), nsb, _p(scales, C.c_float), _p(q, C.c_int8), _p(bsums, C.c_int32),
                          _p(idots, C.c_int32) if want_idots else None)
    return (float(v), idots) if want_idots else float(v)


def dot_q5k(row, act, want_idots: bool = False):
    row = _u8(row)
    scales, q, bsums = act
    nsb = scales.size
    idots = np.empty(nsb * 8, np.int32) if want_idots else None
    v = lib().orc_dot_q5k(_p(row, C.c_uint8), nsb, _p(scales, C.c_float), _p(q, C.c_int8), _p(bsums, C.c_int32),
                          _p(idots, C.c_int32) if want_idots else None)
    return (float(v), idots) if want_idots else float(v)


def dot_q6k(row, act, want_idots: bool = False):
    row = _u8(row)
    scales, q, _ = act
    nsb = scales.size
    idots = np.empty(nsb * 16, np.int32) if want_idots else None
    v = lib().orc_dot_q6k(_p(row, C.c_uint8), nsb, _p(scales, C.c_float), _p(q, C.c_int8),
                          _p(idots, C.c_int32) if want_idots else None)
    return (float(v), idots) if want_idots else float(v)


def dot_q80(row, x) -> float:
    row = _u8(row)
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    return float(lib().orc_dot_q80(_p(row, C.c_uint8), _p(x, C.c_float), x.size))


def dot_iq4nl(row, x) -> float:
    row = _u8(row)
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    return float(lib().orc_dot_iq4nl(_p(row, C.c_uint8), _p(x, C.c_float), x.size))


def dot_iq4xs(row, x) -> float:
    row = _u8(row)
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    return float(lib().orc_dot_iq4xs(_p(row, C.c_uint8), _p(x, C.c_float), x.size))


def matvec_kq(raw, t: int, n: int, k: int, x, threads: int = 0, native: bool = False) -> np.ndarray:
    raw = _u8(raw)
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    assert x.size == k and raw.size == n * row_bytes(t, k), (x.size, k, raw.size, n * row_bytes(t, k))
    out = np.empty(n, np.float32)
    rc = lib(native).orc_matvec_kq(_p(raw, C.c_uint8), t, n, k, _p(x, C.c_float), threads or (os.cpu_count() or 1),
                                   _p(out, C.c_float))
    assert rc == 0, rc
    return out


def matmul_kq(raw, t: int, n: int, k: int, x, threads: int = 0, native: bool = False) -> np.ndarray:
    """m rows of activations -> [m, n], one matvec_kq per row as the reference CPU path does."""
    raw = _u8(raw)
    x = np.ascontiguousarray(x, np.float32).reshape(-1, k)
    m = x.shape[0]
    assert raw.size == n * row_bytes(t, k)
    out = np.empty((m, n), np.float32)
    rc = lib(native).orc_matmul_kq(_p(raw, C.c_uint8), t, n, k, _p(x, C.c_float), m, threads or (os.cpu_count() or 1),
                                   _p(out, C.c_float))
    assert rc == 0, rc
    return out


def rmsnorm(x, w, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x, C.c_float), _p(w, C.c_float), x.size, eps, _p(out, C.c_float))
    return out


def silu_mul(g, u) -> np.ndarray:
    g = np.ascontiguousarray(g, np.float32).reshape(-1)
    u = np.ascontiguousarray(u, np.float32).reshape(-1)
    out = np.empty_like(g)
    lib().orc_silu_mul(_p(g, C.c_float), _p(u, C.c_float), g.size, _p(out, C.c_float))
    return out


def moe_topk(logits, ksel: int) -> tuple[np.ndarray, np.ndarray]:
    lg = np.ascontiguousarray(logits, np.float32)
    lg2 = lg.reshape(-1, lg.shape[-1])
    m, e = lg2.shape
    idx = np.empty((m, ksel), np.uint32)
    wgt = np.empty((m, ksel), np.float32)
    for t in range(m):
        lib().orc_moe_topk(_p(lg2[t], C.c_float), e, ksel, _p(idx[t], C.c_uint32), _p(wgt[t], C.c_float))
    return idx, wgt


def moe_ffn(wg, wu, wd, type_gu: int, type_d: int, h, idx, wgt, d: int, ffn: int, threads: int = 0,
            native: bool = False) -> np.ndarray:
    wg, wu, wd = _u8(wg), _u8(wu), _u8(wd)
    h = np.ascontiguousarray(h, np.float32).reshape(-1, d)
    m = h.shape[0]
    idx = np.ascontiguousarray(idx, np.uint32).reshape(m, -1)
    wgt = np.ascontiguousarray(wgt, np.float32).reshape(m, -1)
    ksel = idx.shape[1]
    out = np.empty((m, d), np.float32)
    rc = lib(native).orc_moe_ffn(_p(wg, C.c_uint8), _p(wu, C.c_uint8), _p(wd, C.c_uint8), type_gu, type_d,
                                 _p(h, C.c_float), _p(idx, C.c_uint32), _p(wgt, C.c_float), m, ksel, d, ffn,
                                 threads or (os.cpu_count() or 1), _p(out, C.c_float))
    assert rc == 0, rc
    return out


def tvec(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_tvec(n, seed & 0xFFFFFFFF, _p(out, C.c_float))
    return out
