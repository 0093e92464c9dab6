"""Host-side mirror of the engine's backend interface for the quantized-matmul path.

``B200Gpu`` plays the part of ``CudaGpu`` (crates/ojas-cuda/src/device.rs:87-146, 418-537): it
owns one device + one stream and offers the ``Device`` calls (alloc / upload / read,
crates/ojas-core/src/lib.rs:26-40) and the ``KernelRuntime`` calls (has_kernel / begin /
dispatch / submit, crates/ojas-core/src/kernel.rs:68-83) with the same names and argument
meaning.  ``Lin`` is the loaded weight (crates/ojas-cuda/src/qwen35.rs:146-226) and ``mm`` the
matmul operator (``CudaSsm::mm``, crates/ojas-cuda/src/qwen35.rs:644-702).  Everything
computes through the C ABI; nothing here falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import lib as _lib

Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS = 8, 12, 13, 14, 20, 23
PLAIN, ACCUM, BIAS = 0, 1, 2
GEMV_MAX_M = 8
_TAGS = {Q4_K: "q4k", Q5_K: "q5k", Q6_K: "q6k", Q8_0: "q80", IQ4_NL: "iq4nl", IQ4_XS: "iq4xs"}


class OjasB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"ojas_b200 error {code}: {message}")
        self.code = code


@dataclass
class Buf:
    """A device allocation (the engine's CuBuf, crates/ojas-cuda/src/device.rs:20-23)."""
    ptr: int
    nbytes: int

    def at(self, byte_offset: int) -> int:
        return self.ptr + byte_offset


@dataclass
class Lin:
    """A weight as it lives on the device: repacked planes + its GGUF type and shape
    ([n, k]: one output per row).  Counterpart of ``Lin`` / ``Repr`` in
    crates/ojas-cuda/src/qwen35.rs:146-226."""
    buf: Buf
    ggml_type: int
    n: int
    k: int

    @property
    def gguf_bytes(self) -> int:
        return _lib.load().ojas_b200_raw_bytes(self.ggml_type, self.n, self.k)


class Enc:
    """A chain of dispatches on the context's stream (``KernelRuntime::begin``)."""

    def __init__(self) -> None:
        self.dispatches = 0


class B200Gpu:
    def __init__(self, device: int = 0, stream: int | None = None):
        self._l = _lib.load()
        ctx = C.c_void_p()
        rc = self._l.ojas_b200_create(device, C.c_void_p(stream) if stream else None, C.byref(ctx))
        if rc != 0:
            why = {-1: "no such device", -2: "CUDA runtime error (no GPU?)", -3: "device is not sm_100 (B200)"}.get(rc, "")
            raise OjasB200Error(rc, f"ojas_b200_create(device={device}) failed: {why}")
        self._ctx = ctx
        self.device = device

    # ------------------------------------------------------------------ plumbing
    def _ck(self, rc: int) -> None:
        if rc != 0:
            raise OjasB200Error(rc, self._l.ojas_b200_last_error(self._ctx).decode())

    def close(self) -> None:
        if getattr(self, "_ctx", None):
            self._l.ojas_b200_destroy(self._ctx)
            self._ctx = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    @property
    def ctx(self) -> C.c_void_p:
        return self._ctx

    @property
    def sm_count(self) -> int:
        return self._l.ojas_b200_sm_count(self._ctx)

    @property
    def launch_count(self) -> int:
        return int(self._l.ojas_b200_launch_count(self._ctx))

    @property
    def stream(self) -> int:
        return int(self._l.ojas_b200_stream(self._ctx) or 0)

    def set_option(self, key: str, value: int) -> None:
        self._ck(self._l.ojas_b200_set_option(self._ctx, key.encode(), int(value)))

    # ------------------------------------------------------------------ Device
    def alloc_bytes(self, nbytes: int) -> Buf:
        p = C.c_void_p()
        self._ck(self._l.ojas_b200_alloc(self._ctx, nbytes, C.byref(p)))
        return Buf(int(p.value), nbytes)

    def alloc(self, len_f32: int) -> Buf:
        """``Device::alloc``: room for ``len_f32`` floats."""
        return self.alloc_bytes(len_f32 * 4)

    def free(self, buf: Buf) -> None:
        self._ck(self._l.ojas_b200_free(self._ctx, C.c_void_p(buf.ptr)))

    def write(self, buf: Buf, data: np.ndarray, byte_offset: int = 0) -> None:
        data = np.ascontiguousarray(data)
        assert byte_offset + data.nbytes <= buf.nbytes
        self._ck(self._l.ojas_b200_upload(self._ctx, C.c_void_p(buf.ptr + byte_offset), data.ctypes.data_as(C.c_void_p), data.nbytes))
        self.sync()  # the host array may be pageable and short-lived

    def upload(self, data: np.ndarray) -> Buf:
        """``Device::upload``: a new buffer holding ``data``."""
        data = np.ascontiguousarray(data)
        buf = self.alloc_bytes(max(data.nbytes, 1))
        if data.nbytes:
            self.write(buf, data)
        return buf

    def read(self, buf: Buf, dtype, count: int, byte_offset: int = 0) -> np.ndarray:
        """``Device::read``: waits for the stream, then copies ``count`` items back."""
        out = np.empty(count, dtype)
        assert byte_offset + out.nbytes <= buf.nbytes
        self._ck(self._l.ojas_b200_download(self._ctx, out.ctypes.data_as(C.c_void_p), C.c_void_p(buf.ptr + byte_offset), out.nbytes))
        self.sync()
        return out

    def memset(self, buf: Buf, value: int = 0) -> None:
        self._ck(self._l.ojas_b200_memset(self._ctx, C.c_void_p(buf.ptr), value, buf.nbytes))

    def sync(self) -> None:
        self._ck(self._l.ojas_b200_sync(self._ctx))

    def profile_report(self) -> list[tuple[str, int, float]]:
        """Per-kernel (name, launches, total ms) of the per-launch profiler (option ``profile``), largest total first."""
        n = self._l.ojas_b200_profile_report(self._ctx, None, 0)
        buf = C.create_string_buffer(n + 1)
        self._l.ojas_b200_profile_report(self._ctx, buf, n + 1)
        rows = []
        for line in buf.value.decode().splitlines():
            name, launches, ms, _ = line.split()
            rows.append((name, int(launches), float(ms)))
        return rows

    def profile_reset(self) -> None:
        self._ck(self._l.ojas_b200_profile_reset(self._ctx))

    # ------------------------------------------------------------------ upload layout
    def load_weight(self, raw: np.ndarray, ggml_type: int, n: int, k: int) -> Lin:
        """``Lin::load_as``: GGUF blocks (host bytes) -> repacked planes on the device."""
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        want = self._l.ojas_b200_raw_bytes(ggml_type, n, k)
        if want == 0 or raw.size != want:
            raise OjasB200Error(-1, f"load_weight: type {ggml_type} [{n},{k}] needs {want} bytes, got {raw.size}")
        tmp = self.upload(raw)
        out = self.alloc_bytes(self._l.ojas_b200_repacked_bytes(ggml_type, n, k))
        try:
            self._ck(self._l.ojas_b200_repack(self._ctx, ggml_type, C.c_void_p(tmp.ptr), n, k, C.c_void_p(out.ptr)))
            self.sync()
        finally:
            self.free(tmp)
        return Lin(out, ggml_type, n, k)

    def load_repacked(self, packed: np.ndarray, ggml_type: int, n: int, k: int) -> Lin:
        """A weight that is already in the tile layout (an entry of the repacked-weight cache): one upload."""
        packed = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
        want = self._l.ojas_b200_repacked_bytes(ggml_type, n, k)
        if want == 0 or packed.size != want:
            raise OjasB200Error(-1, f"load_repacked: type {ggml_type} [{n},{k}] needs {want} bytes, got {packed.size}")
        return Lin(self.upload(packed), ggml_type, n, k)

    # ------------------------------------------------------------------ typed entry points
    def quant_q8k(self, x: Buf, m: int, k: int, q: Buf, scales: Buf, bsums: Buf) -> None:
        self._ck(self._l.ojas_b200_quant_q8k(self._ctx, C.c_void_p(x.ptr), m, k, C.c_void_p(q.ptr), C.c_void_p(scales.ptr), C.c_void_p(bsums.ptr)))

    def rmsnorm_q8k(self, x: Buf, w: Buf, eps: float, m: int, k: int, q: Buf, scales: Buf, bsums: Buf, xn: Buf | None = None) -> None:
        """RMSNorm of the rows of x [m,k] ending in Q8_K (the input of ``gemv_q8k``); ``xn`` also keeps the f32 rows."""
        self._ck(self._l.ojas_b200_rmsnorm_q8k(self._ctx, C.c_void_p(x.ptr), C.c_void_p(w.ptr), C.c_float(eps), m, k,
                                               C.c_void_p(xn.ptr) if xn else None, C.c_void_p(q.ptr), C.c_void_p(scales.ptr), C.c_void_p(bsums.ptr)))

    def silu_mul_q8k(self, g: Buf, u: Buf, m: int, k: int, q: Buf, scales: Buf, bsums: Buf) -> None:
        """act = silu(g) * u per element of [m,k], ending in Q8_K."""
        self._ck(self._l.ojas_b200_silu_mul_q8k(self._ctx, C.c_void_p(g.ptr), C.c_void_p(u.ptr), m, k, C.c_void_p(q.ptr), C.c_void_p(scales.ptr), C.c_void_p(bsums.ptr)))

    def gemv(self, w: Lin, x: Buf, y: Buf, m: int = 1, form: int = PLAIN, bias: Buf | None = None) -> None:
        self._ck(self._l.ojas_b200_gemv(self._ctx, w.ggml_type, form, C.c_void_p(x.ptr), C.c_void_p(w.buf.ptr), C.c_void_p(y.ptr),
                                        C.c_void_p(bias.ptr) if bias else None, w.k, w.n, m))

    def gemv_rmsnorm(self, w: Lin, x: Buf, norm_w: Buf, eps: float, y: Buf, m: int = 1, form: int = PLAIN, bias: Buf | None = None) -> None:
        """``y = W rmsnorm(x)``: the norm is formed in the GEMV's prologue (one launch instead of producer + GEMV)."""
        self._ck(self._l.ojas_b200_gemv_rmsnorm(self._ctx, w.ggml_type, form, C.c_void_p(x.ptr), C.c_void_p(norm_w.ptr), C.c_float(eps),
                                                C.c_void_p(w.buf.ptr), C.c_void_p(y.ptr), C.c_void_p(bias.ptr) if bias else None, w.k, w.n, m))

    def gemv_silu_mul(self, w: Lin, g: Buf, u: Buf, y: Buf, m: int = 1, form: int = PLAIN, bias: Buf | None = None) -> None:
        """``y = W (silu(g) * u)``: SwiGLU is formed in the GEMV's prologue (one launch instead of producer + GEMV)."""
        self._ck(self._l.ojas_b200_gemv_silu_mul(self._ctx, w.ggml_type, form, C.c_void_p(g.ptr), C.c_void_p(u.ptr), C.c_void_p(w.buf.ptr),
                                                 C.c_void_p(y.ptr), C.c_void_p(bias.ptr) if bias else None, w.k, w.n, m))

    def gemv_q8k(self, w: Lin, q: Buf, scales: Buf, bsums: Buf, y: Buf, m: int = 1, form: int = PLAIN, bias: Buf | None = None) -> None:
        self._ck(self._l.ojas_b200_gemv_q8k(self._ctx, w.ggml_type, form, C.c_void_p(q.ptr), C.c_void_p(scales.ptr), C.c_void_p(bsums.ptr),
                                            C.c_void_p(w.buf.ptr), C.c_void_p(y.ptr), C.c_void_p(bias.ptr) if bias else None, w.k, w.n, m))

    def gemm_workspace_bytes(self, m: int, k: int) -> int:
        return int(self._l.ojas_b200_gemm_workspace_bytes(m, k))

    def gemm(self, w: Lin, x: Buf, y: Buf, m: int, accum: bool = False, workspace: Buf | None = None) -> None:
        """Tensor-core prefill GEMM.  Without a caller workspace a grow-only scratch buffer owned by
        this object is used (allocated outside the call path of the C ABI, which never allocates)."""
        need = self.gemm_workspace_bytes(m, w.k)
        if workspace is None:
            ws = getattr(self, "_gemm_ws", None)
            if ws is None or ws.nbytes < need:
                if ws is not None:
                    self.sync()
                    self.free(ws)
                ws = self._gemm_ws = self.alloc_bytes(need)
            workspace = ws
        self._ck(self._l.ojas_b200_gemm(self._ctx, w.ggml_type, C.c_void_p(x.ptr), C.c_void_p(w.buf.ptr), C.c_void_p(y.ptr),
                                        w.k, w.n, m, 1 if accum else 0, C.c_void_p(workspace.ptr), workspace.nbytes))

    def reserve(self, nbytes: int) -> None:
        """Context-owned scratch for the name-based prefill entries (allocates: set-up only)."""
        self._ck(self._l.ojas_b200_reserve(self._ctx, nbytes))

    def moe_topk(self, logits: Buf, idx: Buf, wgt: Buf, m: int, e: int, ksel: int) -> None:
        self._ck(self._l.ojas_b200_moe_topk(self._ctx, C.c_void_p(logits.ptr), C.c_void_p(idx.ptr), C.c_void_p(wgt.ptr), m, e, ksel))

    def moe_workspace_bytes(self, m: int, e: int, ksel: int, d: int, ffn: int) -> int:
        return int(self._l.ojas_b200_moe_workspace_bytes(m, e, ksel, d, ffn))

    def moe_ffn(self, wg: Lin, wu: Lin, wd: Lin, h: Buf, idx: Buf, wgt: Buf, out: Buf, m: int, e: int, ksel: int,
                accum: bool = False, workspace: Buf | None = None) -> None:
        """Expert FFN over stacked experts: wg, wu are [e*ffn, d], wd is [e*d, ffn]."""
        ffn, d = wg.n // e, wg.k
        assert wu.n == wg.n and wu.k == d and wd.n == e * d and wd.k == ffn
        need = self.moe_workspace_bytes(m, e, ksel, d, ffn)
        if workspace is None:
            ws = getattr(self, "_moe_ws", None)
            if ws is None or ws.nbytes < need:
                if ws is not None:
                    self.sync()
                    self.free(ws)
                ws = self._moe_ws = self.alloc_bytes(need)
            workspace = ws
        self._ck(self._l.ojas_b200_moe_ffn(self._ctx, wg.ggml_type, wd.ggml_type, C.c_void_p(h.ptr), C.c_void_p(wg.buf.ptr),
                                           C.c_void_p(wu.buf.ptr), C.c_void_p(wd.buf.ptr), C.c_void_p(idx.ptr), C.c_void_p(wgt.ptr),
                                           m, e, ksel, d, ffn, C.c_void_p(out.ptr), 1 if accum else 0, C.c_void_p(workspace.ptr),
                                           workspace.nbytes))

    def gemm_static(self, w: Lin, x: Buf, y: Buf, m: int, accum: bool = False) -> None:
        """The GEMM for callers that cannot supply scratch: uses the library's built-in 8 MiB array
        (m * k <= 4 194 304), allocates nothing."""
        self._ck(self._l.ojas_b200_gemm_static(self._ctx, w.ggml_type, C.c_void_p(x.ptr), C.c_void_p(w.buf.ptr), C.c_void_p(y.ptr),
                                               w.k, w.n, m, 1 if accum else 0))

    def embed_rows(self, table: Buf, ggml_type: int, rows: int, ids: Buf, m: int, d: int, x: Buf) -> None:
        """``x[m, :]`` = the dequantized row ``ids[m]`` of a token table kept as raw GGUF blocks (``q35_embed_q4k``)."""
        self._ck(self._l.ojas_b200_embed_rows(self._ctx, ggml_type, C.c_void_p(table.ptr), rows, C.c_void_p(ids.ptr), m, d, C.c_void_p(x.ptr)))

    def gemv_idots(self, w: Lin, x: Buf, idots: Buf) -> None:
        self._ck(self._l.ojas_b200_gemv_idots(self._ctx, w.ggml_type, C.c_void_p(x.ptr), C.c_void_p(w.buf.ptr), C.c_void_p(idots.ptr), w.k, w.n))

    # ------------------------------------------------------------------ KernelRuntime
    def has_kernel(self, name: str) -> bool:
        return bool(self._l.ojas_b200_has_kernel(name.encode()))

    def kernel_names(self) -> list[str]:
        return [self._l.ojas_b200_kernel_name(i).decode() for i in range(self._l.ojas_b200_kernel_count())]

    def begin(self) -> Enc:
        return Enc()

    def dispatch(self, enc: Enc, name: str, bufs, consts, grid=(1, 1, 1), block=(1, 1, 1)) -> None:
        """``KernelRuntime::dispatch``: ``bufs`` = [(Buf, byte_offset), ...] positional, then u32 ``consts``."""
        n = len(bufs)
        ptrs = (C.c_void_p * max(n, 1))(*[C.c_void_p(b.ptr) for b, _ in bufs])
        offs = (C.c_uint64 * max(n, 1))(*[int(o) for _, o in bufs])
        cs = (C.c_uint32 * max(len(consts), 1))(*[int(c) for c in consts])
        g = (C.c_uint32 * 3)(*grid)
        bl = (C.c_uint32 * 3)(*block)
        self._ck(self._l.ojas_b200_dispatch(self._ctx, name.encode(), ptrs, offs, n, cs, len(consts), g, bl))
        enc.dispatches += 1

    def submit(self, enc: Enc) -> None:
        """``KernelRuntime::submit``: wait for the chain; device errors surface here."""
        self.sync()

    # ------------------------------------------------------------------ the matmul operator
    def mm(self, x: Buf, w: Lin, y: Buf, m: int, accum: bool = False) -> None:
        """``CudaSsm::mm(st, x, w, y, m, accum)`` (crates/ojas-cuda/src/qwen35.rs:644-702): picks the
        kernel from the weight representation and the row count."""
        form = ACCUM if accum else PLAIN
        if m <= GEMV_MAX_M:
            self.gemv(w, x, y, m, form)
            return
        self.gemm(w, x, y, m, accum)  # tensor-core prefill path

    # ------------------------------------------------------------------ timing / graphs
    def event(self) -> int:
        p = C.c_void_p()
        self._ck(self._l.ojas_b200_event_create(self._ctx, C.byref(p)))
        return int(p.value)

    def record(self, ev: int) -> None:
        self._ck(self._l.ojas_b200_event_record(self._ctx, C.c_void_p(ev)))

    def elapsed_ms(self, start: int, stop: int) -> float:
        ms = C.c_float()
        self._ck(self._l.ojas_b200_event_elapsed_ms(self._ctx, C.c_void_p(start), C.c_void_p(stop), C.byref(ms)))
        return float(ms.value)

    def graph_begin(self) -> None:
        self._ck(self._l.ojas_b200_graph_begin(self._ctx))

    def graph_end(self) -> int:
        p = C.c_void_p()
        self._ck(self._l.ojas_b200_graph_end(self._ctx, C.byref(p)))
        return int(p.value)

    def graph_launch(self, g: int) -> None:
        self._ck(self._l.ojas_b200_graph_launch(self._ctx, C.c_void_p(g)))

    def graph_destroy(self, g: int) -> None:
        self._ck(self._l.ojas_b200_graph_destroy(self._ctx, C.c_void_p(g)))

    def host_alloc(self, nbytes: int, dtype=np.uint8) -> np.ndarray:
        """Pinned host array (kept alive by the returned array's base object)."""
        p = C.c_void_p()
        self._ck(self._l.ojas_b200_host_alloc(self._ctx, nbytes, C.byref(p)))
        raw = (C.c_uint8 * nbytes).from_address(p.value)
        arr = np.frombuffer(raw, dtype=np.uint8).view(dtype)
        return arr


class ExpertCache:
    """Bounded arena of expert slots with LRU eviction (``ExpertCache``, crates/ojas-cuda/src/expert_cache.rs:34-160).
    ``gather(ids, load)`` makes the experts resident and returns their byte offsets into ``arena``; ``load(id)`` returns
    the expert's GGUF blocks as a uint8 array (where a real caller reads from its model file)."""

    def __init__(self, gpu: B200Gpu, ggml_type: int, n: int, k: int, budget_bytes: int):
        self.gpu, self._l = gpu, gpu._l
        h = C.c_void_p()
        gpu._ck(self._l.ojas_b200_expert_cache_create(gpu.ctx, ggml_type, n, k, budget_bytes, C.byref(h)))
        self._h = h
        self.raw_bytes = raw_bytes(ggml_type, n, k)

    @property
    def slots(self) -> int:
        return int(self._l.ojas_b200_expert_cache_slots(self._h))

    @property
    def slot_bytes(self) -> int:
        return int(self._l.ojas_b200_expert_cache_slot_bytes(self._h))

    @property
    def resident_bytes(self) -> int:
        return self.slots * self.slot_bytes

    @property
    def arena(self) -> Buf:
        return Buf(int(self._l.ojas_b200_expert_cache_arena(self._h)), self.resident_bytes)

    @property
    def stats(self) -> dict:
        out = (C.c_size_t * 4)()
        self._l.ojas_b200_expert_cache_stats(self._h, out)
        return {"hits": out[0], "misses": out[1], "evictions": out[2], "bytes_streamed": out[3]}

    def hit_rate(self) -> float:
        st = self.stats
        total = st["hits"] + st["misses"]
        return st["hits"] / total if total else 0.0

    def gather(self, ids, load) -> np.ndarray:
        ids = np.ascontiguousarray(ids, np.uint32)
        offs = np.zeros(ids.size, np.uint64)
        nbytes = self.raw_bytes

        @C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t)
        def cb(_user, expert, dst, n):
            try:
                data = np.ascontiguousarray(load(int(expert))).view(np.uint8).reshape(-1)
                if data.size != n:
                    return 1
                C.memmove(dst, data.ctypes.data, n)
                return 0
            except Exception:
                return 1

        self.gpu._ck(self._l.ojas_b200_expert_cache_gather(self._h, ids.ctypes.data_as(C.POINTER(C.c_uint32)), ids.size, cb, None,
                                                           offs.ctypes.data_as(C.POINTER(C.c_uint64))))
        assert nbytes == self.raw_bytes
        return offs

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._l.ojas_b200_expert_cache_destroy(self._h)
            self._h = None


# ---------------------------------------------------------------------- host utilities (no GPU)
def raw_bytes(ggml_type: int, n: int, k: int) -> int:
    return int(_lib.load().ojas_b200_raw_bytes(ggml_type, n, k))


def repacked_bytes(ggml_type: int, n: int, k: int) -> int:
    return int(_lib.load().ojas_b200_repacked_bytes(ggml_type, n, k))


def encode(ggml_type: int, w: np.ndarray) -> np.ndarray:
    """f32 [n, k] -> GGUF blocks with this library's simple test-input encoder."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    out = np.empty(raw_bytes(ggml_type, n, k), np.uint8)
    rc = _lib.load().ojas_b200_encode_host(ggml_type, w.ctypes.data_as(C.c_void_p), n, k, out.ctypes.data_as(C.c_void_p))
    if rc != 0:
        raise OjasB200Error(rc, f"encode: type {ggml_type} [{n},{k}]")
    return out


def repack_host(ggml_type: int, raw: np.ndarray, n: int, k: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    out = np.empty(repacked_bytes(ggml_type, n, k), np.uint8)
    rc = _lib.load().ojas_b200_repack_host(ggml_type, raw.ctypes.data_as(C.c_void_p), n, k, out.ctypes.data_as(C.c_void_p))
    if rc != 0:
        raise OjasB200Error(rc, f"repack_host: type {ggml_type} [{n},{k}]")
    return out
