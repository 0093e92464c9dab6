"""Row-sharded tensor parallelism for the quantized matmul: one process per GPU, NCCL over NVLink.

The reference engine is single-GPU; this module defines the sharded form of its matmul operator:

* ``col``: the weight's rows (outputs) are split across ranks; every rank computes its slice of y and the
  slices are joined by an all-gather.  Each output element is bit-identical to the single-GPU result.
* ``row``: the weight's K dimension is split on 256-weight super-block boundaries; every rank takes its
  slice of x (Q8_K activation scales are per super-block, so each rank's integer block dots are the ones a
  single GPU forms), computes a full-width partial y, and the partials are joined by an all-reduce (sum).

``torch.distributed`` is used only as plumbing for the collectives.  The compute callable is injected so
the same shard/collective logic runs under ``gloo`` on CPU in the tests.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as _lib
from .runtime import raw_bytes


def shard_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    r0, rows = C.c_size_t(), C.c_size_t()
    rc = _lib.load().ojas_b200_tp_shard_rows(n, world, rank, C.byref(r0), C.byref(rows))
    if rc:
        raise ValueError(f"shard_rows(n={n}, world={world}, rank={rank})")
    return int(r0.value), int(rows.value)


def shard_k(k: int, world: int, rank: int) -> tuple[int, int]:
    k0, klen = C.c_size_t(), C.c_size_t()
    rc = _lib.load().ojas_b200_tp_shard_k(k, world, rank, C.byref(k0), C.byref(klen))
    if rc:
        raise ValueError(f"shard_k(k={k}, world={world}, rank={rank}): K must be a multiple of 256")
    return int(k0.value), int(klen.value)


def slice_rows(raw: np.ndarray, ggml_type: int, n: int, k: int, row0: int, rows: int) -> np.ndarray:
    """GGUF bytes of weight rows [row0, row0+rows)."""
    rb = raw_bytes(ggml_type, 1, k)
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(n, rb)
    return np.ascontiguousarray(raw[row0:row0 + rows]).reshape(-1)


def slice_k(raw: np.ndarray, ggml_type: int, n: int, k: int, k0: int, klen: int) -> np.ndarray:
    """GGUF bytes of the K range [k0, k0+klen) of every row."""
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    out = np.empty(raw_bytes(ggml_type, n, klen), np.uint8)
    rc = _lib.load().ojas_b200_tp_slice_k_host(ggml_type, raw.ctypes.data_as(C.c_void_p), n, k, k0, klen, out.ctypes.data_as(C.c_void_p))
    if rc:
        raise ValueError(f"slice_k(type={ggml_type}, n={n}, k={k}, k0={k0}, klen={klen})")
    return out


class ShardedLinear:
    """One rank's share of a [n, k] weight.

    ``matmul(raw_shard, ggml_type, n_local, k_local, x_local) -> ndarray/tensor [m, n_local]`` is the local
    compute (the B200 kernels in production); ``dist`` is ``torch.distributed`` (or None for world 1).
    """

    def __init__(self, raw: np.ndarray, ggml_type: int, n: int, k: int, mode: str, rank: int, world: int):
        if mode not in ("col", "row"):
            raise ValueError("mode must be 'col' or 'row'")
        self.ggml_type, self.n, self.k, self.mode, self.rank, self.world = ggml_type, n, k, mode, rank, world
        if mode == "col":
            self.row0, self.rows = shard_rows(n, world, rank)
            self.k0, self.klen = 0, k
            self.raw = slice_rows(raw, ggml_type, n, k, self.row0, self.rows)
        else:
            self.row0, self.rows = 0, n
            self.k0, self.klen = shard_k(k, world, rank)
            self.raw = slice_k(raw, ggml_type, n, k, self.k0, self.klen)

    @property
    def local_shape(self) -> tuple[int, int]:
        return self.rows, self.klen

    def local_x(self, x: np.ndarray) -> np.ndarray:
        """This rank's slice of the activations [m, k]."""
        return np.ascontiguousarray(x[:, self.k0:self.k0 + self.klen])

    def join(self, y_local, dist=None):
        """All-gather (col) or all-reduce (row) of torch tensors; returns the full [m, n] tensor."""
        import torch
        if self.world == 1 or dist is None:
            return y_local
        if self.mode == "row":
            dist.all_reduce(y_local, op=dist.ReduceOp.SUM)
            return y_local
        m = y_local.shape[0]
        sizes = [shard_rows(self.n, self.world, r)[1] for r in range(self.world)]
        if len(set(sizes)) == 1:
            gathered = torch.empty((self.world * m, sizes[0]), dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(gathered, y_local.contiguous())
            return gathered.view(self.world, m, sizes[0]).permute(1, 0, 2).reshape(m, self.n)
        parts = [torch.empty((m, s), dtype=y_local.dtype, device=y_local.device) for s in sizes]
        dist.all_gather(parts, y_local.contiguous())
        return torch.cat(parts, dim=1)


class TpGroup:
    """The decode join through peer memory (``ojas_b200_tp_*``): every rank's GEMV stores its results straight into
    all ranks' receive windows (stamped values, no flags) and a join kernel with a bounded wait forms the result.  One process per GPU;
    ``exchange(obj) -> list`` is any host all-gather of Python objects (``torch.distributed.all_gather_object``
    wrapped by the caller): it carries the CUDA IPC handles once, at set-up, and nothing afterwards."""

    COL, ROW = 1, 2

    def __init__(self, gpu, world: int, rank: int, slot_floats: int, exchange):
        self.gpu, self.world, self.rank, self.slot_floats = gpu, world, rank, slot_floats
        self._l = _lib.load()
        h = C.c_void_p()
        gpu._ck(self._l.ojas_b200_tp_create(gpu.ctx, world, rank, slot_floats, C.byref(h)))
        self._h = h
        nbytes = self._l.ojas_b200_tp_handle_bytes()
        mine = (C.c_uint8 * nbytes)()
        gpu._ck(self._l.ojas_b200_tp_export(self._h, mine))
        handles = exchange(bytes(mine))
        for peer, blob in enumerate(handles):
            if peer != rank:
                buf = (C.c_uint8 * nbytes).from_buffer_copy(blob)
                gpu._ck(self._l.ojas_b200_tp_import(self._h, peer, buf))

    def set_wait_us(self, micros: int) -> None:
        self.gpu._ck(self._l.ojas_b200_tp_set_wait_us(self._h, micros))

    def gemv(self, w, x, offset: int = 0) -> None:
        """One activation row through this rank's shard ``w`` (a ``Lin``); results pushed to every rank."""
        self.gpu._ck(self._l.ojas_b200_tp_gemv(self._h, w.ggml_type, C.c_void_p(x.ptr), C.c_void_p(w.buf.ptr), w.k, w.n, offset))

    def join(self, mode: int, y=None, n_total: int = 0) -> None:
        self.gpu._ck(self._l.ojas_b200_tp_join(self._h, mode, C.c_void_p(y.ptr) if y is not None else None, n_total))

    def allgather(self, src, floats: int, y_all) -> None:
        """One kernel: push ``floats`` values of ``src`` to every rank, wait (bounded), copy out ``y_all`` [world][floats]."""
        self.gpu._ck(self._l.ojas_b200_tp_allgather(self._h, C.c_void_p(src.ptr), floats, C.c_void_p(y_all.ptr)))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._l.ojas_b200_tp_destroy(self._h)
            self._h = None
