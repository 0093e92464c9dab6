"""Host-side mirror of the loader entries: a GGUF tensor directory and the cache file of repacked weights
(reference: crates/ojas-formats/src/gguf.rs:158-205 GgufFile::open / read_tensor_raw and
crates/ojas-models/src/weights.rs:14-32, the cache keyed to the source file by size and modification time).
Everything here runs on the host; the bytes an entry hands out are what Engine.upload_repacked takes."""
import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import lib as _lib


class LoaderError(RuntimeError):
    pass


def _check(rc, err):
    if rc != 0:
        raise LoaderError(f"{err.value.decode() or 'loader call failed'} (code {rc})")


@dataclass(frozen=True)
class TensorInfo:
    name: str
    ggml_type: int
    dims: tuple          # GGUF order: dims[0] = K (contiguous), dims[1] = N
    file_offset: int
    nbytes: int          # 0 for a type whose block size the library does not know


class GgufFile:
    def __init__(self, path):
        self._l = _lib.load()
        self._h = C.c_void_p()
        err = C.create_string_buffer(256)
        _check(self._l.ojas_b200_gguf_open(os.fsencode(path), C.byref(self._h), err, len(err)), err)
        self.path = path

    def close(self):
        if self._h:
            self._l.ojas_b200_gguf_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self):
        return self._l.ojas_b200_gguf_tensor_count(self._h)

    def info(self, index):
        name, t, nd = C.c_char_p(), C.c_uint32(), C.c_uint32()
        dims, off, nb = (C.c_uint64 * 4)(), C.c_uint64(), C.c_uint64()
        rc = self._l.ojas_b200_gguf_tensor_info(self._h, index, C.byref(name), C.byref(t), C.byref(nd), dims, C.byref(off), C.byref(nb))
        if rc != 0:
            raise IndexError(index)
        return TensorInfo(name.value.decode(), t.value, tuple(dims[: nd.value]), off.value, nb.value)

    def tensors(self):
        return [self.info(i) for i in range(len(self))]

    def find(self, name):
        i = self._l.ojas_b200_gguf_find(self._h, name.encode())
        if i < 0:
            raise KeyError(name)
        return int(i)

    def read_raw(self, index):
        ti = self.info(index)
        out = np.empty(ti.nbytes, np.uint8)
        if self._l.ojas_b200_gguf_read_raw(self._h, index, out.ctypes.data, out.size) != 0:
            raise LoaderError(f"cannot read tensor {ti.name}")
        return out


@dataclass(frozen=True)
class CacheEntry:
    name: str
    ggml_type: int
    N: int
    K: int
    data: np.ndarray     # a view into the mapped file: valid until the cache is closed


class WeightCache:
    """The repacked-weight cache of one GGUF file.  WeightCache.for_gguf builds it when it is missing or was made from
    another version of the file (weights.rs:24-32 checks the same two fields)."""

    def __init__(self, cache_path, gguf_path=None):
        self._l = _lib.load()
        self._h = C.c_void_p()
        err = C.create_string_buffer(256)
        rc = self._l.ojas_b200_weight_cache_open(os.fsencode(cache_path), os.fsencode(gguf_path) if gguf_path else None, C.byref(self._h), err, len(err))
        _check(rc, err)

    @staticmethod
    def build(gguf_path, cache_path):
        l = _lib.load()
        err = C.create_string_buffer(256)
        _check(l.ojas_b200_weight_cache_build(os.fsencode(gguf_path), os.fsencode(cache_path), err, len(err)), err)

    @classmethod
    def for_gguf(cls, gguf_path, cache_path):
        try:
            return cls(cache_path, gguf_path)
        except LoaderError:
            cls.build(gguf_path, cache_path)
            return cls(cache_path, gguf_path)

    def close(self):
        if self._h:
            self._l.ojas_b200_weight_cache_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self):
        return self._l.ojas_b200_weight_cache_count(self._h)

    def entry(self, index):
        name, t = C.c_char_p(), C.c_uint32()
        n, k, nb, data = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_void_p()
        if self._l.ojas_b200_weight_cache_entry(self._h, index, C.byref(name), C.byref(t), C.byref(n), C.byref(k), C.byref(data), C.byref(nb)) != 0:
            raise IndexError(index)
        view = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nb.value,))
        return CacheEntry(name.value.decode(), t.value, n.value, k.value, view)

    def entries(self):
        return [self.entry(i) for i in range(len(self))]
