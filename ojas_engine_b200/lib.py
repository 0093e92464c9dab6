"""ctypes binding of ``libojas_b200.so`` (the C ABI declared in ``include/ojas_b200.h``).

There is no CPU fallback anywhere in this package: if the library cannot be loaded the
import of :func:`load` raises, and every compute call needs a B200.
"""
from __future__ import annotations

import ctypes as C
import os
import re

from . import _build

_vp, _sz, _u32, _u64 = C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint64
_i = C.c_int

# name -> (restype, argtypes); must cover every symbol the header declares
SIGNATURES = {
    "ojas_b200_create": (_i, [_i, _vp, C.POINTER(_vp)]),
    "ojas_b200_destroy": (None, [_vp]),
    "ojas_b200_set_stream": (_i, [_vp, _vp]),
    "ojas_b200_stream": (_vp, [_vp]),
    "ojas_b200_set_option": (_i, [_vp, C.c_char_p, _i]),
    "ojas_b200_last_error": (C.c_char_p, [_vp]),
    "ojas_b200_sm_count": (_i, [_vp]),
    "ojas_b200_profile_report": (_sz, [_vp, C.c_char_p, _sz]),
    "ojas_b200_profile_reset": (_i, [_vp]),
    "ojas_b200_launch_count": (_u64, [_vp]),
    "ojas_b200_version": (C.c_char_p, []),
    "ojas_b200_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "ojas_b200_free": (_i, [_vp, _vp]),
    "ojas_b200_upload": (_i, [_vp, _vp, _vp, _sz]),
    "ojas_b200_download": (_i, [_vp, _vp, _vp, _sz]),
    "ojas_b200_memset": (_i, [_vp, _vp, _i, _sz]),
    "ojas_b200_sync": (_i, [_vp]),
    "ojas_b200_event_create": (_i, [_vp, C.POINTER(_vp)]),
    "ojas_b200_event_destroy": (_i, [_vp, _vp]),
    "ojas_b200_event_record": (_i, [_vp, _vp]),
    "ojas_b200_event_elapsed_ms": (_i, [_vp, _vp, _vp, C.POINTER(C.c_float)]),
    "ojas_b200_graph_begin": (_i, [_vp]),
    "ojas_b200_graph_end": (_i, [_vp, C.POINTER(_vp)]),
    "ojas_b200_graph_launch": (_i, [_vp, _vp]),
    "ojas_b200_graph_destroy": (_i, [_vp, _vp]),
    "ojas_b200_host_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "ojas_b200_host_free": (_i, [_vp, _vp]),
    "ojas_b200_raw_bytes": (_sz, [_u32, _sz, _sz]),
    "ojas_b200_repacked_bytes": (_sz, [_u32, _sz, _sz]),
    "ojas_b200_repack": (_i, [_vp, _u32, _vp, _sz, _sz, _vp]),
    "ojas_b200_repack_host": (_i, [_u32, _vp, _sz, _sz, _vp]),
    "ojas_b200_quant_q8k": (_i, [_vp, _vp, _sz, _sz, _vp, _vp, _vp]),
    "ojas_b200_rmsnorm_q8k": (_i, [_vp, _vp, _vp, C.c_float, _sz, _sz, _vp, _vp, _vp, _vp]),
    "ojas_b200_silu_mul_q8k": (_i, [_vp, _vp, _vp, _sz, _sz, _vp, _vp, _vp]),
    "ojas_b200_gemv": (_i, [_vp, _u32, _i, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "ojas_b200_gemv_rmsnorm": (_i, [_vp, _u32, _i, _vp, _vp, C.c_float, _vp, _vp, _vp, _sz, _sz, _sz]),
    "ojas_b200_gemv_silu_mul": (_i, [_vp, _u32, _i, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "ojas_b200_gemv_q8k": (_i, [_vp, _u32, _i, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "ojas_b200_gemv_idots": (_i, [_vp, _u32, _vp, _vp, _vp, _sz, _sz]),
    "ojas_b200_gemm_workspace_bytes": (_sz, [_sz, _sz]),
    "ojas_b200_gemm": (_i, [_vp, _u32, _vp, _vp, _vp, _sz, _sz, _sz, _i, _vp, _sz]),
    "ojas_b200_gemm_f16": (_i, [_vp, _u32, _vp, _vp, _vp, _sz, _sz, _sz, _i, _vp, _sz]),
    "ojas_b200_reserve": (_i, [_vp, _sz]),
    "ojas_b200_reserved_bytes": (_sz, [_vp]),
    "ojas_b200_gemm_static_capacity": (_sz, []),
    "ojas_b200_gemm_static": (_i, [_vp, _u32, _vp, _vp, _vp, _sz, _sz, _sz, _i]),
    "ojas_b200_moe_topk": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "ojas_b200_moe_workspace_bytes": (_sz, [_sz, _sz, _sz, _sz, _sz]),
    "ojas_b200_moe_ffn": (_i, [_vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _vp, _i, _vp, _sz]),
    "ojas_b200_embed_rows": (_i, [_vp, _u32, _vp, _sz, _vp, _sz, _sz, _vp]),
    "ojas_b200_gguf_open": (_i, [C.c_char_p, C.POINTER(_vp), C.c_char_p, _sz]),
    "ojas_b200_gguf_close": (None, [_vp]),
    "ojas_b200_gguf_tensor_count": (_sz, [_vp]),
    "ojas_b200_gguf_tensor_info": (_i, [_vp, _sz, C.POINTER(C.c_char_p), C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u64)]),
    "ojas_b200_gguf_find": (C.c_longlong, [_vp, C.c_char_p]),
    "ojas_b200_gguf_read_raw": (_i, [_vp, _sz, _vp, _sz]),
    "ojas_b200_weight_cache_build": (_i, [C.c_char_p, C.c_char_p, C.c_char_p, _sz]),
    "ojas_b200_weight_cache_open": (_i, [C.c_char_p, C.c_char_p, C.POINTER(_vp), C.c_char_p, _sz]),
    "ojas_b200_weight_cache_close": (None, [_vp]),
    "ojas_b200_weight_cache_count": (_sz, [_vp]),
    "ojas_b200_weight_cache_entry": (_i, [_vp, _sz, C.POINTER(C.c_char_p), C.POINTER(_u32), C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_vp), C.POINTER(_u64)]),
    "ojas_b200_expert_lru_create": (_i, [_sz, C.POINTER(_vp)]),
    "ojas_b200_expert_lru_destroy": (None, [_vp]),
    "ojas_b200_expert_lru_plan": (_i, [_vp, C.POINTER(_u32), _sz, C.POINTER(_u32), C.POINTER(C.c_uint8)]),
    "ojas_b200_expert_lru_stats": (None, [_vp, C.POINTER(_sz)]),
    "ojas_b200_expert_cache_create": (_i, [_vp, _u32, _sz, _sz, _sz, C.POINTER(_vp)]),
    "ojas_b200_expert_cache_destroy": (None, [_vp]),
    "ojas_b200_expert_cache_slots": (_sz, [_vp]),
    "ojas_b200_expert_cache_slot_bytes": (_sz, [_vp]),
    "ojas_b200_expert_cache_arena": (_vp, [_vp]),
    "ojas_b200_expert_cache_stats": (None, [_vp, C.POINTER(_sz)]),
    "ojas_b200_expert_cache_gather": (_i, [_vp, C.POINTER(_u32), _sz, _vp, _vp, C.POINTER(_u64)]),
    "ojas_b200_tp_shard_rows": (_i, [_sz, _i, _i, C.POINTER(_sz), C.POINTER(_sz)]),
    "ojas_b200_tp_shard_k": (_i, [_sz, _i, _i, C.POINTER(_sz), C.POINTER(_sz)]),
    "ojas_b200_tp_slice_k_host": (_i, [_u32, _vp, _sz, _sz, _sz, _sz, _vp]),
    "ojas_b200_tp_create": (_i, [_vp, _i, _i, _sz, C.POINTER(_vp)]),
    "ojas_b200_tp_destroy": (None, [_vp]),
    "ojas_b200_tp_handle_bytes": (_sz, []),
    "ojas_b200_tp_export": (_i, [_vp, _vp]),
    "ojas_b200_tp_import": (_i, [_vp, _i, _vp]),
    "ojas_b200_tp_set_wait_us": (_i, [_vp, C.c_uint]),
    "ojas_b200_tp_gemv": (_i, [_vp, _u32, _vp, _vp, _sz, _sz, _sz]),
    "ojas_b200_tp_join": (_i, [_vp, _i, _vp, _sz]),
    "ojas_b200_tp_allgather": (_i, [_vp, _vp, _sz, _vp]),
    "ojas_b200_has_kernel": (_i, [C.c_char_p]),
    "ojas_b200_kernel_count": (_i, []),
    "ojas_b200_kernel_name": (C.c_char_p, [_i]),
    "ojas_b200_dispatch": (_i, [_vp, C.c_char_p, C.POINTER(_vp), C.POINTER(_u64), _i, C.POINTER(_u32), _i,
                                C.POINTER(_u32), C.POINTER(_u32)]),
    "ojas_b200_encode_host": (_i, [_u32, _vp, _sz, _sz, _vp]),
}

_lib: C.CDLL | None = None


def header_symbols() -> list[str]:
    """Every function name declared in include/ojas_b200.h."""
    with open(_build.HEADER) as fh:
        text = fh.read()
    return sorted(set(re.findall(r"OJAS_B200_API[^;(]*?\b(ojas_b200_\w+)\s*\(", text)))


def load() -> C.CDLL:
    """Load (building first when the sources changed and nvcc is present) and bind the library."""
    global _lib
    if _lib is not None:
        return _lib
    if not _build.is_current():
        if _build._nvcc() is not None:
            _build.build()
        elif not os.path.exists(_build.LIB):
            raise RuntimeError(
                f"{_build.LIB} is missing and nvcc is not available to build it; "
                "run `python -m ojas_engine_b200._build` on a machine with the CUDA toolkit")
    lib = C.CDLL(os.environ.get("OJAS_B200_LIBRARY") or _build.LIB)   # the override is for development builds
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library out of step
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib
