"""ojas_engine_b200 — the quantized-matmul hot path of ojas-engine, rebuilt for B200 (sm_100a).

The product is ``libojas_b200.so`` (CUDA kernels behind the C ABI of ``include/ojas_b200.h``);
this package is its host-side mirror of the engine's backend interface.  There is no CPU
fallback: compute calls need the built library and a B200.
"""
from .runtime import (ACCUM, BIAS, GEMV_MAX_M, IQ4_NL, IQ4_XS, PLAIN, Q4_K, Q5_K, Q6_K, Q8_0, B200Gpu, Buf, Enc, ExpertCache, Lin, OjasB200Error, encode,
                      raw_bytes, repack_host, repacked_bytes)

__all__ = ["ACCUM", "BIAS", "GEMV_MAX_M", "IQ4_NL", "IQ4_XS", "PLAIN", "Q4_K", "Q5_K", "Q6_K", "Q8_0", "B200Gpu", "Buf", "Enc", "ExpertCache", "Lin", "OjasB200Error",
           "encode", "raw_bytes", "repack_host", "repacked_bytes"]
