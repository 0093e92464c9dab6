// Warp-level Q8_K activation quantization, shared by the standalone kernel and by the GEMV
// prologue.  One warp quantizes one 256-value super-block: lane l owns values 8l .. 8l+7.
// Bit-identical to quant_q8k (crates/ojas-cpu/src/cpu_math.rs:545-563): scale = amax/127
// (1 when amax == 0), inv = 1/scale, q = clamp(round_half_away(v * inv), -127, 127).
#pragma once
#include "common.cuh"

struct Q8kLane {
    uint2 packed;   // the lane's eight int8 values, little-endian in value order
    int sum8;       // their sum
    float scale;    // the super-block scale (same in every lane)
};

__device__ __forceinline__ Q8kLane quant_q8k_warp(const float *seg /* 256 floats, 32-byte aligned */, int lane) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(seg) + lane * 2);
    const float4 b = __ldg(reinterpret_cast<const float4 *>(seg) + lane * 2 + 1);
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float scale = (m > 0.0f) ? __fdiv_rn(m, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    int qi[8];
    int s = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float r = round_half_away(__fmul_rn(v[i], inv));
        r = fminf(fmaxf(r, -127.0f), 127.0f);
        qi[i] = (r != r) ? 0 : (int)r;
        s += qi[i];
    }
    Q8kLane out;
    out.packed.x = (uint32_t)(qi[0] & 0xff) | ((uint32_t)(qi[1] & 0xff) << 8) | ((uint32_t)(qi[2] & 0xff) << 16) |
                   ((uint32_t)(qi[3] & 0xff) << 24);
    out.packed.y = (uint32_t)(qi[4] & 0xff) | ((uint32_t)(qi[5] & 0xff) << 8) | ((uint32_t)(qi[6] & 0xff) << 16) |
                   ((uint32_t)(qi[7] & 0xff) << 24);
    out.sum8 = s;
    out.scale = scale;
    return out;
}

// Where the GEMV kernels keep quantized activations in shared memory.  A super-block is 16
// units of 16 bytes; unit (c, t) holds values 64c + 16t .. +15.  Units are interleaved over
// pairs of super-blocks so that the eight lanes of a quarter-warp (two super-blocks x four
// chunks) read 128 contiguous bytes for a fixed t: no bank conflicts.
__device__ __forceinline__ int xq_unit(int sb, int c, int t) { return (sb >> 1) * 32 + t * 8 + (sb & 1) * 4 + c; }
