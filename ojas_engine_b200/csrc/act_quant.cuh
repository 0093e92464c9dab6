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

__device__ __forceinline__ Q8kLane quant_q8k_values(const float (&v)[8]);

__device__ __forceinline__ Q8kLane quant_q8k_warp(const float *seg /* 256 floats, 32-byte aligned */, int lane) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(seg) + lane * 2);
    const float4 b = __ldg(reinterpret_cast<const float4 *>(seg) + lane * 2 + 1);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    return quant_q8k_values(v);
}

// The same for values already in registers (lane l holds values 8l .. 8l+7 of the super-block).
__device__ __forceinline__ Q8kLane quant_q8k_values(const float (&v)[8]) {
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
        const bool nan = r != r;   // a NaN quotient quantizes to 0 (Rust's `as i8`)
        r = fminf(fmaxf(r, -127.0f), 127.0f);
        qi[i] = nan ? 0 : (int)r;
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

// Half-warp form: lanes 0-15 quantize one super-block, lanes 16-31 another; lane l owns values
// 16*(l & 15) .. +15 of its super-block.  Fewer, fuller instructions per super-block than the
// one-warp form; same results bit for bit.
struct Q8kHalfLane {
    uint4 packed;   // the lane's sixteen int8 values in value order (one 16-byte unit)
    int sum16;      // their sum
    float scale;
};

__device__ __forceinline__ Q8kHalfLane quant_q8k_halfwarp(const float *seg /* 256 floats of this half-warp's block */, int lane) {
    const int hl = lane & 15;
    float v[16];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(seg) + hl * 4 + j);
        v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
    }
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float scale = (m > 0.0f) ? __fdiv_rn(m, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    uint32_t w[4];
    int s = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float t = __fmul_rn(v[4 * j + i], inv);
            float r = round_half_away(t);
            const bool nan = r != r;
            r = fminf(fmaxf(r, -127.0f), 127.0f);
            const int qi = nan ? 0 : (int)r;
            s += qi;
            word |= (uint32_t)(qi & 0xff) << (8 * i);
        }
        w[j] = word;
    }
    Q8kHalfLane out;
    out.packed = make_uint4(w[0], w[1], w[2], w[3]);
    out.sum16 = s;
    out.scale = scale;
    return out;
}

// Where the GEMV kernels keep quantized activations in shared memory.  A super-block is 16
// units of 16 bytes; unit (c, t) holds values 64c + 16t .. +15.  Units are interleaved over
// pairs of super-blocks so that the eight lanes of a quarter-warp (two super-blocks x four
// chunks) read 128 contiguous bytes for a fixed t: no bank conflicts.
__device__ __forceinline__ int xq_unit(int sb, int c, int t) { return (sb >> 1) * 32 + t * 8 + (sb & 1) * 4 + c; }
