// Device helpers shared by the affine-Q4 kernels (sm_100a).
//
// Format (MLX affine, group 64): a weight row is K/8 little-endian u32 words, eight 4-bit
// values per word with value i at bits [4i,4i+4) (k = 8*word + i); one bf16 scale and one bf16
// bias per 64 consecutive k; w = scale*q + bias. Mirrors shaders/qwen38.metal:18-115 of the
// reference (bf16 conversion, nibble order, byte-wise loads for unaligned tensors).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace q4 {

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits) { return __uint_as_float(bits << 16); }

// round-to-nearest-even without a NaN case: shaders/qwen38.metal:22-26
__device__ __forceinline__ uint32_t float_to_bf16_bits(float v) {
    uint32_t bits = __float_as_uint(v);
    return (bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16;
}

// Streaming 128-bit load: read-only path, no L1 allocation (weights are touched once).
__device__ __forceinline__ uint4 ldg_stream_v4(const void *p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Predicated loads: nothing is fetched and zeros are returned when `pred` is false. Written as
// predicated instructions so a warp whose lanes disagree does not branch.
__device__ __forceinline__ uint4 ldg_stream_v4_pred(const void *p, bool pred) {
    uint4 v;
    asm("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t"
        "@q ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p), "r"((uint32_t)pred));
    return v;
}

// cached variant for data that every warp re-reads (prepared activations)
__device__ __forceinline__ uint4 ldg_v4_pred(const void *p, bool pred) {
    uint4 v;
    asm("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t"
        "@q ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p), "r"((uint32_t)pred));
    return v;
}

__device__ __forceinline__ float2 ldg_f2_pred(const float *p, bool pred) {
    float2 v;
    asm("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %3, 0;\n\tmov.f32 %0, 0f00000000;\n\tmov.f32 %1, 0f00000000;\n\t"
        "@q ld.global.nc.v2.f32 {%0,%1}, [%2];\n\t}"
        : "=f"(v.x), "=f"(v.y)
        : "l"(p), "r"((uint32_t)pred));
    return v;
}

__device__ __forceinline__ uint32_t ldg_u16_pred(const void *p, bool pred) {
    uint32_t v;
    asm("{\n\t.reg .pred q;\n\t.reg .b16 h;\n\tsetp.ne.b32 q, %2, 0;\n\tmov.b16 h, 0;\n\t"
        "@q ld.global.nc.u16 h, [%1];\n\tcvt.u32.u16 %0, h;\n\t}"
        : "=r"(v)
        : "l"(p), "r"((uint32_t)pred));
    return v;
}

// Asynchronous 16-byte global -> shared copy (L2 only: the data is streamed once), its group fence and
// wait, and the matching shared load.
__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_16_pred(uint32_t smem_addr, const void *gmem, bool pred) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t@q cp.async.cg.shared.global [%0], [%1], 16;\n\t}" ::"r"(smem_addr),
                 "l"(gmem), "r"((uint32_t)pred)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t smem_addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_addr) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t smem_addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_addr) : "memory");
    return v;
}

__device__ __forceinline__ uint2 lds_v2(uint32_t smem_addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(smem_addr) : "memory");
    return v;
}

// 16 bytes starting `mis` (0..15) bytes into the 32-byte window {lo, hi}
__device__ __forceinline__ uint4 realign_16(uint4 lo, uint4 hi, uint32_t mis) {
    uint32_t w0 = lo.x, w1 = lo.y, w2 = lo.z, w3 = lo.w, w4 = hi.x, w5 = hi.y, w6 = hi.z, w7 = hi.w;
    // `mis` is the same for every lane of a warp (one tensor), so this is a branch, not a row of selects: offsets
    // below four bytes -- two, for tensors that follow an odd-sized safetensors header -- need the shifts only
    if (mis & 12u) {
        if (mis & 4) { w0 = w1; w1 = w2; w2 = w3; w3 = w4; w4 = w5; w5 = w6; w6 = w7; }
        if (mis & 8) { w0 = w2; w1 = w3; w2 = w4; w3 = w5; w4 = w6; }
    }
    const uint32_t sh = (mis & 3u) * 8u;
    uint4 out;
    out.x = __funnelshift_r(w0, w1, sh);
    out.y = __funnelshift_r(w1, w2, sh);
    out.z = __funnelshift_r(w2, w3, sh);
    out.w = __funnelshift_r(w3, w4, sh);
    return out;
}

// 16 bytes from an arbitrarily aligned address: two aligned 128-bit loads of the enclosing
// window and a funnel shift (the byte-addressed twin of the aligned load; the reference's
// qwen38_load_u32, shaders/qwen38.metal:105-110, reads byte by byte instead).
// `mis` = address & 15, uniform over the warp. Reads up to 16 bytes past p+16 when mis != 0;
// shard allocations are padded for that.
__device__ __forceinline__ uint4 ldg_stream_v4_unaligned(const uint8_t *p, uint32_t mis) {
    const uint8_t *base = p - mis;
    uint4 lo = ldg_stream_v4(base);
    if (mis == 0) return lo;
    uint4 hi = ldg_stream_v4(base + 16);
    uint32_t w0 = lo.x, w1 = lo.y, w2 = lo.z, w3 = lo.w, w4 = hi.x, w5 = hi.y, w6 = hi.z, w7 = hi.w;
    if (mis & 4) { w0 = w1; w1 = w2; w2 = w3; w3 = w4; w4 = w5; w5 = w6; w6 = w7; }
    if (mis & 8) { w0 = w2; w1 = w3; w2 = w4; w3 = w5; w4 = w6; }
    uint32_t sh = (mis & 3u) * 8u;
    uint4 out;
    out.x = __funnelshift_r(w0, w1, sh);
    out.y = __funnelshift_r(w1, w2, sh);
    out.z = __funnelshift_r(w2, w3, sh);
    out.w = __funnelshift_r(w3, w4, sh);
    return out;
}

// one bf16 parameter (scale or bias) at any byte alignment, as raw bits
__device__ __forceinline__ uint32_t ldg_bf16_bits(const uint8_t *p) {
    if ((reinterpret_cast<uintptr_t>(p) & 1u) == 0) {
        return (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(p));
    }
    return (uint32_t)__ldg(p) | ((uint32_t)__ldg(p + 1) << 8);
}

// Constants of the nibble conversion, held in registers the compiler cannot see through so that
// mask-and-or stays one three-input logic instruction (with two immediates it becomes two).
struct Magic {
    uint32_t mask_lo;  // 0x000f000f: nibbles at bits [0,4) of each half
    uint32_t mask_hi;  // 0x00f000f0: nibbles at bits [4,8) of each half
    uint32_t k1024;    // 0x64006400: fp16 1024.0 in both halves
    uint32_t sixteenth;  // 0x2c002c00: fp16 1/16
    uint32_t neg64;    // 0xd400d400: fp16 -64.0
};

__device__ __forceinline__ Magic make_magic() {
    Magic m;
    asm volatile("mov.b32 %0, 0x000f000f;\n\tmov.b32 %1, 0x00f000f0;\n\tmov.b32 %2, 0x64006400;\n\t"
                 "mov.b32 %3, 0x2c002c00;\n\tmov.b32 %4, 0xd400d400;"
                 : "=r"(m.mask_lo), "=r"(m.mask_hi), "=r"(m.k1024), "=r"(m.sixteenth), "=r"(m.neg64));
    return m;
}

// Two nibbles of a packed word -> exact fp16x2. 0x6400|q is the fp16 number 1024+q (ulp 1 in
// [1024,2048)); a nibble four bits higher reads as 1024+16q. Both corrections are exact.
//   lo: nibbles at bits [0,4) and [16,20)      hi: nibbles at bits [4,8) and [20,24)
__device__ __forceinline__ uint32_t nib_lo_to_f16x2(uint32_t v, const Magic &m) {
    uint32_t biased, out;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(biased) : "r"(v), "r"(m.mask_lo), "r"(m.k1024));  // (v & mask) | 1024
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(out) : "r"(biased), "r"(m.k1024));
    return out;
}
__device__ __forceinline__ uint32_t nib_hi_to_f16x2(uint32_t v, const Magic &m) {
    uint32_t biased, out;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(biased) : "r"(v), "r"(m.mask_hi), "r"(m.k1024));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out) : "r"(biased), "r"(m.sixteenth), "r"(m.neg64));  // (1024+16q)/16 - 64
    return out;
}

// Load into registers that keep their old contents when `pred` is false (no zero fill).
__device__ __forceinline__ void ldg_v4_keep(uint4 &v, const void *p, bool pred) {
    asm("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t@q ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "l"(p), "r"((uint32_t)pred));
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float silu(float v) { return v * (1.0f / (1.0f + __expf(-v))); }

// ---- integer tensor-core path (persistent decode kernel, short-batch kernel) ----

// The activation is held as 23-bit fixed point: x' = round(x * 2^e) with 2^e putting the largest magnitude into
// [2^21, 2^22). A bf16 value within 2^14 of the maximum is represented exactly, smaller ones to 2^-22 of the maximum.
// e = 0 for an all-zero vector.
__device__ __forceinline__ int scale_exponent(uint32_t amax_bits) {
    const int e = 21 - ((int)((amax_bits >> 23) & 0xffu) - 127);
    return amax_bits == 0 ? 0 : max(-100, min(100, e));
}


__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// exact for |i| < 2^22
__device__ __forceinline__ float small_int_to_float(int i) { return __int_as_float(i + 0x4B400000) - 12582912.0f; }


}  // namespace q4
