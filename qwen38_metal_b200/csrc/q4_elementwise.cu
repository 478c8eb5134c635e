// Small kernels that sit between projections: SwiGLU, row argmax, dtype casts, and the
// weightless RMS-norm of the synthetic decode stack. Counterparts in the reference:
// qwen38_swiglu_rows (shaders/qwen38.metal:4188-4198), qwen38_argmax_rows (:4201-4245),
// qwen38_f32_to_f16 / qwen38_f16_to_f32 (:4166-4186), qwen38_rms_norm (:4250-4311).
#include "q4_kernels.h"

#include "q4_device.cuh"

namespace q4 {

__global__ void __launch_bounds__(256) swiglu_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                     uint64_t count, float *__restrict__ out_f32,
                                                     uint16_t *__restrict__ out_bf16) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float g = gate[i];
    float h = (g * (1.0f / (1.0f + expf(-g)))) * up[i];
    if (out_f32) out_f32[i] = h;
    if (out_bf16) out_bf16[i] = (uint16_t)float_to_bf16_bits(h);
}

__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float *__restrict__ in, uint64_t count,
                                                          uint16_t *__restrict__ out) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = (uint16_t)float_to_bf16_bits(in[i]);
}

// greatest value wins, equal values -> lower index (shaders/qwen38.metal:4218-4221)
__device__ __forceinline__ void argmax_merge(float &bv, uint32_t &bi, float ov, uint32_t oi) {
    if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
    }
}

__device__ __forceinline__ void argmax_block_reduce(float &bv, uint32_t &bi) {
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
        argmax_merge(bv, bi, ov, oi);
    }
    if ((threadIdx.x & 31u) == 0) {
        sv[threadIdx.x >> 5] = bv;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = threadIdx.x < 8 ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < 8 ? si[threadIdx.x] : 0xffffffffu;
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
            argmax_merge(bv, bi, ov, oi);
        }
    }
}

// stage 1: grid (parts, m). stage 2: grid (1, m) over the `parts` partial pairs.
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float *__restrict__ logits, uint32_t n,
                                                             uint32_t parts, float *__restrict__ pv,
                                                             uint32_t *__restrict__ pi) {
    const uint32_t row = blockIdx.y;
    const float *src = logits + (uint64_t)row * n;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < n; i += parts * 256u) argmax_merge(bv, bi, src[i], i);
    argmax_block_reduce(bv, bi);
    if (threadIdx.x == 0) {
        pv[row * parts + blockIdx.x] = bv;
        pi[row * parts + blockIdx.x] = bi;
    }
}

__global__ void __launch_bounds__(256) argmax_final_kernel(const float *__restrict__ pv, const uint32_t *__restrict__ pi,
                                                           uint32_t parts, uint32_t index_base,
                                                           uint32_t *__restrict__ tokens, float *__restrict__ values) {
    const uint32_t row = blockIdx.x;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < parts; i += 256u) argmax_merge(bv, bi, pv[row * parts + i], pi[row * parts + i]);
    argmax_block_reduce(bv, bi);
    if (threadIdx.x == 0) {
        // an all-NaN / empty row keeps the reference's starting index 0
        tokens[row] = (bi == 0xffffffffu ? 0u : bi) + index_base;
        if (values) values[row] = bv;
    }
}

// y = bf16(d / sqrt(mean(d^2) + eps)) for one vector per block; used by the synthetic stack to
// keep the activation scale near one from layer to layer.
__global__ void __launch_bounds__(1024) rms_unit_bf16_kernel(const float *__restrict__ in, uint32_t n, float eps,
                                                            uint16_t *__restrict__ out) {
    __shared__ float warp_sums[32];
    const float *src = in + (uint64_t)blockIdx.x * n;
    float s = 0.f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) s += src[i] * src[i];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if ((threadIdx.x & 31u) == 0) warp_sums[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        s = threadIdx.x < (blockDim.x >> 5) ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (threadIdx.x == 0) warp_sums[0] = s;
    }
    __syncthreads();
    const float inv = rsqrtf(warp_sums[0] / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x)
        out[(uint64_t)blockIdx.x * n + i] = (uint16_t)float_to_bf16_bits(src[i] * inv);
}

// dequantized_row (src/native.rs:4944-4987): out[i] = q*scale + bias for one row, byte-addressed
__global__ void __launch_bounds__(256) dequantize_row_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ s,
                                                             const uint8_t *__restrict__ b, uint32_t k, uint32_t row,
                                                             float *__restrict__ out) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= k) return;
    const uint8_t *wp = w + ((uint64_t)row * (k / 8) + i / 8) * 4u;
    uint32_t word = (uint32_t)wp[0] | ((uint32_t)wp[1] << 8) | ((uint32_t)wp[2] << 16) | ((uint32_t)wp[3] << 24);
    float q = (float)((word >> ((i % 8u) * 4u)) & 0xfu);
    uint64_t p = ((uint64_t)row * (k / 64) + i / 64) * 2u;
    float scale = bf16_bits_to_float((uint32_t)s[p] | ((uint32_t)s[p + 1] << 8));
    float bias = bf16_bits_to_float((uint32_t)b[p] | ((uint32_t)b[p + 1] << 8));
    out[i] = __fadd_rn(__fmul_rn(q, scale), bias);
}

}  // namespace q4

extern "C" cudaError_t q4k_dequantize_row(const uint8_t *w, const uint8_t *s, const uint8_t *b, uint32_t k, uint32_t row,
                                          float *out, cudaStream_t stream) {
    q4::dequantize_row_kernel<<<(k + 255) / 256, 256, 0, stream>>>(w, s, b, k, row, out);
    return cudaGetLastError();
}

extern "C" cudaError_t q4k_swiglu(const float *gate, const float *up, uint64_t count, float *out_f32,
                                  uint16_t *out_bf16, cudaStream_t stream) {
    q4::swiglu_kernel<<<(uint32_t)((count + 255) / 256), 256, 0, stream>>>(gate, up, count, out_f32, out_bf16);
    return cudaGetLastError();
}

extern "C" cudaError_t q4k_f32_to_bf16(const float *in, uint64_t count, uint16_t *out, cudaStream_t stream) {
    q4::f32_to_bf16_kernel<<<(uint32_t)((count + 255) / 256), 256, 0, stream>>>(in, count, out);
    return cudaGetLastError();
}

extern "C" uint32_t q4k_argmax_parts(uint32_t n) {
    uint32_t parts = (n + 4095u) / 4096u;
    return parts < 1u ? 1u : (parts > 1024u ? 1024u : parts);
}

extern "C" cudaError_t q4k_argmax_rows(const float *logits, uint32_t m, uint32_t n, uint32_t index_base, float *pv,
                                       uint32_t *pi, uint32_t *tokens, float *values, cudaStream_t stream) {
    uint32_t parts = q4k_argmax_parts(n);
    q4::argmax_partial_kernel<<<dim3(parts, m), 256, 0, stream>>>(logits, n, parts, pv, pi);
    q4::argmax_final_kernel<<<m, 256, 0, stream>>>(pv, pi, parts, index_base, tokens, values);
    return cudaGetLastError();
}

extern "C" cudaError_t q4k_rms_unit_bf16(const float *in, uint32_t rows, uint32_t n, float eps, uint16_t *out,
                                         cudaStream_t stream) {
    q4::rms_unit_bf16_kernel<<<rows, 1024, 0, stream>>>(in, n, eps, out);
    return cudaGetLastError();
}
