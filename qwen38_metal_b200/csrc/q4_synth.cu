// Seeded synthetic tensors generated directly in HBM (the benchmark's stand-in for a
// checkpoint: ~14 GB of packed weights cannot be staged through the host in reasonable time).
//
// value(seed, tensor, index) = (sum of twelve 16-bit uniforms - 6*65535) / 65536, the uniforms
// being the 16-bit fields of three splitmix64 outputs: an integer-only Irwin-Hall normal, so
// this generator and the CPU one agree bit for bit. Quantisation is the MLX affine recipe:
// per 64 inputs of a row, bias = min, scale = (max-min)/15, q = clamp(rint((w-bias)/scale)),
// scale and bias stored as bf16 (RNE).
#include "q4_kernels.h"

#include "q4_device.cuh"

namespace q4 {

__device__ __forceinline__ uint64_t splitmix64(uint64_t value) {
    value += 0x9e3779b97f4a7c15ull;
    uint64_t z = value;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float synth_normal(uint64_t base, uint64_t index) {
    int32_t total = 0;
#pragma unroll
    for (uint64_t j = 0; j < 3; ++j) {
        uint64_t r = splitmix64(base ^ (index * 3u + j));
        total += (int32_t)(r & 0xffffu) + (int32_t)((r >> 16) & 0xffffu) + (int32_t)((r >> 32) & 0xffffu) +
                 (int32_t)((r >> 48) & 0xffffu);
    }
    return __fmul_rn((float)(total - 6 * 65535), 1.0f / 65536.0f);
}

// one thread per (row, group); values are regenerated for the second pass instead of kept
__global__ void __launch_bounds__(128) synth_q4_kernel(uint64_t base, float sigma, uint64_t row0, uint64_t rows,
                                                       uint32_t k, uint8_t *__restrict__ w, uint8_t *__restrict__ s,
                                                       uint8_t *__restrict__ b) {
    const uint32_t groups = k / 64;
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * groups) return;
    uint64_t r = idx / groups;
    uint32_t g = (uint32_t)(idx % groups);
    uint64_t first = (row0 + r) * k + (uint64_t)g * 64u;
    float lo = 0.f, hi = 0.f;
    for (uint32_t i = 0; i < 64; ++i) {
        float v = __fmul_rn(sigma, synth_normal(base, first + i));
        lo = (i == 0 || v < lo) ? v : lo;
        hi = (i == 0 || v > hi) ? v : hi;
    }
    const float scale = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
    const float bias = lo;
    uint8_t *wp = w + (r * (k / 8) + (uint64_t)g * 8u) * 4u;
    for (uint32_t word = 0; word < 8; ++word) {
        uint32_t packed = 0;
        for (uint32_t i = 0; i < 8; ++i) {
            float q = 0.f;
            if (scale != 0.f) {
                float v = __fmul_rn(sigma, synth_normal(base, first + word * 8 + i));
                q = rintf(__fdiv_rn(__fsub_rn(v, bias), scale));
                q = q < 0.f ? 0.f : (q > 15.f ? 15.f : q);
            }
            packed |= (uint32_t)q << (4 * i);
        }
        // byte stores: the destination may be misaligned on purpose
        wp[4 * word + 0] = (uint8_t)packed;
        wp[4 * word + 1] = (uint8_t)(packed >> 8);
        wp[4 * word + 2] = (uint8_t)(packed >> 16);
        wp[4 * word + 3] = (uint8_t)(packed >> 24);
    }
    uint32_t sbits = float_to_bf16_bits(scale), bbits = float_to_bf16_bits(bias);
    uint64_t p = (r * groups + g) * 2u;
    s[p] = (uint8_t)sbits;
    s[p + 1] = (uint8_t)(sbits >> 8);
    b[p] = (uint8_t)bbits;
    b[p + 1] = (uint8_t)(bbits >> 8);
}

__global__ void __launch_bounds__(256) synth_bf16_kernel(uint64_t base, uint64_t count, uint16_t *__restrict__ out) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = (uint16_t)float_to_bf16_bits(synth_normal(base, i));
}

}  // namespace q4

static uint64_t host_splitmix64(uint64_t value) {
    value += 0x9e3779b97f4a7c15ull;
    uint64_t z = value;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

extern "C" cudaError_t q4k_synth_q4(uint64_t seed, uint64_t tensor, float sigma, uint64_t row0, uint64_t rows,
                                    uint32_t k, uint8_t *w, uint8_t *s, uint8_t *b, cudaStream_t stream) {
    uint64_t base = host_splitmix64(seed ^ host_splitmix64(tensor));
    uint64_t total = rows * (k / 64);
    if (total == 0) return cudaSuccess;
    q4::synth_q4_kernel<<<(uint32_t)((total + 127) / 128), 128, 0, stream>>>(base, sigma, row0, rows, k, w, s, b);
    return cudaGetLastError();
}

extern "C" cudaError_t q4k_synth_bf16(uint64_t seed, uint64_t tensor, uint64_t count, uint16_t *out,
                                      cudaStream_t stream) {
    uint64_t base = host_splitmix64(seed ^ host_splitmix64(tensor));
    if (count == 0) return cudaSuccess;
    q4::synth_bf16_kernel<<<(uint32_t)((count + 255) / 256), 256, 0, stream>>>(base, count, out);
    return cudaGetLastError();
}
