// q4b_matvec_noalloc: a single-projection decode matvec for callers that cannot allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a stream-ordered region whose owner
// forbids allocator traffic, in a process whose memory budget was fixed up front by another component, or in a
// plug-in that is only handed pointers and a stream. The regular entry points grow scratch pools on first use
// (prepared activations, per-group sums, partial sums of split tiles, arrival counters); this one keeps all of
// that in one file-scope device array that every GPU loading the library holds until the process exits.
//
// Rules of the shared array:
//   - it is one array per device, shared by every call: calls that overlap on the GPU race on it; order them on
//     one stream or with events;
//   - it keeps the previous call's contents; the arrival counters, the only part that must start at zero, are
//     cleared on the caller's stream at the start of every call;
//   - the first call on a device looks up the array's device address (cudaGetSymbolAddress) and the kernel
//     occupancy; make that first call outside any stream capture.
// Limits: one projection, one bf16 activation row, K <= 32768; larger shapes are rejected, not truncated.
#include "../../include/q4b200.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "q4_kernels.h"

namespace {

constexpr uint32_t kMaxK = 32768;
constexpr uint32_t kMaxWorkers = 2048;  // warps of one launch; each owns two 512-byte partial slots
constexpr size_t kXpBytes = (size_t)kMaxK * 2 + 1024;               // one fp16 column plus over-read slack
constexpr size_t kXsumBytes = (size_t)(kMaxK / 64) * 4 * 4 + 1024;  // [groups][4 columns] fp32
constexpr size_t kRowInvBytes = 256;
constexpr size_t kPartialBytes = (size_t)kMaxWorkers * 2 * 512;
constexpr size_t kCounterBytes = (size_t)kMaxWorkers * 4;
constexpr size_t kOffXsum = kXpBytes;
constexpr size_t kOffRowInv = kOffXsum + kXsumBytes;
constexpr size_t kOffPartials = (kOffRowInv + kRowInvBytes + 255) & ~(size_t)255;
constexpr size_t kOffCounters = kOffPartials + kPartialBytes;
constexpr size_t kScratchBytes = kOffCounters + kCounterBytes;  // about 1.1 MB

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char q4_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
    unsigned char *scratch = nullptr;  // device address of q4_noalloc_scratch on this device
    uint32_t warps_fast = 0, warps_generic = 0;
    int sm_count = 0;
};
PerDevice g_devices[kMaxDevices];
std::mutex g_setup_mutex;

thread_local char g_noalloc_error[256];

int noalloc_fail(int status, const char *message) {
    snprintf(g_noalloc_error, sizeof g_noalloc_error, "%s", message);
    return status;
}

// once per device, with that device current
int setup_device(int device, PerDevice **out) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    PerDevice &d = g_devices[device];
    if (!d.scratch) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, q4_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return noalloc_fail(Q4B_CUDA_ERROR, "cudaGetSymbolAddress failed for the static scratch array");
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess || sms <= 0) return noalloc_fail(Q4B_CUDA_ERROR, "cannot read the SM count");
        d.warps_fast = q4k_gemv_occupancy(1, 1);
        d.warps_generic = q4k_gemv_occupancy(1, 0);
        if (!d.warps_fast || !d.warps_generic) return noalloc_fail(Q4B_CUDA_ERROR, "projection kernel cannot be resident on this device");
        d.sm_count = sms;
        d.scratch = static_cast<unsigned char *>(ptr);
    }
    *out = &d;
    return Q4B_OK;
}

}  // namespace

extern "C" const char *q4b_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" int q4b_matvec_noalloc(int device, const void *x_bf16_dev, uint64_t k, const void *weights_dev,
                                  const void *scales_dev, const void *biases_dev, uint64_t n, float *out_dev, void *stream) {
    if (!x_bf16_dev || !weights_dev || !scales_dev || !biases_dev || !out_dev)
        return noalloc_fail(Q4B_INVALID_ARGUMENT, "a device pointer is null");
    if (device < 0 || device >= kMaxDevices) return noalloc_fail(Q4B_NO_DEVICE, "device ordinal out of range");
    if (k == 0 || n == 0) return noalloc_fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    if (k % 64 != 0) return noalloc_fail(Q4B_INPUT_NOT_GROUPED, "input dimension is not divisible by affine group size 64");
    if (k > kMaxK) return noalloc_fail(Q4B_UNSUPPORTED, "K exceeds the 32768 inputs the static scratch array is sized for");
    if (n > 0xffffffffull) return noalloc_fail(Q4B_DIMENSION_OVERFLOW, "output rows exceeds runtime limits");
    if ((uintptr_t)x_bf16_dev & 15u) return noalloc_fail(Q4B_INVALID_ARGUMENT, "device activations must be 16-byte aligned");
    int current = -1;
    if (cudaGetDevice(&current) != cudaSuccess) return noalloc_fail(Q4B_NO_DEVICE, "no CUDA device is available");
    if (current != device && cudaSetDevice(device) != cudaSuccess) return noalloc_fail(Q4B_NO_DEVICE, "cannot select the device");
    PerDevice *d = nullptr;
    int st = setup_device(device, &d);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (st == Q4B_OK) {
        const uint32_t k32 = (uint32_t)k, kp = (k32 + 127u) & ~127u, groups = k32 / 64, vpad = 4;
        uint16_t *xp = reinterpret_cast<uint16_t *>(d->scratch);
        float *xsum = reinterpret_cast<float *>(d->scratch + kOffXsum);
        float *row_inv = reinterpret_cast<float *>(d->scratch + kOffRowInv);
        float *partials = reinterpret_cast<float *>(d->scratch + kOffPartials);
        unsigned int *counters = reinterpret_cast<unsigned int *>(d->scratch + kOffCounters);
        // the counters are the only state that must start at zero (a previous call may have been cut short)
        cudaError_t e = cudaMemsetAsync(counters, 0, kCounterBytes, s);
        if (e == cudaSuccess) e = q4k_prepare_x(x_bf16_dev, 0, 1, k32, kp, vpad, xp, xsum, row_inv, s);
        if (e == cudaSuccess) {
            q4::GemvParams p;
            memset(&p, 0, sizeof p);
            const uint8_t *w = static_cast<const uint8_t *>(weights_dev), *sc = static_cast<const uint8_t *>(scales_dev),
                          *bi = static_cast<const uint8_t *>(biases_dev);
            const bool fast = ((((uintptr_t)w | (uintptr_t)sc | (uintptr_t)bi) & 15u) == 0) && groups % 8u == 0;
            p.jobs[0].w = w;
            p.jobs[0].s = sc;
            p.jobs[0].b = bi;
            p.jobs[0].out = out_dev;
            p.jobs[0].n = (uint32_t)n;
            p.jobs[0].out_stride = (uint32_t)n;
            p.jobs[0].tile_begin = 0;
            p.jobs[0].w_misalign = (uint32_t)((uintptr_t)w & 15u);
            p.n_jobs = 1;
            p.xp = xp;
            p.xsum = xsum;
            p.row_inv = row_inv;
            p.kp = kp;
            p.v_cols = 1;
            p.vpad = vpad;
            p.m_rows = 1;
            p.k = k32;
            p.groups = groups;
            p.cpt = (groups + 1u) / 2u;
            p.units = (uint64_t)((n + 15) / 16) * p.cpt;
            uint64_t workers = (uint64_t)d->sm_count * (fast ? d->warps_fast : d->warps_generic);
            if (workers > kMaxWorkers) workers = kMaxWorkers;
            const uint64_t min_chunks = (p.cpt + 7u) / 8u;
            if (workers > p.units / min_chunks) workers = p.units / min_chunks;
            if (workers == 0) workers = 1;
            p.workers = (uint32_t)workers;
            p.partials = partials;
            p.counters = counters;
            e = q4k_gemv(&p, 1, fast ? 1 : 0, s);
        }
        if (e != cudaSuccess) {
            snprintf(g_noalloc_error, sizeof g_noalloc_error, "CUDA call failed: %s", cudaGetErrorString(e));
            st = Q4B_CUDA_ERROR;
        }
    }
    if (current != device) cudaSetDevice(current);
    return st;
}
