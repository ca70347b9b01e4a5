// An allocation-free matvec entry point.
//
// Some hosts of this library may not allocate device memory when they call into it: a plugin whose
// embedding application owns every device buffer and forbids allocations after start-up (the llama.cpp
// backend contract: all memory comes from the backend's buffer types, graph_compute allocates nothing), a
// serving loop that must never hit cudaMalloc because it serialises the whole device, or code running
// while memory is already fully committed to weights and KV cache.  The ordinary fp32-activation matvec
// needs a small scratch for the 8-bit copy of the activations (11 * k / 32 ints) that such callers have
// nowhere to put.  kcb_matvec_q4k_f32x_static keeps that scratch in the library image instead: a
// file-scope __device__ array that every GPU loading the library carries until the process exits.
//
// Limits and rules:
//   * k <= kStaticMaxK (16384 columns; 22 KB of scratch per GPU); larger k is refused with InvalidValue;
//   * the first call on a device resolves the array's device address (cudaGetSymbolAddress, once per
//     device, with that device current), loads the kernels' module and may set a kernel attribute.  That
//     warm-up call is the one to make outside any stream capture and before memory is counted; from the
//     second call on, the call makes no CUDA call other than its two launches;
//   * every call uses the same array, so two calls whose GPU work can overlap (different streams, or
//     different host threads) race on it -- serialise them on one stream.  The quantizer rewrites every
//     word the matvec reads, so nothing has to be cleared between calls.
// The call allocates nothing: no cudaMalloc/cudaFree and no library routine that allocates.

#include "../../include/kernelcore_b200.h"

#include "common.cuh"
#include "ops.h"

#include <atomic>

namespace {

constexpr int kStaticMaxK = 16384;
constexpr int kStaticInts = 11 * (kStaticMaxK / 32);  // the reference's per-32 scratch layout, llm_kernels.hpp:82-85
constexpr int kMaxDevices = 64;

static __device__ __align__(256) int g_static_q8_scratch[kStaticInts];

// Host code must not pass g_static_q8_scratch itself to a kernel: on the host that name is only a handle.
// The device address is looked up once per device and cached here (two host threads making their first call on
// one device may both look it up; they store the same value).
std::atomic<int*> g_scratch_addr[kMaxDevices] = {};

int scratch_for_current_device(int** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kcb::KCB_INVALID_DEVICE;
    int* addr = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!addr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_q8_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return kcb::KCB_INTERNAL_ERROR;
        }
        addr = static_cast<int*>(p);
        g_scratch_addr[dev].store(addr, std::memory_order_release);
    }
    *out = addr;
    return kcb::KCB_SUCCESS;
}

}  // namespace

extern "C" int kcb_matvec_q4k_f32x_static(const void* w_dev, const float* x_dev, float* y_dev, int rows, int k, void* stream) {
    if (!w_dev || !x_dev || !y_dev || rows < 0 || k <= 0 || k % 256) return kcb::KCB_INVALID_VALUE;
    if (k > kStaticMaxK) return kcb::KCB_INVALID_VALUE;  // beyond the built-in scratch
    if (rows == 0) return kcb::KCB_SUCCESS;
    int* q = nullptr;
    if (const int e = scratch_for_current_device(&q); e != kcb::KCB_SUCCESS) return e;
    const int nb = k / 32;
    float* xd = reinterpret_cast<float*>(q + nb * 8);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (const int e = kcb::quantize_q8x4(x_dev, q, xd, nb, s); e != kcb::KCB_SUCCESS) return e;
    return kcb::matvec_q4k_q8(w_dev, q, xd, y_dev, rows, k, s);
}

extern "C" int kcb_static_scratch_max_k(void) { return kStaticMaxK; }
