// Matvec for callers whose activations and results live in host memory.
//
// The reference's Backend::matvec (llm/llm_model.cpp:385-397) reads x and writes y in the process's own memory,
// because its "device" is the CPU.  A caller that keeps that habit hands host buffers to every call; this pipe keeps
// the copies off the critical path: two slots of device buffers, a compute stream and one copy stream per direction.
// submit() enqueues x -> device, the single-launch matvec (in-kernel Q8 quantization) and y -> host, and returns at
// once; the copy-in of call s + 1 and the read-back of call s - 1 overlap the kernel of call s.  y_host of a call is complete after sync(), or
// after the second following submit() has returned (its slot is reused only when its copy has finished).
// Host buffers should be pinned (cudaHostAlloc / cudaHostRegister) for the copies to be asynchronous.

#include "../../include/kernelcore_b200.h"

#include "common.cuh"
#include "ops.h"

namespace {

using namespace kcb;

struct HostPipe {
    int rows = 0, k = 0;
    unsigned long long calls = 0;
    cudaStream_t compute = nullptr, copy = nullptr, copy_in = nullptr;
    float* x[2] = {};
    float* y[2] = {};
    cudaEvent_t computed[2] = {}, read_back[2] = {}, x_ready[2] = {};
    ~HostPipe() {
        if (compute) cudaStreamSynchronize(compute);
        if (copy) cudaStreamSynchronize(copy);
        if (copy_in) cudaStreamSynchronize(copy_in);
        for (int i = 0; i < 2; ++i) {
            if (x_ready[i]) cudaEventDestroy(x_ready[i]);
            if (x[i]) cudaFree(x[i]);
            if (y[i]) cudaFree(y[i]);
            if (computed[i]) cudaEventDestroy(computed[i]);
            if (read_back[i]) cudaEventDestroy(read_back[i]);
        }
        if (compute) cudaStreamDestroy(compute);
        if (copy) cudaStreamDestroy(copy);
        if (copy_in) cudaStreamDestroy(copy_in);
    }
};

}  // namespace

extern "C" {

int kcb_host_matvec_create(int rows, int k, void** out) {
    if (!out || rows <= 0 || rows % 8 || k <= 0 || k % 256 || k > 4096) return KCB_INVALID_VALUE;
    *out = nullptr;
    auto* p = new HostPipe;
    p->rows = rows, p->k = k;
    bool ok = cudaStreamCreateWithFlags(&p->compute, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p->copy, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p->copy_in, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < 2 && ok; ++i)
        ok = cudaMalloc(reinterpret_cast<void**>(&p->x[i]), static_cast<size_t>(k) * 4) == cudaSuccess &&
             cudaMalloc(reinterpret_cast<void**>(&p->y[i]), static_cast<size_t>(rows) * 4) == cudaSuccess &&
             cudaEventCreateWithFlags(&p->computed[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&p->read_back[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&p->x_ready[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventRecord(p->read_back[i], p->copy) == cudaSuccess && cudaEventRecord(p->computed[i], p->compute) == cudaSuccess;
    if (!ok) {
        delete p;
        return KCB_OUT_OF_MEMORY;
    }
    *out = p;
    return KCB_SUCCESS;
}

int kcb_host_matvec_submit(void* h, const void* planes_dev, const float* x_host, float* y_host) {
    if (!h || !planes_dev || !x_host || !y_host) return KCB_INVALID_VALUE;
    auto* p = static_cast<HostPipe*>(h);
    const int sl = static_cast<int>(p->calls++ & 1);
    // x travels on its own stream, so the copy of call s + 1 runs under the kernel of call s; it may overwrite the
    // slot's x only after the kernel that last read it
    if (cudaStreamWaitEvent(p->copy_in, p->computed[sl], 0) != cudaSuccess ||
        cudaMemcpyAsync(p->x[sl], x_host, static_cast<size_t>(p->k) * 4, cudaMemcpyHostToDevice, p->copy_in) != cudaSuccess ||
        cudaEventRecord(p->x_ready[sl], p->copy_in) != cudaSuccess || cudaStreamWaitEvent(p->compute, p->x_ready[sl], 0) != cudaSuccess ||
        cudaStreamWaitEvent(p->compute, p->read_back[sl], 0) != cudaSuccess)  // ... and the slot's last y has left
        return KCB_INTERNAL_ERROR;
    if (const int e = matvec_q6k_f32x_sharded(planes_dev, p->x[sl], p->y[sl], nullptr, 0, nullptr, nullptr, nullptr, 0, 1, p->rows, p->k, p->compute);
        e != KCB_SUCCESS)
        return e;
    if (cudaEventRecord(p->computed[sl], p->compute) != cudaSuccess || cudaStreamWaitEvent(p->copy, p->computed[sl], 0) != cudaSuccess ||
        cudaMemcpyAsync(y_host, p->y[sl], static_cast<size_t>(p->rows) * 4, cudaMemcpyDeviceToHost, p->copy) != cudaSuccess ||
        cudaEventRecord(p->read_back[sl], p->copy) != cudaSuccess)
        return KCB_INTERNAL_ERROR;
    return KCB_SUCCESS;
}

int kcb_host_matvec_sync(void* h) {
    if (!h) return KCB_INVALID_VALUE;
    auto* p = static_cast<HostPipe*>(h);
    return cudaStreamSynchronize(p->copy_in) == cudaSuccess && cudaStreamSynchronize(p->compute) == cudaSuccess &&
                   cudaStreamSynchronize(p->copy) == cudaSuccess
               ? KCB_SUCCESS
               : KCB_INTERNAL_ERROR;
}

int kcb_host_matvec_destroy(void* h) {
    delete static_cast<HostPipe*>(h);
    return KCB_SUCCESS;
}

}  // extern "C"
