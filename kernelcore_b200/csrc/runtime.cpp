// The kc* runtime re-backed by CUDA: device memory, streams, events and graphs per visible GPU.
//
// Stands in for the reference's src/runtime.cpp (lifecycle, memory, launch, capture, events, sticky
// fault state), src/stream.cpp (streams; its CPU worker pool has no counterpart) and
// src/allocation_registry.cpp (interval map used to range-check every pointer before a launch).
// Exposed twice: as extern "C" kcb_* functions returning int status codes, and as the reference's
// C++ kc* functions (include/kernelcore/api.hpp), which forward to them.
//
// Semantics kept from the reference (include/kernelcore/api.hpp:15-85, src/runtime.cpp):
//   * launches on the null stream are synchronous and return the kernel's result; on a created stream
//     they are asynchronous and errors surface at the next synchronize (first error wins);
//   * between BeginCapture and EndCapture launches are validated and recorded, not run; copies, memsets,
//     frees and device synchronisation are refused (UnsupportedOperation) while any stream captures;
//   * kcFree takes exact base pointers only and drains the device first; zero-byte kcMalloc is
//     InvalidValue; a device-side failure is sticky (ContextPoisoned) until kcDeviceReset;
//   * a thread-local detail string describes the most recent failure on the calling thread.
// Extension: every visible GPU is a device; kcSetDevice selects the calling thread's current one.

#include "../../include/kernelcore_b200.h"

#include "common.cuh"
#include "dispatch.h"

#include <kernelcore/api.hpp>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <utility>
#include <vector>

using namespace kcb;

struct kcStream_st {
    cudaStream_t s = nullptr;
    int device = 0;
    bool capturing = false;
    bool is_default = false;
};
struct kcEvent_st {
    cudaEvent_t e = nullptr;
    int device = 0;
};
struct kcGraph_st {
    cudaGraph_t g = nullptr;
    cudaGraphExec_t exec = nullptr;
    int device = 0;
};

namespace {

thread_local int tl_device = 0;
thread_local std::string tl_detail;

struct Device {
    bool started = false;
    kcStream_st dflt;
    std::map<uintptr_t, size_t> allocs;  // base -> bytes
    std::set<kcStream_st*> streams;
    std::set<kcEvent_st*> events;
    std::set<kcGraph_st*> graphs;
    int capturing = 0;  // streams of this device in capture
    bool poisoned = false;
    cudaError_t injected = cudaSuccess;  // test hook: reported by the next successful wait or launch
    kc::FaultInfo fault{};
    char props_name[128] = {};
};

struct Runtime {
    std::recursive_mutex m;
    bool initialized = false;
    int ndev = 0;
    std::vector<std::unique_ptr<Device>> dev;
    std::map<std::string, const kc::KernelEntry*> user;
    kc::Codegen codegen = kc::Codegen::Auto;
};
Runtime& rt() {
    static Runtime r;
    return r;
}

int fail(int code, const std::string& why) {
    tl_detail = why;
    return code;
}
std::string cuda_text(const char* what, cudaError_t e) {
    return std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
}

// Brings up the calling thread's current device on first use.
int device_ready(Device*& out) {
    Runtime& r = rt();
    if (!r.initialized) return fail(KCB_NOT_INITIALIZED, "kcInit has not been called");
    if (tl_device < 0 || tl_device >= r.ndev) return fail(KCB_INVALID_DEVICE, "current device index is out of range");
    Device& d = *r.dev[tl_device];
    if (cudaSetDevice(tl_device) != cudaSuccess) return fail(KCB_INVALID_DEVICE, "cudaSetDevice failed");
    if (!d.started) {
        cudaStream_t s;
        const cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
        if (e != cudaSuccess) return fail(KCB_INTERNAL_ERROR, cuda_text("default stream", e));
        d.dflt.s = s;
        d.dflt.device = tl_device;
        d.dflt.is_default = true;
        d.started = true;
    }
    out = &d;
    return KCB_SUCCESS;
}

// Turns a CUDA error seen after device work into the sticky fault state.
int fault(Device& d, const char* what, cudaError_t e) {
    d.poisoned = true;
    d.fault = kc::FaultInfo{};
    d.fault.code = static_cast<uint32_t>(e);
    std::snprintf(d.fault.kernel, sizeof d.fault.kernel, "%s", what);
    cudaGetLastError();
    return fail(KCB_KERNEL_FAULT, cuda_text(what, e));
}

// The result of a call that waited for, or enqueued, device work.  A test can plant one error code per device
// (kcb_test_inject_device_error): the next such call that itself succeeded reports the planted code instead, which
// drives the fault -> poisoned -> reset cycle without any failing kernel.
int after_device_work(Device& d, const char* what, cudaError_t e) {
    if (e == cudaSuccess && d.injected != cudaSuccess) std::swap(e, d.injected);
    return e == cudaSuccess ? KCB_SUCCESS : fault(d, what, e);
}

int usable(Device*& d) {
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    if (d->poisoned) return fail(KCB_CONTEXT_POISONED, "a device fault is pending; call kcDeviceReset");
    return KCB_SUCCESS;
}

// Resolves a stream handle (null = the device's default stream) and checks it belongs to the device.
int resolve(Device& d, kcStream_t h, kcStream_st*& out) {
    if (!h) {
        out = &d.dflt;
        return KCB_SUCCESS;
    }
    if (!d.streams.count(h)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown stream handle for the current device");
    out = h;
    return KCB_SUCCESS;
}

struct Checker final : kc::LaunchContext, kcb::RangeChecker {
    explicit Checker(const Device& d) : dev(d) {}
    const Device& dev;
    int check(const void* p, size_t bytes, const char* what) const override {
        if (bytes == 0) return KCB_SUCCESS;
        if (!p) return fail(KCB_INVALID_POINTER, std::string(what) + ": null device pointer");
        const uintptr_t key = reinterpret_cast<uintptr_t>(p);
        auto it = dev.allocs.upper_bound(key);
        if (it == dev.allocs.begin()) return fail(KCB_INVALID_POINTER, std::string(what) + ": pointer is not inside any allocation");
        --it;
        const uintptr_t off = key - it->first;
        if (off >= it->second) return fail(KCB_INVALID_POINTER, std::string(what) + ": pointer is not inside any allocation");
        if (bytes > it->second - off) {
            char buf[160];
            std::snprintf(buf, sizeof buf, "%s: range of %zu bytes at offset %zu exceeds an allocation of %zu bytes", what, bytes,
                          static_cast<size_t>(off), it->second);
            return fail(KCB_INVALID_POINTER, buf);
        }
        return KCB_SUCCESS;
    }
    kc::Error checkDeviceRange(const void* p, size_t bytes, const char* what) const noexcept override {
        return static_cast<kc::Error>(check(p, bytes, what));
    }
};

void release_everything(Device& d) {
    if (!d.started) return;
    cudaSetDevice(d.dflt.device);
    cudaDeviceSynchronize();
    cudaGetLastError();
    for (auto& [base, bytes] : d.allocs) cudaFree(reinterpret_cast<void*>(base));
    d.allocs.clear();
    for (kcGraph_st* g : d.graphs) {
        if (g->exec) cudaGraphExecDestroy(g->exec);
        if (g->g) cudaGraphDestroy(g->g);
        delete g;
    }
    d.graphs.clear();
    for (kcEvent_st* e : d.events) {
        cudaEventDestroy(e->e);
        delete e;
    }
    d.events.clear();
    for (kcStream_st* s : d.streams) {
        cudaStreamDestroy(s->s);
        delete s;
    }
    d.streams.clear();
    d.capturing = 0;
    d.dflt.capturing = false;
    d.poisoned = false;
    d.injected = cudaSuccess;
    d.fault = kc::FaultInfo{};
}

#define KCB_LOCK std::lock_guard<std::recursive_mutex> lock_(rt().m); tl_detail.clear()

}  // namespace

extern "C" {

int kcb_init(void) {
    KCB_LOCK;
    Runtime& r = rt();
    if (r.initialized) return KCB_SUCCESS;
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n < 1) {
        cudaGetLastError();
        return fail(KCB_INVALID_DEVICE, "no CUDA device is visible (this library has no CPU fallback)");
    }
    r.ndev = n;
    r.dev.clear();
    for (int i = 0; i < n; ++i) r.dev.push_back(std::make_unique<Device>());
    r.initialized = true;
    return KCB_SUCCESS;
}

int kcb_shutdown(void) {
    KCB_LOCK;
    Runtime& r = rt();
    if (!r.initialized) return KCB_SUCCESS;
    for (auto& d : r.dev) {
        release_everything(*d);
        if (d->started) {
            cudaStreamDestroy(d->dflt.s);
            d->started = false;
        }
    }
    r.user.clear();
    r.initialized = false;
    return KCB_SUCCESS;
}

int kcb_device_reset(void) {
    KCB_LOCK;
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    release_everything(*d);
    return KCB_SUCCESS;
}

int kcb_get_device_count(int* count) {
    KCB_LOCK;
    if (!count) return fail(KCB_INVALID_VALUE, "count is null");
    if (!rt().initialized) return fail(KCB_NOT_INITIALIZED, "kcInit has not been called");
    *count = rt().ndev;
    return KCB_SUCCESS;
}

int kcb_set_device(int device) {
    KCB_LOCK;
    if (!rt().initialized) return fail(KCB_NOT_INITIALIZED, "kcInit has not been called");
    if (device < 0 || device >= rt().ndev) return fail(KCB_INVALID_DEVICE, "device index out of range");
    tl_device = device;
    return KCB_SUCCESS;
}

int kcb_get_device(int* device) {
    KCB_LOCK;
    if (!device) return fail(KCB_INVALID_VALUE, "device is null");
    if (!rt().initialized) return fail(KCB_NOT_INITIALIZED, "kcInit has not been called");
    *device = tl_device;
    return KCB_SUCCESS;
}

int kcb_get_device_properties(char* name128, unsigned* sm_count, size_t* total_memory, int device) {
    KCB_LOCK;
    if (!rt().initialized) return fail(KCB_NOT_INITIALIZED, "kcInit has not been called");
    if (device < 0 || device >= rt().ndev) return fail(KCB_INVALID_DEVICE, "device index out of range");
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return fail(KCB_INTERNAL_ERROR, "cudaGetDeviceProperties failed");
    if (name128) std::snprintf(name128, 128, "%s", p.name);
    if (sm_count) *sm_count = static_cast<unsigned>(p.multiProcessorCount);
    if (total_memory) *total_memory = p.totalGlobalMem;
    return KCB_SUCCESS;
}

int kcb_device_synchronize(void) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    if (d->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "device synchronisation while a stream is capturing");
    const cudaError_t e = cudaDeviceSynchronize();
    return after_device_work(*d, "cudaDeviceSynchronize", e);
}

int kcb_malloc(void** ptr, size_t bytes) {
    KCB_LOCK;
    if (!ptr) return fail(KCB_INVALID_VALUE, "ptr is null");
    *ptr = nullptr;
    if (bytes == 0) return fail(KCB_INVALID_VALUE, "zero-byte allocation");
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    if (d->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "allocation while a stream is capturing");
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(KCB_OUT_OF_MEMORY, cuda_text("cudaMalloc", e));
    }
    d->allocs.emplace(reinterpret_cast<uintptr_t>(p), bytes);
    *ptr = p;
    return KCB_SUCCESS;
}

int kcb_free(void* ptr) {
    KCB_LOCK;
    if (!ptr) return KCB_SUCCESS;
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    if (d->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "free while a stream is capturing");
    auto it = d->allocs.find(reinterpret_cast<uintptr_t>(ptr));
    if (it == d->allocs.end()) {
        Checker c(*d);
        if (c.check(ptr, 1, "kcFree") == KCB_SUCCESS) return fail(KCB_INVALID_POINTER, "pointer is interior to an allocation; free takes base pointers");
        return fail(KCB_INVALID_POINTER, "pointer is not a live allocation (unknown or already freed)");
    }
    cudaDeviceSynchronize();  // drain every stream of the device first
    cudaGetLastError();
    cudaFree(ptr);
    d->allocs.erase(it);
    return KCB_SUCCESS;
}

int kcb_memcpy(void* dst, const void* src, size_t bytes, int kind) {
    KCB_LOCK;
    if (kind < 0 || kind > 3) return fail(KCB_INVALID_VALUE, "bad copy kind");
    if (bytes == 0) return KCB_SUCCESS;
    if (!dst || !src) return fail(KCB_INVALID_VALUE, "null pointer");
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    if (d->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "copy while a stream is capturing");
    Checker c(*d);
    if (kind == 0 || kind == 2)
        if (const int e = c.check(dst, bytes, "dst"); e != KCB_SUCCESS) return e;
    if (kind == 1 || kind == 2)
        if (const int e = c.check(src, bytes, "src"); e != KCB_SUCCESS) return e;
    if (kind == 3) {
        std::memmove(dst, src, bytes);
        return KCB_SUCCESS;
    }
    static const cudaMemcpyKind kinds[3] = {cudaMemcpyHostToDevice, cudaMemcpyDeviceToHost, cudaMemcpyDeviceToDevice};
    cudaError_t e = cudaDeviceSynchronize();  // ordered after everything queued on the device
    if (e == cudaSuccess) e = cudaMemcpy(dst, src, bytes, kinds[kind]);
    return after_device_work(*d, "cudaMemcpy", e);
}

int kcb_memset(void* dst, int value, size_t bytes) {
    KCB_LOCK;
    if (bytes == 0) return KCB_SUCCESS;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    if (d->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "memset while a stream is capturing");
    Checker c(*d);
    if (const int e = c.check(dst, bytes, "dst"); e != KCB_SUCCESS) return e;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemset(dst, value, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return after_device_work(*d, "cudaMemset", e);
}

int kcb_check_range(const void* ptr, size_t bytes) {
    KCB_LOCK;
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    return Checker(*d).check(ptr, bytes, "range");
}

// ---- launches -----------------------------------------------------------------------------------
int kcb_launch_kernel(const char* name, const void* typed_args, void* stream_handle) {
    KCB_LOCK;
    if (!name || !typed_args) return fail(KCB_INVALID_VALUE, "null kernel name or arguments");
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    kcStream_st* st;
    if (const int e = resolve(*d, static_cast<kcStream_t>(stream_handle), st); e != KCB_SUCCESS) return e;
    Checker c(*d);
    int status;
    if (const KernelDesc* k = find_kernel(name)) {
        status = k->launch(typed_args, c, st->s);
        if (status != KCB_SUCCESS && tl_detail.empty()) tl_detail = std::string(name) + ": arguments rejected";
    } else {
        auto it = rt().user.find(name);
        if (it == rt().user.end()) return fail(KCB_KERNEL_NOT_FOUND, std::string("no kernel named '") + name + "'");
        if (!it->second->cuda_launch)
            return fail(KCB_UNSUPPORTED_OPERATION, std::string(name) + ": registered without a cuda_launch entry (kernel images are not executed)");
        status = static_cast<int>(it->second->cuda_launch(typed_args, c, st->s));
    }
    if (status != KCB_SUCCESS) return status;
    if (st->capturing || !st->is_default) return KCB_SUCCESS;
    const cudaError_t e = cudaStreamSynchronize(st->s);  // null stream: synchronous, returns the kernel's result
    return after_device_work(*d, name, e);
}

int kcb_register_kernel(const void* entry) {
    KCB_LOCK;
    if (!rt().initialized) return fail(KCB_NOT_INITIALIZED, "kcInit has not been called");
    const auto* e = static_cast<const kc::KernelEntry*>(entry);
    if (!e || !e->name || !*e->name) return fail(KCB_INVALID_VALUE, "entry needs a name");
    if (!e->marshal && !e->cuda_launch) return fail(KCB_INVALID_VALUE, "entry needs a marshal or cuda_launch function");
    if (find_kernel(e->name) || rt().user.count(e->name)) return fail(KCB_INVALID_VALUE, std::string("kernel '") + e->name + "' is already registered");
    rt().user[e->name] = e;
    return KCB_SUCCESS;
}

// ---- streams ---------------------------------------------------------------------------------------
int kcb_stream_create(void** out) {
    KCB_LOCK;
    if (!out) return fail(KCB_INVALID_VALUE, "stream is null");
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    auto* s = new kcStream_st;
    s->device = tl_device;
    const cudaError_t e = cudaStreamCreateWithFlags(&s->s, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete s;
        return fail(KCB_INTERNAL_ERROR, cuda_text("cudaStreamCreate", e));
    }
    d->streams.insert(s);
    *out = s;
    return KCB_SUCCESS;
}

int kcb_stream_destroy(void* h) {
    KCB_LOCK;
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    auto* s = static_cast<kcStream_st*>(h);
    if (!s || !d->streams.count(s)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown stream handle");
    if (s->capturing) {
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(s->s, &g);
        if (g) cudaGraphDestroy(g);
        --d->capturing;
    }
    cudaStreamSynchronize(s->s);
    cudaStreamDestroy(s->s);
    cudaGetLastError();
    d->streams.erase(s);
    delete s;
    return KCB_SUCCESS;
}

int kcb_stream_synchronize(void* h) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(h), s); e != KCB_SUCCESS) return e;
    if (s->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "synchronising a capturing stream");
    const cudaError_t e = cudaStreamSynchronize(s->s);
    return after_device_work(*d, "cudaStreamSynchronize", e);
}

int kcb_stream_query(void* h) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(h), s); e != KCB_SUCCESS) return e;
    if (s->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "querying a capturing stream");
    const cudaError_t e = cudaStreamQuery(s->s);
    if (e == cudaSuccess) return KCB_SUCCESS;
    if (e == cudaErrorNotReady) {
        cudaGetLastError();
        return KCB_NOT_READY;
    }
    return fault(*d, "cudaStreamQuery", e);
}

int kcb_launch_host_func(void* h, void (*fn)(void*), void* user) {
    KCB_LOCK;
    if (!fn) return fail(KCB_INVALID_VALUE, "fn is null");
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(h), s); e != KCB_SUCCESS) return e;
    if (s->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "host function on a capturing stream");
    const cudaError_t e = cudaLaunchHostFunc(s->s, fn, user);
    if (e != cudaSuccess) return fail(KCB_LAUNCH_FAILURE, cuda_text("cudaLaunchHostFunc", e));
    if (s->is_default) cudaStreamSynchronize(s->s);
    return KCB_SUCCESS;
}

// ---- events ----------------------------------------------------------------------------------------
int kcb_event_create(void** out) {
    KCB_LOCK;
    if (!out) return fail(KCB_INVALID_VALUE, "event is null");
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    auto* ev = new kcEvent_st;
    ev->device = tl_device;
    if (cudaEventCreate(&ev->e) != cudaSuccess) {
        delete ev;
        return fail(KCB_INTERNAL_ERROR, "cudaEventCreate failed");
    }
    d->events.insert(ev);
    *out = ev;
    return KCB_SUCCESS;
}
int kcb_event_destroy(void* h) {
    KCB_LOCK;
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    auto* ev = static_cast<kcEvent_st*>(h);
    if (!ev || !d->events.count(ev)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown event handle");
    cudaEventDestroy(ev->e);  // CUDA keeps a recorded event alive until it completes
    d->events.erase(ev);
    delete ev;
    return KCB_SUCCESS;
}
int kcb_event_record(void* h, void* stream) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    auto* ev = static_cast<kcEvent_st*>(h);
    if (!ev || !d->events.count(ev)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown event handle");
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(stream), s); e != KCB_SUCCESS) return e;
    if (s->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "event record on a capturing stream");
    const cudaError_t e = cudaEventRecord(ev->e, s->s);
    return e == cudaSuccess ? KCB_SUCCESS : fail(KCB_INTERNAL_ERROR, cuda_text("cudaEventRecord", e));
}
int kcb_event_synchronize(void* h) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    auto* ev = static_cast<kcEvent_st*>(h);
    if (!ev || !d->events.count(ev)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown event handle");
    const cudaError_t e = cudaEventSynchronize(ev->e);
    return after_device_work(*d, "cudaEventSynchronize", e);
}
int kcb_event_query(void* h) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    auto* ev = static_cast<kcEvent_st*>(h);
    if (!ev || !d->events.count(ev)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown event handle");
    const cudaError_t e = cudaEventQuery(ev->e);
    if (e == cudaSuccess) return KCB_SUCCESS;
    if (e == cudaErrorNotReady) {
        cudaGetLastError();
        return KCB_NOT_READY;
    }
    return fault(*d, "cudaEventQuery", e);
}
int kcb_event_elapsed_ms(void* start, void* stop, float* ms) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    auto *a = static_cast<kcEvent_st*>(start), *b = static_cast<kcEvent_st*>(stop);
    if (!ms || !a || !b || !d->events.count(a) || !d->events.count(b)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown event handle");
    const cudaError_t e = cudaEventElapsedTime(ms, a->e, b->e);
    if (e == cudaErrorNotReady) {
        cudaGetLastError();
        return KCB_NOT_READY;
    }
    return e == cudaSuccess ? KCB_SUCCESS : fail(KCB_INVALID_VALUE, cuda_text("cudaEventElapsedTime", e));
}
int kcb_stream_wait_event(void* stream, void* h) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    auto* ev = static_cast<kcEvent_st*>(h);
    if (!ev || !d->events.count(ev)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown event handle");
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(stream), s); e != KCB_SUCCESS) return e;
    const cudaError_t e = cudaStreamWaitEvent(s->s, ev->e, 0);
    return e == cudaSuccess ? KCB_SUCCESS : fail(KCB_INTERNAL_ERROR, cuda_text("cudaStreamWaitEvent", e));
}

// ---- graphs ----------------------------------------------------------------------------------------
int kcb_stream_begin_capture(void* h) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(h), s); e != KCB_SUCCESS) return e;
    if (s->capturing) return fail(KCB_INVALID_VALUE, "stream is already capturing");
    const cudaError_t e = cudaStreamBeginCapture(s->s, cudaStreamCaptureModeRelaxed);
    if (e != cudaSuccess) return fail(KCB_INTERNAL_ERROR, cuda_text("cudaStreamBeginCapture", e));
    s->capturing = true;
    ++d->capturing;
    return KCB_SUCCESS;
}
int kcb_stream_end_capture(void* h, void** graph) {
    KCB_LOCK;
    if (!graph) return fail(KCB_INVALID_VALUE, "graph is null");
    *graph = nullptr;
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(h), s); e != KCB_SUCCESS) return e;
    if (!s->capturing) return fail(KCB_INVALID_VALUE, "stream is not capturing");
    cudaGraph_t g = nullptr;
    const cudaError_t e = cudaStreamEndCapture(s->s, &g);
    s->capturing = false;
    --d->capturing;
    if (e != cudaSuccess || !g) {
        cudaGetLastError();
        return fail(KCB_INTERNAL_ERROR, cuda_text("cudaStreamEndCapture", e));
    }
    auto* out = new kcGraph_st;
    out->g = g;
    out->device = tl_device;
    d->graphs.insert(out);
    *graph = out;
    return KCB_SUCCESS;
}
int kcb_graph_launch(void* gh, void* stream) {
    KCB_LOCK;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    auto* g = static_cast<kcGraph_st*>(gh);
    if (!g || !d->graphs.count(g)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown graph handle");
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(stream), s); e != KCB_SUCCESS) return e;
    if (s->capturing) return fail(KCB_UNSUPPORTED_OPERATION, "graph launch on a capturing stream");
    if (!g->exec) {
        const cudaError_t e = cudaGraphInstantiate(&g->exec, g->g, 0);
        if (e != cudaSuccess) return fail(KCB_LAUNCH_FAILURE, cuda_text("cudaGraphInstantiate", e));
    }
    cudaError_t e = cudaGraphLaunch(g->exec, s->s);
    if (e != cudaSuccess) return fail(KCB_LAUNCH_FAILURE, cuda_text("cudaGraphLaunch", e));
    if (!s->is_default) return KCB_SUCCESS;
    e = cudaStreamSynchronize(s->s);
    return after_device_work(*d, "graph", e);
}
int kcb_graph_destroy(void* gh) {
    KCB_LOCK;
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    auto* g = static_cast<kcGraph_st*>(gh);
    if (!g || !d->graphs.count(g)) return fail(KCB_INVALID_RESOURCE_HANDLE, "unknown graph handle");
    if (g->exec) cudaGraphExecDestroy(g->exec);  // a launched exec graph stays alive in CUDA until it completes
    cudaGraphDestroy(g->g);
    d->graphs.erase(g);
    delete g;
    return KCB_SUCCESS;
}
int kcb_stream_concurrent(void* h, int begin) {
    KCB_LOCK;
    (void)begin;
    Device* d;
    if (const int e = usable(d); e != KCB_SUCCESS) return e;
    kcStream_st* s;
    if (const int e = resolve(*d, static_cast<kcStream_t>(h), s); e != KCB_SUCCESS) return e;
    if (!s->capturing) return fail(KCB_INVALID_VALUE, "concurrent sections only exist inside a capture");
    return KCB_SUCCESS;  // launches stay ordered; a valid (conservative) schedule of independent launches
}

int kcb_test_inject_device_error(int cuda_error) {
    KCB_LOCK;
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    if (cuda_error < 0) return fail(KCB_INVALID_VALUE, "not a CUDA error code");
    d->injected = static_cast<cudaError_t>(cuda_error);
    return KCB_SUCCESS;
}

int kcb_get_last_fault(void* info) {
    KCB_LOCK;
    if (!info) return fail(KCB_INVALID_VALUE, "info is null");
    Device* d;
    if (const int e = device_ready(d); e != KCB_SUCCESS) return e;
    *static_cast<kc::FaultInfo*>(info) = d->fault;
    return KCB_SUCCESS;
}
const char* kcb_last_error_detail(void) { return tl_detail.c_str(); }
void* kcb_stream_native(void* h) {  // the cudaStream_t behind a handle (NULL handle: the device's default stream)
    KCB_LOCK;
    Device* d;
    if (device_ready(d) != KCB_SUCCESS) return nullptr;
    kcStream_st* s;
    if (resolve(*d, static_cast<kcStream_t>(h), s) != KCB_SUCCESS) return nullptr;
    return s->s;
}

}  // extern "C"

// ---- the reference's C++ entry points ---------------------------------------------------------------
#define E(x) static_cast<kc::Error>(x)
kc::Error kcInit() noexcept { return E(kcb_init()); }
kc::Error kcShutdown() noexcept { return E(kcb_shutdown()); }
kc::Error kcDeviceReset() noexcept { return E(kcb_device_reset()); }
kc::Error kcGetDeviceCount(int* c) noexcept { return E(kcb_get_device_count(c)); }
kc::Error kcGetDeviceProperties(kc::DeviceProperties* p, int device) noexcept {
    if (!p) return kc::Error::InvalidValue;
    *p = kc::DeviceProperties{};
    unsigned sms = 0;
    const int e = kcb_get_device_properties(p->name, &sms, &p->total_memory, device);
    p->worker_count = p->performance_workers = sms;
    p->is_hardware_gpu = true;
    return E(e);
}
kc::Error kcSetDevice(int d) noexcept { return E(kcb_set_device(d)); }
kc::Error kcGetDevice(int* d) noexcept { return E(kcb_get_device(d)); }
kc::Error kcDeviceSynchronize() noexcept { return E(kcb_device_synchronize()); }
kc::Error kcMalloc(void** p, size_t n) noexcept { return E(kcb_malloc(p, n)); }
kc::Error kcFree(void* p) noexcept { return E(kcb_free(p)); }
kc::Error kcMemcpy(void* d, const void* s, size_t n, kc::CopyKind k) noexcept { return E(kcb_memcpy(d, s, n, static_cast<int>(k))); }
kc::Error kcMemset(void* d, int v, size_t n) noexcept { return E(kcb_memset(d, v, n)); }
kc::Error kcRegisterKernel(const kc::KernelEntry* e) noexcept { return E(kcb_register_kernel(e)); }
kc::Error kcLaunchKernel(const char* name, const void* a, kcStream_t s) noexcept { return E(kcb_launch_kernel(name, a, s)); }
kc::Error kcLaunchKernelChunked(const char* name, const void* a, unsigned workers, int64_t, kcStream_t s) noexcept {
    if (workers == 0 || workers > 1024) {
        tl_detail = "workers must be in [1, 1024]";
        return kc::Error::InvalidValue;
    }
    return E(kcb_launch_kernel(name, a, s));
}
kc::Error kcStreamCreate(kcStream_t* s) noexcept { return E(kcb_stream_create(reinterpret_cast<void**>(s))); }
kc::Error kcStreamDestroy(kcStream_t s) noexcept { return E(kcb_stream_destroy(s)); }
kc::Error kcStreamSynchronize(kcStream_t s) noexcept { return E(kcb_stream_synchronize(s)); }
kc::Error kcStreamQuery(kcStream_t s) noexcept { return E(kcb_stream_query(s)); }
kc::Error kcLaunchHostFunc(kcStream_t s, void (*fn)(void*), void* u) noexcept { return E(kcb_launch_host_func(s, fn, u)); }
kc::Error kcEventCreate(kcEvent_t* e) noexcept { return E(kcb_event_create(reinterpret_cast<void**>(e))); }
kc::Error kcEventDestroy(kcEvent_t e) noexcept { return E(kcb_event_destroy(e)); }
kc::Error kcEventRecord(kcEvent_t e, kcStream_t s) noexcept { return E(kcb_event_record(e, s)); }
kc::Error kcEventSynchronize(kcEvent_t e) noexcept { return E(kcb_event_synchronize(e)); }
kc::Error kcEventQuery(kcEvent_t e) noexcept { return E(kcb_event_query(e)); }
kc::Error kcStreamWaitEvent(kcStream_t s, kcEvent_t e) noexcept { return E(kcb_stream_wait_event(s, e)); }
kc::Error kcStreamBeginCapture(kcStream_t s) noexcept { return E(kcb_stream_begin_capture(s)); }
kc::Error kcStreamEndCapture(kcStream_t s, kcGraph_t* g) noexcept { return E(kcb_stream_end_capture(s, reinterpret_cast<void**>(g))); }
kc::Error kcGraphLaunch(kcGraph_t g, kcStream_t s) noexcept { return E(kcb_graph_launch(g, s)); }
kc::Error kcStreamConcurrentBegin(kcStream_t s) noexcept { return E(kcb_stream_concurrent(s, 1)); }
kc::Error kcStreamConcurrentEnd(kcStream_t s) noexcept { return E(kcb_stream_concurrent(s, 0)); }
kc::Error kcGraphDestroy(kcGraph_t g) noexcept { return E(kcb_graph_destroy(g)); }
kc::Error kcSetKernelCodegen(kc::Codegen c) noexcept {
    if (static_cast<int>(c) < 0 || static_cast<int>(c) > 3) return kc::Error::InvalidValue;
    rt().codegen = c;
    return kc::Error::Success;
}
kc::Error kcGetKernelCodegen(kc::Codegen* c) noexcept {
    if (!c) return kc::Error::InvalidValue;
    *c = rt().codegen;
    return kc::Error::Success;
}
kc::Error kcGetKernelCodegenFor(const char* name, kc::Codegen* used) noexcept {
    if (!name || !used) return kc::Error::InvalidValue;
    if (!find_kernel(name) && !rt().user.count(name)) return kc::Error::KernelNotFound;
    *used = kc::Codegen::Native;  // one compiled CUDA path per kernel
    return kc::Error::Success;
}
const char* kcCodegenName(kc::Codegen c) noexcept {
    switch (c) {
    case kc::Codegen::Auto: return "auto";
    case kc::Codegen::Booth: return "booth";
    case kc::Codegen::Native: return "native";
    case kc::Codegen::Simd: return "simd";
    }
    return "?";
}
kc::Error kcGetLastFault(kc::FaultInfo* i) noexcept { return E(kcb_get_last_fault(i)); }
const char* kcGetErrorString(kc::Error e) noexcept { return kcb_error_string(static_cast<int>(e)); }
const char* kcGetLastErrorDetail() noexcept { return kcb_last_error_detail(); }
#undef E
