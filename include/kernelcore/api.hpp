// kernelcore/api.hpp -- the Kernelcore host API, backed by CUDA on B200.
//
// Source-compatible with the reference's include/kernelcore/{api,error,types,kernel_registry,
// backend,kernels}.hpp: same function names, argument order, default arguments, handle types and
// kc::Error values, so code written against the reference compiles against this header.  What the
// calls do underneath is different: kcMalloc returns CUDA device memory of the current device, streams
// are CUDA streams, events CUDA events, a captured graph is a CUDA graph, and kcLaunchKernel runs a
// hand-written sm_100a kernel selected by name.  All functions are noexcept, C++ linkage, and callable
// from any thread.  They are thin wrappers over the C ABI in kernelcore_b200.h (kcb_*).
#pragma once

#include <bit>
#include <cstddef>
#include <cstdint>

namespace kc {

// ---- status codes: values fixed by the reference (include/kernelcore/error.hpp:8-25), append only ----
enum class Error : int {
    Success = 0,
    NotInitialized,         // call made before kcInit or after kcShutdown
    InvalidValue,           // null / negative / malformed argument
    InvalidDevice,          // no such CUDA device
    OutOfMemory,
    InvalidPointer,         // not (inside) a live kcMalloc allocation of the current device
    InvalidResourceHandle,  // unknown stream / event / graph
    UnsupportedOperation,   // refused by design (e.g. a copy while a stream is capturing)
    InvalidKernelImage,     // kept for compatibility; never produced (no kernel images are loaded)
    KernelNotFound,         // no kernel of that name
    DynamicCodeBlocked,     // kept for compatibility; never produced
    LaunchFailure,          // CUDA rejected the launch
    KernelFault,            // a CUDA error surfaced from device work (sticky)
    ContextPoisoned,        // returned after a KernelFault until kcDeviceReset
    NotReady,               // query: work still pending
    InternalError
};

// Filled after a device-side failure (kcGetLastFault).  The reference reports an x86 exception record
// here; this build stores the CUDA error number in `code` and the failing kernel's name.
struct FaultInfo {
    uint32_t code = 0;
    uint64_t fault_address = 0;
    uint32_t access_type = 0;
    uint64_t instruction = 0;
    bool     in_kernel_image = false;
    uint64_t code_offset = 0;
    char     kernel[64] = {};
};

enum class CopyKind : int { HostToDevice = 0, DeviceToHost = 1, DeviceToDevice = 2, HostToHost = 3 };

// The reference chooses between CPU code generators; here there is one code path (CUDA).  The enum and
// its setters are kept so callers compile; every value resolves to the CUDA kernels.
enum class Codegen : int { Auto = 0, Booth = 1, Native = 2, Simd = 3 };

struct DeviceProperties {
    char     name[128] = {};
    unsigned worker_count = 0;         // streaming multiprocessors
    unsigned performance_workers = 0;  // same: every SM is a "fast core"
    size_t   total_memory = 0;         // device memory in bytes
    bool     is_hardware_gpu = false;  // true
    bool     guard_pages = false;
    bool     large_pages = false;
    size_t   kernel_stack_bytes = 0;
};

// ---- kernel registration contract (reference: include/kernelcore/kernel_registry.hpp:16-104) --------
struct LaunchArgs {
    uint64_t gpr[6] = {};
    unsigned n_gpr = 0;
    uint64_t xmm[8] = {};
    unsigned n_xmm = 0;
    int64_t  nthreads = 0;
};

class LaunchContext {
public:
    virtual ~LaunchContext() = default;
    // Success iff [ptr, ptr + bytes) lies inside one live allocation of the current device.
    virtual Error checkDeviceRange(const void* ptr, size_t bytes, const char* what) const noexcept = 0;
};

using NativeKernelFn = void (*)(const LaunchArgs* args);
struct NativeKernel {
    NativeKernelFn scalar = nullptr;
    NativeKernelFn simd = nullptr;
    const char*    note = nullptr;
};

// A user-registered kernel.  The image / native fields of the reference are accepted and ignored (no
// foreign machine code is run).  `cuda_launch`, appended after the reference's fields, is what a
// registration must supply here: it validates the typed arguments and enqueues CUDA work on `stream`
// (a cudaStream_t).  A registered name without it launches as UnsupportedOperation.
struct KernelEntry {
    const char*          name = nullptr;
    const unsigned char* image = nullptr;
    size_t               image_size = 0;
    const char*          image_sha256 = nullptr;
    const char*          provenance = nullptr;
    const NativeKernel*  native = nullptr;
    Error (*marshal)(const void* typed_args, const LaunchContext& ctx, LaunchArgs* out) noexcept = nullptr;
    Error (*extent)(const void* typed_args, int64_t* total) noexcept = nullptr;
    Error (*marshal_chunk)(const void* typed_args, int64_t begin, int64_t length, LaunchArgs* out) noexcept = nullptr;
    Error (*cuda_launch)(const void* typed_args, const LaunchContext& ctx, void* stream) noexcept = nullptr;
};

class ArgPacker {  // kept for adapters written against the reference; packs in declaration order
public:
    explicit ArgPacker(LaunchArgs& out) noexcept : out_(out) { out_ = LaunchArgs{}; }
    ArgPacker& ptr(const void* p) noexcept { return put(static_cast<uint64_t>(reinterpret_cast<uintptr_t>(p))); }
    ArgPacker& i32(int32_t v) noexcept { return put(static_cast<uint64_t>(static_cast<int64_t>(v))); }
    ArgPacker& i64(int64_t v) noexcept { return put(static_cast<uint64_t>(v)); }
    ArgPacker& f32(float v) noexcept {
        if (out_.n_xmm >= 8) full_ = true;
        else out_.xmm[out_.n_xmm++] = std::bit_cast<uint32_t>(v);
        return *this;
    }
    Error finish(int64_t nthreads) noexcept {
        if (nthreads < 0) return Error::InvalidValue;
        put(static_cast<uint64_t>(nthreads));
        if (full_) return Error::UnsupportedOperation;
        out_.nthreads = nthreads;
        return Error::Success;
    }

private:
    ArgPacker& put(uint64_t v) noexcept {
        if (out_.n_gpr >= 6) full_ = true;
        else out_.gpr[out_.n_gpr++] = v;
        return *this;
    }
    LaunchArgs& out_;
    bool full_ = false;
};

// Backend seam of the reference (include/kernelcore/backend.hpp:14-23): allocate / release / copy /
// launch.  The CUDA runtime behind kc* implements exactly this contract.
class IBackend {
public:
    virtual ~IBackend() = default;
    virtual const char* name() const noexcept = 0;
    virtual Error allocate(void** ptr, size_t bytes) noexcept = 0;
    virtual Error release(void* ptr) noexcept = 0;
    virtual Error copy(void* dst, const void* src, size_t bytes, CopyKind kind) noexcept = 0;
    virtual Error launch(const KernelEntry& entry, const LaunchArgs& args) noexcept = 0;
};

}  // namespace kc

struct kcStream_st;
struct kcEvent_st;
struct kcGraph_st;
using kcStream_t = kcStream_st*;  // nullptr = the device's default stream: launches on it are synchronous
using kcEvent_t  = kcEvent_st*;
using kcGraph_t  = kcGraph_st*;

// ---- lifecycle (reference: include/kernelcore/api.hpp:15-18) ----
kc::Error kcInit() noexcept;         // idempotent; creates per-device state lazily
kc::Error kcShutdown() noexcept;     // idempotent; drains, frees every allocation, stream, event, graph
kc::Error kcDeviceReset() noexcept;  // frees everything on the current device, clears ContextPoisoned

// ---- device (api.hpp:20-25).  Unlike the reference (one device), every visible GPU is addressable. ----
kc::Error kcGetDeviceCount(int* count) noexcept;
kc::Error kcGetDeviceProperties(kc::DeviceProperties* props, int device) noexcept;
kc::Error kcSetDevice(int device) noexcept;  // per calling thread
kc::Error kcGetDevice(int* device) noexcept;
kc::Error kcDeviceSynchronize() noexcept;    // first pending error of the current device

// ---- memory (api.hpp:27-31): device memory of the current device ----
kc::Error kcMalloc(void** ptr, size_t bytes) noexcept;  // 256-byte aligned; zero bytes -> InvalidValue
kc::Error kcFree(void* ptr) noexcept;                   // exact base pointers only; drains the device first
kc::Error kcMemcpy(void* dst, const void* src, size_t bytes, kc::CopyKind kind) noexcept;  // synchronous
kc::Error kcMemset(void* dst, int value, size_t bytes) noexcept;

// ---- kernels (api.hpp:33-39) ----
kc::Error kcRegisterKernel(const kc::KernelEntry* entry) noexcept;
kc::Error kcLaunchKernel(const char* name, const void* typed_args, kcStream_t stream = nullptr) noexcept;
// The reference splits a launch over CPU workers; on the GPU a launch already fills the device, so this
// is kcLaunchKernel (workers must still be in [1, 1024]).
kc::Error kcLaunchKernelChunked(const char* name, const void* typed_args, unsigned workers, int64_t min_chunk = 4096,
                                kcStream_t stream = nullptr) noexcept;

// ---- streams and events (api.hpp:41-52) ----
kc::Error kcStreamCreate(kcStream_t* stream) noexcept;
kc::Error kcStreamDestroy(kcStream_t stream) noexcept;
kc::Error kcStreamSynchronize(kcStream_t stream) noexcept;
kc::Error kcStreamQuery(kcStream_t stream) noexcept;
kc::Error kcLaunchHostFunc(kcStream_t stream, void (*fn)(void*), void* user) noexcept;
kc::Error kcEventCreate(kcEvent_t* event) noexcept;
kc::Error kcEventDestroy(kcEvent_t event) noexcept;
kc::Error kcEventRecord(kcEvent_t event, kcStream_t stream = nullptr) noexcept;
kc::Error kcEventSynchronize(kcEvent_t event) noexcept;
kc::Error kcEventQuery(kcEvent_t event) noexcept;
kc::Error kcStreamWaitEvent(kcStream_t stream, kcEvent_t event) noexcept;  // implemented (the reference refuses it)

// ---- graphs (api.hpp:54-70): stream capture into a CUDA graph ----
kc::Error kcStreamBeginCapture(kcStream_t stream) noexcept;
kc::Error kcStreamEndCapture(kcStream_t stream, kcGraph_t* graph) noexcept;
kc::Error kcGraphLaunch(kcGraph_t graph, kcStream_t stream = nullptr) noexcept;  // nullptr: synchronous
kc::Error kcStreamConcurrentBegin(kcStream_t stream = nullptr) noexcept;  // accepted while capturing; ordering kept
kc::Error kcStreamConcurrentEnd(kcStream_t stream = nullptr) noexcept;
kc::Error kcGraphDestroy(kcGraph_t graph) noexcept;

// ---- code generation path (api.hpp:72-77): retained, single CUDA path ----
kc::Error kcSetKernelCodegen(kc::Codegen codegen) noexcept;
kc::Error kcGetKernelCodegen(kc::Codegen* codegen) noexcept;
kc::Error kcGetKernelCodegenFor(const char* name, kc::Codegen* used) noexcept;
const char* kcCodegenName(kc::Codegen codegen) noexcept;

// ---- diagnostics (api.hpp:79-85) ----
kc::Error kcGetLastFault(kc::FaultInfo* info) noexcept;
const char* kcGetErrorString(kc::Error error) noexcept;
const char* kcGetLastErrorDetail() noexcept;  // thread-local text of the most recent call on this thread

// ---- built-in kernel (reference: include/kernelcore/kernels.hpp:10-28) ----
namespace kc::kernels {
struct VectorAddArgs {
    const float* a;
    const float* b;
    float*       out;
    int          count;
};
inline Error launchVectorAdd(const float* a, const float* b, float* out, int count, kcStream_t stream = nullptr) noexcept {
    const VectorAddArgs args{a, b, out, count};
    return kcLaunchKernel("vector_add", &args, stream);
}
inline Error launchVectorAddChunked(const float* a, const float* b, float* out, int count, unsigned workers,
                                    int64_t min_chunk = 4096, kcStream_t stream = nullptr) noexcept {
    const VectorAddArgs args{a, b, out, count};
    return kcLaunchKernelChunked("vector_add", &args, workers, min_chunk, stream);
}
}  // namespace kc::kernels
