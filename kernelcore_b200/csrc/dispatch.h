// Name -> launcher table behind kcLaunchKernel.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace kcb {

// Range oracle handed to the adapters: KCB_SUCCESS iff [p, p + bytes) lies inside one live allocation
// of the current device (the role of kc::LaunchContext::checkDeviceRange in the reference).
struct RangeChecker {
    virtual ~RangeChecker() = default;
    virtual int check(const void* p, size_t bytes, const char* what) const = 0;
};

struct KernelDesc {
    const char* name;
    // Validates the typed argument struct (shapes -> InvalidValue, pointers -> InvalidPointer) and
    // enqueues the kernel on `s`.
    int (*launch)(const void* typed_args, const RangeChecker& rc, cudaStream_t s);
};

const KernelDesc* find_kernel(const char* name);
int kernel_count();
const char* kernel_name(int i);

}  // namespace kcb
