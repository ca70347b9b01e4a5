/* Stand-in for ggml-backend.h: opaque handle types and the few public calls the Kernelcore backend uses.
 * See ggml.h in this directory for what this stand-in is and is not. */
#ifndef KCB_STUB_GGML_BACKEND_H
#define KCB_STUB_GGML_BACKEND_H

#include "ggml.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ggml_backend_buffer_type* ggml_backend_buffer_type_t;
typedef struct ggml_backend_buffer* ggml_backend_buffer_t;
typedef struct ggml_backend* ggml_backend_t;
typedef struct ggml_backend_device* ggml_backend_dev_t;
typedef struct ggml_backend_reg* ggml_backend_reg_t;

enum ggml_backend_buffer_usage { GGML_BACKEND_BUFFER_USAGE_ANY = 0, GGML_BACKEND_BUFFER_USAGE_WEIGHTS = 1, GGML_BACKEND_BUFFER_USAGE_COMPUTE = 2 };
enum ggml_backend_dev_type { GGML_BACKEND_DEVICE_TYPE_CPU = 0, GGML_BACKEND_DEVICE_TYPE_GPU, GGML_BACKEND_DEVICE_TYPE_IGPU, GGML_BACKEND_DEVICE_TYPE_ACCEL };

struct ggml_backend_dev_caps {
    bool async, host_buffer, buffer_from_host_ptr, events, mmap_support;
};
struct ggml_backend_dev_props {
    const char* name;
    const char* description;
    size_t memory_free, memory_total;
    enum ggml_backend_dev_type type;
    struct ggml_backend_dev_caps caps;
};

ggml_backend_buffer_type_t ggml_backend_buffer_get_type(ggml_backend_buffer_t buffer);
enum ggml_backend_buffer_usage ggml_backend_buffer_get_usage(ggml_backend_buffer_t buffer);

#ifdef __cplusplus
}
#endif
#endif
