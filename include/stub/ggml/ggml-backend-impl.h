/* Stand-in for ggml-backend-impl.h: the interface tables a backend fills and the objects that carry them.  The member
 * lists are those the reference's backend initialises, in its order
 * (ggml-kernelcore.cpp:213-225, 272-281, 794-811, 963-979, 998-1003 of the reference project).
 * See ggml.h in this directory for what this stand-in is and is not. */
#ifndef KCB_STUB_GGML_BACKEND_IMPL_H
#define KCB_STUB_GGML_BACKEND_IMPL_H

#include "ggml-backend.h"

#ifdef __cplusplus
extern "C" {
#endif

#define GGML_BACKEND_API_VERSION 2

struct ggml_backend_buffer_type_i {
    const char* (*get_name)(ggml_backend_buffer_type_t buft);
    ggml_backend_buffer_t (*alloc_buffer)(ggml_backend_buffer_type_t buft, size_t size);
    void* alloc_buffer_n;
    size_t (*get_alignment)(ggml_backend_buffer_type_t buft);
    size_t (*get_max_size)(ggml_backend_buffer_type_t buft);
    size_t (*get_alloc_size)(ggml_backend_buffer_type_t buft, const struct ggml_tensor* tensor);
    void* get_alloc_size_n;
    bool (*is_host)(ggml_backend_buffer_type_t buft);
};
struct ggml_backend_buffer_type {
    struct ggml_backend_buffer_type_i iface;
    ggml_backend_dev_t device;
    void* context;
};

struct ggml_backend_buffer_i {
    void (*free_buffer)(ggml_backend_buffer_t buffer);
    void* (*get_base)(ggml_backend_buffer_t buffer);
    void* init_tensor;
    void (*memset_tensor)(ggml_backend_buffer_t buffer, struct ggml_tensor* tensor, uint8_t value, size_t offset, size_t size);
    void (*set_tensor)(ggml_backend_buffer_t buffer, struct ggml_tensor* tensor, const void* data, size_t offset, size_t size);
    void (*get_tensor)(ggml_backend_buffer_t buffer, const struct ggml_tensor* tensor, void* data, size_t offset, size_t size);
    void* set_tensor_2d;
    void* get_tensor_2d;
    void* cpy_tensor;
    void (*clear)(ggml_backend_buffer_t buffer, uint8_t value);
    void* reset;
};
struct ggml_backend_buffer {
    struct ggml_backend_buffer_i iface;
    ggml_backend_buffer_type_t buft;
    void* context;
    size_t size;
    enum ggml_backend_buffer_usage usage;
};
ggml_backend_buffer_t ggml_backend_buffer_init(ggml_backend_buffer_type_t buft, struct ggml_backend_buffer_i iface, void* context, size_t size);

struct ggml_backend_i {
    const char* (*get_name)(ggml_backend_t backend);
    void (*free)(ggml_backend_t backend);
    void* set_tensor_async;
    void* get_tensor_async;
    void* set_tensor_2d_async;
    void* get_tensor_2d_async;
    void* cpy_tensor_async;
    void* synchronize;
    void* graph_plan_create;
    void* graph_plan_free;
    void* graph_plan_update;
    void* graph_plan_compute;
    enum ggml_status (*graph_compute)(ggml_backend_t backend, struct ggml_cgraph* cgraph);
    void* event_record;
    void* event_wait;
    void* graph_optimize;
};
struct ggml_backend {
    ggml_guid_t guid;
    struct ggml_backend_i iface;
    ggml_backend_dev_t device;
    void* context;
};

struct ggml_backend_device_i {
    const char* (*get_name)(ggml_backend_dev_t dev);
    const char* (*get_description)(ggml_backend_dev_t dev);
    void (*get_memory)(ggml_backend_dev_t dev, size_t* free, size_t* total);
    enum ggml_backend_dev_type (*get_type)(ggml_backend_dev_t dev);
    void (*get_props)(ggml_backend_dev_t dev, struct ggml_backend_dev_props* props);
    ggml_backend_t (*init_backend)(ggml_backend_dev_t dev, const char* params);
    ggml_backend_buffer_type_t (*get_buffer_type)(ggml_backend_dev_t dev);
    ggml_backend_buffer_type_t (*get_host_buffer_type)(ggml_backend_dev_t dev);
    void* buffer_from_host_ptr;
    bool (*supports_op)(ggml_backend_dev_t dev, const struct ggml_tensor* op);
    bool (*supports_buft)(ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft);
    void* offload_op;
    void* event_new;
    void* event_free;
    void* event_synchronize;
};
struct ggml_backend_device {
    struct ggml_backend_device_i iface;
    ggml_backend_reg_t reg;
    void* context;
};

struct ggml_backend_reg_i {
    const char* (*get_name)(ggml_backend_reg_t reg);
    size_t (*get_device_count)(ggml_backend_reg_t reg);
    ggml_backend_dev_t (*get_device)(ggml_backend_reg_t reg, size_t index);
    void* (*get_proc_address)(ggml_backend_reg_t reg, const char* name);
};
struct ggml_backend_reg {
    int api_version;
    struct ggml_backend_reg_i iface;
    void* context;
};

/* dynamic-loading entry: the real header emits ggml_backend_init / ggml_backend_score exports for loadable backends */
#define GGML_BACKEND_DL_IMPL(reg_fn)

#ifdef __cplusplus
}
#endif
#endif
