/*
 * Stand-in for llama.cpp's ggml.h, holding ONLY the names that the Kernelcore backend touches, written for this
 * project so that the backend object (kernelcore_b200/csrc/ggml_backend.cpp) compiles and is unit-tested where no
 * llama.cpp source tree is present.  Inside a llama.cpp tree the real headers take its place (GGML_INCLUDE= on the
 * make command line); nothing here is meant to be ABI-compatible with a particular ggml release beyond the member
 * names and meanings the backend relies on.
 *
 * The members are those the reference's backend reads or fills
 * (integrations/llama.cpp/ggml/src/ggml-kernelcore/ggml-kernelcore.cpp of the reference project).
 */
#ifndef KCB_STUB_GGML_H
#define KCB_STUB_GGML_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GGML_MAX_DIMS 4
#define GGML_MAX_SRC 10
#define GGML_MAX_OP_PARAMS 64
#define GGML_MAX_NAME 64
#define GGML_BACKEND_API

/* element types: the numeric values are those GGUF files store for a tensor's type */
enum ggml_type {
    GGML_TYPE_F32 = 0,
    GGML_TYPE_F16 = 1,
    GGML_TYPE_Q4_K = 12,
    GGML_TYPE_Q6_K = 14,
    GGML_TYPE_I32 = 26,
    GGML_TYPE_I64 = 27,
};

/* graph operators the backend distinguishes; anything else is "some other operator" */
enum ggml_op {
    GGML_OP_NONE = 0,
    GGML_OP_ADD,
    GGML_OP_MUL,
    GGML_OP_RMS_NORM,
    GGML_OP_MUL_MAT,
    GGML_OP_RESHAPE,
    GGML_OP_VIEW,
    GGML_OP_PERMUTE,
    GGML_OP_TRANSPOSE,
    GGML_OP_ROPE,
    GGML_OP_SET_ROWS,
    GGML_OP_FLASH_ATTN_EXT,
    GGML_OP_GLU,
    GGML_OP_SOFT_MAX, /* an operator the backend does not claim (for tests) */
    GGML_OP_COUNT,
};

enum ggml_glu_op { GGML_GLU_OP_REGLU = 0, GGML_GLU_OP_GEGLU, GGML_GLU_OP_SWIGLU };
enum ggml_status { GGML_STATUS_FAILED = -1, GGML_STATUS_SUCCESS = 0 };
enum ggml_tensor_flag { GGML_TENSOR_FLAG_INPUT = 1, GGML_TENSOR_FLAG_OUTPUT = 2, GGML_TENSOR_FLAG_PARAM = 4, GGML_TENSOR_FLAG_COMPUTE = 16 };
#define GGML_ROPE_TYPE_NEOX 2

struct ggml_backend_buffer;

struct ggml_tensor {
    enum ggml_type type;
    struct ggml_backend_buffer* buffer;
    int64_t ne[GGML_MAX_DIMS]; /* elements per dimension */
    size_t nb[GGML_MAX_DIMS];  /* strides in bytes */
    enum ggml_op op;
    int32_t op_params[GGML_MAX_OP_PARAMS / sizeof(int32_t)];
    int32_t flags;
    struct ggml_tensor* src[GGML_MAX_SRC];
    struct ggml_tensor* view_src;
    size_t view_offs;
    void* data;
    char name[GGML_MAX_NAME];
};

struct ggml_cgraph {
    int n_nodes;
    struct ggml_tensor** nodes;
};

typedef uint8_t ggml_guid[16];
typedef ggml_guid* ggml_guid_t;

/* helpers (defined inline in ggml-impl.h of this stand-in) */
size_t ggml_nbytes(const struct ggml_tensor* t);
int64_t ggml_nelements(const struct ggml_tensor* t);
int64_t ggml_nrows(const struct ggml_tensor* t);
bool ggml_is_contiguous(const struct ggml_tensor* t);
bool ggml_is_empty(const struct ggml_tensor* t);
bool ggml_are_same_shape(const struct ggml_tensor* a, const struct ggml_tensor* b);
const char* ggml_op_desc(const struct ggml_tensor* t);
const char* ggml_type_name(enum ggml_type t);
enum ggml_glu_op ggml_get_glu_op(const struct ggml_tensor* t);
int32_t ggml_get_op_params_i32(const struct ggml_tensor* t, uint32_t i);
bool ggml_guid_matches(ggml_guid_t a, ggml_guid_t b);

#ifdef __cplusplus
}
#endif
#endif
