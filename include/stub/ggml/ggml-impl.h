/* Stand-in for ggml-impl.h: logging / assertion macros, the fusion query and inline bodies of the helpers declared in
 * this directory's ggml.h.  See ggml.h for what this stand-in is and is not. */
#ifndef KCB_STUB_GGML_IMPL_H
#define KCB_STUB_GGML_IMPL_H

#include "ggml-backend-impl.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define GGML_LOG_ERROR(...) fprintf(stderr, __VA_ARGS__)
#define GGML_LOG_INFO(...) ((void)0)
#define GGML_ASSERT(x)                                                          \
    do {                                                                        \
        if (!(x)) {                                                             \
            fprintf(stderr, "GGML_ASSERT(%s) failed at %s:%d\n", #x, __FILE__, __LINE__); \
            abort();                                                            \
        }                                                                       \
    } while (0)
#define GGML_ABORT(...)               \
    do {                              \
        fprintf(stderr, __VA_ARGS__); \
        abort();                      \
    } while (0)

#ifdef __cplusplus
extern "C" {
#endif

static inline size_t kcb_stub_type_size(enum ggml_type t, int64_t* block) {
    *block = 1;
    switch (t) {
    case GGML_TYPE_F32: case GGML_TYPE_I32: return 4;
    case GGML_TYPE_F16: return 2;
    case GGML_TYPE_I64: return 8;
    case GGML_TYPE_Q4_K: *block = 256; return 144;
    case GGML_TYPE_Q6_K: *block = 256; return 210;
    }
    return 0;
}
inline int64_t ggml_nelements(const struct ggml_tensor* t) { return t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3]; }
inline int64_t ggml_nrows(const struct ggml_tensor* t) { return t->ne[1] * t->ne[2] * t->ne[3]; }
inline bool ggml_is_empty(const struct ggml_tensor* t) { return ggml_nelements(t) == 0; }
inline size_t ggml_nbytes(const struct ggml_tensor* t) {
    int64_t blk;
    const size_t ts = kcb_stub_type_size(t->type, &blk);
    if (ggml_is_empty(t)) return 0;
    size_t n = (size_t)(t->ne[0] / blk) * ts;  /* last byte of the last element, strides respected */
    for (int i = 1; i < GGML_MAX_DIMS; ++i) n += (size_t)(t->ne[i] - 1) * t->nb[i];
    return n;
}
inline bool ggml_is_contiguous(const struct ggml_tensor* t) {
    int64_t blk;
    const size_t ts = kcb_stub_type_size(t->type, &blk);
    size_t expect = ts;
    if (t->ne[0] != blk && t->nb[0] != ts) return false;
    expect = (size_t)(t->ne[0] / blk) * ts;
    for (int i = 1; i < GGML_MAX_DIMS; ++i) {
        if (t->ne[i] != 1 && t->nb[i] != expect) return false;
        expect *= (size_t)t->ne[i];
    }
    return true;
}
inline bool ggml_are_same_shape(const struct ggml_tensor* a, const struct ggml_tensor* b) {
    return a->ne[0] == b->ne[0] && a->ne[1] == b->ne[1] && a->ne[2] == b->ne[2] && a->ne[3] == b->ne[3];
}
inline const char* ggml_op_desc(const struct ggml_tensor* t) {
    static const char* names[GGML_OP_COUNT] = {"NONE", "ADD", "MUL", "RMS_NORM", "MUL_MAT", "RESHAPE", "VIEW", "PERMUTE", "TRANSPOSE",
                                               "ROPE", "SET_ROWS", "FLASH_ATTN_EXT", "GLU", "SOFT_MAX"};
    return (int)t->op >= 0 && t->op < GGML_OP_COUNT ? names[t->op] : "?";
}
inline const char* ggml_type_name(enum ggml_type t) {
    switch (t) {
    case GGML_TYPE_F32: return "f32";
    case GGML_TYPE_F16: return "f16";
    case GGML_TYPE_Q4_K: return "q4_K";
    case GGML_TYPE_Q6_K: return "q6_K";
    case GGML_TYPE_I32: return "i32";
    case GGML_TYPE_I64: return "i64";
    }
    return "?";
}
inline enum ggml_glu_op ggml_get_glu_op(const struct ggml_tensor* t) { return (enum ggml_glu_op)t->op_params[0]; }
inline int32_t ggml_get_op_params_i32(const struct ggml_tensor* t, uint32_t i) { return t->op_params[i]; }
inline bool ggml_guid_matches(ggml_guid_t a, ggml_guid_t b) { return memcmp(a, b, sizeof(ggml_guid)) == 0; }

inline ggml_backend_buffer_type_t ggml_backend_buffer_get_type(ggml_backend_buffer_t buffer) { return buffer->buft; }
inline enum ggml_backend_buffer_usage ggml_backend_buffer_get_usage(ggml_backend_buffer_t buffer) { return buffer->usage; }
inline ggml_backend_buffer_t ggml_backend_buffer_init(ggml_backend_buffer_type_t buft, struct ggml_backend_buffer_i iface, void* context,
                                                      size_t size) {
    ggml_backend_buffer_t b = (ggml_backend_buffer_t)calloc(1, sizeof(struct ggml_backend_buffer));
    b->iface = iface;
    b->buft = buft;
    b->context = context;
    b->size = size;
    b->usage = GGML_BACKEND_BUFFER_USAGE_ANY;
    return b;
}

/* Whether nodes [node_idx, node_idx + num_ops) form a chain of exactly these operators in which every intermediate
 * result feeds only the next node of the chain (so a backend may compute the chain as one step). */
static inline bool ggml_can_fuse(const struct ggml_cgraph* g, int node_idx, const enum ggml_op* ops, int num_ops) {
    if (node_idx + num_ops > g->n_nodes) return false;
    for (int i = 0; i < num_ops; ++i) {
        const struct ggml_tensor* n = g->nodes[node_idx + i];
        if (n->op != ops[i]) return false;
        if (i + 1 == num_ops) break;
        if (n->flags & GGML_TENSOR_FLAG_OUTPUT) return false;
        const struct ggml_tensor* next = g->nodes[node_idx + i + 1];
        if (next->src[0] != n && next->src[1] != n) return false;
        for (int j = 0; j < g->n_nodes; ++j) { /* no other reader of the intermediate */
            if (j == node_idx + i + 1) continue;
            for (int s = 0; s < GGML_MAX_SRC; ++s)
                if (g->nodes[j]->src[s] == n) return false;
        }
    }
    return true;
}

#ifdef __cplusplus
}
#endif
#endif
