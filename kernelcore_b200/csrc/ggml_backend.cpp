// The ggml backend object: registry, device, two buffer types, op support rules and the graph walk.
//
// Stands in for integrations/llama.cpp/ggml/src/ggml-kernelcore/ggml-kernelcore.cpp:156-310 (buffers and buffer
// types), :706-811 (graph_compute and the backend table) and :818-1054 (device, support rules, registry, exports) of
// the reference, over this project's operator layer (ggml_ops.cpp, which covers :471-697).  What is kept is the
// contract llama.cpp sees: the three exported functions, the names "Kernelcore" / "Kernelcore_Host", an ACCEL device
// whose first buffer type takes the weights, which ops are claimed, the fusion patterns of the walk
// ([ADD +] RMS_NORM + MUL by a row vector, RMS_NORM + MUL, SwiGLU with quantized output, matmuls sharing a quantized
// input), a synchronous graph_compute.  What differs, because the device is a B200 and not the host's cores:
//   * both buffer types are device memory (is_host false); ggml moves data through set_tensor / get_tensor, which
//     stage K-quant weights into the device layouts (Q4_K blocks as they are, Q6_K as four planes, fp16 weights as
//     8-row interleaved words) and return canonical GGUF bytes on the way back;
//   * the device layouts are exactly as large as the GGUF tensors, so get_alloc_size is ggml_nbytes;
//   * attention runs on the device for any number of tokens (the reference hands batches above 8 tokens back to the
//     CPU backend, which can read its host-resident cache; a device-resident cache cannot be read that way), limited
//     only by the score row having to fit in shared memory.
// Compiles against llama.cpp's ggml headers, or against the stand-in under include/stub/ggml.

#include "ggml-kernelcore.h"

#include "ggml-backend-impl.h"
#include "ggml-impl.h"

#include "../../include/ggml-kernelcore-ops.h"
#include "../../include/kernelcore_b200.h"

#include <cuda_runtime.h>

#include <climits>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

namespace {

// ---- process-wide settings -----------------------------------------------------------------------------------------
struct Settings {
    bool ok = false;           // a CUDA device is there and the runtime came up
    bool disabled = false;     // GGML_KERNELCORE_DISABLE=1: claim nothing
    bool matmul_only = false;  // GGML_KERNELCORE_MATMUL_ONLY=1: only MUL_MAT
    bool attn = true;          // GGML_KERNELCORE_ATTN=0: leave the KV cache and attention to other backends
    int attn_tokens = INT_MAX; // GGML_KERNELCORE_ATTN_TOKENS: largest batch whose attention is claimed
};
bool env_is(const char* name, const char* value) {
    const char* e = std::getenv(name);
    return e && std::strcmp(e, value) == 0;
}
Settings read_settings(bool need_device) {
    Settings s;
    s.ok = !need_device || kcb_init() == 0;
    if (need_device && !s.ok) GGML_LOG_ERROR("Kernelcore: no CUDA device (%s)\n", kcb_last_error_detail());
    s.disabled = env_is("GGML_KERNELCORE_DISABLE", "1");
    s.matmul_only = env_is("GGML_KERNELCORE_MATMUL_ONLY", "1");
    s.attn = !env_is("GGML_KERNELCORE_ATTN", "0");
    if (const char* n = std::getenv("GGML_KERNELCORE_ATTN_TOKENS")) s.attn_tokens = std::max(0, std::atoi(n));
    return s;
}
const Settings& settings() {
    static const Settings s = read_settings(true);
    return s;
}

ggml_backend_buffer_type_t weight_buffer_type();
ggml_backend_buffer_type_t kv_buffer_type();

// ---- which tensors are staged -----------------------------------------------------------------------------------------
bool is_kquant(ggml_type t) { return t == GGML_TYPE_Q4_K || t == GGML_TYPE_Q6_K; }

// A matrix the matmul kernels take: K-quant super-blocks or fp16 pairs along k, rows in groups of 8 (ggml-kernelcore.cpp:103-109).
bool weight_shape_ok(const ggml_tensor* w) {
    const bool kq = is_kquant(w->type) && w->ne[0] % 256 == 0;
    const bool f16 = w->type == GGML_TYPE_F16 && w->ne[0] % 2 == 0;
    return (kq || f16) && w->ne[2] == 1 && w->ne[3] == 1 && w->ne[1] % 8 == 0 && w->ne[0] <= INT32_MAX && w->ne[1] <= INT32_MAX &&
           ggml_is_contiguous(w);
}
// fp16 tensors are re-laid only when they are weights: an fp16 input (the attention mask) stays as it is.
bool is_f16_weight(ggml_backend_buffer_t buf, const ggml_tensor* t) {
    return t->type == GGML_TYPE_F16 && weight_shape_ok(t) && buf && ggml_backend_buffer_get_usage(buf) == GGML_BACKEND_BUFFER_USAGE_WEIGHTS;
}
bool is_staged(ggml_backend_buffer_t buf, const ggml_tensor* t) { return (is_kquant(t->type) && weight_shape_ok(t)) || is_f16_weight(buf, t); }

// One operator context for uploads (its stream orders the layout conversions).
void* upload_ctx() {
    static void* ctx = [] {
        void* c = nullptr;
        return kcb_ggml_ctx_create(nullptr, &c) == 0 ? c : nullptr;
    }();
    return ctx;
}

// ---- buffers ---------------------------------------------------------------------------------------------------------
struct DeviceBuffer {
    void* base = nullptr;
    size_t size = 0;
};
void buffer_free(ggml_backend_buffer_t b) {
    auto* d = static_cast<DeviceBuffer*>(b->context);
    kcb_free(d->base);
    delete d;
}
void* buffer_base(ggml_backend_buffer_t b) { return static_cast<DeviceBuffer*>(b->context)->base; }
void buffer_memset(ggml_backend_buffer_t, ggml_tensor* t, uint8_t value, size_t offset, size_t size) {
    cudaMemset(static_cast<char*>(t->data) + offset, value, size);
}
void buffer_clear(ggml_backend_buffer_t b, uint8_t value) {
    auto* d = static_cast<DeviceBuffer*>(b->context);
    cudaMemset(d->base, value, d->size);
}
void plain_set(ggml_backend_buffer_t, ggml_tensor* t, const void* data, size_t offset, size_t size) {
    cudaMemcpy(static_cast<char*>(t->data) + offset, data, size, cudaMemcpyHostToDevice);
}
void plain_get(ggml_backend_buffer_t, const ggml_tensor* t, void* data, size_t offset, size_t size) {
    cudaMemcpy(data, static_cast<const char*>(t->data) + offset, size, cudaMemcpyDeviceToHost);
}
// Weights: GGUF bytes in, device layout stored (set_tensor, ggml-kernelcore.cpp:175-190) ...
void weight_set(ggml_backend_buffer_t b, ggml_tensor* t, const void* data, size_t offset, size_t size) {
    if (!is_staged(b, t)) return plain_set(b, t, data, offset, size);
    GGML_ASSERT(offset == 0 && size == ggml_nbytes(t) && "Kernelcore: weights are uploaded whole");
    const int e = kcb_ggml_set_weight(upload_ctx(), t->data, data, static_cast<int>(t->type), static_cast<int>(t->ne[1]), static_cast<int>(t->ne[0]));
    if (e) GGML_LOG_ERROR("Kernelcore: weight upload failed: %s\n", kcb_error_string(e));
}
// ... and canonical GGUF bytes out (get_tensor, :192-206).
void weight_get(ggml_backend_buffer_t b, const ggml_tensor* t, void* data, size_t offset, size_t size) {
    if (!is_staged(b, t) || t->type == GGML_TYPE_Q4_K) return plain_get(b, t, data, offset, size);  // Q4_K blocks are stored as they are
    const size_t bytes = ggml_nbytes(t);
    const int rows = static_cast<int>(t->ne[1]), k = static_cast<int>(t->ne[0]);
    std::vector<uint8_t> full(bytes);
    if (t->type == GGML_TYPE_Q6_K) {
        void* tmp = nullptr;
        if (cudaMalloc(&tmp, bytes) != cudaSuccess) return;
        if (kcb_q6k_from_planes(t->data, tmp, rows, k, nullptr) == 0) cudaMemcpy(full.data(), tmp, bytes, cudaMemcpyDeviceToHost);
        cudaFree(tmp);
    } else {  // fp16 words, rows in groups of 8 interleaved by 32-bit word -> row-major halves
        std::vector<uint32_t> words(bytes / 4);
        cudaMemcpy(words.data(), t->data, bytes, cudaMemcpyDeviceToHost);
        auto* out = reinterpret_cast<uint16_t*>(full.data());
        const int kw = k / 2;
        for (int r = 0; r < rows; ++r)
            for (int j = 0; j < kw; ++j) {
                const uint32_t v = words[(static_cast<size_t>(r / 8) * kw + j) * 8 + r % 8];
                out[static_cast<size_t>(r) * k + 2 * j] = static_cast<uint16_t>(v & 0xFFFFu);
                out[static_cast<size_t>(r) * k + 2 * j + 1] = static_cast<uint16_t>(v >> 16);
            }
    }
    std::memcpy(data, full.data() + offset, size);
}

ggml_backend_buffer_i make_buffer_iface(bool staged) {
    ggml_backend_buffer_i i{};
    i.free_buffer = buffer_free;
    i.get_base = buffer_base;
    i.memset_tensor = buffer_memset;
    i.set_tensor = staged ? weight_set : plain_set;
    i.get_tensor = staged ? weight_get : plain_get;
    i.clear = buffer_clear;
    return i;
}

// ---- buffer types ----------------------------------------------------------------------------------------------------
ggml_backend_buffer_t alloc_device(ggml_backend_buffer_type_t buft, size_t size, bool staged) {
    if (!settings().ok) return nullptr;
    void* p = nullptr;
    const size_t bytes = size ? size : 64;  // llama.cpp probes with empty buffers
    if (kcb_malloc(&p, bytes) != 0) {
        GGML_LOG_ERROR("Kernelcore: allocating %zu bytes failed: %s\n", bytes, kcb_last_error_detail());
        return nullptr;
    }
    return ggml_backend_buffer_init(buft, make_buffer_iface(staged), new DeviceBuffer{p, bytes}, size);
}
const char* weight_buft_name(ggml_backend_buffer_type_t) { return "Kernelcore"; }
const char* kv_buft_name(ggml_backend_buffer_type_t) { return "Kernelcore_Host"; }
ggml_backend_buffer_t weight_buft_alloc(ggml_backend_buffer_type_t t, size_t n) { return alloc_device(t, n, true); }
ggml_backend_buffer_t kv_buft_alloc(ggml_backend_buffer_type_t t, size_t n) { return alloc_device(t, n, false); }
size_t buft_alignment(ggml_backend_buffer_type_t) { return 256; }  // what the 16-byte loads and bulk copies need, with room
size_t buft_alloc_size(ggml_backend_buffer_type_t, const ggml_tensor* t) { return ggml_nbytes(t); }
bool buft_is_host(ggml_backend_buffer_type_t) { return false; }

ggml_backend_buffer_type_i make_buft_iface(bool weights) {
    ggml_backend_buffer_type_i i{};
    i.get_name = weights ? weight_buft_name : kv_buft_name;
    i.alloc_buffer = weights ? weight_buft_alloc : kv_buft_alloc;
    i.get_alignment = buft_alignment;
    i.get_alloc_size = buft_alloc_size;
    i.is_host = buft_is_host;
    return i;
}

// ---- tensors of a graph as the operator layer sees them -------------------------------------------------------------
// One kcb_tensor per ggml tensor and graph, at a stable address: the operator layer recognises "the same input" of two
// matmuls, and a fused norm's already quantized output, by that address.
struct GraphTensors {
    std::deque<kcb_tensor> store;
    std::unordered_map<const ggml_tensor*, kcb_tensor*> seen;
    // Every tensor is converted with all of its sources, however it is first reached (as an operator's result or as
    // somebody's input): a memoised entry is always complete.
    const kcb_tensor* of(const ggml_tensor* t) {
        if (!t) return nullptr;
        if (const auto it = seen.find(t); it != seen.end()) return it->second;
        store.emplace_back();
        kcb_tensor* k = &store.back();
        seen.emplace(t, k);
        k->type = static_cast<int>(t->type);
        for (int i = 0; i < 4; ++i) k->ne[i] = t->ne[i], k->nb[i] = t->nb[i];
        k->data = t->data;
        std::memcpy(k->op_params, t->op_params, sizeof k->op_params);
        for (int i = 0; i < 4; ++i) k->src[i] = of(t->src[i]);
        return k;
    }
};

struct BackendCtx {
    void* ops = nullptr;  // operator-layer context (stream, quantized-input scratch)
    ~BackendCtx() {
        if (ops) kcb_ggml_ctx_destroy(ops);
    }
};

float op_param_f32(const ggml_tensor* t, int i) {
    float v;
    std::memcpy(&v, reinterpret_cast<const int32_t*>(t->op_params) + i, sizeof v);
    return v;
}
bool is_row_vector_of(const ggml_tensor* v, const ggml_tensor* x) {
    return v->type == GGML_TYPE_F32 && ggml_is_contiguous(v) && v->ne[0] == x->ne[0] && ggml_nrows(v) == 1;
}
bool wanted(const ggml_tensor* n) { return (n->flags & GGML_TENSOR_FLAG_COMPUTE) != 0 && !ggml_is_empty(n); }

// ---- the graph walk (ggml-kernelcore.cpp:706-792) -----------------------------------------------------------------------
const char* backend_name(ggml_backend_t) { return "Kernelcore"; }
void backend_free(ggml_backend_t b) {
    delete static_cast<BackendCtx*>(b->context);
    delete b;
}

ggml_status graph_compute(ggml_backend_t backend, ggml_cgraph* g) {
    auto& ctx = *static_cast<BackendCtx*>(backend->context);
    if (kcb_ggml_ctx_begin_graph(ctx.ops) != 0) return GGML_STATUS_FAILED;
    GraphTensors tensors;
    int err = 0;
    for (int i = 0; i < g->n_nodes && !err; ++i) {
        ggml_tensor* node = g->nodes[i];
        if (!wanted(node)) continue;  // flagged off, or nothing to compute (a prompt's early ubatches select no output rows)
        switch (node->op) {
        case GGML_OP_MUL_MAT:
            // matmuls of one input (q, k, v; gate, up) find it already quantized: the operator layer keeps the list
            err = kcb_ggml_mul_mat(ctx.ops, tensors.of(node));
            break;
        case GGML_OP_ADD:
        case GGML_OP_RMS_NORM: {
            // [ADD +] RMS_NORM + MUL by a row vector (the norm weight), n % 256 == 0: one fused step that also leaves the
            // result quantized for the matmuls behind it; otherwise RMS_NORM (+ MUL) or a plain ADD
            static const ggml_op norm_mul[] = {GGML_OP_RMS_NORM, GGML_OP_MUL};
            const int ni = node->op == GGML_OP_ADD ? i + 1 : i;
            ggml_tensor* norm = ni < g->n_nodes ? g->nodes[ni] : nullptr;
            ggml_tensor* mul = ni + 1 < g->n_nodes ? g->nodes[ni + 1] : nullptr;
            const bool fused = norm && mul && norm->op == GGML_OP_RMS_NORM && ggml_can_fuse(g, ni, norm_mul, 2) && mul->src[0] == norm &&
                               is_row_vector_of(mul->src[1], norm) && norm->src[0]->ne[0] % 256 == 0 && ggml_is_contiguous(norm->src[0]) &&
                               (node->op == GGML_OP_RMS_NORM || norm->src[0] == node);
            if (fused) {
                err = kcb_ggml_fused_norm(ctx.ops, node->op == GGML_OP_ADD ? tensors.of(node) : nullptr, tensors.of(norm), tensors.of(mul));
                i = ni + 1;
            } else if (node->op == GGML_OP_ADD) {
                err = kcb_ggml_add(ctx.ops, tensors.of(node));
            } else {
                ggml_tensor* next = i + 1 < g->n_nodes ? g->nodes[i + 1] : nullptr;
                if (next && ggml_can_fuse(g, i, norm_mul, 2) && next->src[0] == node && is_row_vector_of(next->src[1], node)) {
                    err = kcb_ggml_rms_norm(ctx.ops, tensors.of(node), static_cast<const float*>(next->src[1]->data), tensors.of(next));
                    ++i;
                } else {
                    err = kcb_ggml_rms_norm(ctx.ops, tensors.of(node), nullptr, tensors.of(node));
                }
            }
            break;
        }
        case GGML_OP_MUL: err = kcb_ggml_mul(ctx.ops, tensors.of(node)); break;
        case GGML_OP_ROPE: err = kcb_ggml_rope(ctx.ops, tensors.of(node)); break;
        case GGML_OP_GLU: err = node->ne[0] % 256 == 0 ? kcb_ggml_fused_swiglu(ctx.ops, tensors.of(node)) : kcb_ggml_swiglu(ctx.ops, tensors.of(node)); break;
        case GGML_OP_SET_ROWS: err = kcb_ggml_set_rows(ctx.ops, tensors.of(node)); break;
        case GGML_OP_FLASH_ATTN_EXT: err = kcb_ggml_flash_attn(ctx.ops, tensors.of(node)); break;
        case GGML_OP_NONE:
        case GGML_OP_RESHAPE:
        case GGML_OP_VIEW:
        case GGML_OP_PERMUTE:
        case GGML_OP_TRANSPOSE: break;
        default: GGML_ABORT("%s: unsupported op %s\n", __func__, ggml_op_desc(node));
        }
        if (err) GGML_LOG_ERROR("Kernelcore: %s failed: %s\n", ggml_op_desc(node), kcb_error_string(err));
    }
    // synchronous, as the reference's backend is: results are complete when graph_compute returns
    if (kcb_ggml_ctx_sync(ctx.ops) != 0) err = err ? err : 15;
    return err ? GGML_STATUS_FAILED : GGML_STATUS_SUCCESS;
}

ggml_backend_i make_backend_iface() {
    ggml_backend_i i{};
    i.get_name = backend_name;
    i.free = backend_free;
    i.graph_compute = graph_compute;
    return i;
}
ggml_guid_t backend_guid() {
    static ggml_guid guid = {0x6b, 0x63, 0x2d, 0x62, 0x32, 0x30, 0x30, 0x2d, 0x6b, 0x71, 0x75, 0x61, 0x6e, 0x74, 0x2d, 0x31};
    return &guid;
}

// ---- op support rules (ggml-kernelcore.cpp:860-961) ---------------------------------------------------------------------
bool f32c(const ggml_tensor* t) { return t && t->type == GGML_TYPE_F32 && ggml_is_contiguous(t); }
bool in_kv_buffer(const ggml_tensor* t) {  // the tensor, or what it views, lives in a KV-cache buffer of this backend
    const ggml_backend_buffer_t b = t->view_src ? t->view_src->buffer : t->buffer;
    return b && ggml_backend_buffer_get_type(b) == kv_buffer_type();
}
bool f16_rows(const ggml_tensor* t) {  // fp16 with rows and heads at 32-bit word strides
    return t->type == GGML_TYPE_F16 && t->nb[0] == 2 && t->nb[1] % 4 == 0 && t->nb[2] % 4 == 0 && t->ne[3] == 1 && t->nb[1] / 4 <= INT32_MAX &&
           t->nb[2] / 4 <= INT32_MAX;
}
bool flash_attn_ok(const ggml_tensor* op, int max_tokens) {
    const ggml_tensor *q = op->src[0], *k = op->src[1], *v = op->src[2], *mask = op->src[3];
    if (op->src[4] || q->ne[1] > max_tokens) return false;                          // no sinks
    if (op_param_f32(op, 1) != 0.0f || op_param_f32(op, 2) != 0.0f) return false;  // no ALiBi, no softcap
    if (!in_kv_buffer(k) || !in_kv_buffer(v) || !f16_rows(k) || !f16_rows(v)) return false;
    const int64_t D = k->ne[0];
    if (v->ne[0] != D || q->ne[0] != D || D % 8 || k->ne[1] != v->ne[1] || k->ne[2] != v->ne[2] || k->ne[2] <= 0 || q->ne[2] % k->ne[2] ||
        q->ne[3] != 1 || k->ne[1] <= 0 || k->ne[1] > INT32_MAX)
        return false;
    if ((k->ne[1] + D) * 4 > 200 * 1024) return false;  // one row of scores plus a query row in shared memory
    if (q->type != GGML_TYPE_F32 || q->nb[0] != 4 || q->nb[1] % 4 || q->nb[2] % 4) return false;
    if (!f32c(op) || op->ne[0] != D || op->ne[1] != q->ne[2] || op->ne[2] != q->ne[1] || op->ne[3] != 1) return false;
    if (mask && (mask->type != GGML_TYPE_F16 || mask->nb[0] != 2 || mask->nb[1] % 4 || mask->ne[0] < k->ne[1] || mask->ne[1] < q->ne[1] ||
                 mask->ne[2] != 1 || mask->ne[3] != 1))
        return false;
    return true;
}

// The rules alone: pure host arithmetic on the tensor's fields, no device needed.
bool supports_op_rules(const Settings& rt, const ggml_tensor* op) {
    if (!rt.ok || rt.disabled) return false;
    const ggml_tensor *s0 = op->src[0], *s1 = op->src[1];
    switch (op->op) {
    case GGML_OP_NONE:
    case GGML_OP_RESHAPE:
    case GGML_OP_VIEW:
    case GGML_OP_PERMUTE:
    case GGML_OP_TRANSPOSE: return true;
    case GGML_OP_MUL_MAT:  // the weight must live in this backend's weight buffers (staged), any batch size
        return s0->buffer && ggml_backend_buffer_get_type(s0->buffer) == weight_buffer_type() && weight_shape_ok(s0) && f32c(s1) &&
               s1->ne[0] == s0->ne[0] && f32c(op) && op->ne[0] == s0->ne[1] && ggml_nrows(op) == ggml_nrows(s1);
    default: break;
    }
    if (rt.matmul_only) return false;
    switch (op->op) {
    case GGML_OP_RMS_NORM: return f32c(s0) && f32c(op) && ggml_are_same_shape(s0, op);
    case GGML_OP_ADD: return f32c(s0) && f32c(s1) && f32c(op) && ggml_are_same_shape(s0, s1) && ggml_are_same_shape(s0, op);
    case GGML_OP_MUL:  // by a row vector (a norm weight, n % 8 == 0) or elementwise
        return f32c(s0) && f32c(s1) && f32c(op) && ggml_are_same_shape(s0, op) &&
               ((is_row_vector_of(s1, s0) && s0->ne[0] % 8 == 0) || (ggml_are_same_shape(s0, s1) && ggml_nelements(s0) % 8 == 0));
    case GGML_OP_ROPE: {
        const int32_t* p = reinterpret_cast<const int32_t*>(op->op_params);
        const ggml_tensor* ff = op->src[2];
        // NORM or NEOX pairing over the whole head, no context extension (freq_scale 1, ext_factor 0, attn_factor 1), no sections
        return (p[2] == 0 || p[2] == GGML_ROPE_TYPE_NEOX) && p[1] == s0->ne[0] && op_param_f32(op, 6) == 1.0f && op_param_f32(op, 7) == 0.0f &&
               op_param_f32(op, 8) == 1.0f && p[15] == 0 && f32c(s0) && f32c(op) && ggml_are_same_shape(s0, op) && s0->ne[0] % 16 == 0 &&
               s0->ne[3] == 1 && s1 && s1->type == GGML_TYPE_I32 && ggml_is_contiguous(s1) && s1->ne[0] == s0->ne[2] &&
               (!ff || (f32c(ff) && ff->ne[0] >= s0->ne[0] / 2));
    }
    case GGML_OP_SET_ROWS:  // into the fp16 KV cache
        return rt.attn && in_kv_buffer(op) && op->type == GGML_TYPE_F16 && op->nb[0] == 2 && op->nb[1] % 4 == 0 && op->ne[2] == 1 && op->ne[3] == 1 &&
               op->ne[1] <= INT32_MAX && s0->type == GGML_TYPE_F32 && s0->nb[0] == 4 && s0->nb[1] % 4 == 0 && s0->ne[0] == op->ne[0] &&
               s0->ne[0] % 16 == 0 && s0->ne[2] == 1 && s0->ne[3] == 1 && s1->type == GGML_TYPE_I64 && ggml_is_contiguous(s1) &&
               s1->ne[0] == s0->ne[1] && s1->ne[1] == 1 && s1->ne[2] == 1 && s1->ne[3] == 1;
    case GGML_OP_FLASH_ATTN_EXT: return rt.attn && flash_attn_ok(op, rt.attn_tokens);
    case GGML_OP_GLU:
        return ggml_get_glu_op(op) == GGML_GLU_OP_SWIGLU && ggml_get_op_params_i32(op, 1) == 0 && f32c(s0) && f32c(s1) && f32c(op) &&
               ggml_are_same_shape(s0, s1) && ggml_are_same_shape(s0, op);
    default: return false;
    }
}

// ---- device ----------------------------------------------------------------------------------------------------------
const char* dev_name(ggml_backend_dev_t) { return "Kernelcore"; }
const char* dev_description(ggml_backend_dev_t) { return "Kernelcore: K-quant LLM kernels on an NVIDIA B200 (sm_100a)"; }
void dev_memory(ggml_backend_dev_t, size_t* free, size_t* total) {
    *free = *total = 0;
    if (settings().ok) cudaMemGetInfo(free, total);
}
enum ggml_backend_dev_type dev_type(ggml_backend_dev_t) { return GGML_BACKEND_DEVICE_TYPE_ACCEL; }
void dev_props(ggml_backend_dev_t dev, ggml_backend_dev_props* props) {
    props->name = dev_name(dev);
    props->description = dev_description(dev);
    props->type = dev_type(dev);
    dev_memory(dev, &props->memory_free, &props->memory_total);
    // weights are copied into device memory, so a memory-mapped model file would only stay resident as a second copy:
    // no mmap while this backend claims weights (ggml-kernelcore.cpp:835-846)
    const bool claims_weights = settings().ok && !settings().disabled;
    props->caps = {false, false, false, false, !claims_weights};
}
ggml_backend_t dev_init_backend(ggml_backend_dev_t, const char*) { return ggml_backend_kernelcore_init(); }
ggml_backend_buffer_type_t dev_buffer_type(ggml_backend_dev_t) { return weight_buffer_type(); }
// llama.cpp's KV-cache hook asks for this type so that SET_ROWS and FLASH_ATTN_EXT can run here (:853-858)
ggml_backend_buffer_type_t dev_kv_buffer_type(ggml_backend_dev_t) {
    const Settings& rt = settings();
    return rt.ok && !rt.disabled && !rt.matmul_only && rt.attn ? kv_buffer_type() : nullptr;
}
bool dev_supports_op(ggml_backend_dev_t, const ggml_tensor* op) { return supports_op_rules(settings(), op); }
bool dev_supports_buft(ggml_backend_dev_t, ggml_backend_buffer_type_t buft) { return buft == weight_buffer_type() || buft == kv_buffer_type(); }

ggml_backend_device_i make_device_iface() {
    ggml_backend_device_i i{};
    i.get_name = dev_name;
    i.get_description = dev_description;
    i.get_memory = dev_memory;
    i.get_type = dev_type;
    i.get_props = dev_props;
    i.init_backend = dev_init_backend;
    i.get_buffer_type = dev_buffer_type;
    i.get_host_buffer_type = dev_kv_buffer_type;
    i.supports_op = dev_supports_op;
    i.supports_buft = dev_supports_buft;
    return i;
}

// ---- registry ----------------------------------------------------------------------------------------------------------
const char* reg_name(ggml_backend_reg_t) { return "Kernelcore"; }
size_t reg_device_count(ggml_backend_reg_t) { return 1; }
ggml_backend_dev_t reg_device(ggml_backend_reg_t reg, size_t index) {
    GGML_ASSERT(index == 0);
    static ggml_backend_device device = {make_device_iface(), reg, nullptr};
    return &device;
}

}  // namespace

// The support rules and the two buffer types without the device check, for callers that want to know what the backend
// would claim before (or without) bringing a GPU up: flags bit 0 = MUL_MAT only, bit 1 = no attention; attn_tokens < 0 =
// no limit.  Reached through ggml_backend_reg_get_proc_address as "kcb_ggml_supports_op_rules" /
// "kcb_ggml_weight_buffer_type" / "kcb_ggml_kv_buffer_type".
extern "C" int kcb_ggml_supports_op_rules(const ggml_tensor* op, int flags, int attn_tokens) {
    Settings s;
    s.ok = true;
    s.matmul_only = (flags & 1) != 0;
    s.attn = (flags & 2) == 0;
    s.attn_tokens = attn_tokens < 0 ? INT_MAX : attn_tokens;
    return op && supports_op_rules(s, op) ? 1 : 0;
}
extern "C" ggml_backend_buffer_type_t kcb_ggml_weight_buffer_type(void) { return weight_buffer_type(); }
extern "C" ggml_backend_buffer_type_t kcb_ggml_kv_buffer_type(void) { return kv_buffer_type(); }

namespace {
void* reg_proc_address(ggml_backend_reg_t, const char* name) {
    if (!name) return nullptr;
    if (!std::strcmp(name, "kcb_ggml_supports_op_rules")) return reinterpret_cast<void*>(kcb_ggml_supports_op_rules);
    if (!std::strcmp(name, "kcb_ggml_weight_buffer_type")) return reinterpret_cast<void*>(kcb_ggml_weight_buffer_type);
    if (!std::strcmp(name, "kcb_ggml_kv_buffer_type")) return reinterpret_cast<void*>(kcb_ggml_kv_buffer_type);
    return nullptr;
}
ggml_backend_reg_i make_reg_iface() {
    ggml_backend_reg_i i{};
    i.get_name = reg_name;
    i.get_device_count = reg_device_count;
    i.get_device = reg_device;
    i.get_proc_address = reg_proc_address;
    return i;
}
ggml_backend_buffer_type_t weight_buffer_type() {
    static ggml_backend_buffer_type t = {make_buft_iface(true), reg_device(ggml_backend_kernelcore_reg(), 0), nullptr};
    return &t;
}
ggml_backend_buffer_type_t kv_buffer_type() {
    static ggml_backend_buffer_type t = {make_buft_iface(false), reg_device(ggml_backend_kernelcore_reg(), 0), nullptr};
    return &t;
}
}  // namespace

extern "C" {

ggml_backend_t ggml_backend_kernelcore_init(void) {
    if (!settings().ok) return nullptr;
    auto* ctx = new BackendCtx;
    if (kcb_ggml_ctx_create(nullptr, &ctx->ops) != 0) {
        delete ctx;
        return nullptr;
    }
    return new ggml_backend{backend_guid(), make_backend_iface(), reg_device(ggml_backend_kernelcore_reg(), 0), ctx};
}

bool ggml_backend_is_kc(ggml_backend_t backend) { return backend != nullptr && ggml_guid_matches(backend->guid, backend_guid()); }

ggml_backend_reg_t ggml_backend_kernelcore_reg(void) {
    static ggml_backend_reg reg = {GGML_BACKEND_API_VERSION, make_reg_iface(), nullptr};
    return &reg;
}

GGML_BACKEND_DL_IMPL(ggml_backend_kernelcore_reg)

}  // extern "C"
