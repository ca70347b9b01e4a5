// Operator layer of the llama.cpp backend: ggml tensors -> kernel launches.
//
// One function per graph operator, following the reference's rules
// (integrations/llama.cpp/ggml/src/ggml-kernelcore/ggml-kernelcore.cpp:471-711):
//  * mul_mat quantizes its activation input once per graph and shares it between the matrices that read the same
//    tensor (q, k, v; gate, up); one column -> per-32 blocks + matvec, contiguous batches -> per-256 slots + matmul;
//  * fused_norm / fused_swiglu leave their result both as floats and already quantized for the matmuls behind them;
//  * strides of ggml tensors become the row / head strides of the attention and set_rows kernels.
// Launches go straight to the kernels' host functions on the context's stream (no name lookup, no argument
// marshalling: the by-name route exists for callers that hold the reference's argument structs).

#include "../../include/ggml-kernelcore-ops.h"
#include "../../include/kernelcore_b200.h"

#include "common.cuh"
#include "ops.h"

#include <cmath>
#include <cstring>
#include <vector>

namespace {

using namespace kcb;

constexpr int scratch_ints(int nb) { return nb * 11; }   // per-32 slot (llm/llm_kernels.hpp:82-85)
constexpr int scratch_k_ints(int nsb) { return nsb * 85; }  // per-256 slot (:86-89)

struct Quantized {
    const kcb_tensor* t;
    long long ncols;
    int k;
    bool k256;
    int* q;
};

struct Ctx {
    cudaStream_t stream = nullptr;
    std::vector<std::pair<int*, size_t>> chunks;  // scratch, grown by adding chunks (launches in flight keep theirs)
    size_t chunk = 0, used = 0;
    std::vector<Quantized> quantized;
    float* ones = nullptr;
    int ones_n = 0;

    ~Ctx() {
        for (auto& c : chunks) cudaFree(c.first);
        if (ones) cudaFree(ones);
    }
    int* take(size_t ints) {
        ints = (ints + 15) / 16 * 16;
        while (chunk < chunks.size() && used + ints > chunks[chunk].second) ++chunk, used = 0;
        if (chunk == chunks.size()) {
            const size_t n = std::max<size_t>(ints, chunks.empty() ? (1u << 20) : chunks.back().second * 2);
            void* p = nullptr;
            if (cudaMalloc(&p, n * sizeof(int)) != cudaSuccess) return nullptr;
            chunks.emplace_back(static_cast<int*>(p), n);
            used = 0;
        }
        int* base = chunks[chunk].first + used;
        used += ints;
        return base;
    }
    const float* ones_of(int n) {
        if (n <= ones_n) return ones;
        if (ones) {
            cudaStreamSynchronize(stream);
            cudaFree(ones);
            ones = nullptr, ones_n = 0;
        }
        std::vector<float> h(static_cast<size_t>(n), 1.0f);
        if (cudaMalloc(reinterpret_cast<void**>(&ones), h.size() * 4) != cudaSuccess) return nullptr;
        if (cudaMemcpyAsync(ones, h.data(), h.size() * 4, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
            cudaStreamSynchronize(stream) != cudaSuccess)
            return nullptr;
        ones_n = n;
        return ones;
    }
};

long long nrows(const kcb_tensor* t) { return t->ne[1] * t->ne[2] * t->ne[3]; }
long long nelements(const kcb_tensor* t) { return t->ne[0] * nrows(t); }
float param_f32(const kcb_tensor* t, int i) {
    float v;
    std::memcpy(&v, t->op_params + i, sizeof v);
    return v;
}
bool is_contiguous_f32(const kcb_tensor* t) {
    return t->type == KCB_TYPE_F32 && t->nb[0] == 4 && t->nb[1] == static_cast<size_t>(t->ne[0]) * 4 &&
           t->nb[2] == t->nb[1] * t->ne[1] && t->nb[3] == t->nb[2] * t->ne[2];
}
const float* f32(const kcb_tensor* t) { return static_cast<const float*>(t->data); }
float* f32w(const kcb_tensor* t) { return static_cast<float*>(t->data); }

// Batches read activations scaled per 256 values (ggml-kernelcore.cpp:424).
bool batch_k256(long long ncols) { return ncols > 1; }

int* quantized_slots(Ctx& c, const kcb_tensor* x, int k, long long ncols, bool k256, size_t extra = 0) {
    const size_t slot = k256 ? scratch_k_ints(k / 256) : scratch_ints(k / 32);
    int* base = c.take(slot * static_cast<size_t>(ncols) + extra);
    if (base) c.quantized.push_back({x, ncols, k, k256, base});
    return base;
}

// The columns of x as 8-bit activations, quantized once per graph (ggml-kernelcore.cpp:471-497).
int* quantized_input(Ctx& c, const kcb_tensor* x, int k, long long ncols, bool k256, int& err) {
    for (const Quantized& q : c.quantized)
        if (q.t == x && q.ncols == ncols && q.k == k && q.k256 == k256) return q.q;
    int* base = quantized_slots(c, x, k, ncols, k256);
    if (!base) {
        err = KCB_OUT_OF_MEMORY;
        return nullptr;
    }
    if (k256) {
        err = quantize_cols_k(f32(x), base, k, static_cast<int>(ncols), c.stream);
    } else if (ncols > 1 && x->nb[1] == static_cast<size_t>(k) * 4) {
        err = quantize_cols(f32(x), base, k, static_cast<int>(ncols), c.stream);
    } else {
        const int nb = k / 32;
        for (long long col = 0; col < ncols && err == KCB_SUCCESS; ++col) {
            int* q = base + static_cast<size_t>(col) * scratch_ints(nb);
            const float* xc = reinterpret_cast<const float*>(static_cast<const char*>(x->data) + col * x->nb[1]);
            err = quantize_q8x4(xc, q, reinterpret_cast<float*>(q + nb * 8), nb, c.stream);
        }
    }
    return err == KCB_SUCCESS ? base : nullptr;
}

}  // namespace

extern "C" {

int kcb_ggml_ctx_create(void* stream, void** out) {
    if (!out) return KCB_INVALID_VALUE;
    auto* c = new Ctx;
    c->stream = static_cast<cudaStream_t>(stream);
    *out = c;
    return KCB_SUCCESS;
}
int kcb_ggml_ctx_begin_graph(void* h) {
    if (!h) return KCB_INVALID_VALUE;
    auto* c = static_cast<Ctx*>(h);
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) return KCB_INTERNAL_ERROR;
    c->quantized.clear();
    c->chunk = 0, c->used = 0;
    return KCB_SUCCESS;
}
int kcb_ggml_ctx_sync(void* h) {
    if (!h) return KCB_INVALID_VALUE;
    return cudaStreamSynchronize(static_cast<Ctx*>(h)->stream) == cudaSuccess ? KCB_SUCCESS : KCB_INTERNAL_ERROR;
}
int kcb_ggml_ctx_destroy(void* h) {
    if (h) {
        auto* c = static_cast<Ctx*>(h);
        cudaStreamSynchronize(c->stream);
        delete c;
    }
    return KCB_SUCCESS;
}

size_t kcb_ggml_weight_bytes(int type, int rows, int k) {
    if (rows <= 0 || k <= 0) return 0;
    if (type == KCB_TYPE_Q4_K || type == KCB_TYPE_Q6_K) return k % 256 ? 0 : kcb_kquant_bytes(rows, k, type == KCB_TYPE_Q6_K);
    if (type == KCB_TYPE_F16) return k % 2 || rows % 8 ? 0 : static_cast<size_t>(rows) * k * 2;
    return 0;
}
int kcb_ggml_set_weight(void* h, void* dst, const void* src, int type, int rows, int k) {
    const size_t bytes = kcb_ggml_weight_bytes(type, rows, k);
    if (!h || !dst || !src || !bytes) return KCB_INVALID_VALUE;
    auto* c = static_cast<Ctx*>(h);
    if (type == KCB_TYPE_Q4_K) {
        if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream) != cudaSuccess) return KCB_INTERNAL_ERROR;
        return cudaStreamSynchronize(c->stream) == cudaSuccess ? KCB_SUCCESS : KCB_INTERNAL_ERROR;
    }
    if (type == KCB_TYPE_Q6_K) {
        void* tmp = nullptr;
        if (cudaMalloc(&tmp, bytes) != cudaSuccess) return KCB_OUT_OF_MEMORY;
        int e = cudaMemcpyAsync(tmp, src, bytes, cudaMemcpyHostToDevice, c->stream) == cudaSuccess ? KCB_SUCCESS : KCB_INTERNAL_ERROR;
        if (e == KCB_SUCCESS) e = q6k_convert(tmp, dst, rows, k, 1, c->stream);
        cudaStreamSynchronize(c->stream);
        cudaFree(tmp);
        return e;
    }
    // fp16: rows in groups of 8, interleaved by 32-bit word (llm::ref::repackF16, llm/llm_reference.cpp:740-746)
    const uint16_t* w = static_cast<const uint16_t*>(src);
    const int kw = k / 2;
    std::vector<int> words(static_cast<size_t>(rows) * kw);
    for (int r = 0; r < rows; ++r)
        for (int j = 0; j < kw; ++j)
            words[(static_cast<size_t>(r / 8) * kw + j) * 8 + r % 8] =
                static_cast<int>(static_cast<uint32_t>(w[static_cast<size_t>(r) * k + 2 * j]) | (static_cast<uint32_t>(w[static_cast<size_t>(r) * k + 2 * j + 1]) << 16));
    if (cudaMemcpyAsync(dst, words.data(), bytes, cudaMemcpyHostToDevice, c->stream) != cudaSuccess) return KCB_INTERNAL_ERROR;
    return cudaStreamSynchronize(c->stream) == cudaSuccess ? KCB_SUCCESS : KCB_INTERNAL_ERROR;
}

int kcb_ggml_mul_mat(void* h, const kcb_tensor* dst) {
    if (!h || !dst || !dst->src[0] || !dst->src[1]) return KCB_INVALID_VALUE;
    auto& c = *static_cast<Ctx*>(h);
    const kcb_tensor *w = dst->src[0], *x = dst->src[1];
    const int rows = static_cast<int>(w->ne[1]), k = static_cast<int>(w->ne[0]), nb = k / 32;
    const long long ncols = nrows(x);
    if (x->type != KCB_TYPE_F32 || x->ne[0] != k || ncols <= 0) return KCB_INVALID_VALUE;
    if (w->type == KCB_TYPE_F16) {
        if (x->nb[1] != static_cast<size_t>(k) * 4) return KCB_UNSUPPORTED_OPERATION;
        return matmul_f16(static_cast<const int*>(w->data), f32(x), f32w(dst), rows, k, static_cast<int>(ncols), c.stream);
    }
    if (w->type != KCB_TYPE_Q4_K && w->type != KCB_TYPE_Q6_K) return KCB_UNSUPPORTED_OPERATION;
    const bool q6 = w->type == KCB_TYPE_Q6_K;
    const bool k256 = batch_k256(ncols) && x->nb[1] == static_cast<size_t>(k) * 4;
    int err = KCB_SUCCESS;
    int* base = quantized_input(c, x, k, ncols, k256, err);
    if (!base) return err;
    if (ncols > 1)  // several tokens: Y[c * rows + r], the layout of a [rows, ncols] ggml tensor
        return matmul_kq_q8(w->data, base, f32w(dst), rows, k, static_cast<int>(ncols), q6, k256, c.stream);
    float* xd = reinterpret_cast<float*>(base + nb * 8);
    return q6 ? matvec_q6k_q8(w->data, base, xd, f32w(dst), rows, k, c.stream) : matvec_q4k_q8(w->data, base, xd, f32w(dst), rows, k, c.stream);
}

int kcb_ggml_fused_norm(void* h, const kcb_tensor* add, const kcb_tensor* norm, const kcb_tensor* mul) {
    if (!h || !norm || !mul || !norm->src[0] || !mul->src[1]) return KCB_INVALID_VALUE;
    auto& c = *static_cast<Ctx*>(h);
    const kcb_tensor* x = norm->src[0];
    const int n = static_cast<int>(x->ne[0]), rows = static_cast<int>(nrows(x));
    if (n % 256 || rows <= 0) return KCB_INVALID_VALUE;
    const bool k256 = batch_k256(rows);
    // per 256: the slots, then per-row partial sums of squares; per 32: the partial sums live inside the slots
    int* qk = quantized_slots(c, mul, n, rows, k256, k256 ? static_cast<size_t>(rows) * scratch_ints(n / 32) : 0);
    if (!qk) return KCB_OUT_OF_MEMORY;
    int* sq = k256 ? qk + static_cast<size_t>(rows) * scratch_k_ints(n / 256) : nullptr;
    const float* a = add ? f32(add->src[0]) : f32(x);
    const float* t = add ? f32(add->src[1]) : nullptr;
    float* out = add ? f32w(add) : nullptr;
    return add_norm_q8(a, t, out, f32(mul->src[1]), f32w(mul), qk, sq, n, rows, param_f32(norm, 0), 3, k256, c.stream);
}

int kcb_ggml_rms_norm(void* h, const kcb_tensor* norm, const float* weight, const kcb_tensor* out) {
    if (!h || !norm || !out || !norm->src[0]) return KCB_INVALID_VALUE;
    auto& c = *static_cast<Ctx*>(h);
    const kcb_tensor* x = norm->src[0];
    const int n = static_cast<int>(x->ne[0]), rows = static_cast<int>(nrows(x));
    const float* w = weight ? weight : c.ones_of(n);
    if (!w) return KCB_OUT_OF_MEMORY;
    return rms_norm(f32(x), w, f32w(out), n, rows, param_f32(norm, 0), c.stream);
}

int kcb_ggml_mul(void* h, const kcb_tensor* dst) {
    if (!h || !dst || !dst->src[0] || !dst->src[1]) return KCB_INVALID_VALUE;
    auto& c = *static_cast<Ctx*>(h);
    const kcb_tensor *a = dst->src[0], *b = dst->src[1];
    const bool row_vector = b->type == KCB_TYPE_F32 && is_contiguous_f32(b) && b->ne[0] == a->ne[0] && nrows(b) == 1;
    const int n = row_vector ? static_cast<int>(a->ne[0]) : static_cast<int>(nelements(a));  // broadcast or same shape
    return mul_rows(f32(a), f32(b), f32w(dst), n, static_cast<size_t>(nelements(a)), c.stream);
}

int kcb_ggml_add(void* h, const kcb_tensor* dst) {
    if (!h || !dst || !dst->src[0] || !dst->src[1]) return KCB_INVALID_VALUE;
    return vector_add(f32(dst->src[0]), f32(dst->src[1]), f32w(dst), static_cast<size_t>(nelements(dst)), static_cast<Ctx*>(h)->stream);
}

int kcb_ggml_rope(void* h, const kcb_tensor* dst) {
    if (!h || !dst || !dst->src[0] || !dst->src[1]) return KCB_INVALID_VALUE;
    auto& c = *static_cast<Ctx*>(h);
    const kcb_tensor* x = dst->src[0];
    const int hd = static_cast<int>(x->ne[0]), nh = static_cast<int>(x->ne[1]), nt = static_cast<int>(x->ne[2]);
    const float* ff = dst->src[2] ? f32(dst->src[2]) : nullptr;  // no frequency factors: the kernel divides by nothing
    const bool neox = (dst->op_params[2] & KCB_ROPE_TYPE_NEOX) != 0;
    return rope_ggml(f32(x), f32w(dst), static_cast<const int*>(dst->src[1]->data), ff, hd, nh, nt, std::log2(param_f32(dst, 5)), neox, c.stream);
}

int kcb_ggml_swiglu(void* h, const kcb_tensor* dst) {
    if (!h || !dst || !dst->src[0] || !dst->src[1]) return KCB_INVALID_VALUE;
    return silu_mul(f32(dst->src[0]), f32(dst->src[1]), f32w(dst), static_cast<size_t>(nelements(dst)), static_cast<Ctx*>(h)->stream);
}

int kcb_ggml_fused_swiglu(void* h, const kcb_tensor* dst) {
    if (!h || !dst || !dst->src[0] || !dst->src[1]) return KCB_INVALID_VALUE;
    auto& c = *static_cast<Ctx*>(h);
    const int n = static_cast<int>(dst->ne[0]), cols = static_cast<int>(nrows(dst));
    if (n % 256 || cols <= 0) return KCB_INVALID_VALUE;
    const bool k256 = batch_k256(cols);
    int* q = quantized_slots(c, dst, n, cols, k256);
    if (!q) return KCB_OUT_OF_MEMORY;
    if (!k256) return silu_mul_q8(f32(dst->src[0]), f32(dst->src[1]), f32w(dst), q, nullptr, nullptr, n, cols, c.stream);
    const int e = silu_mul(f32(dst->src[0]), f32(dst->src[1]), f32w(dst), static_cast<size_t>(n) * cols, c.stream);
    return e != KCB_SUCCESS ? e : quantize_cols_k(f32(dst), q, n, cols, c.stream);
}

int kcb_ggml_set_rows(void* h, const kcb_tensor* dst) {
    if (!h || !dst || !dst->src[0] || !dst->src[1]) return KCB_INVALID_VALUE;
    const kcb_tensor *src = dst->src[0], *idx = dst->src[1];
    if (dst->type != KCB_TYPE_F16 || idx->type != KCB_TYPE_I64) return KCB_UNSUPPORTED_OPERATION;
    return set_rows_f16(f32(src), static_cast<const long long*>(idx->data), dst->data, static_cast<int>(src->ne[0] / 2), static_cast<int>(src->ne[1]),
                        static_cast<int>(src->nb[1] / 4), static_cast<int>(dst->nb[1] / 4), static_cast<int>(dst->ne[1]), static_cast<Ctx*>(h)->stream);
}

int kcb_ggml_flash_attn(void* h, const kcb_tensor* dst) {
    if (!h || !dst || !dst->src[0] || !dst->src[1] || !dst->src[2]) return KCB_INVALID_VALUE;
    const kcb_tensor *q = dst->src[0], *k = dst->src[1], *v = dst->src[2], *mask = dst->src[3];
    if (k->type != KCB_TYPE_F16 || v->type != KCB_TYPE_F16 || (mask && mask->type != KCB_TYPE_F16)) return KCB_UNSUPPORTED_OPERATION;
    int d[15];
    const int D = static_cast<int>(k->ne[0]), T = static_cast<int>(k->ne[1]), Hkv = static_cast<int>(k->ne[2]);
    const int H = static_cast<int>(q->ne[2]), N = static_cast<int>(q->ne[1]);
    if (Hkv <= 0 || H % Hkv) return KCB_INVALID_VALUE;
    // field order of llm::FaDims (llm/llm_kernels.hpp:316-332); K, V and mask strides in 32-bit words, q strides in floats
    d[0] = H, d[1] = T, d[2] = D, d[3] = H / Hkv, d[4] = (T + 7) / 8 * 8;
    d[5] = static_cast<int>(k->nb[1] / 4), d[6] = static_cast<int>(k->nb[2] / 4);
    d[7] = static_cast<int>(v->nb[1] / 4), d[8] = static_cast<int>(v->nb[2] / 4);
    d[9] = N, d[10] = static_cast<int>(q->nb[1] / 4), d[11] = static_cast<int>(q->nb[2] / 4);
    d[12] = mask ? static_cast<int>(mask->nb[1] / 4) : 0, d[13] = mask ? 1 : 0, d[14] = Hkv;
    return flash_attn_f16(f32(q), k->data, v->data, mask ? mask->data : nullptr, f32w(dst), d, param_f32(dst, 0), static_cast<Ctx*>(h)->stream);
}

}  // extern "C"
