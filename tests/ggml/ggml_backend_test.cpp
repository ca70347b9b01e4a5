// Test driver for the ggml backend object (kernelcore_b200/csrc/ggml_backend.cpp), compiled against the ggml stand-in
// headers and linked with libkernelcore_b200.so.  Two modes:
//   rules                        no GPU: registry / device / buffer-type properties and the supports_op accept / reject
//                                table, checked against the reference's rules
//                                (integrations/llama.cpp/ggml/src/ggml-kernelcore/ggml-kernelcore.cpp:860-961);
//   graph <model.bin> <out.bin>  GPU: uploads a tiny Llama-style model through the buffer type's set_tensor, builds the
//                                graph llama.cpp would build for a prompt of n tokens (norm + mul, q/k/v, rope, SET_ROWS
//                                into an fp16 cache, FLASH_ATTN_EXT, wo, add + norm + mul, gate/up, SwiGLU, down, ...,
//                                last row: add + norm + mul + lm_head), runs graph_compute and writes the logits, plus
//                                the canonical bytes get_tensor returns for one Q4_K and one Q6_K weight.
// Prints "ok" and exits 0, or a message and exits 1.
#include "ggml-kernelcore.h"

#include "ggml-backend-impl.h"
#include "ggml-impl.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <string>
#include <vector>

#define CHECK(x)                                                     \
    do {                                                             \
        if (!(x)) {                                                  \
            std::printf("FAILED %s (line %d)\n", #x, __LINE__);      \
            return 1;                                                \
        }                                                            \
    } while (0)

namespace {

size_t type_size(ggml_type t, int64_t& blk) { return kcb_stub_type_size(t, &blk); }

// Tensors with stable addresses; contiguous strides unless changed afterwards.
struct Pool {
    std::deque<ggml_tensor> store;
    ggml_tensor* make(ggml_type type, int64_t n0, int64_t n1 = 1, int64_t n2 = 1, int64_t n3 = 1) {
        store.emplace_back();
        ggml_tensor* t = &store.back();
        std::memset(t, 0, sizeof *t);
        t->type = type;
        t->ne[0] = n0, t->ne[1] = n1, t->ne[2] = n2, t->ne[3] = n3;
        int64_t blk;
        const size_t ts = type_size(type, blk);
        t->nb[0] = ts;
        t->nb[1] = static_cast<size_t>(n0 / blk) * ts;
        t->nb[2] = t->nb[1] * n1;
        t->nb[3] = t->nb[2] * n2;
        t->flags = GGML_TENSOR_FLAG_COMPUTE;
        return t;
    }
    ggml_tensor* op(ggml_op o, ggml_type type, std::vector<ggml_tensor*> src, int64_t n0, int64_t n1 = 1, int64_t n2 = 1) {
        ggml_tensor* t = make(type, n0, n1, n2);
        t->op = o;
        for (size_t i = 0; i < src.size(); ++i) t->src[i] = src[i];
        return t;
    }
};
void set_f32(ggml_tensor* t, int i, float v) { std::memcpy(t->op_params + i, &v, 4); }

using RulesFn = int (*)(const ggml_tensor*, int, int);
using BuftFn = ggml_backend_buffer_type_t (*)(void);

int run_rules() {
    ggml_backend_reg_t reg = ggml_backend_kernelcore_reg();
    CHECK(reg && reg->api_version == GGML_BACKEND_API_VERSION);
    CHECK(std::string(reg->iface.get_name(reg)) == "Kernelcore" && reg->iface.get_device_count(reg) == 1);
    ggml_backend_dev_t dev = reg->iface.get_device(reg, 0);
    CHECK(dev && dev->reg == reg && std::string(dev->iface.get_name(dev)) == "Kernelcore");
    CHECK(dev->iface.get_type(dev) == GGML_BACKEND_DEVICE_TYPE_ACCEL);
    CHECK(!ggml_backend_is_kc(nullptr));
    auto rules = reinterpret_cast<RulesFn>(reg->iface.get_proc_address(reg, "kcb_ggml_supports_op_rules"));
    auto wtype = reinterpret_cast<BuftFn>(reg->iface.get_proc_address(reg, "kcb_ggml_weight_buffer_type"));
    auto ktype = reinterpret_cast<BuftFn>(reg->iface.get_proc_address(reg, "kcb_ggml_kv_buffer_type"));
    CHECK(rules && wtype && ktype && !reg->iface.get_proc_address(reg, "nothing"));
    ggml_backend_buffer_type_t wt = wtype(), kt = ktype();
    CHECK(dev->iface.get_buffer_type(dev) == wt);
    CHECK(std::string(wt->iface.get_name(wt)) == "Kernelcore" && std::string(kt->iface.get_name(kt)) == "Kernelcore_Host");
    CHECK(!wt->iface.is_host(wt) && !kt->iface.is_host(kt) && wt->iface.get_alignment(wt) >= 64);
    CHECK(dev->iface.supports_buft(dev, wt) && dev->iface.supports_buft(dev, kt) && !dev->iface.supports_buft(dev, nullptr));

    Pool p;
    ggml_backend_buffer wbuf{}, kbuf{}, other{};
    wbuf.buft = wt, wbuf.usage = GGML_BACKEND_BUFFER_USAGE_WEIGHTS;
    kbuf.buft = kt;
    ggml_backend_buffer_type foreign{};
    other.buft = &foreign;
    // device layouts are as large as the GGUF tensors
    ggml_tensor* w4 = p.make(GGML_TYPE_Q4_K, 512, 64);
    ggml_tensor* w6 = p.make(GGML_TYPE_Q6_K, 512, 64);
    CHECK(wt->iface.get_alloc_size(wt, w4) == 64 * 2 * 144 && wt->iface.get_alloc_size(wt, w6) == 64 * 2 * 210);
    w4->buffer = w6->buffer = &wbuf;

    auto ok = [&](const ggml_tensor* t, int flags = 0, int tokens = -1) { return rules(t, flags, tokens) == 1; };
    // --- MUL_MAT: weight in this backend's weight buffer, K-quant or fp16, rows % 8, f32 contiguous activations
    ggml_tensor* x = p.make(GGML_TYPE_F32, 512, 5);
    ggml_tensor* mm = p.op(GGML_OP_MUL_MAT, GGML_TYPE_F32, {w4, x}, 64, 5);
    CHECK(ok(mm) && ok(mm, 1));                                        // also when only matmuls are claimed
    mm->src[0] = w6;
    CHECK(ok(mm));
    ggml_tensor* wf = p.make(GGML_TYPE_F16, 512, 64);
    wf->buffer = &wbuf;
    mm->src[0] = wf;
    CHECK(ok(mm));
    ggml_tensor* w_else = p.make(GGML_TYPE_Q4_K, 512, 64);
    w_else->buffer = &other;
    mm->src[0] = w_else;
    CHECK(!ok(mm));                                                    // weight lives in another backend's buffer
    ggml_tensor* w_rows = p.make(GGML_TYPE_Q4_K, 512, 60);
    w_rows->buffer = &wbuf;
    ggml_tensor* mm60 = p.op(GGML_OP_MUL_MAT, GGML_TYPE_F32, {w_rows, x}, 60, 5);
    CHECK(!ok(mm60));                                                  // rows % 8
    ggml_tensor* w32 = p.make(GGML_TYPE_F32, 512, 64);
    w32->buffer = &wbuf;
    mm->src[0] = w32;
    CHECK(!ok(mm));                                                    // f32 weights stay with the CPU backend
    mm->src[0] = w4;
    ggml_tensor* xs = p.make(GGML_TYPE_F32, 512, 5);
    xs->nb[1] *= 2, xs->nb[2] *= 2, xs->nb[3] *= 2;
    mm->src[1] = xs;
    CHECK(!ok(mm));                                                    // strided activations
    mm->src[1] = x;
    ggml_tensor* mm_bad = p.op(GGML_OP_MUL_MAT, GGML_TYPE_F32, {w4, x}, 64, 4);
    CHECK(!ok(mm_bad));                                                // output columns != input columns
    // --- elementwise and norm
    ggml_tensor* a = p.make(GGML_TYPE_F32, 512, 5);
    ggml_tensor* wrow = p.make(GGML_TYPE_F32, 512);
    ggml_tensor* norm = p.op(GGML_OP_RMS_NORM, GGML_TYPE_F32, {a}, 512, 5);
    CHECK(ok(norm) && !ok(norm, 1));
    CHECK(ok(p.op(GGML_OP_ADD, GGML_TYPE_F32, {a, x}, 512, 5)) && !ok(p.op(GGML_OP_ADD, GGML_TYPE_F32, {a, wrow}, 512, 5)));
    CHECK(ok(p.op(GGML_OP_MUL, GGML_TYPE_F32, {a, wrow}, 512, 5)) && ok(p.op(GGML_OP_MUL, GGML_TYPE_F32, {a, x}, 512, 5)));
    ggml_tensor* odd = p.make(GGML_TYPE_F32, 7, 3);
    CHECK(!ok(p.op(GGML_OP_MUL, GGML_TYPE_F32, {odd, p.make(GGML_TYPE_F32, 7, 3)}, 7, 3)));   // 21 elements: not a multiple of 8
    CHECK(!ok(p.op(GGML_OP_SOFT_MAX, GGML_TYPE_F32, {a}, 512, 5)));    // not an operator of this backend
    CHECK(ok(p.op(GGML_OP_RESHAPE, GGML_TYPE_F32, {a}, 512 * 5)) && ok(p.op(GGML_OP_VIEW, GGML_TYPE_F32, {a}, 512)));
    // --- SwiGLU
    ggml_tensor* glu = p.op(GGML_OP_GLU, GGML_TYPE_F32, {a, x}, 512, 5);
    glu->op_params[0] = GGML_GLU_OP_SWIGLU;
    CHECK(ok(glu));
    glu->op_params[1] = 1;                                             // swapped halves: not claimed
    CHECK(!ok(glu));
    glu->op_params[1] = 0, glu->op_params[0] = GGML_GLU_OP_GEGLU;
    CHECK(!ok(glu));
    // --- RoPE: whole head, NORM or NEOX, no context extension
    ggml_tensor* q = p.make(GGML_TYPE_F32, 64, 4, 5);
    ggml_tensor* pos = p.make(GGML_TYPE_I32, 5);
    ggml_tensor* rope = p.op(GGML_OP_ROPE, GGML_TYPE_F32, {q, pos}, 64, 4, 5);
    rope->op_params[1] = 64, rope->op_params[2] = 0;
    set_f32(rope, 5, 10000.0f), set_f32(rope, 6, 1.0f), set_f32(rope, 7, 0.0f), set_f32(rope, 8, 1.0f);
    CHECK(ok(rope));
    rope->op_params[2] = GGML_ROPE_TYPE_NEOX;
    CHECK(ok(rope));
    rope->op_params[2] = 8;                                            // another rope mode
    CHECK(!ok(rope));
    rope->op_params[2] = 0, rope->op_params[1] = 32;                   // partial rotation
    CHECK(!ok(rope));
    rope->op_params[1] = 64;
    set_f32(rope, 6, 0.5f);                                            // frequency scaling
    CHECK(!ok(rope));
    set_f32(rope, 6, 1.0f);
    rope->src[1] = p.make(GGML_TYPE_I32, 4);                           // positions != tokens
    CHECK(!ok(rope));
    // --- KV cache: SET_ROWS into, FLASH_ATTN_EXT over, tensors in this backend's KV buffers
    const int D = 64, Hkv = 2, H = 4, T = 24, N = 3;
    ggml_tensor* cache = p.make(GGML_TYPE_F16, Hkv * D, 32);
    cache->buffer = &kbuf;
    ggml_tensor* krows = p.make(GGML_TYPE_F32, Hkv * D, N);
    ggml_tensor* idx = p.make(GGML_TYPE_I64, N);
    ggml_tensor* sr = p.op(GGML_OP_SET_ROWS, GGML_TYPE_F16, {krows, idx}, Hkv * D, 32);
    sr->view_src = cache;
    CHECK(ok(sr) && !ok(sr, 2) && !ok(sr, 1));
    sr->src[1] = p.make(GGML_TYPE_I32, N);                             // 32-bit row indices
    CHECK(!ok(sr));
    sr->src[1] = idx, sr->view_src = nullptr, sr->buffer = &other;     // cache in another backend's buffer
    CHECK(!ok(sr));
    auto cache_view = [&]() {
        ggml_tensor* v = p.make(GGML_TYPE_F16, D, T, Hkv);
        v->nb[1] = static_cast<size_t>(Hkv) * D * 2, v->nb[2] = static_cast<size_t>(D) * 2, v->nb[3] = v->nb[1] * T;
        v->view_src = cache;
        return v;
    };
    ggml_tensor* qf = p.make(GGML_TYPE_F32, D, N, H);
    qf->nb[1] = static_cast<size_t>(H) * D * 4, qf->nb[2] = static_cast<size_t>(D) * 4;
    ggml_tensor* mask = p.make(GGML_TYPE_F16, 32, 8);
    ggml_tensor* fa = p.op(GGML_OP_FLASH_ATTN_EXT, GGML_TYPE_F32, {qf, cache_view(), cache_view(), mask}, D, H, N);
    set_f32(fa, 0, 0.125f);
    CHECK(ok(fa) && ok(fa, 0, 3) && !ok(fa, 0, 2) && !ok(fa, 2));     // token limit, attention switched off
    set_f32(fa, 2, 30.0f);                                             // logit softcap
    CHECK(!ok(fa));
    set_f32(fa, 2, 0.0f), set_f32(fa, 1, 8.0f);                        // ALiBi
    CHECK(!ok(fa));
    set_f32(fa, 1, 0.0f);
    fa->src[4] = mask;                                                 // sinks
    CHECK(!ok(fa));
    fa->src[4] = nullptr;
    ggml_tensor* k_host = cache_view();
    k_host->view_src = nullptr, k_host->buffer = &other;
    fa->src[1] = k_host;                                               // K not in a KV buffer of this backend
    CHECK(!ok(fa));
    fa->src[1] = cache_view();
    fa->src[3] = p.make(GGML_TYPE_F32, 32, 8);                         // f32 mask
    CHECK(!ok(fa));
    std::printf("ok\n");
    return 0;
}

// ---- graph mode ------------------------------------------------------------------------------------------------------
struct Blob {
    std::vector<uint8_t> bytes;
    size_t at = 0;
    template <class T>
    const T* take(size_t n) {
        const T* p = reinterpret_cast<const T*>(bytes.data() + at);
        at += (n * sizeof(T) + 15) / 16 * 16;
        return p;
    }
};

int run_graph(const char* model_path, const char* out_path) {
    Blob blob;
    {
        FILE* f = std::fopen(model_path, "rb");
        CHECK(f);
        std::fseek(f, 0, SEEK_END);
        blob.bytes.resize(static_cast<size_t>(std::ftell(f)));
        std::fseek(f, 0, SEEK_SET);
        CHECK(std::fread(blob.bytes.data(), 1, blob.bytes.size(), f) == blob.bytes.size());
        std::fclose(f);
    }
    // header: hidden, inter, layers, heads, kv_heads, head_dim, vocab, n_tokens, neox, then eps and rope base as floats
    const int* hdr = blob.take<int>(16);
    const int hidden = hdr[0], inter = hdr[1], layers = hdr[2], H = hdr[3], Hkv = hdr[4], D = hdr[5], vocab = hdr[6], n = hdr[7], neox = hdr[8];
    float eps, base;
    std::memcpy(&eps, hdr + 9, 4), std::memcpy(&base, hdr + 10, 4);
    const int qd = H * D, kv = Hkv * D, tp = (n + 7) / 8 * 8;

    ggml_backend_t be = ggml_backend_kernelcore_init();
    CHECK(be && ggml_backend_is_kc(be));
    ggml_backend_dev_t dev = be->device;
    ggml_backend_buffer_type_t wt = dev->iface.get_buffer_type(dev), kt = dev->iface.get_host_buffer_type(dev);
    CHECK(wt && kt);
    ggml_backend_buffer_t wbuf = wt->iface.alloc_buffer(wt, 64u << 20), abuf = wt->iface.alloc_buffer(wt, 64u << 20), kbuf = kt->iface.alloc_buffer(kt, 16u << 20);
    CHECK(wbuf && abuf && kbuf);
    wbuf->usage = GGML_BACKEND_BUFFER_USAGE_WEIGHTS;
    kbuf->iface.clear(kbuf, 0);

    Pool p;
    size_t woff = 0, aoff = 0, koff = 0;
    auto place = [&](ggml_tensor* t, ggml_backend_buffer_t b, size_t& off) {
        t->buffer = b;
        t->data = static_cast<char*>(b->iface.get_base(b)) + off;
        off += (ggml_nbytes(t) + 255) / 256 * 256;
        return t;
    };
    auto weight = [&](ggml_type type, int rows, int k) {
        ggml_tensor* t = place(p.make(type, k, rows), wbuf, woff);
        const size_t bytes = ggml_nbytes(t);
        wbuf->iface.set_tensor(wbuf, t, blob.take<uint8_t>(bytes), 0, bytes);
        return t;
    };
    auto vec = [&](int count) {
        ggml_tensor* t = place(p.make(GGML_TYPE_F32, count), wbuf, woff);
        wbuf->iface.set_tensor(wbuf, t, blob.take<float>(count), 0, static_cast<size_t>(count) * 4);
        return t;
    };
    auto act = [&](ggml_op o, std::vector<ggml_tensor*> src, int64_t n0, int64_t n1 = 1, int64_t n2 = 1) {
        return place(p.op(o, GGML_TYPE_F32, src, n0, n1, n2), abuf, aoff);
    };
    std::vector<ggml_tensor*> nodes;
    auto node = [&](ggml_tensor* t) {
        nodes.push_back(t);
        return t;
    };

    // inputs: embedded tokens, positions, row indices, causal mask
    ggml_tensor* x = place(p.make(GGML_TYPE_F32, hidden, n), abuf, aoff);
    abuf->iface.set_tensor(abuf, x, blob.take<float>(static_cast<size_t>(hidden) * n), 0, static_cast<size_t>(hidden) * n * 4);
    ggml_tensor* pos = place(p.make(GGML_TYPE_I32, n), abuf, aoff);
    ggml_tensor* idx = place(p.make(GGML_TYPE_I64, n), abuf, aoff);
    ggml_tensor* mask = place(p.make(GGML_TYPE_F16, tp, n), abuf, aoff);
    {
        std::vector<int32_t> pv(n);
        std::vector<int64_t> iv(n);
        std::vector<uint16_t> mv(static_cast<size_t>(tp) * n, 0xFC00);  // -inf
        for (int i = 0; i < n; ++i) {
            pv[i] = i, iv[i] = i;
            for (int j = 0; j <= i; ++j) mv[static_cast<size_t>(i) * tp + j] = 0;
        }
        abuf->iface.set_tensor(abuf, pos, pv.data(), 0, pv.size() * 4);
        abuf->iface.set_tensor(abuf, idx, iv.data(), 0, iv.size() * 8);
        abuf->iface.set_tensor(abuf, mask, mv.data(), 0, mv.size() * 2);
    }
    ggml_tensor *first_q4 = nullptr, *first_q6 = nullptr;
    ggml_tensor* resid = x;       // the residual stream
    ggml_tensor* ffn_out = nullptr;
    for (int l = 0; l < layers; ++l) {
        ggml_tensor* wq = weight(GGML_TYPE_Q4_K, qd, hidden);
        ggml_tensor* wk = weight(GGML_TYPE_Q4_K, kv, hidden);
        ggml_tensor* wv = weight(GGML_TYPE_Q6_K, kv, hidden);
        ggml_tensor* wo = weight(GGML_TYPE_Q4_K, hidden, qd);
        ggml_tensor* wg = weight(GGML_TYPE_Q4_K, inter, hidden);
        ggml_tensor* wu = weight(GGML_TYPE_Q4_K, inter, hidden);
        ggml_tensor* wd = weight(GGML_TYPE_Q6_K, hidden, inter);
        ggml_tensor* attn_norm = vec(hidden);
        ggml_tensor* ffn_norm = vec(hidden);
        if (!first_q4) first_q4 = wq, first_q6 = wv;
        ggml_tensor* kc = place(p.make(GGML_TYPE_F16, kv, n), kbuf, koff);
        ggml_tensor* vc = place(p.make(GGML_TYPE_F16, kv, n), kbuf, koff);

        if (ffn_out) resid = node(act(GGML_OP_ADD, {resid, ffn_out}, hidden, n));   // fused with the norm behind it
        ggml_tensor* nrm = node(act(GGML_OP_RMS_NORM, {resid}, hidden, n));
        set_f32(nrm, 0, eps);
        ggml_tensor* cur = node(act(GGML_OP_MUL, {nrm, attn_norm}, hidden, n));
        ggml_tensor* Q = node(act(GGML_OP_MUL_MAT, {wq, cur}, qd, n));
        ggml_tensor* K = node(act(GGML_OP_MUL_MAT, {wk, cur}, kv, n));
        ggml_tensor* V = node(act(GGML_OP_MUL_MAT, {wv, cur}, kv, n));
        auto heads_view = [&](ggml_tensor* t, int nh) {   // [D, nh, n] over the same memory
            ggml_tensor* v = p.op(GGML_OP_RESHAPE, GGML_TYPE_F32, {t}, D, nh, n);
            v->buffer = t->buffer, v->data = t->data, v->view_src = t;
            return node(v);
        };
        auto rope = [&](ggml_tensor* t, int nh) {
            ggml_tensor* r = node(act(GGML_OP_ROPE, {heads_view(t, nh), pos}, D, nh, n));
            r->op_params[1] = D, r->op_params[2] = neox ? GGML_ROPE_TYPE_NEOX : 0;
            set_f32(r, 5, base), set_f32(r, 6, 1.0f), set_f32(r, 7, 0.0f), set_f32(r, 8, 1.0f);
            return r;
        };
        ggml_tensor* Qr = rope(Q, H);
        ggml_tensor* Kr = rope(K, Hkv);
        auto rows_view = [&](ggml_tensor* t) {            // [kv, n]
            ggml_tensor* v = p.op(GGML_OP_RESHAPE, GGML_TYPE_F32, {t}, kv, n);
            v->buffer = t->buffer, v->data = t->data, v->view_src = t;
            return node(v);
        };
        auto set_rows = [&](ggml_tensor* cache, ggml_tensor* src) {
            ggml_tensor* s = p.op(GGML_OP_SET_ROWS, GGML_TYPE_F16, {src, idx}, kv, n);
            s->buffer = cache->buffer, s->data = cache->data, s->view_src = cache;
            return node(s);
        };
        set_rows(kc, rows_view(Kr));
        set_rows(vc, V);
        auto cache_heads = [&](ggml_tensor* cache) {      // [D, n, Hkv] view of the cache rows
            ggml_tensor* v = p.op(GGML_OP_VIEW, GGML_TYPE_F16, {cache}, D, n, Hkv);
            v->nb[1] = static_cast<size_t>(kv) * 2, v->nb[2] = static_cast<size_t>(D) * 2, v->nb[3] = v->nb[1] * n;
            v->buffer = cache->buffer, v->data = cache->data, v->view_src = cache;
            return node(v);
        };
        ggml_tensor* qperm = p.op(GGML_OP_PERMUTE, GGML_TYPE_F32, {Qr}, D, n, H);   // [D, n, H] over [D, H, n]
        qperm->nb[1] = static_cast<size_t>(qd) * 4, qperm->nb[2] = static_cast<size_t>(D) * 4, qperm->nb[3] = qperm->nb[1] * n;
        qperm->buffer = Qr->buffer, qperm->data = Qr->data, qperm->view_src = Qr;
        node(qperm);
        ggml_tensor* fa = node(act(GGML_OP_FLASH_ATTN_EXT, {qperm, cache_heads(kc), cache_heads(vc), mask}, D, H, n));
        set_f32(fa, 0, 1.0f / std::sqrt(static_cast<float>(D)));
        CHECK(dev->iface.supports_op(dev, fa));
        ggml_tensor* flat = p.op(GGML_OP_RESHAPE, GGML_TYPE_F32, {fa}, qd, n);
        flat->buffer = fa->buffer, flat->data = fa->data, flat->view_src = fa;
        node(flat);
        ggml_tensor* attn_out = node(act(GGML_OP_MUL_MAT, {wo, flat}, hidden, n));
        resid = node(act(GGML_OP_ADD, {resid, attn_out}, hidden, n));
        ggml_tensor* n2 = node(act(GGML_OP_RMS_NORM, {resid}, hidden, n));
        set_f32(n2, 0, eps);
        ggml_tensor* c2 = node(act(GGML_OP_MUL, {n2, ffn_norm}, hidden, n));
        ggml_tensor* g = node(act(GGML_OP_MUL_MAT, {wg, c2}, inter, n));
        ggml_tensor* u = node(act(GGML_OP_MUL_MAT, {wu, c2}, inter, n));
        ggml_tensor* sw = node(act(GGML_OP_GLU, {g, u}, inter, n));
        sw->op_params[0] = GGML_GLU_OP_SWIGLU;
        ffn_out = node(act(GGML_OP_MUL_MAT, {wd, sw}, hidden, n));
        for (ggml_tensor* t : {Q, K, V, attn_out, g, u, ffn_out, sw}) CHECK(dev->iface.supports_op(dev, t));
    }
    // last token: residual add, final norm, logits
    ggml_tensor* out_norm = vec(hidden);
    ggml_tensor* lm_head = weight(GGML_TYPE_Q6_K, vocab, hidden);
    auto last_row = [&](ggml_tensor* t) {
        ggml_tensor* v = p.op(GGML_OP_VIEW, GGML_TYPE_F32, {t}, hidden, 1);
        v->buffer = t->buffer, v->data = static_cast<char*>(t->data) + static_cast<size_t>(n - 1) * hidden * 4, v->view_src = t;
        return node(v);
    };
    ggml_tensor* xl = node(act(GGML_OP_ADD, {last_row(resid), last_row(ffn_out)}, hidden, 1));
    ggml_tensor* nl = node(act(GGML_OP_RMS_NORM, {xl}, hidden, 1));
    set_f32(nl, 0, eps);
    ggml_tensor* cl = node(act(GGML_OP_MUL, {nl, out_norm}, hidden, 1));
    ggml_tensor* logits = node(act(GGML_OP_MUL_MAT, {lm_head, cl}, vocab, 1));

    ggml_cgraph graph{static_cast<int>(nodes.size()), nodes.data()};
    CHECK(be->iface.graph_compute(be, &graph) == GGML_STATUS_SUCCESS);
    CHECK(be->iface.graph_compute(be, &graph) == GGML_STATUS_SUCCESS);   // a second run over the same graph: same result, scratch reused

    std::vector<float> lg(vocab);
    abuf->iface.get_tensor(abuf, logits, lg.data(), 0, lg.size() * 4);
    std::vector<uint8_t> b4(ggml_nbytes(first_q4)), b6(ggml_nbytes(first_q6));
    wbuf->iface.get_tensor(wbuf, first_q4, b4.data(), 0, b4.size());
    wbuf->iface.get_tensor(wbuf, first_q6, b6.data(), 0, b6.size());
    FILE* f = std::fopen(out_path, "wb");
    CHECK(f);
    std::fwrite(lg.data(), 4, lg.size(), f);
    std::fwrite(b4.data(), 1, b4.size(), f);
    std::fwrite(b6.data(), 1, b6.size(), f);
    std::fclose(f);
    for (ggml_backend_buffer_t b : {wbuf, abuf, kbuf}) {
        b->iface.free_buffer(b);
        std::free(b);
    }
    be->iface.free(be);
    std::printf("ok %zu nodes\n", nodes.size());
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc >= 2 && std::string(argv[1]) == "rules") return run_rules();
    if (argc >= 4 && std::string(argv[1]) == "graph") return run_graph(argv[2], argv[3]);
    std::printf("usage: %s rules | graph <model.bin> <out.bin>\n", argv[0]);
    return 2;
}
