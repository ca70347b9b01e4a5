// llm::makeKcBackend: the decode step's operations as CUDA launches on the kc runtime's default stream.
//
// Interface: llm::Backend (llm/llm_model.hpp:152-207 of the reference; its own KcBackend, llm/llm_model.cpp:366-503,
// packs an argument struct per call and launches kernels by name).  Here every call goes straight to the launcher the
// graph decoder uses (ops.h), which buys two things: the residual add, RMSNorm and quantization of addRmsNormQuant are
// one launch instead of two, and nothing is looked up or range-checked per call.  Results are those of the named
// kernels bit for bit (the fused form is tested against the two-kernel form).  All four synthetic formats of
// buildModels are served beside the K-quants.
#include <llm_model.hpp>

#include "common.cuh"
#include "llm_host.hpp"
#include "ops.h"

#include <cmath>
#include <stdexcept>
#include <string>

extern "C" void* kcb_stream_native(void* stream);
extern "C" const char* kcb_error_string(int status);

namespace llm {
namespace {

class CudaBackend final : public Backend {
public:
    CudaBackend(const Model& model, bool graphs) : m_(model), c_(model.cfg), graphs_(graphs), ctx_(model.cfg.max_ctx) {
        stream_ = static_cast<cudaStream_t>(kcb_stream_native(nullptr));
        if (c_.neox) {  // the half-split rotation reads its position and frequency factors from device memory
            host::require(kcMalloc(reinterpret_cast<void**>(&pos_dev_), sizeof(int)), "kcMalloc");
            if (!m_.rope_ff) {
                const std::vector<float> ones(size_t(c_.head_dim / 2), 1.0f);
                host::require(kcMalloc(reinterpret_cast<void**>(&ones_dev_), ones.size() * sizeof(float)), "kcMalloc");
                host::require(kcMemcpy(ones_dev_, ones.data(), ones.size() * sizeof(float), kc::CopyKind::HostToDevice), "kcMemcpy H2D");
            }
        }
    }
    ~CudaBackend() override {
        discardRecording();
        kcFree(pos_dev_);
        kcFree(ones_dev_);
    }

    // ---- per-token set-up ----
    void setScratch(int* q) override { xq_ = q; }
    void setContext(int ctx) override {
        ctx_ = ctx;
        dims_ = c_.attnDims(ctx);
        const auto ints = host::attnDimsInts(dims_);
        host::require(kcMemcpy(m_.attn_dims, ints.data(), sizeof ints, kc::CopyKind::HostToDevice), "kcMemcpy H2D");
        if (pos_dev_) {
            const int pos = ctx - 1;
            host::require(kcMemcpy(pos_dev_, &pos, sizeof pos, kc::CopyKind::HostToDevice), "kcMemcpy H2D");
        }
    }
    void beginToken(bool profiling) override {
        discardRecording();  // a token that threw half way leaves a capture open
        if (graphs_ && !profiling) {
            host::require(kcStreamBeginCapture(nullptr), "kcStreamBeginCapture");
            recording_ = true;
        }
    }
    void endToken() override {
        if (!recording_) return;
        recording_ = false;
        kcGraph_t graph = nullptr;
        host::require(kcStreamEndCapture(nullptr, &graph), "kcStreamEndCapture");
        const kc::Error ran = kcGraphLaunch(graph, nullptr);  // returns when the token's launches have finished
        std::string why;
        if (ran != kc::Error::Success) why = std::string(kcGetErrorString(ran)) + " (" + kcGetLastErrorDetail() + ")";
        kcGraphDestroy(graph);
        if (ran != kc::Error::Success) throw std::runtime_error("kcGraphLaunch: " + why);
    }
    void finish() override { host::require(kcDeviceSynchronize(), "kcDeviceSynchronize"); }

    // ---- matrix times vector ----
    void matvec(const Mat& w, const float* x, float* y) override {
        switch (w.format) {
        case Weights::Q8: return ran("matvec_q8", kcb::matvec_q8w(static_cast<const int8_t*>(w.q), w.s, x, y, w.rows, w.k, stream_));
        case Weights::Q4:
        case Weights::Q4X8:
            return ran("matvec_q4", kcb::matvec_q4w(static_cast<const uint8_t*>(w.q), w.s, x, y, w.rows, w.k, w.format == Weights::Q4X8, stream_));
        default:  // 8-bit activations: quantize into the scratch, where the caller's next matvecQuantized finds them too
            ran("quantize_q8x4", kcb::quantize_q8x4(x, xq_, scales(w.k), w.k / 32, stream_));
            matvecQuantized(w, y);
        }
    }
    void matvecQuantized(const Mat& w, float* y) override {
        const int* xq = xq_;
        const float* xd = scales(w.k);
        switch (w.format) {
        case Weights::Q4K: return ran("matvec_q4k_q8", kcb::matvec_q4k_q8(w.q, xq, xd, y, w.rows, w.k, stream_));
        case Weights::Q6K: return ran("matvec_q6k_q8", kcb::matvec_q6k_q8(w.q, xq, xd, y, w.rows, w.k, stream_));
        case Weights::Q4X8Q8: return ran("matvec_q4x8_q8", kcb::matvec_q4x8_q8(static_cast<const int*>(w.q), xq, xd, y, w.rows, w.k, stream_));
        default: throw std::runtime_error(std::string("no quantized-activation matvec for ") + weightsName(w.format));
        }
    }

    // ---- normalisation, residual, SwiGLU ----
    void rmsNorm(const float* x, const float* w, float* y) override { ran("rms_norm", kcb::rms_norm(x, w, y, c_.hidden, 1, c_.eps, stream_)); }
    void rmsNormRows(float* x, const float* w, int n, int rows) override { ran("rms_norm", kcb::rms_norm(x, w, x, n, rows, c_.eps, stream_)); }
    void addRmsNorm(float* x, const float* t, const float* w, float* y) override {
        ran("add_rms_norm", kcb::add_rms_norm(x, t, w, y, c_.hidden, c_.eps, stream_));
    }
    void addRmsNormQuant(float* x, const float* t, const float* w) override {
        ran("add + norm + quantize", kcb::add_norm_q8_fast(x, t, w, xq_, scales(c_.hidden), c_.hidden, c_.eps, stream_));
    }
    void siluMul(const float* g, const float* u, float* out, int n) override { ran("silu_mul", kcb::silu_mul(g, u, out, size_t(n), stream_)); }
    void siluMulQuant(const float* g, const float* u, int n) override {
        ran("silu_mul_q8x4", kcb::silu_mul_q8(g, u, nullptr, nullptr, xq_, scales(n), n, 1, stream_));
    }
    void add(float* x, const float* t, int n) override { ran("vector_add", kcb::vector_add(x, t, x, size_t(n), stream_)); }

    // ---- attention over the fp32 caches ----
    void rope(float* x, int heads, int pos) override {
        const float log2_base = std::log2(c_.rope_base);
        if (c_.neox) {
            atLastPosition(pos, "rope");
            ran("rope_ggml", kcb::rope_ggml(x, x, pos_dev_, m_.rope_ff ? m_.rope_ff : ones_dev_, c_.head_dim, heads, 1, log2_base, 1, stream_));
        } else {
            const int pairs = c_.head_dim / 2;
            ran("rope", kcb::rope(x, m_.rope_ff, pairs, pos, heads * pairs, log2_base, stream_));
        }
    }
    void appendKv(const float* k, const float* v, float* kt, float* vc, int pos) override {
        atLastPosition(pos, "appendKv");
        ran("kv_append", kcb::kv_append(k, v, kt, vc, dims_.kv_stride, dims_.k_stride, pos, stream_));
    }
    void attnScores(const float* q, const float* k, float* scores) override {
        const float scale = 1.0f / std::sqrt(float(c_.head_dim));
        ran("attn_scores",
            kcb::attn_scores(q, k, scores, dims_.n_heads, dims_.ctx, dims_.head_dim, dims_.group, dims_.ctx_pad, dims_.k_stride, scale, stream_));
    }
    void softmax(float* scores) override { ran("softmax", kcb::softmax(scores, dims_.ctx, dims_.ctx_pad, dims_.n_heads, stream_)); }
    void attnValues(const float* p, const float* v, float* out) override {
        ran("attn_values", kcb::attn_values(p, v, out, dims_.n_heads, dims_.ctx, dims_.head_dim, dims_.kv_stride, dims_.group, dims_.ctx_pad, stream_));
    }

    // ---- data movement (ordered with the launches by the runtime) ----
    void copy(float* dst, const float* src, int n) override {
        host::require(kcMemcpy(dst, src, size_t(n) * sizeof(float), kc::CopyKind::DeviceToDevice), "kcMemcpy D2D");
    }
    void upload(float* dst, const float* src, int n) override {
        host::require(kcMemcpy(dst, src, size_t(n) * sizeof(float), kc::CopyKind::HostToDevice), "kcMemcpy H2D");
    }

private:
    float* scales(int k) const { return scratchScales(xq_, k / 32); }
    static void ran(const char* what, int status) {
        if (status != kcb::KCB_SUCCESS) throw std::runtime_error(std::string(what) + ": " + kcb_error_string(status));
    }
    void atLastPosition(int pos, const char* who) const {
        if (pos != ctx_ - 1) throw std::logic_error(std::string(who) + ": position must be the last of the context");
    }
    void discardRecording() noexcept {
        if (!recording_) return;
        recording_ = false;
        kcGraph_t graph = nullptr;
        if (kcStreamEndCapture(nullptr, &graph) == kc::Error::Success) kcGraphDestroy(graph);
    }

    const Model& m_;
    const Config& c_;
    const bool graphs_;
    bool recording_ = false;
    int ctx_;
    AttnDims dims_{};
    cudaStream_t stream_ = nullptr;
    int* xq_ = nullptr;
    int* pos_dev_ = nullptr;
    float* ones_dev_ = nullptr;
};

}  // namespace

std::unique_ptr<Backend> makeKcBackend(const Model& m, unsigned /*workers*/, bool graphs, bool /*two_rows*/) {
    return std::make_unique<CudaBackend>(m, graphs);
}

}  // namespace llm
