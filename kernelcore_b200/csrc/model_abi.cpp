// extern "C" view of the decoder model and decode loop (include/kernelcore_b200.h, kcb_model_*).
#include "../../include/kernelcore_b200.h"

#include "common.cuh"

#include <llm_model.hpp>

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

struct OpenModel {
    llm::KcAllocator alloc;
    llm::Model model;
    llm::Acts acts;
    std::unique_ptr<llm::Backend> backend;
    std::vector<float> logits;
};

thread_local std::string tl_what;

llm::HostMat host_mat(const kcb_mat& m) { return {static_cast<const uint8_t*>(m.blocks), m.rows, m.k, m.fmt == 6}; }

}  // namespace

extern "C" {

int kcb_model_create(const kcb_model_desc* d, int graphs, void** out) {
    if (!d || !out || !d->layers || d->n_layers <= 0) return kcb::KCB_INVALID_VALUE;
    *out = nullptr;
    try {
        llm::HostModel h;
        llm::Config& c = h.cfg;
        c.name = "kcb model";
        c.hidden = d->hidden, c.inter = d->inter, c.layers = d->n_layers, c.heads = d->heads, c.kv_heads = d->kv_heads;
        c.head_dim = d->head_dim, c.vocab = d->vocab, c.max_ctx = d->max_ctx, c.eps = d->eps, c.rope_base = d->rope_base;
        c.neox = d->neox != 0, c.qk_norm = d->qk_norm != 0, c.weights = llm::Weights::Gguf;
        for (int l = 0; l < d->n_layers; ++l) {
            const kcb_layer& s = d->layers[l];
            h.layers.push_back({host_mat(s.wq), host_mat(s.wk), host_mat(s.wv), host_mat(s.wo), host_mat(s.wg), host_mat(s.wu),
                                host_mat(s.wd), s.attn_norm, s.ffn_norm, s.q_norm, s.k_norm});
        }
        h.out_norm = d->out_norm;
        h.lm_head = host_mat(d->lm_head);
        h.rope_ff = d->rope_ff;
        auto om = std::make_unique<OpenModel>();
        om->model = llm::uploadModel(h, om->alloc);
        om->acts = llm::allocActs(om->model.cfg, om->alloc, 1);
        om->backend = llm::makeKcBackend(om->model, 0, graphs != 0);
        om->logits.resize(size_t(c.vocab));
        *out = om.release();
    } catch (const std::exception& e) {
        tl_what = e.what();
        return kcb::KCB_INTERNAL_ERROR;
    }
    return kcb::KCB_SUCCESS;
}

int kcb_model_create_synthetic(const kcb_model_desc* d, int weights, unsigned long long model_seed, unsigned long long start_seed, int graphs,
                               void** out) {
    if (!d || !out || weights < 0 || weights > 3) return kcb::KCB_INVALID_VALUE;
    *out = nullptr;
    try {
        llm::Config c;
        c.name = "kcb synthetic model";
        c.hidden = d->hidden, c.inter = d->inter, c.layers = d->n_layers, c.heads = d->heads, c.kv_heads = d->kv_heads;
        c.head_dim = d->head_dim, c.vocab = d->vocab, c.max_ctx = d->max_ctx, c.eps = d->eps, c.rope_base = d->rope_base;
        c.weights = static_cast<llm::Weights>(weights);
        auto om = std::make_unique<OpenModel>();
        std::vector<llm::Model> built;
        llm::buildModels(c, model_seed, {&om->alloc}, built);
        om->model = std::move(built.front());
        om->acts = llm::allocActs(c, om->alloc, start_seed);
        om->backend = llm::makeKcBackend(om->model, 0, graphs != 0);
        om->logits.resize(size_t(c.vocab));
        *out = om.release();
    } catch (const std::invalid_argument& e) {
        tl_what = e.what();
        return kcb::KCB_INVALID_VALUE;
    } catch (const std::exception& e) {
        tl_what = e.what();
        return kcb::KCB_INTERNAL_ERROR;
    }
    return kcb::KCB_SUCCESS;
}

int kcb_model_decode(void* h, int token, int pos, float* logits_host, int* argmax) {
    auto* om = static_cast<OpenModel*>(h);
    if (!om || (token < 0 && om->model.embed)) return kcb::KCB_INVALID_VALUE;
    try {
        llm::decodeToken(*om->backend, om->model, om->acts, pos, nullptr, token);
        om->backend->finish();
        float* dst = logits_host ? logits_host : om->logits.data();
        om->alloc.download(dst, om->acts.logits, om->logits.size() * sizeof(float));
        if (argmax) {
            int best = 0;
            for (int i = 1; i < int(om->logits.size()); ++i)
                if (dst[i] > dst[best]) best = i;
            *argmax = best;
        }
    } catch (const std::out_of_range& e) {
        tl_what = e.what();
        return kcb::KCB_INVALID_VALUE;
    } catch (const std::exception& e) {
        tl_what = e.what();
        return kcb::KCB_INTERNAL_ERROR;
    }
    return kcb::KCB_SUCCESS;
}

int kcb_model_destroy(void* h) {
    delete static_cast<OpenModel*>(h);
    return kcb::KCB_SUCCESS;
}

const char* kcb_model_last_error(void) { return tl_what.c_str(); }

}  // extern "C"
