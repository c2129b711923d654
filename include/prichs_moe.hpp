// prichs_moe.hpp -- C++ host side of the B200 MoE layer, mirroring the reference's Rust API one to one.
//
// The reference is compiled code (Rust); this header is the compiled-language host shim above the C ABI of
// prichs_moe.h. Names, argument order, meaning and error behaviour follow
//   crates/prichs-core/src/tensor.rs:7-89     Tensor (f32, row-major; from_f32_slice copies, dims(), as_f32_slice())
//   crates/prichs-model/src/moe.rs:6-29       Expert { gate_proj, up_proj, down_proj }
//   crates/prichs-model/src/moe.rs:44-53      MoEStash (routing fields)
//   crates/prichs-model/src/moe.rs:58-245     MoELayer { router, router_bias, shared_expert, experts, top_k },
//                                             new / forward / forward_with_memory / forward_train /
//                                             update_aux_free_bias
// `anyhow::Result` errors become prichs::Error (shape mismatches, like the `bail!` of ops.rs:11-18).
// Header only; link against libprichs_moe.so. Everything is computed on the GPU: there is no CPU path here.
#ifndef PRICHS_MOE_HPP_
#define PRICHS_MOE_HPP_

#include <cmath>
#include <cstdint>
#include <random>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "prichs_moe.h"

namespace prichs {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error("[" + std::to_string(c) + "] " + m), code(c) {}
};

inline void check(int rc) {
    if (rc != PRICHS_OK) throw Error(rc, prichs_last_error());
}

// f32 row-major tensor, the only storage the reference has (tensor.rs:7-29, storage.rs:54-57).
class Tensor {
   public:
    Tensor() = default;
    static Tensor from_f32_slice(const float* data, std::vector<size_t> dims) {
        Tensor t;
        t.dims_ = std::move(dims);
        t.data_.assign(data, data + t.elem_count());
        return t;
    }
    static Tensor from_vec(std::vector<float> data, std::vector<size_t> dims) {
        Tensor t;
        t.dims_ = std::move(dims);
        if (data.size() != t.elem_count()) throw Error(PRICHS_ERR_BAD_SHAPE, "data length does not match the shape");
        t.data_ = std::move(data);
        return t;
    }
    static Tensor zeros(std::vector<size_t> dims) {
        Tensor t;
        t.dims_ = std::move(dims);
        t.data_.assign(t.elem_count(), 0.0f);
        return t;
    }
    // Tensor::randn (tensor.rs:49-63): Box-Muller on two uniforms, u1 clamped at 1e-7. The reference draws from
    // an unseeded thread_rng; here the engine is the caller's.
    template <class Rng>
    static Tensor randn(std::vector<size_t> dims, float mean, float std_, Rng& rng) {
        Tensor t = zeros(std::move(dims));
        std::uniform_real_distribution<float> uni(0.0f, 1.0f);
        for (float& v : t.data_) {
            const float u1 = std::max(uni(rng), 1e-7f), u2 = uni(rng);
            v = mean + std::sqrt(-2.0f * std::log(u1)) * std::cos(2.0f * 3.14159265358979f * u2) * std_;
        }
        return t;
    }
    const std::vector<size_t>& dims() const { return dims_; }
    size_t elem_count() const {
        size_t n = 1;
        for (size_t d : dims_) n *= d;
        return n;
    }
    const float* as_f32_slice() const { return data_.data(); }
    float* as_f32_slice_mut() { return data_.data(); }
    const std::vector<float>& to_vec() const { return data_; }

   private:
    std::vector<float> data_;
    std::vector<size_t> dims_;
};

// moe.rs:6-20. Weights in the reference's x.W layout: gate/up [hidden, intermediate], down [intermediate, hidden].
struct Expert {
    Tensor gate_proj, up_proj, down_proj;
    Expert() = default;
    template <class Rng>
    Expert(size_t hidden_dim, size_t intermediate_dim, Rng& rng) {
        const float s = std::sqrt(2.0f / (float)(hidden_dim + intermediate_dim));
        gate_proj = Tensor::randn({hidden_dim, intermediate_dim}, 0.0f, s, rng);
        up_proj = Tensor::randn({hidden_dim, intermediate_dim}, 0.0f, s, rng);
        down_proj = Tensor::randn({intermediate_dim, hidden_dim}, 0.0f, s, rng);
    }
};

// moe.rs:32-42: what one routed expert contributes to the stash (experts without tokens have no entry).
struct ExpertForwardStash {
    size_t expert_idx = 0;
    std::vector<size_t> token_indices;  // ascending
    std::vector<float> weights;         // gate weights of those tokens
    std::vector<float> x, gate, up, act, out;  // [n, d], [n, f], [n, f], [n, f], [n, d]
};

// moe.rs:44-53. expert_token_counts are the lengths of the expert bins (moe.rs:121,140). The activation vectors are
// filled by forward_train (they are downloaded from the device stash the training forward keeps).
struct MoEStash {
    std::vector<float> router_logits;       // [T, E]
    std::vector<size_t> selected_experts;   // [T * k], slot order = descending selection logit
    std::vector<float> gating_weights;      // [T * k]
    std::vector<float> shared_gate, shared_up, shared_act, shared_out;  // [T, f] x 3, [T, d]
    std::vector<ExpertForwardStash> routed_stashes;
    std::vector<size_t> expert_token_counts;  // [E]
};

class MoELayer {
   public:
    // public fields of the reference (moe.rs:59-63)
    Tensor router;                   // [hidden_dim, num_experts]
    std::vector<float> router_bias;  // [num_experts], starts at zero
    Expert shared_expert;
    std::vector<Expert> experts;
    size_t top_k = 0;

    // MoELayer::new(hidden_dim, intermediate_dim, num_experts, top_k) (moe.rs:67-90)
    MoELayer(size_t hidden_dim, size_t intermediate_dim, size_t num_experts, size_t top_k_, uint64_t seed = std::random_device{}(),
             int mode = PRICHS_MODE_BF16)
        : top_k(top_k_), hidden_(hidden_dim), inter_(intermediate_dim), mode_(mode) {
        std::mt19937_64 rng(seed);
        router = Tensor::randn({hidden_dim, num_experts}, 0.0f, std::sqrt(2.0f / (float)(hidden_dim + num_experts)), rng);
        router_bias.assign(num_experts, 0.0f);
        shared_expert = Expert(hidden_dim, intermediate_dim, rng);
        experts.reserve(num_experts);
        for (size_t i = 0; i < num_experts; ++i) experts.emplace_back(hidden_dim, intermediate_dim, rng);
    }
    MoELayer(const MoELayer&) = delete;
    MoELayer& operator=(const MoELayer&) = delete;
    ~MoELayer() {
        if (h_) prichs_moe_destroy(h_);
    }

    // Call after editing the weight fields so that the next forward uploads them again.
    void mark_weights_changed() { dirty_ = true; }

    // moe.rs:223-225
    Tensor forward(const Tensor& x) { return forward_with_memory(x, nullptr); }

    // moe.rs:214-221. `residual`, when given, fuses the caller's add of block.rs:67: y = residual + moe(x).
    Tensor forward_with_memory(const Tensor& x, const std::vector<float>* starkdb_concept_bias, const Tensor* residual = nullptr) {
        if (x.dims().size() != 2 || x.dims()[1] != hidden_)
            throw Error(PRICHS_ERR_BAD_SHAPE, "Incompatible shapes for matmul: x must be [seq_len, hidden_dim]");
        if (residual && residual->dims() != x.dims()) throw Error(PRICHS_ERR_BAD_SHAPE, "Tensor length mismatch in addition");
        const size_t T = x.dims()[0];
        ensure(T);
        check(prichs_moe_set_bias(h_, router_bias.data(), (int)router_bias.size()));  // the field may have been edited
        Tensor y = Tensor::zeros({T, hidden_});
        const float* cb = starkdb_concept_bias ? starkdb_concept_bias->data() : nullptr;
        const int ncb = starkdb_concept_bias ? (int)starkdb_concept_bias->size() : 0;
        check(prichs_moe_forward_host(h_, x.as_f32_slice(), residual ? residual->as_f32_slice() : nullptr, cb, ncb,
                                      y.as_f32_slice_mut(), (int)T));
        last_T_ = T;
        return y;
    }

    // moe.rs:93-211. Runs the engine-shaped call sequence (the order of model.rs:1327-1408): one grouped training
    // forward on the device, then views of its result.
    std::pair<Tensor, MoEStash> forward_train(const Tensor& x, const std::vector<float>* starkdb_concept_bias) {
        if (starkdb_concept_bias || mode_ != PRICHS_MODE_BF16) {  // the engine call shape has no concept bias argument
            Tensor y0 = forward_with_memory(x, starkdb_concept_bias);
            return {std::move(y0), routing_stash()};
        }
        if (x.dims().size() != 2 || x.dims()[1] != hidden_)
            throw Error(PRICHS_ERR_BAD_SHAPE, "Incompatible shapes for matmul: x must be [seq_len, hidden_dim]");
        const size_t T = x.dims()[0], E = experts.size();
        ensure(T);
        check(prichs_moe_set_bias(h_, router_bias.data(), (int)router_bias.size()));
        MoEStash st;
        st.shared_gate.resize(T * inter_);
        st.shared_up.resize(T * inter_);
        st.shared_act.resize(T * inter_);
        st.shared_out.resize(T * hidden_);
        check(prichs_engine_moe_forward_shared(h_, x.as_f32_slice(), 0, PRICHS_DTYPE_F32, T, st.shared_gate.data(), st.shared_up.data(),
                                               st.shared_act.data(), st.shared_out.data()));
        last_T_ = T;
        st.router_logits.resize(T * E);
        st.selected_experts.resize(T * top_k);
        st.gating_weights.resize(T * top_k);
        check(prichs_engine_moe_routing(h_, st.router_logits.data(), st.selected_experts.data(), st.gating_weights.data(), T));
        st.expert_token_counts.assign(E, 0);
        for (size_t e = 0; e < E; ++e) {
            size_t n = 0;
            check(prichs_engine_moe_forward_expert(h_, (int)e, nullptr, nullptr, 0, &n, nullptr, nullptr, nullptr, nullptr, nullptr));
            st.expert_token_counts[e] = n;
            if (n == 0) continue;  // model.rs:1366
            ExpertForwardStash es;
            es.expert_idx = e;
            std::vector<int32_t> idx(n);
            es.weights.resize(n);
            es.x.resize(n * hidden_);
            es.out.resize(n * hidden_);
            es.gate.resize(n * inter_);
            es.up.resize(n * inter_);
            es.act.resize(n * inter_);
            check(prichs_engine_moe_forward_expert(h_, (int)e, idx.data(), es.weights.data(), n, &n, es.x.data(), es.gate.data(),
                                                   es.up.data(), es.act.data(), es.out.data()));
            es.token_indices.assign(idx.begin(), idx.end());
            st.routed_stashes.push_back(std::move(es));
        }
        Tensor y = Tensor::zeros({T, hidden_});
        check(prichs_engine_moe_finalize_forward(h_, y.as_f32_slice_mut(), T * hidden_));
        return {std::move(y), std::move(st)};
    }

    // moe.rs:228-245: b_i += gamma * (top_k/E - counts[i]/total_tokens); no-op when total_tokens == 0.
    void update_aux_free_bias(const std::vector<size_t>& expert_token_counts, size_t total_tokens, float gamma) {
        if (expert_token_counts.size() != experts.size())
            throw Error(PRICHS_ERR_BAD_SHAPE, "expert_token_counts length differs from the number of experts");
        ensure(1);
        check(prichs_moe_set_bias(h_, router_bias.data(), (int)router_bias.size()));
        check(prichs_moe_update_aux_free_bias(h_, expert_token_counts.data(), (int)expert_token_counts.size(), total_tokens, gamma));
        check(prichs_moe_get_bias(h_, router_bias.data(), (int)router_bias.size()));
    }

   private:
    MoEStash routing_stash() {
        MoEStash st;
        const size_t T = last_T_, E = experts.size();
        st.router_logits.resize(T * E);
        st.gating_weights.resize(T * top_k);
        std::vector<int32_t> sel(T * top_k);
        if (T) check(prichs_moe_get_routing(h_, st.router_logits.data(), sel.data(), st.gating_weights.data(), (int)T));
        st.selected_experts.assign(sel.begin(), sel.end());
        std::vector<int64_t> counts(E, 0);
        check(prichs_moe_get_counts(h_, counts.data(), (int)E));
        st.expert_token_counts.assign(counts.begin(), counts.end());
        return st;
    }

    void ensure(size_t T) {
        if (!h_ || T > cap_) {
            if (h_) prichs_moe_destroy(h_);
            h_ = nullptr;
            prichs_moe_config_t cfg{};
            cfg.hidden_dim = (int)hidden_;
            cfg.intermediate_dim = (int)inter_;
            cfg.num_experts = (int)experts.size();
            cfg.top_k = (int)top_k;
            cfg.max_tokens = (int)std::max<size_t>(T, 1);
            cfg.mode = mode_;
            cfg.device = -1;
            cfg.ep_world = 1;
            check(prichs_moe_create(&cfg, &h_));
            cap_ = (size_t)cfg.max_tokens;
            dirty_ = true;
        }
        if (dirty_) {
            const std::vector<size_t> dr = {hidden_, experts.size()}, dg = {hidden_, inter_}, dd = {inter_, hidden_};
            auto shape_ok = [&](const Expert& e) { return e.gate_proj.dims() == dg && e.up_proj.dims() == dg && e.down_proj.dims() == dd; };
            bool ok = router.dims() == dr && shape_ok(shared_expert) && router_bias.size() == experts.size();
            for (const Expert& e : experts) ok = ok && shape_ok(e);
            if (!ok) throw Error(PRICHS_ERR_BAD_SHAPE, "Incompatible shapes for matmul: a weight tensor does not match the layer dimensions");
            std::vector<const float*> ptrs = {router.as_f32_slice(), shared_expert.gate_proj.as_f32_slice(),
                                              shared_expert.up_proj.as_f32_slice(), shared_expert.down_proj.as_f32_slice()};
            for (const Expert& e : experts) {
                ptrs.push_back(e.gate_proj.as_f32_slice());
                ptrs.push_back(e.up_proj.as_f32_slice());
                ptrs.push_back(e.down_proj.as_f32_slice());
            }
            check(prichs_moe_upload_weights(h_, ptrs.data(), (int)ptrs.size()));
            dirty_ = false;
        }
    }

    size_t hidden_, inter_;
    int mode_;
    prichs_moe_t* h_ = nullptr;
    size_t cap_ = 0, last_T_ = 0;
    bool dirty_ = true;
};

}  // namespace prichs

#endif  // PRICHS_MOE_HPP_
