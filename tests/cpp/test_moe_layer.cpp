// C++ test of prichs::MoELayer (include/prichs_moe.hpp), written the way the reference tests its GPU MoE path
// (crates/prichs-cuda/src/engine.rs:3067-3134 `test_gpu_moe_forward_backward`: every weight 0.1, every input 0.5,
// lengths and "output non-zero" asserted) -- plus the closed form those constants have, which the reference does
// not assert, the bias update of moe.rs:228-245 and the error behaviour of ops.rs:11-18.
#include <cmath>
#include <cstdio>
#include <cstdlib>

#include "prichs_moe.hpp"

#define REQUIRE(cond)                                                        \
    do {                                                                     \
        if (!(cond)) {                                                       \
            std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                        \
        }                                                                    \
    } while (0)

using prichs::Tensor;

static Tensor filled(std::vector<size_t> dims, float v) {
    Tensor t = Tensor::zeros(dims);
    for (size_t i = 0; i < t.elem_count(); ++i) t.as_f32_slice_mut()[i] = v;
    return t;
}

int main() {
    // The reference fixture uses hidden 4, intermediate 8, 2 experts; the tensor-core tiles need multiples of
    // 256 / 128, so the same constants are used at hidden 256, intermediate 128 with weights scaled to keep the
    // pre-activations at the fixture's 0.2: w_gate = w_up = 0.1 * 4/256, w_down = 0.1 * 8/128.
    const size_t d = 256, f = 128, E = 2, k = 2, T = 2;
    prichs::MoELayer layer(d, f, E, k, /*seed=*/1);
    REQUIRE(layer.router.dims() == (std::vector<size_t>{d, E}));
    REQUIRE(layer.router_bias == std::vector<float>(E, 0.0f));
    REQUIRE(layer.experts.size() == E && layer.top_k == k);
    const float wg = 0.1f * 4.0f / (float)d, wd = 0.1f * 8.0f / (float)f;
    layer.router = filled({d, E}, 0.1f);
    auto fill_expert = [&](prichs::Expert& e) {
        e.gate_proj = filled({d, f}, wg);
        e.up_proj = filled({d, f}, wg);
        e.down_proj = filled({f, d}, wd);
    };
    fill_expert(layer.shared_expert);
    for (auto& e : layer.experts) fill_expert(e);
    layer.mark_weights_changed();

    Tensor x = filled({T, d}, 0.5f);
    auto [out, stash] = layer.forward_train(x, nullptr);
    REQUIRE(out.dims() == (std::vector<size_t>{T, d}));
    REQUIRE(stash.selected_experts.size() == T * k && stash.gating_weights.size() == T * k);
    REQUIRE(stash.router_logits.size() == T * E);
    bool nonzero = false;
    for (float v : out.to_vec()) nonzero = nonzero || std::fabs(v) > 1e-6f;
    REQUIRE(nonzero);  // what the reference asserts
    // closed form: gate = up = 0.2 (in bf16 arithmetic), act = silu(0.2) * 0.2, expert row = 8 * act * 0.1;
    // equal logits pick experts (0, 1) with gates 0.5 each, so out = shared + 0.5 e0 + 0.5 e1 = 2 * row
    const double act = (0.2 / (1.0 + std::exp(-0.2))) * 0.2, row = 8.0 * act * 0.1;
    for (float v : out.to_vec()) REQUIRE(std::fabs(v - 2.0 * row) <= 2e-2 * 2.0 * (2.0 * row));
    for (size_t t = 0; t < T; ++t) {
        REQUIRE(stash.selected_experts[t * k] == 0 && stash.selected_experts[t * k + 1] == 1);  // ties -> lower index
        REQUIRE(std::fabs(stash.gating_weights[t * k] - 0.5f) < 1e-6f);
    }
    REQUIRE(stash.expert_token_counts == (std::vector<size_t>{T, T}));
    REQUIRE(std::fabs(stash.router_logits[0] - 256 * 0.5f * 0.1f) < 1e-3f);
    // the activation stash (moe.rs:32-53): lengths as the reference's test expects them, values from the closed form
    REQUIRE(stash.shared_gate.size() == T * f && stash.shared_up.size() == T * f && stash.shared_act.size() == T * f);
    REQUIRE(stash.shared_out.size() == T * d && stash.routed_stashes.size() == E);
    for (float v : stash.shared_gate) REQUIRE(std::fabs(v - 0.2f) <= 2e-3f);
    for (float v : stash.shared_act) REQUIRE(std::fabs(v - act) <= 2e-2 * act);
    for (float v : stash.shared_out) REQUIRE(std::fabs(v - row) <= 2e-2 * row);
    for (size_t e = 0; e < E; ++e) {
        const prichs::ExpertForwardStash& es = stash.routed_stashes[e];
        REQUIRE(es.expert_idx == e && es.token_indices == (std::vector<size_t>{0, 1}) && es.weights.size() == T);
        REQUIRE(es.x.size() == T * d && es.gate.size() == T * f && es.up.size() == T * f && es.out.size() == T * d);
        for (float v : es.x) REQUIRE(v == 0.5f);
        for (float v : es.up) REQUIRE(std::fabs(v - 0.2f) <= 2e-3f);
        for (float v : es.out) REQUIRE(std::fabs(v - row) <= 2e-2 * row);
    }

    // forward == forward_with_memory(None); a concept bias only moves the selection (moe.rs:128-132)
    Tensor out2 = layer.forward(x);
    REQUIRE(out2.to_vec() == out.to_vec());
    // the fused residual equals the caller's add (block.rs:67)
    Tensor res = filled({T, d}, 0.25f);
    Tensor out3 = layer.forward_with_memory(x, nullptr, &res);
    for (size_t i = 0; i < out3.elem_count(); ++i) REQUIRE(std::fabs(out3.to_vec()[i] - (0.25f + out.to_vec()[i])) < 1e-6f);

    // update_aux_free_bias: b_i += gamma * (k/E - count_i / total), f32 step by step; total_tokens == 0 is a no-op
    layer.router_bias = {0.5f, -0.25f};
    layer.update_aux_free_bias({3, 1}, 4, 0.001f);
    const float t_load = (float)k / (float)E;
    const float e0 = 0.5f + 0.001f * (t_load - 3.0f / 4.0f), e1 = -0.25f + 0.001f * (t_load - 1.0f / 4.0f);
    REQUIRE(layer.router_bias[0] == e0 && layer.router_bias[1] == e1);
    layer.update_aux_free_bias({3, 1}, 0, 0.001f);
    REQUIRE(layer.router_bias[0] == e0 && layer.router_bias[1] == e1);
    // the edited field steers the next forward: a large bias on expert 1 puts it first in the selection
    layer.router_bias = {0.0f, 5.0f};
    auto [o4, s4] = layer.forward_train(x, nullptr);
    REQUIRE(s4.selected_experts[0] == 1 && s4.selected_experts[1] == 0);

    // errors: shape mismatch bails (ops.rs:11-18); top_k > num_experts is rejected (ops.rs:224)
    bool threw = false;
    try {
        layer.forward(filled({T, d + 256}, 0.5f));
    } catch (const prichs::Error& e) {
        threw = e.code == PRICHS_ERR_BAD_SHAPE;
    }
    REQUIRE(threw);
    threw = false;
    try {
        prichs::MoELayer bad(d, f, 1, 2, 1);
        bad.forward(x);
    } catch (const prichs::Error& e) {
        threw = e.code == PRICHS_ERR_BAD_SHAPE;
    }
    REQUIRE(threw);
    std::printf("CPP_OK\n");
    return 0;
}
