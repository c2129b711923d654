// CPU oracle for the PRICHS MoE-layer forward path.
//
// TEST INFRASTRUCTURE ONLY. This file restates, in plain C++, the arithmetic of the reference's CPU path
// so that the CUDA kernels can be checked against it. Nothing in the shipped library links, loads or
// calls it; only the test-suite, the smoke check and the CPU-baseline leg of the benchmark do.
//
// PARITY UNPINNED BY REFERENCE VECTORS: the reference has no golden vectors, known-answer tests or
// numeric fixtures for this path (its MoE test asserts only lengths and "non-zero",
// crates/prichs-cuda/src/engine.rs:3067-3182), and it cannot be compiled here (no Rust toolchain).
// The restatement is pinned instead by closed-form answers derived from the constants of the
// reference's own fixture (all weights 0.1, x = 0.5; engine.rs:3091-3118) and by an independent
// numpy restatement kept in the test-suite.
//
// What is followed, line by line:
//   crates/prichs-core/src/ops.rs:33-58    matmul_2d, CPU branch: out zero-initialised, for k ascending
//                                          out[j] += a[k] * b[k,j]  (separate multiply and add; this file
//                                          must be compiled with -ffp-contract=off), rows in parallel.
//                                          The opportunistic cuBLAS branch (ops.rs:27-31) is left out.
//   crates/prichs-core/src/ops.rs:137-159  silu(x) = x / (1 + exp(-x)),  swiglu = silu(g) * u
//   crates/prichs-core/src/ops.rs:219-248  top_k_gating_unbiased
//   crates/prichs-core/src/ops.rs:250-267  add_tensors (the residual add of block.rs:67)
//   crates/prichs-model/src/moe.rs:93-211  MoELayer::forward_train
//   crates/prichs-model/src/moe.rs:228-245 MoELayer::update_aux_free_bias
//   crates/prichs-core/src/ops.rs:109-135  rms_norm (the caller's pre-norm of the MoE sub-layer, block.rs:64)
//   crates/prichs-model/src/model.rs:566-766  MoE part of the backward pass (second half of this file)
//
// Build: see oracle/Makefile (g++ -O3 -march=native -ffp-contract=off -pthread; the image has no OpenMP runtime).

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <utility>
#include <vector>

#include <algorithm>
#include <thread>

namespace {

// Row-parallel helper standing in for rayon's par_chunks / par_iter (ops.rs:45-48,150-156): the range is
// cut into contiguous chunks, one per thread. Per-element arithmetic does not depend on the partition.
int g_threads = 0;  // 0 = hardware concurrency

int thread_count() {
    if (g_threads > 0) return g_threads;
    const unsigned hc = std::thread::hardware_concurrency();
    return hc ? (int)hc : 1;
}

template <class F>
void parallel_for(size_t n, F&& body) {
    const size_t nt = std::min<size_t>((size_t)thread_count(), n);
    if (nt <= 1) {
        for (size_t i = 0; i < n; ++i) body(i);
        return;
    }
    std::vector<std::thread> pool;
    pool.reserve(nt);
    for (size_t w = 0; w < nt; ++w) {
        const size_t lo = n * w / nt, hi = n * (w + 1) / nt;
        pool.emplace_back([lo, hi, &body] {
            for (size_t i = lo; i < hi; ++i) body(i);
        });
    }
    for (auto& t : pool) t.join();
}

// ops.rs:33-58. `m == 1` and `m > 1` branches of the reference perform the same per-element arithmetic;
// only the row loop is parallel (rayon par_chunks_exact_mut there, std::thread chunks here).
void matmul_2d(const float* a, const float* b, float* out, size_t m, size_t k1, size_t n) {
    std::memset(out, 0, m * n * sizeof(float));
    parallel_for(m, [=](size_t i) {
        const float* a_row = a + i * k1;
        float* out_row = out + i * n;
        for (size_t k = 0; k < k1; ++k) {
            const float a_val = a_row[k];
            const float* b_row = b + k * n;
            for (size_t j = 0; j < n; ++j) {
                out_row[j] += a_val * b_row[j];
            }
        }
    });
}

// ops.rs:137-140
inline float silu(float x) { return x / (1.0f + std::exp(-x)); }

// ops.rs:142-159
void swiglu(const float* gate, const float* up, float* out, size_t n) {
    const size_t chunk = 4096, nchunks = (n + chunk - 1) / chunk;
    parallel_for(nchunks, [=](size_t c) {
        const size_t hi = std::min(n, (c + 1) * chunk);
        for (size_t i = c * chunk; i < hi; ++i) out[i] = silu(gate[i]) * up[i];
    });
}

// ops.rs:219-248. The reference sorts (index, routing_logit) pairs with the standard library's stable
// sort_by and the comparator  b.1.partial_cmp(&a.1).unwrap_or(Equal)  -- descending, ties keep the lower
// index first, incomparable (NaN) pairs count as equal. For slices of at most 20 elements that stable sort
// is a left-shifting insertion sort, restated here so that the result agrees for every input.
void top_k_gating_unbiased(const float* raw, const float* routing, size_t n, size_t k,
                           size_t* idx_out, float* w_out) {
    std::vector<std::pair<size_t, float>> indexed(n);
    for (size_t i = 0; i < n; ++i) indexed[i] = {i, routing[i]};
    for (size_t i = 1; i < n; ++i) {
        std::pair<size_t, float> tmp = indexed[i];
        size_t j = i;
        // is_less(tmp, indexed[j-1])  <=>  indexed[j-1].1 < tmp.1
        while (j > 0 && indexed[j - 1].second < tmp.second) {
            indexed[j] = indexed[j - 1];
            --j;
        }
        indexed[j] = tmp;
    }
    float max_val = -INFINITY;
    for (size_t i = 0; i < k; ++i) {
        idx_out[i] = indexed[i].first;
        // f32::max semantics: a NaN operand is ignored.
        max_val = std::fmax(max_val, raw[idx_out[i]]);
    }
    float sum_exp = 0.0f;
    for (size_t i = 0; i < k; ++i) {
        const float e = std::exp(raw[idx_out[i]] - max_val);
        w_out[i] = e;
        sum_exp += e;
    }
    const float inv_sum = 1.0f / (sum_exp + 1e-9f);
    for (size_t i = 0; i < k; ++i) w_out[i] = w_out[i] * inv_sum;
}

}  // namespace

extern "C" {

int oracle_num_threads(void) { return thread_count(); }

void oracle_set_num_threads(int n) { g_threads = n > 0 ? n : 0; }

void oracle_matmul_2d(const float* a, const float* b, float* out, size_t m, size_t k, size_t n) {
    matmul_2d(a, b, out, m, k, n);
}

void oracle_swiglu(const float* gate, const float* up, float* out, size_t n) { swiglu(gate, up, out, n); }

void oracle_top_k_gating_unbiased(const float* raw, const float* routing, size_t n, size_t k,
                                  size_t* idx_out, float* w_out) {
    top_k_gating_unbiased(raw, routing, n, k, idx_out, w_out);
}

// ops.rs:250-267 (used for the residual add outside the layer, block.rs:67: x_residual + moe_out).
void oracle_add_tensors(const float* a, const float* b, float* out, size_t n) {
    const size_t chunk = 4096, nchunks = (n + chunk - 1) / chunk;
    parallel_for(nchunks, [=](size_t c) {
        const size_t hi = std::min(n, (c + 1) * chunk);
        for (size_t i = c * chunk; i < hi; ++i) out[i] = a[i] + b[i];
    });
}

// Routing only (moe.rs:114-142): logits = x . W_r; per token  s_e = logit_e + bias_e (+ concept_e for
// e < n_concept); top-k on s, gates from the raw logits. If `logits_in` is non-null the matmul is skipped
// and those logits are used (how the tests check the GPU's selection given the GPU's own fp32 logits).
// Outputs: selected [T*k] (usize), gating [T*k], counts [E] = length of each expert's assignment list.
void oracle_route(const float* x, const float* router, const float* router_bias, const float* concept_bias,
                  size_t n_concept, size_t T, size_t d, size_t E, size_t top_k, const float* logits_in,
                  float* logits_out, size_t* selected, float* gating, size_t* counts) {
    std::vector<float> logits(T * E);
    if (logits_in) {
        std::memcpy(logits.data(), logits_in, T * E * sizeof(float));
    } else {
        matmul_2d(x, router, logits.data(), T, d, E);
    }
    if (logits_out) std::memcpy(logits_out, logits.data(), T * E * sizeof(float));
    for (size_t e = 0; e < E; ++e) counts[e] = 0;
    std::vector<float> adjusted(E);
    for (size_t t = 0; t < T; ++t) {
        const float* raw = logits.data() + t * E;
        for (size_t e = 0; e < E; ++e) {
            float logit = raw[e] + router_bias[e];
            if (concept_bias && e < n_concept) logit += concept_bias[e];
            adjusted[e] = logit;
        }
        top_k_gating_unbiased(raw, adjusted.data(), E, top_k, selected + t * top_k, gating + t * top_k);
        for (size_t j = 0; j < top_k; ++j) counts[selected[t * top_k + j]] += 1;
    }
}

// MoELayer::forward_train (moe.rs:93-211).
//   weights: 1 + 3*(1+E) pointers in the reference's parameter order (model.rs:353-361):
//            router [d,E], shared gate [d,f], up [d,f], down [f,d], then expert e gate, up, down.
//   out [T,d]; optional stash outputs (may be null): logits [T,E], selected [T*k], gating [T*k],
//   counts [E], shared_out [T,d].
// `token_mask` (may be null): when given, only experts' rows for tokens with mask != 0 are computed and
// only those rows of `out` are meaningful -- the layer is token-wise independent once routing is fixed, so
// this gives exact reference values on a sample of a large batch in bounded time. Routing always runs on
// all T tokens.
int oracle_moe_forward_train(const float* const* weights, const float* router_bias, size_t d, size_t f,
                             size_t E, size_t top_k, const float* x, size_t T, const float* concept_bias,
                             size_t n_concept, const unsigned char* token_mask, float* out, float* logits_out,
                             size_t* selected_out, float* gating_out, size_t* counts_out, float* shared_out) {
    if (top_k > E) return -1;
    const float* router = weights[0];
    const float* sg = weights[1];
    const float* su = weights[2];
    const float* sd = weights[3];

    std::vector<size_t> selected(T * top_k), counts(E);
    std::vector<float> gating(T * top_k);
    oracle_route(x, router, router_bias, concept_bias, n_concept, T, d, E, top_k, nullptr, logits_out,
                 selected.data(), gating.data(), counts.data());
    if (selected_out) std::memcpy(selected_out, selected.data(), selected.size() * sizeof(size_t));
    if (gating_out) std::memcpy(gating_out, gating.data(), gating.size() * sizeof(float));
    if (counts_out) std::memcpy(counts_out, counts.data(), counts.size() * sizeof(size_t));

    // Token list to evaluate (all tokens when no mask).
    std::vector<size_t> toks;
    toks.reserve(T);
    for (size_t t = 0; t < T; ++t)
        if (!token_mask || token_mask[t]) toks.push_back(t);
    const size_t n = toks.size();

    // 1. shared expert on the evaluated tokens (moe.rs:103-106); rows are independent, so evaluating a
    //    subset of rows gives the same values as evaluating all of them.
    std::vector<float> xb(n * d), gate(n * f), up(n * f), act(n * f), yo(n * d);
    for (size_t i = 0; i < n; ++i) std::memcpy(&xb[i * d], x + toks[i] * d, d * sizeof(float));
    matmul_2d(xb.data(), sg, gate.data(), n, d, f);
    matmul_2d(xb.data(), su, up.data(), n, d, f);
    swiglu(gate.data(), up.data(), act.data(), n * f);
    matmul_2d(act.data(), sd, yo.data(), n, f, d);
    for (size_t i = 0; i < n; ++i) {
        std::memcpy(out + toks[i] * d, &yo[i * d], d * sizeof(float));
        if (shared_out) std::memcpy(shared_out + toks[i] * d, &yo[i * d], d * sizeof(float));
    }

    // 2./3. binning in token order (moe.rs:121,140), experts ascending, empty bins skipped (moe.rs:149-153),
    //       gather (155-164), expert MLP (166-170), scatter-add out[tok] += w * row (178-184).
    for (size_t e = 0; e < E; ++e) {
        std::vector<size_t> tok_idx;
        std::vector<float> w;
        for (size_t i = 0; i < n; ++i) {
            const size_t t = toks[i];
            for (size_t j = 0; j < top_k; ++j) {
                if (selected[t * top_k + j] == e) {
                    tok_idx.push_back(t);
                    w.push_back(gating[t * top_k + j]);
                }
            }
        }
        const size_t ne = tok_idx.size();
        if (ne == 0) continue;
        const float* wg = weights[4 + 3 * e];
        const float* wu = weights[5 + 3 * e];
        const float* wd = weights[6 + 3 * e];
        std::vector<float> xe(ne * d), ge(ne * f), ue(ne * f), ae(ne * f), ye(ne * d);
        for (size_t i = 0; i < ne; ++i) std::memcpy(&xe[i * d], x + tok_idx[i] * d, d * sizeof(float));
        matmul_2d(xe.data(), wg, ge.data(), ne, d, f);
        matmul_2d(xe.data(), wu, ue.data(), ne, d, f);
        swiglu(ge.data(), ue.data(), ae.data(), ne * f);
        matmul_2d(ae.data(), wd, ye.data(), ne, f, d);
        for (size_t i = 0; i < ne; ++i) {
            const float weight = w[i];
            const float* exp_row = &ye[i * d];
            float* out_row = out + tok_idx[i] * d;
            for (size_t c = 0; c < d; ++c) out_row[c] += weight * exp_row[c];
        }
    }
    return 0;
}

// rms_norm (ops.rs:109-135): per row sum of squares in index order, rms = sqrt(sum/d + eps), inv = 1/rms,
// out = (x * inv) * weight. Used for the MoE sub-layer of the block (block.rs:64): the caller-side step that the
// library can fuse in front of the layer.
void oracle_rms_norm(const float* x, const float* weight, float eps, float* out, size_t rows, size_t d) {
    parallel_for(rows, [=](size_t r) {
        const float* row = x + r * d;
        float sum_sq = 0.0f;
        for (size_t c = 0; c < d; ++c) sum_sq += row[c] * row[c];
        const float rms = std::sqrt(sum_sq / (float)d + eps);
        const float inv_rms = 1.0f / rms;
        for (size_t c = 0; c < d; ++c) out[r * d + c] = row[c] * inv_rms * weight[c];
    });
}

// MoELayer::update_aux_free_bias (moe.rs:228-245).
void oracle_update_aux_free_bias(float* router_bias, size_t E, size_t top_k, const size_t* expert_token_counts,
                                 size_t total_tokens, float gamma) {
    if (total_tokens == 0 || E == 0) return;
    const float target_load = (float)top_k / (float)E;
    for (size_t i = 0; i < E; ++i) {
        const float actual_load = (float)expert_token_counts[i] / (float)total_tokens;
        const float diff = target_load - actual_load;
        router_bias[i] += gamma * diff;
    }
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Backward of the MoE sub-layer: part A of the per-block loop of PrichsModel::forward_backward
// (crates/prichs-model/src/model.rs:566-783). Restated for the next stage of the GPU work (the layer's backward
// pass); the helpers follow
//   crates/prichs-core/src/ops.rs:64-82      matmul_at_b   dW[i,j] += sum_t a[t,i] * b[t,j]   (t ascending, accumulates)
//   crates/prichs-core/src/ops.rs:86-104     matmul_a_bt   dX[i,j]  = sum_c dy[i,c] * w[j,c]  (c ascending, overwrites)
//   crates/prichs-core/src/backward.rs:247-266  swiglu_activation_backward
//   crates/prichs-core/src/backward.rs:269-287  moe_router_unbiased_backward

namespace {

// ops.rs:64-82, CPU branch (rows of dW in parallel, t ascending inside).
void matmul_at_b(const float* a, const float* b, float* dw, size_t m, size_t k, size_t n) {
    parallel_for(k, [=](size_t i) {
        float* dw_row = dw + i * n;
        for (size_t t = 0; t < m; ++t) {
            const float a_val = a[t * k + i];
            const float* b_row = b + t * n;
            for (size_t j = 0; j < n; ++j) dw_row[j] += a_val * b_row[j];
        }
    });
}

// ops.rs:86-104, CPU branch.
void matmul_a_bt(const float* dy, const float* w, float* dx, size_t m, size_t k, size_t n) {
    parallel_for(m, [=](size_t i) {
        const float* dy_row = dy + i * k;
        for (size_t j = 0; j < n; ++j) {
            const float* w_row = w + j * k;
            float dot = 0.0f;
            for (size_t c = 0; c < k; ++c) dot += dy_row[c] * w_row[c];
            dx[i * n + j] = dot;
        }
    });
}

// backward.rs:247-266
void swiglu_activation_backward(const float* d_y, const float* gate_pre_act, const float* up_proj, float* d_gate,
                                float* d_up, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        const float g = gate_pre_act[i], u = up_proj[i], dy = d_y[i];
        const float sig_g = 1.0f / (1.0f + std::exp(-g));
        const float silu_g = g * sig_g;
        const float d_silu_g = sig_g * (1.0f + g * (1.0f - sig_g));
        d_up[i] = dy * silu_g;
        d_gate[i] = dy * u * d_silu_g;
    }
}

// Expert MLP backward shared by the shared expert (model.rs:571-635) and a routed expert (model.rs:664-719):
// given the expert's input rows xe [n,d], its stashed gate/up/act [n,f] and the gradient of its output dy [n,d],
// accumulates dW_gate, dW_up, dW_down and writes dx = d_gate . W_gate^T and dx_tmp = d_up . W_up^T (kept apart:
// the callers add them in the reference's order).
void expert_backward(const float* xe, const float* gate, const float* up, const float* act, const float* dy,
                     const float* wg, const float* wu, const float* wd, float* gwg, float* gwu, float* gwd, float* dx,
                     float* dx_tmp, size_t n, size_t d, size_t f) {
    matmul_at_b(act, dy, gwd, n, f, d);
    std::vector<float> d_act(n * f), d_gate(n * f), d_up(n * f);
    matmul_a_bt(dy, wd, d_act.data(), n, d, f);
    swiglu_activation_backward(d_act.data(), gate, up, d_gate.data(), d_up.data(), n * f);
    matmul_at_b(xe, d_gate.data(), gwg, n, d, f);
    matmul_at_b(xe, d_up.data(), gwu, n, d, f);
    matmul_a_bt(d_gate.data(), wg, dx, n, f, d);
    matmul_a_bt(d_up.data(), wu, dx_tmp, n, f, d);
}

}  // namespace

extern "C" {

// backward.rs:269-287
void oracle_moe_router_unbiased_backward(const float* d_expert_weights, const float* gating_weights,
                                         const size_t* selected_indices, size_t top_k, float* d_router_logits,
                                         size_t E) {
    for (size_t e = 0; e < E; ++e) d_router_logits[e] = 0.0f;
    float weighted_sum = 0.0f;
    for (size_t k = 0; k < top_k; ++k) weighted_sum += gating_weights[k] * d_expert_weights[k];
    for (size_t k = 0; k < top_k; ++k) {
        const float g_i = gating_weights[k];
        const float dl_dg = d_expert_weights[k];
        d_router_logits[selected_indices[k]] = g_i * (dl_dg - weighted_sum);
    }
}

// rmsnorm_backward (backward.rs:94-131): per row, sum of squares and dot(d_out * gamma, x) in index order, then
//   d_gamma[i] += d_out[i] * x[i] * rms_inv,   d_x[i] += gamma[i] * rms_inv * (d_out[i] - x[i] * coeff),
//   coeff = (dot / d) * rms_inv^2.  Both outputs ACCUMULATE: the caller seeds d_x with the gradient that reaches the
// residual connection (model.rs:777-789: d_x_res starts as a clone of the block's output gradient). Rows in order on
// one thread, as in the reference (d_gamma is shared between rows). Note: the x-term of d_x carries gamma[i], which
// the gradient of x * rms_inv * gamma does not (it is -x[i] * coeff * rms_inv); the two agree for gamma = 1, the
// reference's initial norm weight. Restated as the reference computes it.
void oracle_rmsnorm_backward(const float* d_out, const float* x, const float* gamma, float* d_x, float* d_gamma,
                             size_t rows, size_t d_model, float eps) {
    const float inv_d = 1.0f / (float)d_model;
    for (size_t t = 0; t < rows; ++t) {
        const float* x_row = x + t * d_model;
        const float* dout_row = d_out + t * d_model;
        float* dx_row = d_x + t * d_model;
        float sum_sq = 0.0f, dot_dout_gamma_x = 0.0f;
        for (size_t i = 0; i < d_model; ++i) {
            const float xi = x_row[i];
            sum_sq += xi * xi;
            dot_dout_gamma_x += dout_row[i] * gamma[i] * xi;
        }
        const float rms_inv = 1.0f / std::sqrt(sum_sq * inv_d + eps);
        const float coeff = (dot_dout_gamma_x * inv_d) * (rms_inv * rms_inv);
        for (size_t i = 0; i < d_model; ++i) {
            const float xi = x_row[i], di = dout_row[i];
            d_gamma[i] += di * xi * rms_inv;
            dx_row[i] += gamma[i] * rms_inv * (di - xi * coeff);
        }
    }
}

// MoE part of the backward pass of one block (model.rs:566-766), for a layer input x [T,d] (`normed2` there) and
// the gradient d_out [T,d] of the layer's output (`d_moe`). The forward stashes (moe.rs:103-111,166-175,186-208)
// are recomputed here with the same arithmetic as oracle_moe_forward_train.
//   grads: 1 + 3*(1+E) buffers in the parameter order of `weights`; the gradients are ACCUMULATED into them, as the
//          reference accumulates into grads.grads[base_idx + 6 ...] (matmul_at_b adds).
//   d_x [T,d]: overwritten with d_normed2 = shared + routed (experts ascending) + router contributions.
// The router-bias update that the reference performs at this point (model.rs:768-775) is oracle_update_aux_free_bias.
int oracle_moe_backward(const float* const* weights, const float* router_bias, size_t d, size_t f, size_t E,
                        size_t top_k, const float* x, size_t T, const float* concept_bias, size_t n_concept,
                        const float* d_out, float* const* grads, float* d_x) {
    if (top_k > E) return -1;
    const float* router = weights[0];
    std::vector<size_t> selected(T * top_k), counts(E);
    std::vector<float> gating(T * top_k);
    oracle_route(x, router, router_bias, concept_bias, n_concept, T, d, E, top_k, nullptr, nullptr, selected.data(),
                 gating.data(), counts.data());

    std::vector<float> d_normed2(T * d, 0.0f);

    // 1. shared expert (model.rs:571-635)
    {
        std::vector<float> gate(T * f), up(T * f), act(T * f), dx(T * d), dx_tmp(T * d);
        matmul_2d(x, weights[1], gate.data(), T, d, f);
        matmul_2d(x, weights[2], up.data(), T, d, f);
        swiglu(gate.data(), up.data(), act.data(), T * f);
        expert_backward(x, gate.data(), up.data(), act.data(), d_out, weights[1], weights[2], weights[3], grads[1],
                        grads[2], grads[3], dx.data(), dx_tmp.data(), T, d, f);
        for (size_t i = 0; i < T * d; ++i) d_normed2[i] += dx[i] + dx_tmp[i];
    }

    // 2. routed experts, ascending, empty ones skipped (model.rs:637-733)
    std::vector<float> token_expert_scalars(T * E, 0.0f);
    for (size_t e = 0; e < E; ++e) {
        std::vector<size_t> tok_idx;
        std::vector<float> w;
        for (size_t t = 0; t < T; ++t)
            for (size_t j = 0; j < top_k; ++j)
                if (selected[t * top_k + j] == e) {
                    tok_idx.push_back(t);
                    w.push_back(gating[t * top_k + j]);
                }
        const size_t n = tok_idx.size();
        if (n == 0) continue;
        const float *wg = weights[4 + 3 * e], *wu = weights[5 + 3 * e], *wd = weights[6 + 3 * e];
        std::vector<float> xe(n * d), gate(n * f), up(n * f), act(n * f), ye(n * d);
        for (size_t i = 0; i < n; ++i) std::memcpy(&xe[i * d], x + tok_idx[i] * d, d * sizeof(float));
        matmul_2d(xe.data(), wg, gate.data(), n, d, f);
        matmul_2d(xe.data(), wu, up.data(), n, d, f);
        swiglu(gate.data(), up.data(), act.data(), n * f);
        matmul_2d(act.data(), wd, ye.data(), n, f, d);

        // dY_e = gate weight * d_out[token]; scalar = <expert output row, d_out[token]> (model.rs:647-659)
        std::vector<float> d_y_e(n * d);
        for (size_t i = 0; i < n; ++i) {
            const float* d_moe_row = d_out + tok_idx[i] * d;
            const float* exp_out_row = &ye[i * d];
            float dot = 0.0f;
            for (size_t c = 0; c < d; ++c) {
                d_y_e[i * d + c] = w[i] * d_moe_row[c];
                dot += exp_out_row[c] * d_moe_row[c];
            }
            token_expert_scalars[tok_idx[i] * E + e] = dot;
        }
        std::vector<float> dx(n * d), dx_tmp(n * d);
        expert_backward(xe.data(), gate.data(), up.data(), act.data(), d_y_e.data(), wg, wu, wd, grads[4 + 3 * e],
                        grads[5 + 3 * e], grads[6 + 3 * e], dx.data(), dx_tmp.data(), n, d, f);
        // scatter-add into d_normed2 (model.rs:724-732). dY_e above already carries the gate weight, so the
        // reference's input gradient of a routed expert ends up scaled by w twice (w^2 J^T d_out instead of the
        // gradient w J^T d_out); restated as the reference computes it. The weight gradients are not affected.
        for (size_t i = 0; i < n; ++i) {
            float* out_row = &d_normed2[tok_idx[i] * d];
            for (size_t c = 0; c < d; ++c) out_row[c] += w[i] * (dx[i * d + c] + dx_tmp[i * d + c]);
        }
    }

    // 3. router VJP (model.rs:735-766)
    std::vector<float> d_router_logits(T * E, 0.0f);
    for (size_t t = 0; t < T; ++t) {
        std::vector<float> d_expert_weights(top_k);
        for (size_t j = 0; j < top_k; ++j) d_expert_weights[j] = token_expert_scalars[t * E + selected[t * top_k + j]];
        oracle_moe_router_unbiased_backward(d_expert_weights.data(), &gating[t * top_k], &selected[t * top_k], top_k,
                                            &d_router_logits[t * E], E);
    }
    matmul_at_b(x, d_router_logits.data(), grads[0], T, d, E);
    std::vector<float> d_normed2_router(T * d);
    matmul_a_bt(d_router_logits.data(), router, d_normed2_router.data(), T, E, d);
    for (size_t i = 0; i < T * d; ++i) d_normed2[i] += d_normed2_router[i];

    std::memcpy(d_x, d_normed2.data(), T * d * sizeof(float));
    return 0;
}

}  // extern "C"
