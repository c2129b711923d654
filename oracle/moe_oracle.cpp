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
