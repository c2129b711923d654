// Activation stash read-out and the engine-shaped entry points. Included at the end of prichs_moe.cu (it needs the
// handle's definition); everything here is host code around buffers the forward already filled.
//
// The reference's training loops keep, per layer, the vectors of MoEStash / ExpertForwardStash
// (crates/prichs-model/src/moe.rs:32-53): router logits, selection, gates, the shared expert's gate / up / act / out
// and, per routed expert with tokens, its token indices, gate weights and x / gate / up / act / out rows. Its GPU
// path produces them with one engine call per piece (crates/prichs-cuda/src/engine.rs:1917-2239, call order in
// crates/prichs-model/src/model.rs:1327-1408): gpu_moe_forward_shared, forward_gemm(router) + top-k on the host,
// gpu_moe_forward_expert per expert, gpu_moe_finalize_forward. Here one grouped forward computes all of it on the
// device; the engine-shaped calls below start that forward (…_forward_shared) and then hand out views of its result.
#pragma once

namespace {

inline float bf16_bits_to_float(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// Rows [row0, row0 + n) of a bf16 device matrix with `ld` columns -> host floats, columns [col0, col0 + width).
int copy_rows_bf16(const bf16* dev, size_t row0, size_t n, size_t ld, size_t col0, size_t width, float* dst) {
    std::vector<uint16_t> tmp(n * ld);
    CUDA_TRY(cudaMemcpy(tmp.data(), dev + row0 * ld, n * ld * sizeof(uint16_t), cudaMemcpyDeviceToHost));
    for (size_t r = 0; r < n; ++r)
        for (size_t c = 0; c < width; ++c) dst[r * width + c] = bf16_bits_to_float(tmp[r * ld + col0 + c]);
    return PRICHS_OK;
}

// [gate | up] rows in the blocked column order (128 gate then 128 up per 256) -> gate or up [n, f] floats.
int copy_rows_gate_up(const bf16* dev, size_t row0, size_t n, int f, bool want_up, float* dst) {
    const size_t ld = 2 * (size_t)f;
    std::vector<uint16_t> tmp(n * ld);
    CUDA_TRY(cudaMemcpy(tmp.data(), dev + row0 * ld, n * ld * sizeof(uint16_t), cudaMemcpyDeviceToHost));
    for (size_t r = 0; r < n; ++r)
        for (int j = 0; j < f; ++j)
            dst[r * f + j] = bf16_bits_to_float(tmp[r * ld + (size_t)(j >> 7) * 256 + (want_up ? 128 : 0) + (j & 127)]);
    return PRICHS_OK;
}

int stash_check(prichs_moe* h) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if (h->world > 1 || h->mode != PRICHS_MODE_BF16) return fail(PRICHS_ERR_BAD_ARG, "activation stashes exist with all experts local in the bf16 mode");
    if (h->last_T <= 0 || !h->last_a_shared) return fail(PRICHS_ERR_BAD_ARG, "no forward pass has run on this handle");
    if (h->last_chunked) return fail(PRICHS_ERR_BAD_ARG, "the last forward went through host buffers in chunks: only its last chunk's rows remain");
    return PRICHS_OK;
}

}  // namespace

extern "C" {

int prichs_moe_get_expert_assignments(prichs_moe_t* h, int expert, int32_t* token_indices_host, float* weights_host, size_t capacity,
                                      size_t* n_tokens) {
    int rc = stash_check(h);
    if (rc != PRICHS_OK) return rc;
    if (expert < 0 || expert >= h->E || !n_tokens) return fail(PRICHS_ERR_BAD_ARG, "expert index out of range or null count pointer");
    DeviceGuard guard(h->device);
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    const int T = h->last_T;
    std::vector<int> sel((size_t)T * 2);
    std::vector<float> gates((size_t)T * 2);
    CUDA_TRY(cudaMemcpy(sel.data(), h->sel, sel.size() * sizeof(int), cudaMemcpyDeviceToHost));
    CUDA_TRY(cudaMemcpy(gates.data(), h->gates, gates.size() * sizeof(float), cudaMemcpyDeviceToHost));
    // tokens ascending, as the reference fills expert_assignments[e] (moe.rs:121,140); this is also the row order of the
    // expert's segment
    size_t n = 0;
    for (int t = 0; t < T; ++t)
        for (int j = 0; j < h->k; ++j) {
            const int s = sel[(size_t)t * 2 + j];
            if (s >= 0 && (s & 0xff) == expert) {
                if (n < capacity) {
                    if (token_indices_host) token_indices_host[n] = t;
                    if (weights_host) weights_host[n] = gates[(size_t)t * 2 + j];
                }
                ++n;
            }
        }
    *n_tokens = n;
    if (n > capacity && (token_indices_host || weights_host))
        return fail(PRICHS_ERR_CAPACITY, "expert %d has %zu assignments, the arrays hold %zu", expert, n, capacity);
    return PRICHS_OK;
}

int prichs_moe_get_stash(prichs_moe_t* h, int slot, int which, float* host_dst, size_t n_floats) {
    int rc = stash_check(h);
    if (rc != PRICHS_OK) return rc;
    if (slot < 0 || slot > h->E || which < 0 || which > 4 || !host_dst) return fail(PRICHS_ERR_BAD_ARG, "slot, field or destination out of range");
    DeviceGuard guard(h->device);
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    const size_t d = h->d, f = h->f;
    size_t n = h->last_T, row0 = 0, xrow0 = 0;
    if (slot > 0) {
        route::RouteMeta m;
        CUDA_TRY(cudaMemcpy(&m, h->meta, sizeof(m), cudaMemcpyDeviceToHost));
        if (m.overflow) return fail(PRICHS_ERR_CAPACITY, "the forward pass overflowed its permuted region");
        n = (size_t)m.counts[slot - 1];
        xrow0 = (size_t)m.seg_base[slot - 1];
        row0 = (size_t)h->Tcap + xrow0;
    }
    const size_t width = (which == 0 || which == 4) ? d : f;
    if (n_floats != n * width) return fail(PRICHS_ERR_BAD_SHAPE, "this field has %zu x %zu floats, the destination holds %zu", n, width, n_floats);
    if (n == 0) return PRICHS_OK;
    switch (which) {
        case 0:  // x: the rows the expert saw (ExpertForwardStash::x); for the shared expert the layer input
            return slot == 0 ? copy_rows_bf16(h->last_a_shared, 0, n, d, 0, d, host_dst) : copy_rows_bf16(h->xp, xrow0, n, d, 0, d, host_dst);
        case 1:
        case 2:
            if (!h->gu_valid) return fail(PRICHS_ERR_BAD_ARG, "gate / up pre-activations are kept by prichs_moe_forward_train only");
            return copy_rows_gate_up(h->bwd.gu, row0, n, (int)f, which == 2, host_dst);
        case 3: return copy_rows_bf16(h->hbuf, row0, n, f, 0, f, host_dst);
        default: return copy_rows_bf16(reinterpret_cast<const bf16*>(h->ybuf), row0, n, d, 0, d, host_dst);
    }
}

}  // extern "C"

// ---- the engine's call shape (crates/prichs-cuda/src/engine.rs:1917-2239, driven as in model.rs:1327-1408) ----------
extern "C" {

// gpu_moe_forward_shared(normed2, ...): takes the sub-layer's normalised input and starts the forward. Here this one
// call enqueues the WHOLE layer (router and top-2 on the device, shared and routed experts as grouped GEMMs, combine)
// as a training forward, so that every stash the later calls hand out exists. `normed2` is [seq_len, d] fp32 on the
// host (the reference's slice) or, with on_device != 0, a device pointer of element type dtype -- then nothing
// crosses PCIe; the work is then enqueued on the legacy default stream, like all of the reference engine's work. The four outputs (host, any may be null) are the shared expert's stash vectors.
int prichs_engine_moe_forward_shared(prichs_moe_t* h, const void* normed2, int on_device, int dtype, size_t seq_len, float* shared_gate,
                                     float* shared_up, float* shared_act, float* shared_out) {
    if (!h || !normed2) return fail(PRICHS_ERR_BAD_ARG, "null handle or input");
    if (seq_len == 0 || seq_len > (size_t)h->Tmax) return fail(PRICHS_ERR_CAPACITY, "MoE shared dimensions exceed workspace");  // engine.rs:1936
    DeviceGuard guard(h->device);
    int rc = host_path_setup(h);
    if (rc != PRICHS_OK) return rc;
    const int T = (int)seq_len;
    // Host input: the library's own stream, after its own upload. Device input: the legacy default stream, the one the
    // reference's engine does all its work on (engine.rs passes a null stream everywhere), so the forward is ordered
    // after whatever produced the rows there.
    cudaStream_t st = on_device ? nullptr : h->own_stream;
    const void* x_dev = normed2;
    int x_dtype = dtype;
    if (!on_device) {
        CUDA_TRY(cudaMemcpyAsync(h->stage_x, normed2, (size_t)T * h->d * sizeof(float), cudaMemcpyHostToDevice, st));
        x_dev = h->stage_x;
        x_dtype = PRICHS_DTYPE_F32;
    }
    rc = prichs_moe_forward_train(h, x_dev, x_dtype, nullptr, nullptr, 0, h->stage_y, PRICHS_DTYPE_F32, T, st);
    if (rc != PRICHS_OK) return rc;
    float* outs[4] = {shared_gate, shared_up, shared_act, shared_out};
    for (int i = 0; i < 4 && rc == PRICHS_OK; ++i)
        if (outs[i]) rc = prichs_moe_get_stash(h, 0, i + 1, outs[i], (size_t)T * (i == 3 ? h->d : h->f));
    return rc;
}

// forward_gemm(router) + the host loop over top_k_gating_unbiased (model.rs:1340-1361): the router ran on the device
// inside the call above; this hands out its results. selected is [seq_len, top_k] (usize in the reference).
int prichs_engine_moe_routing(prichs_moe_t* h, float* router_logits, size_t* selected_experts, float* gating_weights, size_t seq_len) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if ((int)seq_len != h->last_T) return fail(PRICHS_ERR_BAD_SHAPE, "seq_len differs from the forward started by gpu_moe_forward_shared");
    std::vector<int32_t> sel(selected_experts ? seq_len * (size_t)h->k : 0);
    int rc = prichs_moe_get_routing(h, router_logits, selected_experts ? sel.data() : nullptr, gating_weights, (int)seq_len);
    for (size_t i = 0; i < sel.size(); ++i) selected_experts[i] = (size_t)sel[i];
    return rc;
}

// gpu_moe_forward_expert(token_indices, weights, ...): in the reference this gathers the expert's rows, runs its three
// GEMMs and scatter-adds into the output. The grouped forward has done all of that already, so the call computes
// nothing: it returns the expert's assignment list (which the reference's caller builds on the host) and, where asked,
// copies of its stash rows. *n_tokens == 0 for an expert without tokens (the reference skips those, model.rs:1366).
int prichs_engine_moe_forward_expert(prichs_moe_t* h, int expert, int32_t* token_indices, float* weights, size_t capacity, size_t* n_tokens,
                                     float* exp_x, float* exp_gate, float* exp_up, float* exp_act, float* exp_out) {
    int rc = prichs_moe_get_expert_assignments(h, expert, token_indices, weights, capacity, n_tokens);
    if (rc != PRICHS_OK) return rc;
    const size_t n = *n_tokens;
    float* outs[5] = {exp_x, exp_gate, exp_up, exp_act, exp_out};
    for (int i = 0; i < 5 && rc == PRICHS_OK; ++i)
        if (outs[i]) rc = prichs_moe_get_stash(h, 1 + expert, i, outs[i], n * (size_t)((i == 0 || i == 4) ? h->d : h->f));
    return rc;
}

// gpu_moe_finalize_forward(total_out): downloads the layer's output [seq_len, d] (without the residual: the reference
// adds it on the host, model.rs:1392-1394) and waits for it, like the reference's cudaDeviceSynchronize there.
int prichs_engine_moe_finalize_forward(prichs_moe_t* h, float* total_out, size_t n_floats) {
    if (!h || !total_out) return fail(PRICHS_ERR_BAD_ARG, "null handle or output");
    if (n_floats != (size_t)h->last_T * h->d) return fail(PRICHS_ERR_BAD_SHAPE, "total_out holds %zu floats, the forward produced %zu", n_floats, (size_t)h->last_T * h->d);
    DeviceGuard guard(h->device);
    CUDA_TRY(cudaMemcpyAsync(total_out, h->stage_y, n_floats * sizeof(float), cudaMemcpyDeviceToHost, h->last_stream));
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    int s = 0;
    CUDA_TRY(cudaMemcpy(&s, h->status, sizeof(int), cudaMemcpyDeviceToHost));
    return translate_status(s);
}

}  // extern "C"
