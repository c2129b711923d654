/*
 * prichs_moe.h -- C ABI of the B200 (sm_100a) MoE-layer forward library, libprichs_moe.so.
 *
 * The library replaces ONE path of DanyaStark553/PRICHS: the forward pass of `MoELayer`
 * (crates/prichs-model/src/moe.rs:58-246) and the kernels and engine calls the reference's GPU path uses
 * for it (crates/prichs-cuda/src/kernels.cu:444-457,888-924; crates/prichs-cuda/src/engine.rs:1917-2239).
 * The convention follows the reference's own FFI (crates/prichs-cuda/src/engine.rs:89-272): plain
 * pointers, size_t/int dimensions, the CUDA stream passed as `void*`. Unlike the reference's `launch_*`
 * wrappers, which return void and drop every error, each function here returns an int status.
 *
 * Data layout. Every matrix is row-major. Weights are handed over in the reference's "x . W" layout:
 * router [d,E], gate_proj and up_proj [d,f], down_proj [f,d] (moe.rs:16-18,73-74). Activations are [T,d].
 *
 * There is no CPU fallback: without a CUDA device every call that touches the device returns
 * PRICHS_ERR_CUDA.
 */
#ifndef PRICHS_MOE_H_
#define PRICHS_MOE_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define PRICHS_API __attribute__((visibility("default")))
#else
#define PRICHS_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------------------------------- */
#define PRICHS_OK 0
#define PRICHS_ERR_BAD_SHAPE (-1) /* the reference bails on shape mismatch in matmul_2d, ops.rs:11-18    */
#define PRICHS_ERR_CAPACITY (-2)  /* more tokens / rows than the handle was created for                   */
#define PRICHS_ERR_CUDA (-3)      /* a CUDA runtime or driver call failed (or no device)                  */
#define PRICHS_ERR_COMM (-4)      /* expert-parallel exchange failed or is not initialised                */
#define PRICHS_ERR_TIMEOUT (-5)   /* a bounded device-side wait gave up (status word set by a kernel)     */
#define PRICHS_ERR_BAD_ARG (-6)   /* null pointer, unknown dtype, weights not uploaded, ...               */
#define PRICHS_ERR_BOUNDS (-7)    /* checking build only: a kernel computed a row index outside its buffer  */

/* element types at the boundary (activations x / residual / y) */
#define PRICHS_DTYPE_F32 0
#define PRICHS_DTYPE_BF16 1

/* compute modes */
#define PRICHS_MODE_BF16 0 /* bf16 operands, fp32 accumulate on the tensor cores                        */
#define PRICHS_MODE_F32 1  /* fp32 fidelity: every operand split into bf16 hi+lo parts, three products   */

typedef struct prichs_moe prichs_moe_t;

/* Mirrors the arguments of MoELayer::new(hidden_dim, intermediate_dim, num_experts, top_k)
 * (moe.rs:67-72) plus what a device handle needs to size its buffers once. */
typedef struct prichs_moe_config {
    int hidden_dim;       /* d; multiple of 256                                                        */
    int intermediate_dim; /* f; multiple of 128                                                        */
    int num_experts;      /* E routed experts, 1..8 (one shared expert is always present, moe.rs:76)   */
    int top_k;            /* 1 or 2, <= num_experts                                                    */
    int max_tokens;       /* largest T a forward call may pass                                         */
    int mode;             /* PRICHS_MODE_*                                                             */
    int device;           /* CUDA device ordinal, or -1 for the current device                         */
    int ep_world;         /* expert-parallel ranks (1 = all experts local); must divide num_experts    */
    int ep_rank;          /* this rank, 0..ep_world-1; owns experts [rank*E/world, (rank+1)*E/world)   */
    int ep_max_recv_rows; /* capacity of the receive side in rows (0 = worst case ep_world*max_tokens*top_k) */
    int ep_waves;         /* expert-parallel only: the batch is cut into this many token waves (1..4) whose
                             exchanges overlap the other waves' GEMMs; 0 = choose from max_tokens. Must be the
                             same on every rank.                                                          */
    /* ---- tuning. Zero selects the default everywhere, so a zero-initialised tail is the product path; the
     *      other values exist so that the alternatives can be measured and tested against each other. The
     *      library reads no environment variable. ------------------------------------------------------ */
    int route_kernel;     /* all experts local, bf16 rows: 0 = choose (single pass from 1024 tokens up), 1 = route,
                             place and dispatch in one pass (one kernel), 2 = router / scan / dispatch launches   */
    int scan_placement;   /* three-launch path: 0 = prefix sums at the router's tail under 1024 tokens, else a
                             launch of their own; 1 = always at the tail; 2 = always their own launch          */
    int separate_prenorm; /* block entry point: 1 = the RMSNorm runs as its own launch (0: folded into the router)  */
    int gemm_kernel;      /* 0 = CTA-pair kernel (tcgen05 cta_group::2, 256-row tiles; batches under 1024 tokens run
                             on the one-CTA kernel), 1 = one-CTA kernel for every batch size, 2 = as 0 with the down
                             projection of small batches on 128-column tiles (faster for one stream of dependent
                             layers, slower when several layers overlap)                                           */
    int pdl;              /* programmatic dependent launch between the kernels of a single-GPU forward (a kernel's
                             set-up overlaps the tail of its predecessor): 0 / 1 = on, 2 = off                     */
    int host_chunk_tokens;/* host-buffer entry point: tokens per pipelined chunk (0 = choose from T)                */
    int router_ctas_per_sm; /* router grid cap in CTAs per SM (0 = default; -1 = one CTA per 16-token tile)         */
    int ep_reserve_sms;   /* expert parallel: SMs the GEMM launches leave to the exchange kernels (0 = default 20,
                             -1 = none)                                                                            */
    int ep_shared_copy_sms; /* expert parallel: 1 = dispatch / combine may share SMs with GEMM CTAs                 */
    int ep_combine_mode;  /* expert parallel: which combine launches keep off the GEMM SMs: 0 = all but the last
                             wave's (default), 1 = all, 2 = none                                                   */
    int ep_dispatch_kernel; /* expert parallel: 0 = rows travel as bulk copies through shared memory on the reserved SMs,
                             1 = one warp per token with 16-byte loads and stores                                  */
    int ep_timeout_ms;    /* expert parallel: how long prichs_moe_sync_status waits for a forward before it aborts the
                             communicators and returns PRICHS_ERR_COMM (0 = 60 s)                                  */
    int ep_nccl_barriers; /* expert parallel: 1 = "rows landed" / "outputs ready" are NCCL all-gathers used as barriers
                             (0: readiness flags the ranks write into each other's memory over NVLink)           */
} prichs_moe_config_t;

/* ---- lifetime ------------------------------------------------------------------------------------ */

/* Replaces MoELayer::new (moe.rs:67-90) and the engine's buffer set-up (engine.rs:363-649): allocates the
 * weights, the workspace for max_tokens and the TMA descriptors. Weights start undefined, the router bias
 * at zero (moe.rs:75). */
PRICHS_API int prichs_moe_create(const prichs_moe_config_t* cfg, prichs_moe_t** out_handle);

/* Replaces Drop for GpuModelEngine (engine.rs:2792-2854). */
PRICHS_API int prichs_moe_destroy(prichs_moe_t* h);

/* Replaces GpuModelEngine::upload_weights (engine.rs:668-689) for the layer's tensors. `host_ptrs` holds
 * 1 + 3*(1+E) fp32 host arrays in the reference's parameter order (model.rs:353-361): router [d,E]; shared
 * gate [d,f], up [d,f], down [f,d]; then for each routed expert gate, up, down. In expert-parallel mode
 * the pointers of experts this rank does not own may be null. The arrays are repacked once on the device
 * (transposed to K-major, gate and up interleaved in 128-column blocks, rounded to bf16 -- or split into
 * bf16 hi/lo parts in PRICHS_MODE_F32). */
PRICHS_API int prichs_moe_upload_weights(prichs_moe_t* h, const float* const* host_ptrs, int n_ptrs);

/* The public field MoELayer::router_bias (moe.rs:60): read and write, host side, length E. */
PRICHS_API int prichs_moe_set_bias(prichs_moe_t* h, const float* host_bias, int n);
PRICHS_API int prichs_moe_get_bias(prichs_moe_t* h, float* host_bias, int n);

/* ---- forward ------------------------------------------------------------------------------------- */

/* Replaces MoELayer::forward / forward_with_memory (moe.rs:214-225) and the engine call sequence
 * gpu_moe_forward_shared + forward_gemm(router) + host top-k + gpu_moe_forward_expert (per expert) +
 * gpu_moe_finalize_forward (engine.rs:1917-2239, model.rs:1327-1408) with device-resident activations.
 *   x_dev        [T,d] device pointer, element type x_dtype
 *   resid_dev    optional [T,d] device pointer (same element type as x): when non-null the caller's
 *                residual add of block.rs:67 is fused, y = resid + moe(x); when null y = moe(x)
 *   concept_bias optional HOST array (the reference's Option<&[f32]>, moe.rs:96,128-132): added to the
 *                selection logit of expert e for e < n_concept; copied by value, no device pointer needed
 *   y_dev        [T,d] device pointer, element type y_dtype
 * All work is enqueued on `stream` (a cudaStream_t; null = legacy default stream, as in the reference).
 * No allocation and no host synchronisation happen inside. One handle is one stream-ordered context: calls
 * on the same handle must not overlap; independent handles are independent. */
PRICHS_API int prichs_moe_forward(prichs_moe_t* h, const void* x_dev, int x_dtype, const void* resid_dev,
                       const float* concept_bias, int n_concept, void* y_dev, int y_dtype, int T,
                       void* stream);

/* MoELayer::forward_train (moe.rs:93-211): the same forward, which also keeps what the backward pass needs. The
 * reference copies gate / up / act / out of every expert into host vectors on every call, also from forward()
 * (moe.rs:108-111,172-175,186-208,219); here the stash is this separate entry point and stays on the device:
 * act (H) and out (Y) are the forward's own buffers, x is the permuted-row buffer, and the [gate | up]
 * pre-activations -- which the plain forward never writes to memory -- are stored by the first GEMM's epilogue (bf16).
 * prichs_moe_backward after this call skips its recomputation of them; prichs_moe_get_stash and
 * prichs_moe_get_expert_assignments hand the pieces out in the reference's shapes. All experts local, bf16 mode;
 * the stash buffer (rows x 2f bf16) is allocated by the first call. */
PRICHS_API int prichs_moe_forward_train(prichs_moe_t* h, const void* x_dev, int x_dtype, const void* resid_dev,
                                        const float* concept_bias, int n_concept, void* y_dev, int y_dtype, int T,
                                        void* stream);

/* One stash vector of the last forward as host fp32, in the reference's shape (MoEStash / ExpertForwardStash,
 * moe.rs:32-53). slot 0 = shared expert (n = T rows), slot 1 + e = routed expert e (n = its assignment count, rows in
 * ascending token order). which: 0 x [n,d], 1 gate [n,f], 2 up [n,f], 3 act [n,f], 4 out [n,d]. n_floats must equal
 * the field's size. gate and up exist after prichs_moe_forward_train only. Waits for the forward. */
PRICHS_API int prichs_moe_get_stash(prichs_moe_t* h, int slot, int which, float* host_dst, size_t n_floats);

/* ExpertForwardStash::token_indices / weights of routed expert e for the last forward (the reference's
 * expert_assignments[e], moe.rs:121,140): token indices ascending and their gate weights. *n_tokens receives the
 * count; the arrays (may be null to ask for the count only) hold `capacity` entries. */
PRICHS_API int prichs_moe_get_expert_assignments(prichs_moe_t* h, int expert, int32_t* token_indices_host, float* weights_host,
                                                 size_t capacity, size_t* n_tokens);

/* ---- the engine's call shape ---------------------------------------------------------------------
 * Replacements for GpuModelEngine::gpu_moe_forward_shared / gpu_moe_forward_expert / gpu_moe_finalize_forward
 * (crates/prichs-cuda/src/engine.rs:1917-2239) and for forward_gemm(router) + the host top-k loop between them, to
 * be called in the order of crates/prichs-model/src/model.rs:1327-1408 (training) or :1124-1182 (forward_gpu_only):
 *   1. prichs_engine_moe_forward_shared  takes normed2 [seq_len,d] (host fp32 slice as in the reference, or a device
 *      pointer with on_device = 1; the work then goes to the legacy default stream, where the reference's engine does
 *      all of its work) and enqueues the WHOLE layer as a training forward: router and top-2 on the device,
 *      shared and routed experts as grouped GEMMs, combine. Optional outputs: the shared expert's stash vectors.
 *   2. prichs_engine_moe_routing         router_logits [seq_len,E], selected_experts [seq_len,k] (usize), gating
 *      weights [seq_len,k]: what the reference computes with an Sgemm round trip and top_k_gating_unbiased on the host.
 *   3. prichs_engine_moe_forward_expert  per expert, ascending: computes nothing (the grouped forward already ran the
 *      expert); returns its token indices and weights and, where asked, its stash rows x, gate, up, act, out.
 *   4. prichs_engine_moe_finalize_forward downloads the layer output [seq_len,d] (no residual) and waits.
 * With on_device = 1 and null stash pointers nothing but the final output crosses PCIe. */
PRICHS_API int prichs_engine_moe_forward_shared(prichs_moe_t* h, const void* normed2, int on_device, int dtype, size_t seq_len,
                                                float* shared_gate, float* shared_up, float* shared_act, float* shared_out);
PRICHS_API int prichs_engine_moe_routing(prichs_moe_t* h, float* router_logits, size_t* selected_experts, float* gating_weights,
                                         size_t seq_len);
PRICHS_API int prichs_engine_moe_forward_expert(prichs_moe_t* h, int expert, int32_t* token_indices, float* weights, size_t capacity,
                                                size_t* n_tokens, float* exp_x, float* exp_gate, float* exp_up, float* exp_act,
                                                float* exp_out);
PRICHS_API int prichs_engine_moe_finalize_forward(prichs_moe_t* h, float* total_out, size_t n_floats);

/* The MoE sub-layer of the reference's block in one call (crates/prichs-model/src/block.rs:64-67):
 *   y = x_res + MoELayer::forward_with_memory(rms_norm(x_res, norm_weight, eps), concept_bias)
 * with rms_norm as in crates/prichs-core/src/ops.rs:109-135 (the engine's counterpart is gpu_rmsnorm_forward,
 * crates/prichs-cuda/src/kernels.cu:329-362). x_res_dev [T,d] of element type x_dtype is both the input of the
 * norm and the residual; norm_weight_dev is [d] fp32 on the device. hidden_dim <= 2048. */
PRICHS_API int prichs_moe_block_forward(prichs_moe_t* h, const void* x_res_dev, int x_dtype, const float* norm_weight_dev,
                                        float eps, const float* concept_bias, int n_concept, void* y_dev, int y_dtype, int T,
                                        void* stream);

/* The same call with HOST buffers, the shape in which the reference's MoELayer::forward(&Tensor) -> Tensor
 * is used (f32 row-major slices, tensor.rs:14-29): copies x (and resid) to the device, runs the forward,
 * copies y back and waits for it. Pinned host memory makes the copies asynchronous; pageable memory works.
 * Batches of 4096 tokens or more are fed through in chunks on three streams (upload, kernels, download
 * overlap); the results, the routing stash and the counts are identical to one pass. An expert-parallel handle cuts
 * every rank's batch into max_tokens / 8192 (at most 8) chunks, each a collective forward: every rank runs the same
 * number of chunks whatever its own T, which must be at least 16 tokens per chunk. */
PRICHS_API int prichs_moe_forward_host(prichs_moe_t* h, const float* x_host, const float* resid_host,
                            const float* concept_bias, int n_concept, float* y_host, int T);

/* Waits for the handle's last stream and returns the device status word of the work enqueued so far:
 * PRICHS_OK, PRICHS_ERR_CAPACITY (an expert's segment did not fit) or PRICHS_ERR_TIMEOUT (a bounded wait
 * inside a kernel gave up); a reported error is cleared. After PRICHS_ERR_CAPACITY the outputs of that forward
 * are undefined (the exchange was skipped on every rank) but the handle stays usable. The reference has no
 * counterpart: its launches report nothing. */
PRICHS_API int prichs_moe_sync_status(prichs_moe_t* h);

/* ---- routing results of the last forward (the MoEStash fields, moe.rs:44-53) ---------------------- */

/* counts[e] = number of (token, slot) assignments expert e received in the last forward on this rank
 * (the lengths of expert_assignments, moe.rs:121,140). Waits for the handle's last stream. */
PRICHS_API int prichs_moe_get_counts(prichs_moe_t* h, int64_t* counts_host, int n);

/* router_logits [T,E] fp32, selected_experts [T,k] int32, gating_weights [T,k] fp32 of the last forward;
 * any pointer may be null. Waits for the handle's last stream. */
PRICHS_API int prichs_moe_get_routing(prichs_moe_t* h, float* logits_host, int32_t* selected_host, float* gating_host,
                           int T);

/* ---- aux-loss-free bias update ------------------------------------------------------------------- */

/* Backward of the last forward on this handle: the MoE section of the reference's per-block backward pass
 * (crates/prichs-model/src/model.rs:566-766; helpers crates/prichs-core/src/ops.rs:64-104 matmul_at_b / matmul_a_bt,
 * crates/prichs-core/src/backward.rs:247-287 swiglu_activation_backward / moe_router_unbiased_backward; the engine's
 * counterparts are gpu_moe_backward_* in crates/prichs-cuda/src/engine.rs:2242-2789).
 *   x_dev     the layer input of that forward, [T,d] of x_dtype, unchanged since (`normed2` in the reference)
 *   dy_dev    gradient of the layer output, [T,d] of dy_dtype (`d_moe`)
 *   dx_dev    [T,d] fp32, overwritten with the gradient of the layer input (`d_normed2`): shared expert + routed
 *             experts in ascending order + router. As in the reference, a routed expert's input gradient carries the
 *             gate weight twice (dY_e = w * d_out, model.rs:647-656, and w * dX_e in the scatter-add, model.rs:724-732)
 *   grads_dev n_grads = 1 + 3 * (1 + E) device pointers to fp32 buffers in the order and [in, out] layouts of
 *             prichs_moe_upload_weights (router [d,E], shared gate [d,f], up [d,f], down [f,d], expert e ...); the
 *             gradients are ADDED to them (the reference's matmul_at_b accumulates). Null entries are skipped; a null
 *             array computes dx only. Experts that received no token are left untouched (model.rs:641-643).
 * All experts local (ep_world = 1), bf16 mode, intermediate_dim a multiple of 256. T is the T of the last forward.
 * Operands are bf16 with fp32 accumulation; the gate/up pre-activations are recomputed, not stashed. The call
 * waits for the forward, reads its placement, enqueues its work on `stream` and returns when that has finished;
 * its workspace is allocated by the first call. */
PRICHS_API int prichs_moe_backward(prichs_moe_t* h, const void* x_dev, int x_dtype, const void* dy_dev, int dy_dtype,
                                   float* dx_dev, float* const* grads_dev, int n_grads, void* stream);

/* Backward of the last prichs_moe_block_forward on this handle: prichs_moe_backward on the normalised rows, then the
 * pre-norm's backward (rmsnorm_backward, crates/prichs-core/src/backward.rs:94-131, as called at
 * crates/prichs-model/src/model.rs:777-789):
 *   dx_res = dy + gamma * rms_inv * (d_normed - x_res * coeff),  d_norm_weight += sum_t d_normed * x_res * rms_inv
 * dy_dev [T,d] is the gradient of the sub-layer's output; it reaches dx_res_dev [T,d] (fp32, overwritten) directly
 * through the residual connection and through the sub-layer. d_norm_weight_dev: [d] fp32, accumulated, may be null.
 * As in the reference the x-term of dx_res carries gamma (the true gradient for gamma = 1, its initial value).
 * grads_dev / n_grads as in prichs_moe_backward. Same restrictions; hidden_dim <= 2048. */
PRICHS_API int prichs_moe_block_backward(prichs_moe_t* h, const void* x_res_dev, int x_dtype, const float* norm_weight_dev,
                                         float eps, const void* dy_dev, int dy_dtype, float* dx_res_dev,
                                         float* d_norm_weight_dev, float* const* grads_dev, int n_grads, void* stream);

/* MoELayer::update_aux_free_bias(expert_token_counts, total_tokens, gamma) (moe.rs:228-245) with host
 * counts, as the reference's call sites pass them (model.rs:786-792,1541-1548):
 *   b_i += gamma * (top_k/E - counts[i]/total_tokens);   no-op when total_tokens == 0.
 * The counts travel as kernel arguments: no allocation, no copy, no device-wide synchronisation. The one-warp kernel is
 * enqueued on the stream of the handle's last forward (after the router that read the bias, before the next forward
 * there); prichs_moe_get_bias waits for it. */
PRICHS_API int prichs_moe_update_aux_free_bias(prichs_moe_t* h, const size_t* expert_token_counts, int n,
                                    size_t total_tokens, float gamma);

/* The same update taken from the counts of the last forward without leaving the device (enqueued on
 * `stream`). total_tokens == 0 means "the T of the last forward". In expert-parallel mode the counts are the
 * sums over all ranks and total_tokens must be the global token count too, so that every rank applies the
 * identical update; 0 then stands for T of this rank times the number of ranks (right when all ranks pass
 * the same T). */
PRICHS_API int prichs_moe_update_bias_from_last(prichs_moe_t* h, float gamma, size_t total_tokens, void* stream);

/* ---- expert parallelism (no counterpart in the reference, which is single-GPU) --------------------- */

/* One process per GPU; rank r owns routed experts [r*E/G, (r+1)*E/G); the shared expert, router and bias are
 * replicated; every rank routes its own tokens. The data path is inside the library's own kernels: the
 * dispatch kernel writes each permuted row straight into the owner's receive buffer over NVLink (peer-mapped
 * memory) and the combine kernel reads expert outputs straight from the owners' buffers, so no separate
 * all-to-all copy exists. NCCL carries only the control plane: one 32-byte all-gather of the per-rank expert
 * counts per wave (placement plan + global counts for the bias update). "Rows landed" and "outputs ready" are
 * readiness flags: each rank stores the forward's sequence number into a slot of every peer's flag array after the
 * producing kernel, and a bounded wait on the local slots precedes the consuming kernel (a wait that runs out is
 * reported as PRICHS_ERR_TIMEOUT by prichs_moe_sync_status; nothing hangs). ep_nccl_barriers = 1 uses two
 * token-sized NCCL all-gathers as barriers instead.
 * Set-up, with any host channel (MPI, torch.distributed, a file) moving the bytes:
 *   1. rank 0: prichs_moe_ep_unique_id(id) and broadcast the PRICHS_EP_ID_BYTES bytes;
 *   2. every rank: prichs_moe_ep_export(h, blob) and all-gather the 128-byte blobs in rank order;
 *   3. every rank: prichs_moe_ep_init(h, id, all_blobs)  (collective: creates the communicator, maps peers).
 * All ranks must then call prichs_moe_forward in the same order. libnccl.so.2 is loaded at run time.
 * Waves: tokens are independent, so a forward cuts its batch into ep_waves token ranges, each with its own
 * receive region, stream and communicator: while the experts of one wave compute, the rows of the next wave
 * travel and the outputs of the previous wave are combined. The shared expert runs on a further stream. */
#define PRICHS_EP_ID_BYTES 1024 /* one communicator id per wave */
#define PRICHS_EP_BLOB_BYTES 128
PRICHS_API int prichs_moe_ep_unique_id(void* id_bytes);
PRICHS_API int prichs_moe_ep_export(prichs_moe_t* h, void* blob128);
PRICHS_API int prichs_moe_ep_init(prichs_moe_t* h, const void* id_bytes, const void* all_blobs);

/* Host-side watchdog of the control plane (no counterpart in the reference, which has no communication). Polls
 * query(ctx) -- 0 = finished, 1 = still running, anything else = failed -- every poll_us microseconds for at most
 * timeout_ms milliseconds; when the time runs out it calls abort_fn(ctx) once (may be null) and returns PRICHS_ERR_COMM.
 * prichs_moe_sync_status uses it for expert-parallel handles with a query on the forward's stream and the
 * communicators' asynchronous error state, and an abort function that calls ncclCommAbort, so that a peer which
 * never joins a collective costs ep_timeout_ms, not the process. After such an abort the handle refuses further
 * forwards with PRICHS_ERR_COMM. Needs no GPU: the tests drive it with CPU ranks. */
PRICHS_API int prichs_ep_wait_or_abort(int (*query)(void*), void (*abort_fn)(void*), void* ctx, int timeout_ms, int poll_us);

/* Rows this rank's experts received in the last forward (expert-parallel load), host value. */
PRICHS_API int prichs_moe_ep_recv_rows(prichs_moe_t* h, int64_t* rows);

/* ---- diagnostics --------------------------------------------------------------------------------- */

/* Message of the last error on the calling thread ("" if none). */
PRICHS_API const char* prichs_last_error(void);

/* 1 when this library was built with -DPRICHS_BOUNDS_CHECK (libprichs_moe_check.so): the routing-side kernels then
 * compare every row index they compute with the extent of its buffer before a scatter or gather, record a violation
 * in the status word (PRICHS_ERR_BOUNDS from prichs_moe_sync_status) and skip the access. The reference has no
 * sanitizer use at all; this build stands in for a memory checker where none may be run. */
PRICHS_API int prichs_bounds_checking(void);

/* Number of kernels this library has launched since it was loaded (all handles). */
PRICHS_API int64_t prichs_kernel_launches(void);

/* Device-time breakdown of the last forward on this handle, in milliseconds, measured with CUDA events
 * recorded on the forward's stream when timing was enabled: router, scan, dispatch, gate_up, down,
 * combine (6 floats). Enabling timing adds event records only. Handles with all experts local only; the
 * expert-parallel forward overlaps its kernels on several streams and reports prichs_moe_get_ep_timeline. */
PRICHS_API int prichs_moe_enable_timing(prichs_moe_t* h, int on);
PRICHS_API int prichs_moe_get_stage_ms(prichs_moe_t* h, float* ms6);

/* Expert-parallel timeline of the last forward (timing enabled): device times in milliseconds since the router
 * finished, ms[0..1] = shared gate|up done, shared down done; then for every wave w eight marks at
 * ms[2 + 8 w + i]: i = 0 counts scanned, 1 plan ready, 2 rows dispatched, 3 all ranks' rows landed, 4 gate|up
 * done, 5 down done, 6 all ranks' outputs ready, 7 combined. n must be at least 2 + 8 * waves. */
PRICHS_API int prichs_moe_get_ep_timeline(prichs_moe_t* h, float* ms, int n);

/* Copies `bytes` bytes at `offset_bytes` of one internal device buffer of the last forward to the host (waits
 * for the handle's last stream). For tests and diagnostics of the intermediate stages; the reference exposes
 * the same intermediates as the stash vectors of forward_train (moe.rs:32-53).
 *   which: 0 converted activations [T,K1] bf16   1 permuted rows [Rcap,K1] bf16   2 hidden H [Tcap+Rcap,K2] bf16
 *          3 expert outputs [Tcap+Rcap,d] (bf16; fp32 in PRICHS_MODE_F32)          4 row map pos [T,2] int32
 *          5 routing summary (struct of ints: counts[8], seg_base[8], src_off[8], total[8], n_mtiles,
 *            recv_rows, overflow, pad, cmat[64])   6 per-tile histograms [ceil(T/16),8] int32
 *          7 their exclusive prefix sums           8 m-tile -> weight slot table int32
 *          after prichs_moe_backward, in the same row space: 9 recomputed [gate | up] [Tcap+Rcap,2f] bf16 (blocks of
 *          128 gate then 128 up columns)   10 dY rows [.,d] bf16   11 d_act [.,f] bf16   12 [d_gate | d_up] [.,2f] bf16
 *          13 dX rows [.,d] bf16   14 <expert row, d_out> [T,2] fp32   15 d_logits [T,8] fp32
 *          16 m-tile -> 128-row tile index inside the permuted region, int32 (all experts local)
 *   K1 = d, K2 = f (2d, 2f in PRICHS_MODE_F32); Tcap = max_tokens rounded up to 256. With all experts local
 *   Rcap = E * Tcap: expert e's rows start at row e * Tcap of the permuted region (fixed-capacity segments). */
PRICHS_API int prichs_moe_debug_copy(prichs_moe_t* h, int which, size_t offset_bytes, void* host_dst, size_t bytes);

/* Test knobs of the single-pass routing kernel (no counterpart in the reference). key 0: index of a 16-token tile
 * that does not publish its counts in the following forwards, so that the look-back of the tiles after it runs out
 * and the forward reports PRICHS_ERR_TIMEOUT through prichs_moe_sync_status (-1 = none, the default). key 1: budget
 * of that kernel's bounded waits, and of the expert-parallel readiness waits, in clock cycles (default 4e9, about two
 * seconds). key 2: 1 + kind * 4 + wave of a readiness signal this rank does not send in the following expert-parallel
 * forwards (kind 0 rows landed, 1 outputs ready; 0 = none), so that the other ranks' bounded wait for it runs out.
 * key 3: nanoseconds a warp of the single-pass routing kernel pauses before it looks again at tiles that have not
 * published their counts yet (default 100; 0 = poll back to back). */
PRICHS_API int prichs_moe_debug_set(prichs_moe_t* h, int key, long long value);

/* ---- routing without any allocation ---------------------------------------------------------------
 * This entry point has no counterpart in the reference. It exists for callers that are not allowed to
 * allocate device memory at the point where they need routing decisions -- a plugin running inside a host
 * application that owns the whole memory pool, a real-time loop that must not enter the allocator, a hook
 * invoked where cudaMalloc would synchronise the device. Such callers cannot create a handle (create
 * allocates), so they get the router stage on its own: logits, top-k experts, gates and per-expert counts for
 * one batch, computed with the same kernels as prichs_moe_forward.
 *
 * Every intermediate (transposed router weights, per-tile histograms, prefix sums, packed selections) lives in
 * ONE fixed 1 MiB array that is part of the library image on each GPU that loads it and stays there until the
 * process exits. The call performs no cudaMalloc/cudaFree and calls no allocating library routine (the very
 * first kernel launch of a process may still make the CUDA runtime load the library's device code).
 *   x_dev        [T,d] bf16, device          router_dev   [d,E] fp32, device (the reference's layout)
 *   bias_dev     [E] fp32 device, or null for a zero bias
 *   outputs (device, caller-owned): logits_dev [T,E] fp32, selected_dev [T,top_k] int32,
 *   gating_dev [T,top_k] fp32, counts_dev [E] int32
 * Limits: T <= PRICHS_ROUTE_STATIC_MAX_TOKENS, d <= PRICHS_ROUTE_STATIC_MAX_HIDDEN (d a multiple of 256),
 * E <= 8, top_k <= 2; anything larger returns PRICHS_ERR_CAPACITY and does nothing.
 * The first call on a device looks up the array's device address (once per device, with that device
 * current); make that first call before starting any stream capture. All calls on a device share the array
 * and it keeps the previous call's contents (what must start at zero is cleared on `stream` by the call
 * itself): two calls whose work overlaps on the GPU -- different streams, no ordering between them -- race on
 * it. Order them on one stream or with events. */
#define PRICHS_ROUTE_STATIC_MAX_TOKENS 16384
#define PRICHS_ROUTE_STATIC_MAX_HIDDEN 2048
PRICHS_API int prichs_moe_route_static(const void* x_dev, const float* router_dev, const float* bias_dev, int T, int d,
                                       int E, int top_k, float* logits_dev, int32_t* selected_dev, float* gating_dev,
                                       int32_t* counts_dev, void* stream);

/* ---- stand-alone kernels with the reference's signatures ----------------------------------------- */

/* Same symbols, arguments and semantics as the reference's wrappers, so engine.rs links unchanged:
 *   launch_moe_gather       kernels.cu:993-1007   out[i,:] = in[idx[i],:]
 *   launch_moe_scatter_add  kernels.cu:1009-1024  acc[idx[i],:] += w[i] * exp_out[i,:]
 *   launch_swiglu_forward   kernels.cu:482-496    out = silu(gate) * up
 * fp32 device pointers, `stream` a cudaStream_t, zero sizes return at once, no status (as there). */
PRICHS_API void launch_moe_gather(const float* dev_in, const int* dev_token_indices, float* dev_out, size_t n_tokens,
                       size_t hidden_dim, void* stream);
PRICHS_API void launch_moe_scatter_add(const float* dev_exp_out, const int* dev_token_indices, const float* dev_weights,
                            float* dev_accum_out, size_t n_tokens, size_t hidden_dim, void* stream);
PRICHS_API void launch_swiglu_forward(const float* dev_gate, const float* dev_up, float* dev_out, size_t total_elements,
                           void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PRICHS_MOE_H_ */
