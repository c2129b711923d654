// Routing-side kernels of the MoE layer: fused router (logits + bias + top-2 + gates + histogram),
// prefix-sum / placement plan, token dispatch (permute), gate-weighted combine (+ residual), bias update.
// All of them are bound by HBM traffic: 16-byte accesses, one warp per token row (or 16-token MMA tile),
// no atomics on the data path, results independent of scheduling.
//
// Reference semantics restated here (and nowhere copied from):
//   crates/prichs-model/src/moe.rs:114-142   router logits, bias add, per-token top-k, expert bins
//   crates/prichs-core/src/ops.rs:219-248    top_k_gating_unbiased (selection on biased logits, gates
//                                            from the raw logits of the selected experts)
//   crates/prichs-model/src/moe.rs:146-184   combine: out = shared; experts ascending: out += w * row
//   crates/prichs-model/src/block.rs:64-67   residual add around the layer
//   crates/prichs-model/src/moe.rs:228-245   update_aux_free_bias
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

// Index checking build (-DPRICHS_BOUNDS_CHECK, libprichs_moe_check.so): every row index the routing-side kernels
// compute before a scatter or a gather is compared with the extent of its buffer; a violation records -7 in the
// status word (PRICHS_ERR_BOUNDS) and the access is skipped -- no trap, no fault. The product build compiles the
// checks away. Stands in for a memory checker on machines where none may be run.
#ifdef PRICHS_BOUNDS_CHECK
#define PRICHS_ROW_OK(idx, limit, status) \
    (((long long)(idx) >= 0 && (long long)(idx) < (long long)(limit)) ? true : (atomicExch((status), -7), false))
#else
#define PRICHS_ROW_OK(idx, limit, status) true
#endif

namespace route {

constexpr int MAX_E = 8;      // routed experts supported by the 8-column router MMA
constexpr int MAX_RANKS = 8;  // expert-parallel group size limit
constexpr int TILE_TOKENS = 16;

// Optional per-expert additive term on the selection logit (moe.rs:128-132), passed by value.
struct ConceptBias {
    float v[MAX_E];
};

// Device-resident routing summary of one forward call.
struct RouteMeta {
    int counts[MAX_E];    // assignments this rank produced per expert (lengths of the bins, moe.rs:121,140)
    int seg_base[MAX_E];  // row, in the owner's permuted buffer, where expert e's segment starts (x128)
    int src_off[MAX_E];   // rows of lower ranks that precede this rank's rows inside that segment
    int total[MAX_E];     // per-expert totals over all ranks
    int n_routed_mtiles;  // 128-row tiles of the local permuted region
    int recv_rows;        // rows this rank's experts receive (unpadded)
    int overflow;         // 1 when the local permuted region would exceed its capacity
    int pad;
    int cmat[MAX_RANKS * MAX_E];  // counts of every rank, [rank][expert]
};

struct PeerPtrs {
    void* p[MAX_RANKS];
};

// ---------------------------------------------------------------------------------------------------
// Per-token selection shared by both router kernels. Called by all 32 lanes of a warp; `active` lanes own
// one token row each, `lower_mask` has a bit for every lane whose token precedes this lane's token.
//   selection logit  s_e = (L_e + bias_e) + concept_e          (moe.rs:126-134)
//   top-k of s, ties to the lower index (stable descending sort, ops.rs:226-229); NaN logits are outside
//   the contract (the reference's result then depends on its sort's internals)
//   gates from the RAW logits of the selected experts: exp(L_i - max) / (sum + 1e-9)   (ops.rs:233-245)
// Writes logits [T,8], sel [T,2] (expert | rank-in-tile << 8, or -1), gates [T,2] and the tile's histogram.
// Returns what the lane selected (i2 = -1: one expert only; inactive lanes: i1 = 0, i2 = -1, unused) and, in lane
// e < 8, the tile's count for expert e.
struct RouteSel {
    int i1, i2, r1, r2, my_count;
};
__device__ __forceinline__ RouteSel route_finish(const float (&L)[MAX_E], bool active, uint32_t lower_mask, int row,
                                                 int tile, int lane, const float* __restrict__ bias,
                                                 const ConceptBias& cb, int E, int top_k, float* __restrict__ logits,
                                                 int* __restrict__ sel, float* __restrict__ gates,
                                                 int* __restrict__ tile_counts) {
    int i1 = 0, i2 = -1;
    float l1 = 0.f, l2 = 0.f;
    if (active) {
        float s[MAX_E];
#pragma unroll
        for (int e = 0; e < MAX_E; ++e) s[e] = (L[e] + bias[e]) + cb.v[e];
        float v1 = s[0];
#pragma unroll
        for (int e = 1; e < MAX_E; ++e) {
            if (e < E && s[e] > v1) {
                v1 = s[e];
                i1 = e;
            }
        }
        if (top_k > 1) {
            float v2 = 0.f;
#pragma unroll
            for (int e = 0; e < MAX_E; ++e) {
                if (e < E && e != i1 && (i2 < 0 || s[e] > v2)) {
                    v2 = s[e];
                    i2 = e;
                }
            }
        }
#pragma unroll
        for (int e = 0; e < MAX_E; ++e) {
            l1 = (e == i1) ? L[e] : l1;
            l2 = (e == i2) ? L[e] : l2;
        }
        float4* lo = reinterpret_cast<float4*>(logits + (size_t)row * MAX_E);
        lo[0] = make_float4(L[0], L[1], L[2], L[3]);
        lo[1] = make_float4(L[4], L[5], L[6], L[7]);
    }
    // histogram of the tile and rank of each assignment among the tile's earlier tokens
    int r1 = 0, r2 = 0, my_count = 0;
#pragma unroll
    for (int e = 0; e < MAX_E; ++e) {
        const uint32_t m = __ballot_sync(0xffffffffu, active && (i1 == e || i2 == e));
        if (i1 == e) r1 = __popc(m & lower_mask);
        if (i2 == e) r2 = __popc(m & lower_mask);
        if (lane == e) my_count = __popc(m);
    }
    if (lane < MAX_E) tile_counts[(size_t)tile * MAX_E + lane] = my_count;
    if (active) {
        float g1, g2 = 0.f;
        if (i2 >= 0) {
            const float mx = fmaxf(l1, l2);
            const float e1 = expf(l1 - mx);
            const float e2 = expf(l2 - mx);
            float sum = 0.0f;
            sum = __fadd_rn(sum, e1);
            sum = __fadd_rn(sum, e2);
            const float inv = 1.0f / (sum + 1e-9f);
            g1 = e1 * inv;
            g2 = e2 * inv;
        } else {
            const float e1 = expf(l1 - l1);
            const float inv = 1.0f / (e1 + 1e-9f);
            g1 = e1 * inv;
        }
        *reinterpret_cast<int2*>(sel + (size_t)row * 2) = make_int2(i1 | (r1 << 8), i2 >= 0 ? (i2 | (r2 << 8)) : -1);
        *reinterpret_cast<float2*>(gates + (size_t)row * 2) = make_float2(g1, g2);
    }
    return RouteSel{i1, i2, r1, r2, my_count};
}

// ---------------------------------------------------------------------------------------------------
// Router for bf16 operands. One CTA of 8 warps owns a tile of 16 tokens; the warps split K between them
// (warp w takes the 32-element slices w, w+8, w+16, ... so that the CTA reads 512 contiguous bytes of every
// row per step) and each computes partial logits with mma.sync m16n8k16 (N = 8 is exactly the expert count):
// lane (g = lane/4, q = lane%4) reads 16 contiguous bytes of token row g (and g+8) and 16 contiguous bytes of
// row g of the transposed router weight. The dot product does not care in which order k is visited, so those
// 8 consecutive elements are fed to two MMAs as the fragment slots (2q, 2q+1, 2q+8, 2q+9) of A and B alike --
// every global access is a full 16-byte vector. The partial sums meet in shared memory and warp 0 adds them
// in a fixed order, then selects. With T/16 CTAs of 8 warps the whole batch is in flight at once, which is
// what an HBM-bound kernel with ~3 KB per token needs.
// wrt: [NSPLIT][8][d] bf16; NSPLIT = 3 holds hi/mid/lo parts of fp32 router weights (their sum is exact to
// 2^-24), NSPLIT = 1 is used when the weights are bf16 values already.
// XF32: x is fp32 [T,d]; it is rounded to bf16 (RNE) for the product and the bf16 copy is written to `xs`
// for the expert GEMMs (saves a separate conversion pass).
// NORM: the rows are RMS-normalised (weight norm_w, epsilon norm_eps) before they are rounded to bf16; `xs`
// receives the normalised rows. The un-normalised rows stay the caller's residual.
constexpr int ROUTER_WARPS = 8;
constexpr int ROUTER_KB = 6;

template <int NT, int SCAN_KEEP>
__device__ __forceinline__ const int* scan_tiles(const int* tile_counts, int* __restrict__ tile_prefix, int ntiles,
                                                 RouteMeta* meta, int rank);
__device__ __forceinline__ void plan_from_cmat(RouteMeta* meta, int* __restrict__ mtile_slot, int* __restrict__ mtile_row,
                                               int E, int El, int world, int rank, int cap_rows, int pad_rows,
                                               int seg_stride, int* __restrict__ status, const int* local_counts);

// Work the last CTA of the router launch does when all experts are local: the prefix sums over the tile
// histograms and the placement plan, which would otherwise be a one-CTA launch of their own between the router
// and the dispatch. `done` counts finished CTAs (zero before the launch, reset by the last CTA); null = no tail.
struct ScanTail {
    int* done;
    int* tile_prefix;
    RouteMeta* meta;
    int* mtile_slot;
    int* mtile_row;
    int El, cap_rows, pad_rows, seg_stride;
    int* status;
};

template <int NSPLIT, bool XF32, bool NORM>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_mma_kernel(const void* __restrict__ x, __nv_bfloat16* __restrict__ xs, const __nv_bfloat16* __restrict__ wrt,
                  const float* __restrict__ bias, const ConceptBias cb, int T, int d, int E, int top_k,
                  float* __restrict__ logits, int* __restrict__ sel, float* __restrict__ gates,
                  int* tile_counts, const float* __restrict__ norm_w, float norm_eps, const ScanTail tail) {
    __shared__ float4 partial[2][ROUTER_WARPS][32];
    __shared__ float ssq[NORM ? TILE_TOKENS : 1][32], inv_rms_s[TILE_TOKENS];
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int ntiles = (T + TILE_TOKENS - 1) / TILE_TOKENS;
    constexpr int KSTEP = ROUTER_WARPS * 32;  // elements of a row the CTA covers per slice
    constexpr int XV = XF32 ? 4 : 2;          // 16-byte vectors a lane reads per slice (rows g and g + 8)
    // grid-stride over tiles; `partial` is double buffered, so a tile costs one barrier and warps 1..7 start the
    // loads of the next tile while warp 0 still selects for this one
    int buf = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, buf ^= 1) {
    const int r0 = tile * TILE_TOKENS + g, r1 = r0 + 8;
    const size_t r0c = (size_t)min(r0, T - 1), r1c = (size_t)min(r1, T - 1);

    float acc[NSPLIT][2][4];
#pragma unroll
    for (int s = 0; s < NSPLIT; ++s)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[s][h][i] = 0.f;

    const __nv_bfloat16* wl = wrt + (size_t)g * d + 8 * q;
    const size_t wsplit = (size_t)MAX_E * d;

    // A pass covers ROUTER_KB slices (the whole row for d <= 1536). All of its loads are issued before the first
    // MMA, so a warp has up to ROUTER_KB * XV 16-byte requests in flight instead of one slice's worth: with
    // ~3 KB per token and no reuse, memory-level parallelism is what sets the speed of this kernel.
    for (int kb = warp * 32; kb < d; kb += ROUTER_KB * KSTEP) {
        uint4 xv[ROUTER_KB][XV], wv[ROUTER_KB][NSPLIT];
#pragma unroll
        for (int i = 0; i < ROUTER_KB; ++i) {
            const int kk = kb + i * KSTEP;
            if (kk < d) {
                if constexpr (XF32) {
                    const float* x0 = reinterpret_cast<const float*>(x) + r0c * d + kk + 8 * q;
                    const float* x1 = reinterpret_cast<const float*>(x) + r1c * d + kk + 8 * q;
                    xv[i][0] = ptx::ld_stream_16(x0);
                    xv[i][1] = ptx::ld_stream_16(x0 + 4);
                    xv[i][2] = ptx::ld_stream_16(x1);
                    xv[i][3] = ptx::ld_stream_16(x1 + 4);
                } else {
                    const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
                    xv[i][0] = ptx::ld_stream_16(xb + r0c * d + kk + 8 * q);
                    xv[i][1] = ptx::ld_stream_16(xb + r1c * d + kk + 8 * q);
                }
#pragma unroll
                for (int s = 0; s < NSPLIT; ++s) wv[i][s] = __ldg(reinterpret_cast<const uint4*>(wl + s * wsplit + kk));
            }
        }
        // the 8 consecutive elements of row half `hf` (0: row g, 1: row g + 8) in slice i, widened to fp32
        auto unpack8 = [&](int i, int hf, float (&v)[8]) {
            if constexpr (XF32) {
                const uint4 a = xv[i][(2 * hf) % XV], b = xv[i][(2 * hf + 1) % XV];
                v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
                v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
            } else {
                const uint4 a = xv[i][hf];
                const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[2 * j] = __uint_as_float(w[j] << 16);
                    v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                }
            }
        };
        auto pack8 = [](const float (&v)[8]) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<uint32_t*>(&b2);
            }
            return make_uint4(w[0], w[1], w[2], w[3]);
        };
        // Pre-norm folded into the read (rms_norm of crates/prichs-core/src/ops.rs:109-135 ahead of the layer,
        // crates/prichs-model/src/block.rs:64). Thread (warp, q) holds for its two rows exactly the elements lane
        // 4 * warp + q of rmsnorm_rows_kernel holds, and sums their squares in the same order; the 32 partial sums
        // of a row then go through the same butterfly, so inv_rms and the normalised bf16 rows are bit-identical to
        // the stand-alone kernel's. Needs the whole row in one pass (d <= ROUTER_KB * 256).
        float inv0 = 1.f, inv1 = 1.f;
        if constexpr (NORM) {
            float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
            for (int i = 0; i < ROUTER_KB; ++i) {
                if (kb + i * KSTEP < d) {
                    float v0[8], v1[8];
                    unpack8(i, 0, v0);
                    unpack8(i, 1, v1);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        ss0 = fmaf(v0[j], v0[j], ss0);
                        ss1 = fmaf(v1[j], v1[j], ss1);
                    }
                }
            }
            ssq[g][4 * warp + q] = ss0;
            ssq[g + 8][4 * warp + q] = ss1;
            __syncthreads();
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                float sv = ssq[2 * warp + rr][lane];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sv += __shfl_xor_sync(0xffffffffu, sv, o);
                if (lane == 0) inv_rms_s[2 * warp + rr] = 1.0f / sqrtf(sv / (float)d + norm_eps);
            }
            __syncthreads();
            inv0 = inv_rms_s[g];
            inv1 = inv_rms_s[g + 8];
        }
#pragma unroll
        for (int i = 0; i < ROUTER_KB; ++i) {
            const int kk = kb + i * KSTEP;
            if (kk < d) {
                uint4 a0, a1;
                if constexpr (NORM) {
                    const float4 n0 = __ldg(reinterpret_cast<const float4*>(norm_w + kk + 8 * q));
                    const float4 n1 = __ldg(reinterpret_cast<const float4*>(norm_w + kk + 8 * q + 4));
                    const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
                    float v0[8], v1[8];
                    unpack8(i, 0, v0);
                    unpack8(i, 1, v1);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        v0[j] = __fmul_rn(__fmul_rn(v0[j], inv0), nw[j]);
                        v1[j] = __fmul_rn(__fmul_rn(v1[j], inv1), nw[j]);
                    }
                    a0 = pack8(v0);
                    a1 = pack8(v1);
                } else if constexpr (XF32) {
                    float v0[8], v1[8];
                    unpack8(i, 0, v0);
                    unpack8(i, 1, v1);
                    a0 = pack8(v0);
                    a1 = pack8(v1);
                } else {
                    a0 = xv[i][0];
                    a1 = xv[i][1];
                }
                if constexpr (NORM || XF32) {
                    if (r0 < T) *reinterpret_cast<uint4*>(xs + (size_t)r0 * d + kk + 8 * q) = a0;
                    if (r1 < T) *reinterpret_cast<uint4*>(xs + (size_t)r1 * d + kk + 8 * q) = a1;
                }
#pragma unroll
                for (int s = 0; s < NSPLIT; ++s) {
                    const uint4 w = wv[i][s];
                    ptx::mma_m16n8k16_bf16(acc[s][0], a0.x, a1.x, a0.y, a1.y, w.x, w.y);
                    ptx::mma_m16n8k16_bf16(acc[s][1], a0.z, a1.z, a0.w, a1.w, w.z, w.w);
                }
            }
        }
    }
    // c[0..1]: row g, experts 2q, 2q+1; c[2..3]: row g+8. Small parts are summed first.
    float c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float v = 0.f;
#pragma unroll
        for (int s = NSPLIT - 1; s >= 0; --s) v += acc[s][0][i] + acc[s][1][i];
        c[i] = v;
    }
    partial[buf][warp][lane] = make_float4(c[0], c[1], c[2], c[3]);
    __syncthreads();
    if (warp == 0) {
#pragma unroll
    for (int w = 1; w < ROUTER_WARPS; ++w) {
        const float4 p = partial[buf][w][lane];
        c[0] += p.x; c[1] += p.y; c[2] += p.z; c[3] += p.w;
    }
    // lanes q = 0 / q = 1 of each quad take row g / g + 8; gather the row's 8 logits from the quad
    float L[MAX_E];
    const int qbase = lane & ~3;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float t0 = __shfl_sync(0xffffffffu, c[0], qbase + j);
        const float t1 = __shfl_sync(0xffffffffu, c[1], qbase + j);
        const float t2 = __shfl_sync(0xffffffffu, c[2], qbase + j);
        const float t3 = __shfl_sync(0xffffffffu, c[3], qbase + j);
        L[2 * j] = (q == 0) ? t0 : t2;
        L[2 * j + 1] = (q == 0) ? t1 : t3;
    }
    const int row = (q == 0) ? r0 : r1;
    const bool active = (q < 2) && (row < T);
    // tokens that precede this lane's token inside the tile: q=0 lanes hold rows 0..7, q=1 lanes rows 8..15
    const uint32_t below = (1u << (4 * g)) - 1u;
    const uint32_t lower_mask = (q == 0) ? (below & 0x11111111u) : (0x11111111u | (below & 0x22222222u));
    route_finish(L, active, lower_mask, row, tile, lane, bias, cb, E, top_k, logits, sel, gates, tile_counts);
    }
    }
    if (tail.done != nullptr) {
        // last-CTA-done: every CTA publishes its histograms (fence) and takes a ticket; the CTA that draws the last
        // ticket sees all of them and finishes the routing metadata
        __shared__ int s_last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicAdd(tail.done, 1) == (int)gridDim.x - 1;
        __syncthreads();
        if (s_last) {
            __threadfence();
            const int* totals = scan_tiles<ROUTER_WARPS * 32, 8>(tile_counts, tail.tile_prefix, ntiles, tail.meta, 0);
            plan_from_cmat(tail.meta, tail.mtile_slot, tail.mtile_row, E, tail.El, 1, 0, tail.cap_rows, tail.pad_rows, tail.seg_stride, tail.status, totals);
            if (threadIdx.x == 0) *tail.done = 0;
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Route, place and dispatch in ONE pass over the tokens (all experts local, bf16 rows). A row is read from
// global memory once, into shared memory, and leaves it twice -- to the segments of its two experts -- without
// passing through registers; in between a warp computes the row's logits from the shared-memory copy.
//
// One persistent CTA per SM. A producer thread draws 16-token tiles from a global ticket counter and copies each
// tile's rows with untiled bulk copies into a ring of `stages` buffers (full / empty mbarrier per stage). Consumer
// warp w owns stage w:
//   1. logits of the tile's 16 tokens on mma.sync m16n8k16 out of shared memory, arithmetic and summation order of
//      router_mma_kernel<NSPLIT, false, false> (bit-identical logits); bias, top-2, gates, the tile's per-expert
//      counts and each token's rank among the tile's earlier tokens (route_finish);
//   2. the tile's exclusive per-expert prefix over all earlier tiles by decoupled look-back: the warp publishes its
//      counts as "aggregate" words, reads the state words of the 32 tiles before it (one tile per lane), adds
//      aggregates back to the nearest "inclusive" word, moves the window further back if there is none, and then
//      publishes its own inclusive prefix. A state word carries its flag and its value together (2 + 30 bits), so
//      no fence sits on this path. Tickets are drawn in order and a tile's rows are requested as soon as its ticket
//      is drawn, so every earlier tile is already being worked on by a running CTA: the walk cannot wait on work
//      that has not been scheduled.
//   3. row of assignment (token, expert e) = e * seg_stride + prefix[e] + rank; the rows go from the stage buffer to
//      the permuted region with bulk copies issued by the lanes that own the tokens; the stage is handed back to
//      the producer when those copies have read it.
// The warp that handles the last tile knows the totals and writes the routing summary and the GEMM's tile table.
// The CTA that leaves last (counter in ctl[1]) returns tile_state and the ticket counter to zero, so a launch
// leaves the scratch state as it found it and the kernel can be replayed from a CUDA graph.
// Every wait (mbarriers, look-back) is bounded by `wait_cycles`; one that gives up raises the CTA's abort flag,
// every role leaves its loop, in-flight copies are waited for, and the status word reports -5.
constexpr int RD_MAX_STAGES = 4;
constexpr int RD_THREADS = (RD_MAX_STAGES + 1) * 32;
constexpr int RD_ROW_PAD = 64;  // bytes: the two rows a quarter-warp reads fall on disjoint banks
constexpr uint32_t RD_AGG = 1u << 30, RD_INCL = 2u << 30, RD_VAL = (1u << 30) - 1u;

__host__ __device__ inline int rd_stage_bytes(int d) { return TILE_TOKENS * (2 * d + RD_ROW_PAD); }
__host__ __device__ inline int rd_weight_bytes(int d, int nsplit) { return nsplit * MAX_E * (2 * d + RD_ROW_PAD); }
__host__ __device__ inline int rd_smem_bytes(int d, int nsplit, int stages) {
    return stages * rd_stage_bytes(d) + rd_weight_bytes(d, nsplit) + 2 * RD_MAX_STAGES * 8 + RD_MAX_STAGES * 4 + 16;
}

struct RouteDispatchArgs {
    const __nv_bfloat16* x;    // [T, d] token rows
    const __nv_bfloat16* wrt;  // [NSPLIT][8][d] transposed router weights
    const float* bias;
    int T, d, E, top_k, stages;
    float* logits;
    int* sel;
    float* gates;
    int* pos;
    int* tile_counts;
    int* tile_prefix;
    uint32_t* tile_state;  // [ceil(T/16)][8] look-back words, all zero between launches
    int* ctl;              // [0] next ticket, [1] CTAs that have left; both zero between launches
    __nv_bfloat16* xp;     // permuted region, expert e's segment at row e * seg_stride
    int seg_stride, pad_rows;
    RouteMeta* meta;
    int* mtile_slot;
    int* mtile_row;
    int* status;
    long long wait_cycles;
    int stall_tile;  // test knob: this tile never publishes its counts, so its successors' look-back runs out (-1: none)
    int poll_sleep_ns;  // pause between two looks at a window whose tiles have not all published yet
};

__device__ __forceinline__ uint4 ld_relaxed_16(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_4(void* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Routing summary and GEMM tile table for fixed-stride segments, by one warp; lane e < 8 passes expert e's total.
__device__ __forceinline__ void plan_fixed_stride_warp(RouteMeta* meta, int* __restrict__ mtile_slot, int* __restrict__ mtile_row,
                                                       int E, int seg_stride, int pad_rows, int total, int lane) {
    const uint32_t full = 0xffffffffu;
    if (lane >= E) total = 0;
    const int tiles = (total + pad_rows - 1) / pad_rows * (pad_rows / 128);
    int inc = tiles;
#pragma unroll
    for (int o = 1; o < MAX_E; o <<= 1) {
        const int n = __shfl_up_sync(full, inc, o);
        if (lane >= o) inc += n;
    }
    const int tile0 = inc - tiles;
    const int ntot = __shfl_sync(full, inc, MAX_E - 1);
    const int recv = __reduce_add_sync(full, lane < MAX_E ? total : 0);
    if (lane < MAX_E) {
        meta->counts[lane] = total;
        meta->total[lane] = total;
        meta->src_off[lane] = 0;
        meta->seg_base[lane] = lane < E ? lane * seg_stride : 0;
        meta->cmat[lane] = total;
    }
    if (lane == 0) {
        meta->n_routed_mtiles = ntot;
        meta->recv_rows = recv;
        meta->overflow = 0;
    }
    int t0s[MAX_E], tots[MAX_E];
#pragma unroll
    for (int e = 0; e < MAX_E; ++e) {
        t0s[e] = __shfl_sync(full, tile0, e);
        tots[e] = __shfl_sync(full, total, e);
    }
    for (int i = lane; i < ntot; i += 32) {
        int le = 0, t0 = 0, tot = tots[0];
#pragma unroll
        for (int e = 1; e < MAX_E; ++e) {
            if (e < E && i >= t0s[e]) {
                le = e;
                t0 = t0s[e];
                tot = tots[e];
            }
        }
        const int j = i - t0;
        mtile_slot[i] = (j * 128 >= tot) ? -1 - le : le;
        mtile_row[i] = le * (seg_stride / 128) + j;
    }
}

template <int NSPLIT>
__global__ void __launch_bounds__(RD_THREADS, 1)
route_dispatch_kernel(const __grid_constant__ RouteDispatchArgs a, const ConceptBias cb) {
    extern __shared__ __align__(128) uint8_t rsm[];
    const int d = a.d, stages = a.stages, T = a.T;
    const int rowb = 2 * d + RD_ROW_PAD;
    const int stage_bytes = TILE_TOKENS * rowb;
    uint8_t* wsm = rsm + (size_t)stages * stage_bytes;  // router weights, [NSPLIT][8][rowb]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(wsm + NSPLIT * MAX_E * rowb);
    uint64_t* empty_bar = full_bar + RD_MAX_STAGES;
    volatile int* tile_of_stage = reinterpret_cast<volatile int*>(empty_bar + RD_MAX_STAGES);
    volatile int* abort_flag = tile_of_stage + RD_MAX_STAGES;
    __shared__ int s_last;

    ptx::grid_dep_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full = 0xffffffffu;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    __syncthreads();  // barriers are initialised: the producer starts its copies at once
    const int ntiles = (T + TILE_TOKENS - 1) / TILE_TOKENS;
    // Everything above, and the staging of the router weights below (they only change at upload, which synchronises
    // the device), is independent of the previous kernel of the stream; under programmatic dependent launch it runs
    // while that kernel drains. Tokens, bias and the scratch state are touched after the wait only.
    if (warp == RD_MAX_STAGES) ptx::grid_dep_wait();
    if (warp < RD_MAX_STAGES) {
        // the consumer warps stage the transposed router weights in padded shared-memory rows (16 bytes per thread and
        // step) while the first tiles are on their way, and meet at a barrier of their own
        for (int i = threadIdx.x; i < NSPLIT * MAX_E * (d / 8); i += RD_MAX_STAGES * 32) {
            const int r = i / (d / 8), c = i - r * (d / 8);
            *reinterpret_cast<uint4*>(wsm + (size_t)r * rowb + 16 * c) = __ldg(reinterpret_cast<const uint4*>(a.wrt + (size_t)r * d) + c);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(RD_MAX_STAGES * 32) : "memory");
        ptx::grid_dep_wait();
    }

    if (warp == RD_MAX_STAGES) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            int loads = 0, stops = 0;
            bool ok = true, more = true;
            for (int n = 0; ok; ++n) {
                const int s = n % stages;
                const uint32_t ph = (uint32_t)((n / stages) & 1);
                if (!ptx::mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag, a.wait_cycles)) {
                    ok = false;
                    break;
                }
                int tile = -1;
                if (more) {
                    tile = atomicAdd(a.ctl, 1);
                    if (tile >= ntiles) {
                        tile = -1;
                        more = false;
                    }
                }
                tile_of_stage[s] = tile;
                if (tile >= 0) {
                    const int rows = min(TILE_TOKENS, T - tile * TILE_TOKENS);
                    uint8_t* dst = rsm + (size_t)s * stage_bytes;
                    ptx::mbar_expect_tx(&full_bar[s], (uint32_t)(rows * 2 * d));
                    for (int r = 0; r < rows; ++r)
                        ptx::bulk_load_1d(dst + (size_t)r * rowb, a.x + ((size_t)tile * TILE_TOKENS + r) * d, (uint32_t)(2 * d), &full_bar[s]);
                    ++loads;
                } else {
                    ptx::mbar_arrive(&full_bar[s]);  // tells the stage's consumer that no tile follows
                    if (++stops == stages) break;
                }
            }
            if (!ok) {
                // leaving early: the copies already in flight must land before this CTA's shared memory goes away
                for (int i = max(0, loads - stages); i < loads; ++i) {
                    const long long t0 = clock64();
                    while (!ptx::mbar_try_wait(&full_bar[i % stages], (uint32_t)((i / stages) & 1)) && clock64() - t0 < a.wait_cycles) {
                    }
                }
            }
        }
    } else if (warp < stages) {
        // ---------------------------------------------------------------- consumer warp of stage `warp`
        const int g = lane >> 2, q = lane & 3;
        uint8_t* stage = rsm + (size_t)warp * stage_bytes;
        const uint8_t* r0p = stage + (size_t)g * rowb + 16 * q;
        const uint8_t* r1p = r0p + 8 * (size_t)rowb;
        const uint8_t* wp = wsm + (size_t)g * rowb + 16 * q;
        for (int n = 0;; ++n) {
            // the vote keeps the warp converged for the warp-wide operations below
            if (!__all_sync(full, ptx::mbar_wait_bounded(&full_bar[warp], (uint32_t)(n & 1), abort_flag, a.wait_cycles))) break;
            const int tile = tile_of_stage[warp];
            if (tile < 0) break;
            // ---- 1. logits: NSPLIT passes over K (small parts first), eight accumulator sets per pass, one per warp
            //         of the lock-step kernel, added in that kernel's order
            float cw[ROUTER_WARPS][4];
#pragma unroll
            for (int w = 0; w < ROUTER_WARPS; ++w)
#pragma unroll
                for (int i = 0; i < 4; ++i) cw[w][i] = 0.f;
#pragma unroll 1
            for (int s = NSPLIT - 1; s >= 0; --s) {
                float acc[ROUTER_WARPS][2][4];
#pragma unroll
                for (int w = 0; w < ROUTER_WARPS; ++w)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[w][hh][i] = 0.f;
                const uint8_t* wps = wp + (size_t)s * MAX_E * rowb;
                for (int kc = 0; kc < d; kc += ROUTER_WARPS * 32) {
#pragma unroll
                    for (int w = 0; w < ROUTER_WARPS; ++w) {
                        const int kb = 2 * (kc + 32 * w);
                        const uint4 a0 = *reinterpret_cast<const uint4*>(r0p + kb);
                        const uint4 a1 = *reinterpret_cast<const uint4*>(r1p + kb);
                        const uint4 wv = *reinterpret_cast<const uint4*>(wps + kb);
                        ptx::mma_m16n8k16_bf16(acc[w][0], a0.x, a1.x, a0.y, a1.y, wv.x, wv.y);
                        ptx::mma_m16n8k16_bf16(acc[w][1], a0.z, a1.z, a0.w, a1.w, wv.z, wv.w);
                    }
                }
#pragma unroll
                for (int w = 0; w < ROUTER_WARPS; ++w)
#pragma unroll
                    for (int i = 0; i < 4; ++i) cw[w][i] += acc[w][0][i] + acc[w][1][i];
            }
            float c[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) c[i] = cw[0][i];
#pragma unroll
            for (int w = 1; w < ROUTER_WARPS; ++w)
#pragma unroll
                for (int i = 0; i < 4; ++i) c[i] += cw[w][i];
            float L[MAX_E];
            const int qbase = lane & ~3;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float t0 = __shfl_sync(full, c[0], qbase + j);
                const float t1 = __shfl_sync(full, c[1], qbase + j);
                const float t2 = __shfl_sync(full, c[2], qbase + j);
                const float t3 = __shfl_sync(full, c[3], qbase + j);
                L[2 * j] = (q == 0) ? t0 : t2;
                L[2 * j + 1] = (q == 0) ? t1 : t3;
            }
            const int lrow = (q == 0) ? g : g + 8;  // this lane's token inside the tile (lanes q < 2)
            const int row = tile * TILE_TOKENS + lrow;
            const bool active = (q < 2) && (row < T);
            const uint32_t below = (1u << (4 * g)) - 1u;
            const uint32_t lower_mask = (q == 0) ? (below & 0x11111111u) : (0x11111111u | (below & 0x22222222u));
            const RouteSel rs = route_finish(L, active, lower_mask, row, tile, lane, a.bias, cb, a.E, a.top_k, a.logits, a.sel, a.gates,
                                             a.tile_counts);

            // ---- 2. exclusive prefix of this tile's counts over all earlier tiles (decoupled look-back)
            uint32_t* my_state = a.tile_state + (size_t)tile * MAX_E;
            const bool publish = tile != a.stall_tile;
            int run[MAX_E];
#pragma unroll
            for (int e = 0; e < MAX_E; ++e) run[e] = 0;
            bool ok = true;
            if (tile > 0) {
                if (publish && lane < MAX_E) st_relaxed_4(my_state + lane, RD_AGG | (uint32_t)rs.my_count);
                uint32_t open = 0xffu;  // experts whose walk has not yet met an inclusive prefix (warp-uniform)
                int base = tile - 1;
                const long long t_start = clock64();
                while (open) {
                    const int p = base - lane;
                    uint4 w0 = make_uint4(RD_INCL, RD_INCL, RD_INCL, RD_INCL), w1 = w0;  // before tile 0: prefix 0
                    if (p >= 0) {
                        w0 = ld_relaxed_16(a.tile_state + (size_t)p * MAX_E);
                        w1 = ld_relaxed_16(a.tile_state + (size_t)p * MAX_E + 4);
                    }
                    const uint32_t w[MAX_E] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                    uint32_t incl_m[MAX_E], need_m[MAX_E];
                    bool usable = true;
#pragma unroll
                    for (int e = 0; e < MAX_E; ++e) {
                        const uint32_t flag = w[e] >> 30;
                        incl_m[e] = __ballot_sync(full, flag == 2u);
                        const uint32_t unset = __ballot_sync(full, flag == 0u);
                        // lanes up to and including the nearest inclusive word (all 32 when the window has none)
                        need_m[e] = incl_m[e] ? ((2u << (__ffs(incl_m[e]) - 1)) - 1u) : full;
                        if (((open >> e) & 1u) && (unset & need_m[e])) usable = false;
                    }
                    if (!usable) {
                        // some earlier tile has not published yet: look at the same window again
                        const bool give_up = __shfl_sync(full, (int)(clock64() - t_start > a.wait_cycles || *abort_flag != 0), 0) != 0;
                        if (give_up) {
                            ok = false;
                            break;
                        }
                        if (a.poll_sleep_ns > 0) __nanosleep(a.poll_sleep_ns);
                        continue;
                    }
#pragma unroll
                    for (int e = 0; e < MAX_E; ++e) {
                        if ((open >> e) & 1u) {
                            const int v = ((need_m[e] >> lane) & 1u) ? (int)(w[e] & RD_VAL) : 0;
                            run[e] += __reduce_add_sync(full, v);
                            if (incl_m[e]) open &= ~(1u << e);
                        }
                    }
                    base -= 32;
                }
            }
            if (!ok) {
                if (lane == 0) *abort_flag = 1;
                break;
            }
            int mine = 0;  // lane e < 8: exclusive prefix of expert e
#pragma unroll
            for (int e = 0; e < MAX_E; ++e) mine = (lane == e) ? run[e] : mine;
            if (lane < MAX_E) {
                if (publish) st_relaxed_4(my_state + lane, RD_INCL | (uint32_t)(mine + rs.my_count));
                a.tile_prefix[(size_t)tile * MAX_E + lane] = mine;
            }
            if (tile == ntiles - 1)
                plan_fixed_stride_warp(a.meta, a.mtile_slot, a.mtile_row, a.E, a.seg_stride, a.pad_rows, mine + rs.my_count, lane);

            // ---- 3. rows to their segments, straight out of the stage buffer
            if (active) {
                int e1 = 0, e2 = 0;
#pragma unroll
                for (int e = 0; e < MAX_E; ++e) {
                    e1 = (rs.i1 == e) ? run[e] : e1;
                    e2 = (rs.i2 == e) ? run[e] : e2;
                }
                int p1 = rs.i1 * a.seg_stride + e1 + rs.r1;
                int p2 = rs.i2 >= 0 ? rs.i2 * a.seg_stride + e2 + rs.r2 : -1;
                if (!PRICHS_ROW_OK(e1 + rs.r1, a.seg_stride, a.status)) p1 = -1;
                if (p2 >= 0 && !PRICHS_ROW_OK(e2 + rs.r2, a.seg_stride, a.status)) p2 = -1;
                *reinterpret_cast<int2*>(a.pos + (size_t)row * 2) = make_int2(p1, p2);
                const uint8_t* src = stage + (size_t)lrow * rowb;
                if (p1 >= 0) ptx::bulk_store_1d(a.xp + (size_t)p1 * d, src, (uint32_t)(2 * d));
                if (p2 >= 0) ptx::bulk_store_1d(a.xp + (size_t)p2 * d, src, (uint32_t)(2 * d));
                ptx::bulk_commit();
                ptx::bulk_wait_read<0>();
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[warp]);
        }
        ptx::bulk_wait_all();  // this lane's copies have been written before the CTA leaves
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int aborted = *abort_flag;
        if (aborted) atomicExch(a.status, -5);
        // Every ticket of this CTA has been drawn and every look-back of its warps has ended (barrier above). The CTA
        // that leaves last therefore sees no reader or writer of the scratch state any more and clears it.
        s_last = (atomicAdd(a.ctl + 1, 1) == (int)gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        for (int i = threadIdx.x; i < ntiles * MAX_E / 4; i += RD_THREADS) reinterpret_cast<uint4*>(a.tile_state)[i] = make_uint4(0, 0, 0, 0);
        if (threadIdx.x == 0) {
            a.ctl[0] = 0;
            a.ctl[1] = 0;
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Router of the fp32-fidelity mode: x and W_r stay fp32 (FMA accumulation), one warp per token, one CTA
// (16 warps) per 16-token tile. Also writes the bf16 hi/lo split of x, [T, 2d] = [hi | lo], which the
// expert GEMMs consume.  wr8: [d][8] fp32 (columns >= E are zero).
__global__ void __launch_bounds__(512)
router_f32_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ xs, const float* __restrict__ wr8,
                  const float* __restrict__ bias, const ConceptBias cb, int T, int d, int E, int top_k,
                  float* __restrict__ logits, int* __restrict__ sel, float* __restrict__ gates,
                  int* __restrict__ tile_counts) {
    __shared__ float sl[TILE_TOKENS][MAX_E];
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x;
    const int row = tile * TILE_TOKENS + warp;
    if (row < T) {
        float acc[MAX_E];
#pragma unroll
        for (int e = 0; e < MAX_E; ++e) acc[e] = 0.f;
        const float* xr = x + (size_t)row * d;
        __nv_bfloat16* xo = xs + (size_t)row * 2 * d;
        for (int k = lane * 4; k < d; k += 128) {
            const float4 v = *reinterpret_cast<const float4*>(xr + k);
            const float xv[4] = {v.x, v.y, v.z, v.w};
            __nv_bfloat16 hi[4], lo[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                hi[j] = __float2bfloat16_rn(xv[j]);
                lo[j] = __float2bfloat16_rn(xv[j] - __bfloat162float(hi[j]));
                const float4 w0 = __ldg(reinterpret_cast<const float4*>(wr8 + (size_t)(k + j) * MAX_E));
                const float4 w1 = __ldg(reinterpret_cast<const float4*>(wr8 + (size_t)(k + j) * MAX_E + 4));
                acc[0] = fmaf(xv[j], w0.x, acc[0]);
                acc[1] = fmaf(xv[j], w0.y, acc[1]);
                acc[2] = fmaf(xv[j], w0.z, acc[2]);
                acc[3] = fmaf(xv[j], w0.w, acc[3]);
                acc[4] = fmaf(xv[j], w1.x, acc[4]);
                acc[5] = fmaf(xv[j], w1.y, acc[5]);
                acc[6] = fmaf(xv[j], w1.z, acc[6]);
                acc[7] = fmaf(xv[j], w1.w, acc[7]);
            }
            *reinterpret_cast<uint2*>(xo + k) = *reinterpret_cast<const uint2*>(hi);
            *reinterpret_cast<uint2*>(xo + d + k) = *reinterpret_cast<const uint2*>(lo);
        }
#pragma unroll
        for (int e = 0; e < MAX_E; ++e) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
        }
        if (lane == 0) {
#pragma unroll
            for (int e = 0; e < MAX_E; ++e) sl[warp][e] = acc[e];
        }
    }
    __syncthreads();
    if (warp == 0) {
        const int r = tile * TILE_TOKENS + lane;
        const bool active = lane < TILE_TOKENS && r < T;
        float L[MAX_E];
#pragma unroll
        for (int e = 0; e < MAX_E; ++e) L[e] = active ? sl[lane][e] : 0.f;
        route_finish(L, active, (1u << lane) - 1u, r, tile, lane, bias, cb, E, top_k, logits, sel, gates,
                     tile_counts);
    }
}

// ---------------------------------------------------------------------------------------------------
// Placement plan from the counts matrix (one CTA). For every expert e, owned by rank e / El:
//   total[e] = sum_s cmat[s][e],  src_off[e] = sum_{s < rank} cmat[s][e],
//   seg_base[e] = row, in the owner's permuted region, where expert e's segment starts:
//     seg_stride == 0 (expert parallel): the padded totals (to pad_rows, a multiple of 128) of the owner's lower
//                     experts, so the region is dense;
//     seg_stride > 0  (all experts local): le * seg_stride -- every expert has a segment of fixed capacity, so a
//                     row's place depends only on the rows before it, never on the totals (this is what lets one
//                     pass over the tokens route and place them).
// For the local experts it also fills the table the grouped GEMM walks: entry i is the i-th 128-row tile that
// holds rows, mtile_row[i] its tile index inside the region (null = dense region, tile i is entry i) and
// mtile_slot[i] its weight slot. A segment contributes whole pad_rows blocks; a 128-row tile of such a block that
// holds only padding rows is marked (-1 - slot).
// `local_counts` (single rank only): the totals in shared memory, straight from the scan, so that this plan
// reads nothing back from global memory; null = take them from meta->cmat.
__device__ __forceinline__ void plan_from_cmat(RouteMeta* meta, int* __restrict__ mtile_slot, int* __restrict__ mtile_row,
                                               int E, int El, int world, int rank, int cap_rows, int pad_rows,
                                               int seg_stride, int* __restrict__ status, const int* local_counts) {
    __shared__ int s_total[MAX_E], s_base[MAX_E + 1], s_tile0[MAX_E + 1], s_over;
    const int tid = threadIdx.x;
    if (tid < MAX_E) {
        int tot = 0, off = 0;
        if (tid < E) {
            if (local_counts != nullptr) {
                tot = local_counts[tid];
            } else {
                for (int s = 0; s < world; ++s) {
                    const int c = meta->cmat[s * MAX_E + tid];
                    tot += c;
                    if (s < rank) off += c;
                }
            }
        }
        s_total[tid] = tot;
        meta->total[tid] = tot;
        meta->src_off[tid] = off;
    }
    __syncthreads();
    if (tid == 0) {
        int recv = 0, over = 0;
        for (int o = 0; o < world; ++o) {
            int base = 0, tiles = 0;
            for (int le = 0; le < El; ++le) {
                const int e = o * El + le;
                const int padded = (s_total[e] + pad_rows - 1) / pad_rows * pad_rows;
                if (seg_stride > 0) {
                    base = le * seg_stride;
                    if (padded > seg_stride) over = 1;
                }
                meta->seg_base[e] = base;
                if (o == rank) {
                    s_base[le] = base;
                    s_tile0[le] = tiles;
                    recv += s_total[e];
                }
                base += padded;
                tiles += padded / 128;
            }
            // every rank evaluates every owner's region, so that all of them skip the exchange together
            if (base > cap_rows) over = 1;
            if (o == rank) {
                s_base[El] = base;
                s_tile0[El] = tiles;
            }
        }
        s_over = over;
        meta->overflow = over;
        meta->recv_rows = recv;
        meta->n_routed_mtiles = over ? 0 : s_tile0[El];
        if (over) atomicExch(status, -2);
    }
    __syncthreads();
    const int ntiles = s_over ? 0 : s_tile0[El];
    for (int i = tid; i < ntiles; i += blockDim.x) {
        int le = 0;
        while (le + 1 < El && i >= s_tile0[le + 1]) ++le;
        const int j = i - s_tile0[le];  // tile inside the segment
        const bool padding_only = j * 128 >= s_total[rank * El + le];
        mtile_slot[i] = padding_only ? -1 - le : le;
        if (mtile_row != nullptr) mtile_row[i] = s_base[le] / 128 + j;
    }
}

// Exclusive prefix sum of the per-tile histograms over tiles by one CTA of NT threads (each thread owns a
// contiguous run of tiles), totals into meta->counts and row `rank` of meta->cmat; returns the totals in shared
// memory (valid for all threads after the next barrier; this function ends with one). The histograms are read
// with ld.global.cg: when this runs at the tail of the router kernel they were written by other CTAs of the same
// launch. A run of up to SCAN_KEEP tiles stays in registers between the two passes, so the CTA makes one trip to
// memory, not two.
template <int NT, int SCAN_KEEP>
__device__ __forceinline__ const int* scan_tiles(const int* tile_counts, int* __restrict__ tile_prefix, int ntiles,
                                                 RouteMeta* meta, int rank) {
    constexpr int NW = NT / 32;
    __shared__ int warp_tot[NW][MAX_E];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = (ntiles + NT - 1) / NT;
    const int t0 = min(tid * per, ntiles), t1 = min(t0 + per, ntiles);
    const bool keep = per <= SCAN_KEEP;
    int4 ka[SCAN_KEEP], kb[SCAN_KEEP];
    int tot[MAX_E];
#pragma unroll
    for (int e = 0; e < MAX_E; ++e) tot[e] = 0;
    auto add = [&](const int4& a, const int4& b, int (&v)[MAX_E]) {
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
        v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
    };
    if (keep) {
#pragma unroll
        for (int j = 0; j < SCAN_KEEP; ++j) {
            ka[j] = kb[j] = make_int4(0, 0, 0, 0);
            if (t0 + j < t1) {
                ka[j] = __ldcg(reinterpret_cast<const int4*>(tile_counts + (size_t)(t0 + j) * MAX_E));
                kb[j] = __ldcg(reinterpret_cast<const int4*>(tile_counts + (size_t)(t0 + j) * MAX_E + 4));
            }
        }
#pragma unroll
        for (int j = 0; j < SCAN_KEEP; ++j) add(ka[j], kb[j], tot);
    } else {
        for (int t = t0; t < t1; ++t)
            add(__ldcg(reinterpret_cast<const int4*>(tile_counts + (size_t)t * MAX_E)),
                __ldcg(reinterpret_cast<const int4*>(tile_counts + (size_t)t * MAX_E + 4)), tot);
    }
    int inc[MAX_E];
#pragma unroll
    for (int e = 0; e < MAX_E; ++e) {
        int v = tot[e];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += n;
        }
        inc[e] = v;
        if (lane == 31) warp_tot[warp][e] = v;
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int e = 0; e < MAX_E; ++e) {
            int v = lane < NW ? warp_tot[lane][e] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += n;
            }
            if (lane < NW) warp_tot[lane][e] = v;  // inclusive over warps
        }
    }
    __syncthreads();
    int run[MAX_E];
#pragma unroll
    for (int e = 0; e < MAX_E; ++e) run[e] = inc[e] - tot[e] + (warp > 0 ? warp_tot[warp - 1][e] : 0);
    auto put = [&](int t) {
        *reinterpret_cast<int4*>(tile_prefix + (size_t)t * MAX_E) = make_int4(run[0], run[1], run[2], run[3]);
        *reinterpret_cast<int4*>(tile_prefix + (size_t)t * MAX_E + 4) = make_int4(run[4], run[5], run[6], run[7]);
    };
    if (keep) {
#pragma unroll
        for (int j = 0; j < SCAN_KEEP; ++j) {
            if (t0 + j < t1) {
                put(t0 + j);
                add(ka[j], kb[j], run);
            }
        }
    } else {
        for (int t = t0; t < t1; ++t) {
            put(t);
            add(__ldcg(reinterpret_cast<const int4*>(tile_counts + (size_t)t * MAX_E)),
                __ldcg(reinterpret_cast<const int4*>(tile_counts + (size_t)t * MAX_E + 4)), run);
        }
    }
    if (tid < MAX_E) {
        const int c = warp_tot[NW - 1][tid];
        meta->counts[tid] = c;
        meta->cmat[rank * MAX_E + tid] = c;
    }
    __syncthreads();
    return &warp_tot[NW - 1][0];
}

// The scan as its own launch (one CTA of 1024 threads). With `fuse_plan` (single rank) the placement plan follows
// in the same launch.
__global__ void __launch_bounds__(1024)
scan_kernel(const int* tile_counts, int* __restrict__ tile_prefix, int ntiles, RouteMeta* meta,
            int* __restrict__ mtile_slot, int* __restrict__ mtile_row, int E, int El, int world, int rank, int cap_rows,
            int fuse_plan, int pad_rows, int seg_stride, int* __restrict__ status) {
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    const int* totals = scan_tiles<1024, 2>(tile_counts, tile_prefix, ntiles, meta, rank);
    if (fuse_plan)
        plan_from_cmat(meta, mtile_slot, mtile_row, E, El, world, rank, cap_rows, pad_rows, seg_stride, status, world == 1 ? totals : nullptr);
}

// Placement plan as its own launch (expert-parallel mode, after the counts of all ranks were gathered).
__global__ void __launch_bounds__(256)
plan_kernel(RouteMeta* meta, int* __restrict__ mtile_slot, int E, int El, int world, int rank, int cap_rows,
            int pad_rows, int* __restrict__ status) {
    plan_from_cmat(meta, mtile_slot, nullptr, E, El, world, rank, cap_rows, pad_rows, 0, status, nullptr);
}

// ---------------------------------------------------------------------------------------------------
// Dispatch (token permute): one warp per token. The token's row (row_elems bf16, a multiple of 256) is read
// once and written to the segment of each selected expert, tokens in ascending order inside a segment, as in
// the reference's bins (moe.rs:140,155-164). The destination buffer belongs to the expert's owner rank: a
// plain pointer for local experts, a peer-mapped pointer over NVLink otherwise. pos[t,j] keeps the row.
__global__ void __launch_bounds__(256)
dispatch_kernel(const __nv_bfloat16* __restrict__ xs, int row_elems, int T, const int* __restrict__ sel,
                const int* __restrict__ tile_prefix, const RouteMeta* __restrict__ meta, const __grid_constant__ PeerPtrs dst, int El,
                int* __restrict__ pos, int cap_rows, int* __restrict__ status) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    if (meta->overflow) return;
    // grid-stride over tokens: the expert-parallel forward caps the grid so that this NVLink-bound kernel
    // does not flood the SMs it shares with a concurrently running GEMM
    for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    int my_row = -1, my_owner = 0;
    if (lane < 2) {
        const int s = sel[(size_t)t * 2 + lane];
        if (s >= 0) {
            const int e = s & 0xff, lr = s >> 8;
            my_row = meta->seg_base[e] + meta->src_off[e] + tile_prefix[(size_t)(t / TILE_TOKENS) * MAX_E + e] + lr;
            my_owner = e / El;
            if (!PRICHS_ROW_OK(my_row, cap_rows, status)) my_row = -1;
            pos[(size_t)t * 2 + lane] = my_row;
        } else {
            pos[(size_t)t * 2 + lane] = -1;
        }
    }
    const int row0 = __shfl_sync(0xffffffffu, my_row, 0), row1 = __shfl_sync(0xffffffffu, my_row, 1);
    const int own0 = __shfl_sync(0xffffffffu, my_owner, 0), own1 = __shfl_sync(0xffffffffu, my_owner, 1);
    const uint4* src = reinterpret_cast<const uint4*>(xs + (size_t)t * row_elems);
    uint4* d0 = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[own0]) + (size_t)max(row0, 0) * row_elems);
    uint4* d1 = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[own1]) + (size_t)max(row1, 0) * row_elems);
    const int nvec = row_elems / 8;
#pragma unroll 6
    for (int c = lane; c < nvec; c += 32) {
        const uint4 v = ptx::ld_stream_16(src + c);
        if (row0 >= 0) d0[c] = v;
        if (row1 >= 0) d1[c] = v;
    }
    }
}

// ---------------------------------------------------------------------------------------------------
// Dispatch for the expert-parallel exchange, on a handful of SMs: the same placement as dispatch_kernel, but a row
// travels global memory -> shared memory -> owner's receive region as bulk copies (one load, one or two stores of
// the whole row), so a CTA keeps its whole ring of tile buffers in flight with three instructions per token instead
// of one 16-byte load and two stores per lane and step. Stores over NVLink are posted: a few such CTAs saturate the
// link, and the SMs the grouped GEMMs must leave free for the exchange shrink accordingly.
// One producer thread per CTA copies 16-token tiles (tile = blockIdx.x, + gridDim.x, ...) into a ring of `stages`
// buffers; consumer warp w owns stage w: lanes 0..15 look up their token's rows, record them in `pos`, and issue the
// stores; the stage goes back to the producer when the stores have read it. Waits are bounded (status -5).
constexpr int DB_MAX_STAGES = 4;
constexpr int DB_THREADS = (DB_MAX_STAGES + 1) * 32;
__host__ __device__ inline int db_smem_bytes(int row_bytes, int stages) { return stages * TILE_TOKENS * row_bytes + 2 * DB_MAX_STAGES * 8 + 16; }

__global__ void __launch_bounds__(DB_THREADS, 1)
dispatch_bulk_kernel(const __nv_bfloat16* __restrict__ xs, int row_elems, int T, const int* __restrict__ sel,
                     const int* __restrict__ tile_prefix, const RouteMeta* __restrict__ meta, const __grid_constant__ PeerPtrs dst, int El,
                     int* __restrict__ pos, int cap_rows, int stages, long long wait_cycles, int* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t dsm[];
    const int row_bytes = row_elems * 2;
    const int stage_bytes = TILE_TOKENS * row_bytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(dsm + (size_t)stages * stage_bytes);
    uint64_t* empty_bar = full_bar + DB_MAX_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + DB_MAX_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    __syncthreads();
    const int ntiles = (T + TILE_TOKENS - 1) / TILE_TOKENS;
    const int my_tiles = (int)blockIdx.x < ntiles ? (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const bool skip = meta->overflow != 0;  // the plan did not fit: every rank skips the exchange
    if (warp == DB_MAX_STAGES) {
        if (lane == 0 && !skip) {
            int issued = 0;
            bool ok = true;
            for (int it = 0; it < my_tiles; ++it) {
                const int s = it % stages;
                if (!ptx::mbar_wait_bounded(&empty_bar[s], (uint32_t)(((it / stages) & 1) ^ 1), abort_flag, wait_cycles)) {
                    ok = false;
                    break;
                }
                const int tile = blockIdx.x + it * gridDim.x;
                const int rows = min(TILE_TOKENS, T - tile * TILE_TOKENS);
                ptx::mbar_expect_tx(&full_bar[s], (uint32_t)(rows * row_bytes));
                ptx::bulk_load_1d(dsm + (size_t)s * stage_bytes, xs + (size_t)tile * TILE_TOKENS * row_elems, (uint32_t)(rows * row_bytes), &full_bar[s]);
                ++issued;
            }
            if (!ok) {
                for (int i = max(0, issued - stages); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!ptx::mbar_try_wait(&full_bar[i % stages], (uint32_t)((i / stages) & 1)) && clock64() - t0 < wait_cycles) {
                    }
                }
            }
        }
    } else if (warp < stages && !skip) {
        const uint8_t* stage = dsm + (size_t)warp * stage_bytes;
        for (int it = warp, n = 0; it < my_tiles; it += stages, ++n) {
            const int tile = blockIdx.x + it * gridDim.x;
            const int t = tile * TILE_TOKENS + lane;
            // the routing look-ups do not need the rows: they overlap the copy
            int row0 = -1, row1 = -1, own0 = 0, own1 = 0;
            if (lane < TILE_TOKENS && t < T) {
                const int2 s2 = *reinterpret_cast<const int2*>(sel + (size_t)t * 2);
                if (s2.x >= 0) {
                    const int e = s2.x & 0xff;
                    row0 = meta->seg_base[e] + meta->src_off[e] + tile_prefix[(size_t)tile * MAX_E + e] + (s2.x >> 8);
                    own0 = e / El;
                }
                if (s2.y >= 0) {
                    const int e = s2.y & 0xff;
                    row1 = meta->seg_base[e] + meta->src_off[e] + tile_prefix[(size_t)tile * MAX_E + e] + (s2.y >> 8);
                    own1 = e / El;
                }
                if (row0 >= 0 && !PRICHS_ROW_OK(row0, cap_rows, status)) row0 = -1;
                if (row1 >= 0 && !PRICHS_ROW_OK(row1, cap_rows, status)) row1 = -1;
                *reinterpret_cast<int2*>(pos + (size_t)t * 2) = make_int2(row0, row1);
            }
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(&full_bar[warp], (uint32_t)(n & 1), abort_flag, wait_cycles))) break;
            if (row0 >= 0 || row1 >= 0) {
                const uint8_t* src = stage + (size_t)lane * row_bytes;
                if (row0 >= 0) ptx::bulk_store_1d(reinterpret_cast<__nv_bfloat16*>(dst.p[own0]) + (size_t)row0 * row_elems, src, (uint32_t)row_bytes);
                if (row1 >= 0) ptx::bulk_store_1d(reinterpret_cast<__nv_bfloat16*>(dst.p[own1]) + (size_t)row1 * row_elems, src, (uint32_t)row_bytes);
                ptx::bulk_commit();
                ptx::bulk_wait_read<0>();
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[warp]);
        }
        ptx::bulk_wait_all();
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(status, -5);
}

// ---------------------------------------------------------------------------------------------------
// Readiness flags of the expert-parallel exchange. Every rank owns a small array of ints, flags[kind][wave][source],
// that its peers write over NVLink: after the kernel that produced something a peer will read (kind 0: this rank's
// rows of a wave have been stored into the peers' receive regions; kind 1: this rank's expert outputs of a wave are
// complete) a one-warp kernel stores the forward's sequence number into slot [kind][wave][this rank] of EVERY
// rank's array, with release semantics at system scope; stream order puts it after the producing kernel. Before the
// kernel that consumes the data a one-warp kernel polls the local slots of all sources until they carry at least
// that sequence number (acquire at system scope). Sequence numbers only grow, so nothing is ever reset.
// The wait is bounded: after `budget_cycles` it records -5 in the status word and returns; the stream goes on, the
// forward's result is then undefined and prichs_moe_sync_status reports PRICHS_ERR_TIMEOUT.
constexpr int EP_FLAG_INTS = 2 * 4 * MAX_RANKS;  // [kind][wave][source]
__host__ __device__ inline int ep_flag_index(int kind, int wave, int source) { return (kind * 4 + wave) * MAX_RANKS + source; }

__global__ void ep_signal_kernel(const __grid_constant__ PeerPtrs flag_arrays, int kind, int wave, int rank, int world, int seq) {
    const int r = threadIdx.x;
    if (r < world) {
        int* dst = reinterpret_cast<int*>(flag_arrays.p[r]) + ep_flag_index(kind, wave, rank);
        __threadfence_system();
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(seq) : "memory");
    }
}

__global__ void ep_wait_kernel(const int* __restrict__ flags, int kind, int wave, int world, int seq, long long budget_cycles,
                               int* __restrict__ status) {
    const int r = threadIdx.x;
    if (r < world) {
        const int* src = flags + ep_flag_index(kind, wave, r);
        const long long t0 = clock64();
        for (;;) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
            if ((int)((unsigned)v - (unsigned)seq) >= 0) break;  // wrap-safe comparison of sequence numbers
            if (clock64() - t0 > budget_cycles) {
                atomicExch(status, -5);
                break;
            }
            __nanosleep(100);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Combine: one warp per token, gather-based (no atomics; the reference's GPU path uses atomicAdd,
// crates/prichs-cuda/src/kernels.cu:906-924). Follows the CPU order: out = shared row; then the selected
// experts in ascending expert index, out += gate * row (multiply and add rounded separately, moe.rs:178-184);
// finally the optional residual, resid + out (block.rs:67).
// Y rows: the shared expert's at row t of the local buffer, a routed expert's at (routed_base + pos) of its
// owner's buffer. YF32: expert outputs are fp32 (fp32-fidelity mode) else bf16. RES: 0 none, 1 bf16, 2 fp32.
template <bool YF32, bool OUTF32, int RES>
__global__ void __launch_bounds__(256)
combine_kernel(const void* __restrict__ y_local, const __grid_constant__ PeerPtrs y_peers, long long routed_base_rows,
               const int* __restrict__ sel, const float* __restrict__ gates, const int* __restrict__ pos,
               const void* __restrict__ resid, void* __restrict__ out, int T, int d, int El, int cap_rows, int* __restrict__ status) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {  // grid-stride (see dispatch_kernel)
    const int2 s = *reinterpret_cast<const int2*>(sel + (size_t)t * 2);
    const float2 gw = *reinterpret_cast<const float2*>(gates + (size_t)t * 2);
    const int2 p = *reinterpret_cast<const int2*>(pos + (size_t)t * 2);
    int ea = s.x & 0xff, eb = (s.y >= 0) ? (s.y & 0xff) : -1;
    float ga = gw.x, gb = gw.y;
    int pa = p.x, pb = p.y;
    if (eb >= 0 && eb < ea) {
        int ti = ea; ea = eb; eb = ti;
        ti = pa; pa = pb; pb = ti;
        const float tf = ga; ga = gb; gb = tf;
    }
    const bool has_b = eb >= 0;
#ifdef PRICHS_BOUNDS_CHECK
    if (!PRICHS_ROW_OK(pa, cap_rows, status) || (has_b && !PRICHS_ROW_OK(pb, cap_rows, status)) || ea / El >= MAX_RANKS) continue;
#endif
    using YT = typename std::conditional<YF32, float, __nv_bfloat16>::type;
    const YT* ys = reinterpret_cast<const YT*>(y_local) + (size_t)t * d;
    const YT* ya = reinterpret_cast<const YT*>(y_peers.p[ea / El]) + (size_t)(routed_base_rows + pa) * d;
    const YT* yb = has_b ? reinterpret_cast<const YT*>(y_peers.p[eb / El]) + (size_t)(routed_base_rows + pb) * d : ys;

    auto load8 = [](const YT* ptr, float (&v)[8]) {
        if constexpr (YF32) {
            const uint4 a = ptx::ld_stream_16(ptr), b = ptx::ld_stream_16(ptr + 4);
            v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
            v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
        } else {
            const uint4 a = ptx::ld_stream_16(ptr);
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[2 * j] = __uint_as_float(w[j] << 16);
                v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
        }
    };

#pragma unroll 2
    for (int c = lane * 8; c < d; c += 256) {
        float o[8], a[8], b[8];
        load8(ys + c, o);
        load8(ya + c, a);
        if (has_b) load8(yb + c, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            o[j] = __fadd_rn(o[j], __fmul_rn(ga, a[j]));
            if (has_b) o[j] = __fadd_rn(o[j], __fmul_rn(gb, b[j]));
        }
        if (RES == 1) {
            const uint4 r = ptx::ld_stream_16(reinterpret_cast<const __nv_bfloat16*>(resid) + (size_t)t * d + c);
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o[2 * j] = __fadd_rn(__uint_as_float(w[j] << 16), o[2 * j]);
                o[2 * j + 1] = __fadd_rn(__uint_as_float(w[j] & 0xffff0000u), o[2 * j + 1]);
            }
        } else if (RES == 2) {
            const float* rp = reinterpret_cast<const float*>(resid) + (size_t)t * d + c;
            const uint4 r0 = ptx::ld_stream_16(rp), r1 = ptx::ld_stream_16(rp + 4);
            const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __fadd_rn(__uint_as_float(w[j]), o[j]);
        }
        if (OUTF32) {
            float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)t * d + c);
            op[0] = make_float4(o[0], o[1], o[2], o[3]);
            op[1] = make_float4(o[4], o[5], o[6], o[7]);
        } else {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 v = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
                w[j] = *reinterpret_cast<uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)t * d + c) =
                make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    }
}

// ---------------------------------------------------------------------------------------------------
// Pre-norm of the block's MoE sub-layer (crates/prichs-model/src/block.rs:64, rms_norm of
// crates/prichs-core/src/ops.rs:109-135): out = (x * inv_rms) * weight with inv_rms = 1 / sqrt(mean(x^2) + eps).
// One warp per row, the row stays in registers between the two passes. XF32: x is fp32 (else bf16);
// OF32: the normalised row is written as fp32 (fp32-fidelity mode) else bf16. d is a multiple of 256.
template <bool XF32, bool OF32, int MAXC>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const void* __restrict__ x, const float* __restrict__ weight, float eps, void* __restrict__ out, int T, int d) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + warp;
    if (t >= T) return;
    float v[MAXC][8];
    float ss = 0.f;
    const int nchunk = d / 256;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        if (i < nchunk) {
            const int c = i * 256 + lane * 8;
            if (XF32) {
                const float* p = reinterpret_cast<const float*>(x) + (size_t)t * d + c;
                const uint4 a = ptx::ld_stream_16(p), b = ptx::ld_stream_16(p + 4);
                v[i][0] = __uint_as_float(a.x); v[i][1] = __uint_as_float(a.y); v[i][2] = __uint_as_float(a.z); v[i][3] = __uint_as_float(a.w);
                v[i][4] = __uint_as_float(b.x); v[i][5] = __uint_as_float(b.y); v[i][6] = __uint_as_float(b.z); v[i][7] = __uint_as_float(b.w);
            } else {
                const uint4 a = ptx::ld_stream_16(reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)t * d + c);
                const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[i][2 * j] = __uint_as_float(w[j] << 16);
                    v[i][2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv_rms = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        if (i < nchunk) {
            const int c = i * 256 + lane * 8;
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(weight + c)), w1 = __ldg(reinterpret_cast<const float4*>(weight + c + 4));
            const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            float o8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o8[j] = __fmul_rn(__fmul_rn(v[i][j], inv_rms), wv[j]);
            if (OF32) {
                float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)t * d + c);
                op[0] = make_float4(o8[0], o8[1], o8[2], o8[3]);
                op[1] = make_float4(o8[4], o8[5], o8[6], o8[7]);
            } else {
                uint32_t pk[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(o8[2 * j], o8[2 * j + 1]);
                    pk[j] = *reinterpret_cast<uint32_t*>(&b2);
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)t * d + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// b_i += gamma * (top_k / E - count_i / total_tokens), each operation rounded on its own like the
// reference's f32 arithmetic (moe.rs:237-244). count_i is the total over all ranks.
// The counts come from the routing summary of the last forward (`meta`) or, when it is null, from the kernel
// arguments (`host_counts`, the reference's call shape with host-side counts).
struct ExpertCounts {
    unsigned long long c[MAX_E];
};
__global__ void bias_update_kernel(float* __restrict__ bias, const RouteMeta* __restrict__ meta, const ExpertCounts host_counts,
                                   int E, int top_k, float gamma, unsigned long long total_tokens) {
    const int i = threadIdx.x;
    if (i >= E || total_tokens == 0ull) return;
    const unsigned long long count = meta != nullptr ? (unsigned long long)meta->total[i] : host_counts.c[i];
    const float target_load = __fdiv_rn((float)top_k, (float)E);
    const float actual_load = __fdiv_rn((float)count, (float)total_tokens);
    const float diff = __fsub_rn(target_load, actual_load);
    bias[i] = __fadd_rn(bias[i], __fmul_rn(gamma, diff));
}

}  // namespace route
