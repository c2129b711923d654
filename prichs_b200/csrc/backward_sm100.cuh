// Element-wise and data-movement kernels of the MoE layer's backward pass (the MoE part of the reference's block
// backward, crates/prichs-model/src/model.rs:566-766). The matrix products of the backward pass run on the grouped
// tcgen05 GEMM of expert_gemm_sm100.cuh; this file holds what sits between them:
//
//   dy_prepare_kernel   d_out -> the A operand of the first backward GEMM, in the row space of the forward
//                       (rows [0,T): d_out itself for the shared expert; row Tcap + pos: gate * d_out[token] for a
//                       routed assignment, model.rs:647-656) and the scalars <expert output row, d_out[token]> the
//                       router VJP needs (model.rs:654-658)
//   swiglu_bwd_kernel   d_act -> d_gate, d_up from the recomputed pre-activations (backward.rs:247-266)
//   router_vjp_kernel   scalars + gates -> d_logits (backward.rs:269-287, model.rs:735-748)
//   dwr_partial_kernel / dwr_reduce_kernel   dW_router += X^T d_logits in a fixed summation order (model.rs:750-757)
//   dx_combine_kernel   d_x = shared dX + sum over the token's experts (ascending) of gate * routed dX + d_logits W_r^T
//                       (model.rs:629-631, 724-732, 759-766); the gate weight enters a routed expert's input
//                       gradient twice, once through dY_e and once here, exactly as in the reference
//   rmsnorm_bwd_rows_kernel / dgamma_*   the block's pre-norm backward after the MoE backward (backward.rs:94-131)
//   transpose_bf16_kernel   [rows, cols] -> [cols, rows]: the weight-gradient products contract over rows, so both
//                       of their operands are fed to the K-major GEMM as transposed copies
//   grad_unpack_*       staged fp32 weight gradients -> accumulated (+=) into the caller's buffers in the reference's
//                       [in, out] layouts (matmul_at_b accumulates, ops.rs:64-82)
#pragma once

#include <cuda_bf16.h>

#include "ptx_sm100.cuh"
#include "route_sm100.cuh"

namespace bwd {

using route::MAX_E;

__device__ __forceinline__ void unpack_bf16x8(const uint4& a, float (&v)[8]) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&b2);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// One warp per token. dy: [T,d] fp32 (DYF32) or bf16. y: the forward's expert outputs (bf16), shared rows at
// [0,T), permuted row r at Tcap + r. dyall: bf16, same row space. scal: [T,2] fp32. d is a multiple of 256.
template <bool DYF32>
__global__ void __launch_bounds__(256)
dy_prepare_kernel(const void* __restrict__ dy, const __nv_bfloat16* __restrict__ y, const int* __restrict__ sel,
                  const float* __restrict__ gates, const int* __restrict__ pos, __nv_bfloat16* __restrict__ dyall,
                  float* __restrict__ scal, int T, int d, long long tcap) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + warp;
    if (t >= T) return;
    const int2 s = *reinterpret_cast<const int2*>(sel + (size_t)t * 2);
    const float2 gw = *reinterpret_cast<const float2*>(gates + (size_t)t * 2);
    const int2 p = *reinterpret_cast<const int2*>(pos + (size_t)t * 2);
    const bool has_a = s.x >= 0 && p.x >= 0, has_b = s.y >= 0 && p.y >= 0;
    float dot_a = 0.f, dot_b = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
        float v[8];
        if (DYF32) {
            const float* src = reinterpret_cast<const float*>(dy) + (size_t)t * d + c;
            const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            unpack_bf16x8(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(dy) + (size_t)t * d + c), v);
        }
        *reinterpret_cast<uint4*>(dyall + (size_t)t * d + c) = pack_bf16x8(v);
        if (has_a) {
            float ya[8], o[8];
            unpack_bf16x8(*reinterpret_cast<const uint4*>(y + (size_t)(tcap + p.x) * d + c), ya);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                o[j] = __fmul_rn(gw.x, v[j]);
                dot_a = fmaf(ya[j], v[j], dot_a);
            }
            *reinterpret_cast<uint4*>(dyall + (size_t)(tcap + p.x) * d + c) = pack_bf16x8(o);
        }
        if (has_b) {
            float yb[8], o[8];
            unpack_bf16x8(*reinterpret_cast<const uint4*>(y + (size_t)(tcap + p.y) * d + c), yb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                o[j] = __fmul_rn(gw.y, v[j]);
                dot_b = fmaf(yb[j], v[j], dot_b);
            }
            *reinterpret_cast<uint4*>(dyall + (size_t)(tcap + p.y) * d + c) = pack_bf16x8(o);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        dot_a += __shfl_xor_sync(0xffffffffu, dot_a, o);
        dot_b += __shfl_xor_sync(0xffffffffu, dot_b, o);
    }
    if (lane == 0) *reinterpret_cast<float2*>(scal + (size_t)t * 2) = make_float2(has_a ? dot_a : 0.f, has_b ? dot_b : 0.f);
}

// d_up = d_act * silu(g), d_gate = d_act * u * sig(g) * (1 + g * (1 - sig(g)))   (backward.rs:247-266).
// gu / dgu: [rows, 2f] bf16 in the column order of the first forward GEMM's B operand: blocks of 256 columns, 128
// gate columns then 128 up columns of the same hidden units. dh: [rows, f] bf16. Rows [0, T) (shared expert) and
// the 128-row tiles of the permuted region the GEMM tile table lists (tile i at row tcap + 128 * mtile_row[i]; padding
// rows included: nothing reads what is computed for them, the weight-gradient products stop at each expert's row count).
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ dgu,
                  int T, int f, long long tcap, const int* __restrict__ n_routed_mtiles, const int* __restrict__ mtile_row) {
    const long long routed_rows = 128LL * *n_routed_mtiles;
    const int vec_per_row = f / 8;  // 8 hidden units per thread and step; f is a multiple of 128
    const long long total = ((long long)T + routed_rows) * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / vec_per_row;
        const int j0 = (int)(i - r * vec_per_row) * 8;
        long long row = r;
        if (r >= T) {
            const long long rr = r - T;
            const int ti = (int)(rr >> 7);
            row = tcap + 128LL * (mtile_row ? mtile_row[ti] : ti) + (rr & 127);
        }
        const int blk = j0 >> 7, within = j0 & 127;
        const size_t gcol = (size_t)blk * 256 + within;
        float dy[8], g[8], u[8], dg[8], du[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(dh + (size_t)row * f + j0), dy);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(gu + (size_t)row * 2 * f + gcol), g);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(gu + (size_t)row * 2 * f + gcol + 128), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float sig = 1.0f / (1.0f + expf(-g[j]));
            const float silu = g[j] * sig;
            const float dsilu = sig * (1.0f + g[j] * (1.0f - sig));
            du[j] = dy[j] * silu;
            dg[j] = dy[j] * u[j] * dsilu;
        }
        *reinterpret_cast<uint4*>(dgu + (size_t)row * 2 * f + gcol) = pack_bf16x8(dg);
        *reinterpret_cast<uint4*>(dgu + (size_t)row * 2 * f + gcol + 128) = pack_bf16x8(du);
    }
}

// d_logits of every token (backward.rs:269-287): weighted = sum_k g_k s_k; d_logit[sel_k] = g_k (s_k - weighted);
// all other experts 0. dlog: [T, 8] fp32.
__global__ void __launch_bounds__(256)
router_vjp_kernel(const int* __restrict__ sel, const float* __restrict__ gates, const float* __restrict__ scal,
                  float* __restrict__ dlog, int T) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int2 s = *reinterpret_cast<const int2*>(sel + (size_t)t * 2);
    const float2 g = *reinterpret_cast<const float2*>(gates + (size_t)t * 2);
    const float2 sc = *reinterpret_cast<const float2*>(scal + (size_t)t * 2);
    float out[MAX_E];
#pragma unroll
    for (int e = 0; e < MAX_E; ++e) out[e] = 0.f;
    float weighted = 0.0f;
    if (s.x >= 0) weighted += g.x * sc.x;
    if (s.y >= 0) weighted += g.y * sc.y;
    const int ea = s.x >= 0 ? (s.x & 0xff) : -1, eb = s.y >= 0 ? (s.y & 0xff) : -1;
#pragma unroll
    for (int e = 0; e < MAX_E; ++e) {
        if (e == ea) out[e] = g.x * (sc.x - weighted);
        if (e == eb) out[e] = g.y * (sc.y - weighted);
    }
    float4* o = reinterpret_cast<float4*>(dlog + (size_t)t * MAX_E);
    o[0] = make_float4(out[0], out[1], out[2], out[3]);
    o[1] = make_float4(out[4], out[5], out[6], out[7]);
}

// dW_router[k, e] += sum_t x[t, k] * d_logits[t, e]. Stage 1: CTA (column block of 64, token split s) sums its
// tokens in ascending order into part[s][k][e]; stage 2 adds the splits in ascending order into the caller's
// [d, E] buffer. Both orders are fixed, so the result does not depend on scheduling.
constexpr int DWR_SPLITS = 64;

__global__ void __launch_bounds__(512)
dwr_partial_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ dlog, float* __restrict__ part, int T, int d) {
    const int c = threadIdx.x & 63, e = threadIdx.x >> 6;  // 64 columns x 8 experts
    const int k = blockIdx.x * 64 + c;
    const int per = (T + DWR_SPLITS - 1) / DWR_SPLITS;
    const int t0 = min(T, (int)blockIdx.y * per), t1 = min(T, t0 + per);
    float acc = 0.f;
    for (int t = t0; t < t1; ++t) acc = fmaf(__bfloat162float(x[(size_t)t * d + k]), dlog[(size_t)t * MAX_E + e], acc);
    part[((size_t)blockIdx.y * d + k) * MAX_E + e] = acc;
}

__global__ void __launch_bounds__(256)
dwr_reduce_kernel(const float* __restrict__ part, float* __restrict__ grad_router, int d, int E) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;  // over d * 8
    if (i >= d * MAX_E) return;
    const int k = i / MAX_E, e = i - k * MAX_E;
    if (e >= E) return;
    float acc = 0.f;
    for (int s = 0; s < DWR_SPLITS; ++s) acc += part[(size_t)s * d * MAX_E + i];
    grad_router[(size_t)k * E + e] += acc;
}

// One warp per token: d_x[t] = dX_shared[t] + (experts ascending) gate * dX_routed[row] + sum_e d_logits[t,e] W_r[:,e].
// dxall: bf16 [rows, d] in the forward's row space; wr8: [d][8] fp32 router weights; dx: [T,d] fp32.
__global__ void __launch_bounds__(256)
dx_combine_kernel(const __nv_bfloat16* __restrict__ dxall, const int* __restrict__ sel, const float* __restrict__ gates,
                  const int* __restrict__ pos, const float* __restrict__ dlog, const float* __restrict__ wr8,
                  float* __restrict__ dx, int T, int d, long long tcap) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + warp;
    if (t >= T) return;
    const int2 s = *reinterpret_cast<const int2*>(sel + (size_t)t * 2);
    const float2 gw = *reinterpret_cast<const float2*>(gates + (size_t)t * 2);
    const int2 p = *reinterpret_cast<const int2*>(pos + (size_t)t * 2);
    int ea = s.x >= 0 ? (s.x & 0xff) : -1, eb = s.y >= 0 ? (s.y & 0xff) : -1;
    int pa = p.x, pb = p.y;
    float ga = gw.x, gb = gw.y;
    if (eb >= 0 && (ea < 0 || eb < ea)) {  // ascending expert index, as the reference's loop over the experts
        int ti = ea; ea = eb; eb = ti;
        ti = pa; pa = pb; pb = ti;
        const float tf = ga; ga = gb; gb = tf;
    }
    const bool has_a = ea >= 0 && pa >= 0, has_b = eb >= 0 && pb >= 0;
    float dl[MAX_E];
    {
        const float4 l0 = *reinterpret_cast<const float4*>(dlog + (size_t)t * MAX_E);
        const float4 l1 = *reinterpret_cast<const float4*>(dlog + (size_t)t * MAX_E + 4);
        dl[0] = l0.x; dl[1] = l0.y; dl[2] = l0.z; dl[3] = l0.w; dl[4] = l1.x; dl[5] = l1.y; dl[6] = l1.z; dl[7] = l1.w;
    }
    for (int c = lane * 8; c < d; c += 256) {
        float o[8], a[8], b[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(dxall + (size_t)t * d + c), o);
        if (has_a) {
            unpack_bf16x8(*reinterpret_cast<const uint4*>(dxall + (size_t)(tcap + pa) * d + c), a);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __fadd_rn(o[j], __fmul_rn(ga, a[j]));
        }
        if (has_b) {
            unpack_bf16x8(*reinterpret_cast<const uint4*>(dxall + (size_t)(tcap + pb) * d + c), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __fadd_rn(o[j], __fmul_rn(gb, b[j]));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(wr8 + (size_t)(c + j) * MAX_E));
            const float4 w1 = __ldg(reinterpret_cast<const float4*>(wr8 + (size_t)(c + j) * MAX_E + 4));
            float r = 0.0f;  // dot over the experts in index order (matmul_a_bt, ops.rs:86-104)
            r += dl[0] * w0.x; r += dl[1] * w0.y; r += dl[2] * w0.z; r += dl[3] * w0.w;
            r += dl[4] * w1.x; r += dl[5] * w1.y; r += dl[6] * w1.z; r += dl[7] * w1.w;
            o[j] = __fadd_rn(o[j], r);
        }
        float4* op = reinterpret_cast<float4*>(dx + (size_t)t * d + c);
        op[0] = make_float4(o[0], o[1], o[2], o[3]);
        op[1] = make_float4(o[4], o[5], o[6], o[7]);
    }
}

// Backward of the block's pre-norm (rmsnorm_backward, backward.rs:94-131) for the MoE sub-layer: one warp per row.
//   rms_inv = 1 / sqrt(mean(x^2) + eps),  coeff = (sum_i dn_i * gamma_i * x_i / d) * rms_inv^2,
//   dx_res_i = dy_i + gamma_i * rms_inv * (dn_i - x_i * coeff)
// dn: gradient of the normalised rows (the MoE backward's d_x), fp32; dy: the gradient that reaches the residual
// connection (the reference seeds d_x_res with a clone of it, model.rs:777-789). The x-term carries gamma as in the
// reference. Also writes rms_inv per row for the weight gradient. d is a multiple of 256, at most 256 * MAXC.
template <bool XF32, bool DYF32, int MAXC>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_rows_kernel(const void* __restrict__ x, const float* __restrict__ dn, const float* __restrict__ gamma,
                        const void* __restrict__ dy, float eps, float* __restrict__ dx_res, float* __restrict__ rinv, int T,
                        int d) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + warp;
    if (t >= T) return;
    const int nchunk = d / 256;
    float xv[MAXC][8], dv[MAXC][8];
    float sum_sq = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        if (i < nchunk) {
            const int c = i * 256 + lane * 8;
            if (XF32) {
                const float* p = reinterpret_cast<const float*>(x) + (size_t)t * d + c;
                const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
                xv[i][0] = a.x; xv[i][1] = a.y; xv[i][2] = a.z; xv[i][3] = a.w; xv[i][4] = b.x; xv[i][5] = b.y; xv[i][6] = b.z; xv[i][7] = b.w;
            } else {
                unpack_bf16x8(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)t * d + c), xv[i]);
            }
            const float* q = dn + (size_t)t * d + c;
            const float4 a = *reinterpret_cast<const float4*>(q), b = *reinterpret_cast<const float4*>(q + 4);
            dv[i][0] = a.x; dv[i][1] = a.y; dv[i][2] = a.z; dv[i][3] = a.w; dv[i][4] = b.x; dv[i][5] = b.y; dv[i][6] = b.z; dv[i][7] = b.w;
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c + 4));
            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sum_sq = fmaf(xv[i][j], xv[i][j], sum_sq);
                dot = fmaf(dv[i][j] * gv[j], xv[i][j], dot);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, o);
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
    }
    const float inv_d = 1.0f / (float)d;
    const float rms_inv = 1.0f / sqrtf(sum_sq * inv_d + eps);
    const float coeff = (dot * inv_d) * (rms_inv * rms_inv);
    if (lane == 0) rinv[t] = rms_inv;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        if (i < nchunk) {
            const int c = i * 256 + lane * 8;
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c + 4));
            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            float seed[8];
            if (DYF32) {
                const float* p = reinterpret_cast<const float*>(dy) + (size_t)t * d + c;
                const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
                seed[0] = a.x; seed[1] = a.y; seed[2] = a.z; seed[3] = a.w; seed[4] = b.x; seed[5] = b.y; seed[6] = b.z; seed[7] = b.w;
            } else {
                unpack_bf16x8(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(dy) + (size_t)t * d + c), seed);
            }
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = seed[j] + gv[j] * rms_inv * (dv[i][j] - xv[i][j] * coeff);
            float4* op = reinterpret_cast<float4*>(dx_res + (size_t)t * d + c);
            op[0] = make_float4(o[0], o[1], o[2], o[3]);
            op[1] = make_float4(o[4], o[5], o[6], o[7]);
        }
    }
}

// d_gamma[i] += sum_t dn[t,i] * x[t,i] * rms_inv[t] (backward.rs:127), in a fixed order: grid (d / 256, DWR_SPLITS)
// sums token ranges into part[s][i]; the reduce kernel adds the splits in ascending order.
template <bool XF32>
__global__ void __launch_bounds__(256)
dgamma_partial_kernel(const void* __restrict__ x, const float* __restrict__ dn, const float* __restrict__ rinv,
                      float* __restrict__ part, int T, int d) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    const int per = (T + DWR_SPLITS - 1) / DWR_SPLITS;
    const int t0 = min(T, (int)blockIdx.y * per), t1 = min(T, t0 + per);
    float acc = 0.f;
    for (int t = t0; t < t1; ++t) {
        const float xi = XF32 ? reinterpret_cast<const float*>(x)[(size_t)t * d + i]
                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[(size_t)t * d + i]);
        acc += dn[(size_t)t * d + i] * xi * rinv[t];
    }
    part[(size_t)blockIdx.y * d + i] = acc;
}

__global__ void __launch_bounds__(256)
dgamma_reduce_kernel(const float* __restrict__ part, float* __restrict__ d_gamma, int d) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d) return;
    float acc = 0.f;
    for (int s = 0; s < DWR_SPLITS; ++s) acc += part[(size_t)s * d + i];
    d_gamma[i] += acc;
}

// dst[c, r] = src[r, c] for r < rows, c < cols (bf16). src row pitch src_pitch, dst row pitch dst_pitch (elements).
// 64 x 64 tiles through shared memory (padded against bank conflicts); grid = (ceil(cols/64), ceil(rows/64)).
// src_nkt > 0: the source is stored tile by tile (256 x 64 blocks, src_nkt blocks per 256 rows; see egemm::Args::b_nkt)
// instead of row-major with src_pitch.
__global__ void __launch_bounds__(256)
transpose_bf16_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows, int cols,
                      long long src_pitch, long long dst_pitch, int src_nkt) {
    __shared__ __nv_bfloat16 tile[64][66];
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
    const long long r0 = (long long)blockIdx.y * 64;
    const int c0 = blockIdx.x * 64;
    for (int i = ty; i < 64; i += 4) {
        const long long r = r0 + i;
        const int c = c0 + tx;
        const size_t at = src_nkt > 0 ? ((((size_t)(r >> 8) * src_nkt + (c >> 6)) << 8) + (r & 255)) * 64 + (c & 63) : (size_t)r * src_pitch + c;
        tile[i][tx] = (r < rows && c < cols) ? src[at] : __float2bfloat16(0.f);
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 4) {
        const int c = c0 + i;
        const long long r = r0 + tx;
        if (c < cols && r < rows) dst[(size_t)c * dst_pitch + r] = tile[tx][i];
    }
}

// Staged weight gradients of one expert -> the caller's buffers (+=), reference layouts.
//   gu_stage [d, 2f] fp32 in the blocked column order (128 gate | 128 up per 256)  ->  grad_gate [d,f], grad_up [d,f]
__global__ void __launch_bounds__(256)
grad_unpack_gate_up_kernel(const float* __restrict__ gu_stage, float* __restrict__ grad_gate, float* __restrict__ grad_up, int d, int f) {
    const size_t total = (size_t)d * 2 * f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t k = i / (2 * (size_t)f);
        const int n = (int)(i - k * 2 * (size_t)f);
        const int blk = n >> 8, r = n & 255;
        const int col = blk * 128 + (r & 127);
        float* dst = (r < 128 ? grad_gate : grad_up);
        if (dst) dst[k * f + col] += gu_stage[i];
    }
}

//   dn_stage [f, d] fp32  ->  grad_down [f, d]
__global__ void __launch_bounds__(256)
grad_accumulate_kernel(const float* __restrict__ stage, float* __restrict__ grad, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) grad[i] += stage[i];
}

}  // namespace bwd
