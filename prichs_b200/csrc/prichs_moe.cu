// libprichs_moe.so -- C ABI (include/prichs_moe.h) over the sm_100a kernels of the PRICHS MoE-layer forward.
//
// One handle = the device state of one MoELayer (crates/prichs-model/src/moe.rs:58-64): repacked weights,
// router bias, workspace for max_tokens, TMA descriptors. With all experts local a forward is six launches (five
// for batches under 1024 tokens, where the scan rides at the tail of the router launch) on
// the caller's stream:
//   router -> scan/plan -> dispatch -> grouped gate|up GEMM (+SwiGLU) -> grouped down GEMM -> combine.
// The expert-parallel forward (forward_ep) runs the same kernels in token waves on several streams and
// exchanges rows through peer-mapped buffers.
// There is no CPU fallback: every entry point that needs the device fails with PRICHS_ERR_CUDA without one.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <chrono>
#include <cstring>
#include <mutex>
#include <thread>
#include <type_traits>
#include <vector>

#include "../../include/prichs_moe.h"
#include "expert_gemm_pair_sm100.cuh"
#include "expert_gemm_sm100.cuh"
#include "route_sm100.cuh"
#include "backward_sm100.cuh"

namespace {

thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define CUDA_TRY(expr)                                                                              \
    do {                                                                                            \
        cudaError_t e__ = (expr);                                                                   \
        if (e__ != cudaSuccess)                                                                     \
            return fail(PRICHS_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                        __FILE__, __LINE__);                                                        \
    } while (0)

#define LAUNCH_CHECK(name)                                                                    \
    do {                                                                                      \
        g_launches.fetch_add(1, std::memory_order_relaxed);                                   \
        cudaError_t e__ = cudaGetLastError();                                                 \
        if (e__ != cudaSuccess)                                                               \
            return fail(PRICHS_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

using bf16 = __nv_bfloat16;

// Kernel launch with the programmatic-dependent-launch attribute when `pdl` is set: the kernel may then be
// scheduled while its predecessor in the stream still runs and blocks at its griddepcontrol.wait until that one
// has completed. Kernel names that contain commas go in parentheses.
#define LAUNCH_K(pdl, kern, grid, block, smem, st, ...)                                        \
    do {                                                                                       \
        cudaLaunchConfig_t c__ = {};                                                           \
        c__.gridDim = dim3((unsigned)(grid));                                                  \
        c__.blockDim = dim3((unsigned)(block));                                                \
        c__.dynamicSmemBytes = (size_t)(smem);                                                 \
        c__.stream = (st);                                                                     \
        cudaLaunchAttribute a__[1];                                                            \
        a__[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                        \
        a__[0].val.programmaticStreamSerializationAllowed = 1;                                 \
        c__.attrs = a__;                                                                       \
        c__.numAttrs = (pdl) ? 1 : 0;                                                          \
        cudaLaunchKernelEx(&c__, kern, __VA_ARGS__);                                           \
    } while (0)

// cuTensorMapEncodeTiled is fetched through the runtime so that the library does not link libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Row-major matrix [rows, cols] of bf16 (or fp32) -> tensor map whose box is 128 bytes wide (64 bf16 or 32
// fp32 elements) and box_rows tall, with the 128-byte swizzle.
// `pitch` (elements, 0 = cols): distance between rows when the map covers a window of a wider matrix.
int make_tmap(CUtensorMap* tm, const void* base, size_t rows, size_t cols, int box_rows, bool f32 = false, size_t pitch = 0) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(PRICHS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const size_t esz = f32 ? 4 : 2;
    if (pitch == 0) pitch = cols;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch * esz) % 16 != 0)
        return fail(PRICHS_ERR_BAD_ARG, "tensor map base and row pitch must be 16-byte aligned");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(pitch * esz)};
    cuuint32_t box[2] = {(cuuint32_t)(128 / esz), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PRICHS_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return PRICHS_OK;
}

// ---- weight repacking (once, at upload) -------------------------------------------------------------
// Both GEMM weights are stored tile by tile: element (n, k) of a slot's K-major [rows, kw] matrix sits at
//   (((n / 256) * (kw / 64) + k / 64) * 256 + n % 256) * 64 + k % 64,
// i.e. every 256 x 64 block the GEMM loads per pipeline stage is one contiguous 32 KB run (egemm::Args::b_nkt).
__device__ __forceinline__ size_t tiled_at(int n, int k, int kw) {
    return ((((size_t)(n >> 8) * (kw >> 6) + (k >> 6)) << 8) + (n & 255)) * 64 + (k & 63);
}

// gate/up [d,f] fp32 (x.W layout) -> the stacked K-major B operand of the first GEMM:
// row n of a slot, n = blk*256 + r, holds hidden unit blk*128 + (r % 128) of gate (r < 128) or up (r >= 128).
// kw = d (bf16 mode) or 2d ([hi | lo], fp32-fidelity mode).
__global__ void repack_gate_up_kernel(const float* __restrict__ wg, const float* __restrict__ wu,
                                      bf16* __restrict__ dst, int d, int f, int split) {
    const int kw = split ? 2 * d : d;
    const size_t total = (size_t)2 * f * d;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int n = (int)(i / d), k = (int)(i % d);
        const int blk = n / 256, r = n % 256;
        const int col = blk * 128 + (r & 127);
        const float v = (r < 128 ? wg : wu)[(size_t)k * f + col];
        const bf16 hi = __float2bfloat16_rn(v);
        dst[tiled_at(n, k, kw)] = hi;
        if (split) dst[tiled_at(n, d + k, kw)] = __float2bfloat16_rn(v - __bfloat162float(hi));
    }
}

// down [f,d] fp32 -> rows n < d of the K-major B operand of the second GEMM, K = f (or [hi | lo] = 2f).
__global__ void repack_down_kernel(const float* __restrict__ wd, bf16* __restrict__ dst, int d, int f, int split) {
    const int kw = split ? 2 * f : f;
    const size_t total = (size_t)d * f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int n = (int)(i / f), k = (int)(i % f);
        const float v = wd[(size_t)k * d + n];
        const bf16 hi = __float2bfloat16_rn(v);
        dst[tiled_at(n, k, kw)] = hi;
        if (split) dst[tiled_at(n, f + k, kw)] = __float2bfloat16_rn(v - __bfloat162float(hi));
    }
}

// router [d,E] fp32 -> transposed bf16 parts [3][8][d] (hi, mid, lo; rows >= E zero) and the padded fp32
// copy [d][8] used by the fp32-fidelity router.
__global__ void repack_router_kernel(const float* __restrict__ wr, bf16* __restrict__ wrt, float* __restrict__ wr8,
                                     int d, int E) {
    const int total = d * route::MAX_E;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int e = i / d, k = i % d;
        const float v = e < E ? wr[(size_t)k * E + e] : 0.f;
        const bf16 p0 = __float2bfloat16_rn(v);
        const float r1 = v - __bfloat162float(p0);
        const bf16 p1 = __float2bfloat16_rn(r1);
        const bf16 p2 = __float2bfloat16_rn(r1 - __bfloat162float(p1));
        wrt[i] = p0;
        wrt[total + i] = p1;
        wrt[2 * total + i] = p2;
        wr8[(size_t)k * route::MAX_E + e] = v;
    }
}

// ---- the reference's stand-alone kernels, same semantics (kernels.cu:444-457,888-924) -----------------
__global__ void compat_gather_kernel(const float* __restrict__ in, const int* __restrict__ idx, float* __restrict__ out,
                                     size_t n, size_t d) {
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n) return;
    const float* src = in + (size_t)idx[warp] * d;
    float* dst = out + warp * d;
    if ((d & 3) == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        for (size_t c = lane; c < d / 4; c += 32)
            reinterpret_cast<float4*>(dst)[c] = reinterpret_cast<const float4*>(src)[c];
    } else {
        for (size_t c = lane; c < d; c += 32) dst[c] = src[c];
    }
}

__global__ void compat_scatter_add_kernel(const float* __restrict__ exp_out, const int* __restrict__ idx,
                                          const float* __restrict__ w, float* __restrict__ acc, size_t n, size_t d) {
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n) return;
    const float wi = w[warp];
    const float* src = exp_out + warp * d;
    float* dst = acc + (size_t)idx[warp] * d;
    // rows of one call may repeat an index, so the accumulation stays atomic like the reference's
    for (size_t c = lane; c < d; c += 32) atomicAdd(dst + c, wi * src[c]);
}

__global__ void compat_swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                     float* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float g = gate[i];
        out[i] = (g * (1.0f / (1.0f + __expf(-g)))) * up[i];
    }
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Ring depth of the single-pass routing kernel for hidden_dim d and `nsplit` router-weight parts: the deepest ring of
// 2..4 tile buffers that fits the 227 KB of shared memory next to the weights, 0 if not even two fit.
int rd_stages_for(int d, int nsplit) {
    for (int st = route::RD_MAX_STAGES; st >= 2; --st)
        if (route::rd_smem_bytes(d, nsplit, st) <= 227 * 1024 - 256) return st;
    return 0;
}

// Token waves of the expert-parallel forward shrink towards the end: the last wave's combine is the only
// exchange nothing can hide, so it is kept small. Cumulative fractions of the batch (per mille) per wave count.
inline int wave_begin(int T, int n_waves, int w) {
    static const int cum[5][5] = {{0, 0, 0, 0, 0}, {0, 1000, 0, 0, 0}, {0, 640, 1000, 0, 0}, {0, 440, 790, 1000, 0}, {0, 350, 650, 870, 1000}};
    if (w >= n_waves) return T;
    const long long b = (long long)T * cum[n_waves][w] / 1000;
    return (int)std::min<long long>(T, (b + 15) / 16 * 16);
}

// Every expert's segment of a permuted region starts on a multiple of this many rows (one CTA-pair tile).
constexpr int SEG_PAD = 256;

// ---- NCCL, loaded at run time (control plane of the expert-parallel mode only) -------------------------
// Only five entry points with a stable ABI are used; the library is opened by soname so that a process
// that already carries an NCCL (for example through torch) shares it.
struct NcclApi {
    struct Id128 { char b[128]; };  // ncclUniqueId, passed by value
    typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
    typedef int (*CommDestroyFn)(void*);
    typedef const char* (*GetErrorStringFn)(int);
    int (*get_unique_id)(void*) = nullptr;
    int (*comm_init_rank)(void**, int, Id128, int) = nullptr;
    AllGatherFn all_gather = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GetErrorStringFn error_string = nullptr;
    int (*comm_abort)(void*) = nullptr;             // optional: frees a collective that a missing peer keeps waiting
    int (*comm_async_error)(void*, int*) = nullptr;  // optional: ncclCommGetAsyncError
    bool ok = false;
};
constexpr int NCCL_INT32 = 2;  // ncclInt32 in nccl.h

NcclApi& nccl() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (lib) {
            api.get_unique_id = reinterpret_cast<int (*)(void*)>(dlsym(lib, "ncclGetUniqueId"));
            api.comm_init_rank = reinterpret_cast<int (*)(void**, int, NcclApi::Id128, int)>(dlsym(lib, "ncclCommInitRank"));
            api.all_gather = reinterpret_cast<NcclApi::AllGatherFn>(dlsym(lib, "ncclAllGather"));
            api.comm_destroy = reinterpret_cast<NcclApi::CommDestroyFn>(dlsym(lib, "ncclCommDestroy"));
            api.error_string = reinterpret_cast<NcclApi::GetErrorStringFn>(dlsym(lib, "ncclGetErrorString"));
            api.comm_abort = reinterpret_cast<int (*)(void*)>(dlsym(lib, "ncclCommAbort"));
            api.comm_async_error = reinterpret_cast<int (*)(void*, int*)>(dlsym(lib, "ncclCommGetAsyncError"));
            api.ok = api.get_unique_id && api.comm_init_rank && api.all_gather && api.comm_destroy && api.error_string;
        }
    }
    return api;
}

#define NCCL_TRY(expr)                                                                                    \
    do {                                                                                                  \
        int r__ = (expr);                                                                                 \
        if (r__ != 0) return fail(PRICHS_ERR_COMM, "%s failed: %s", #expr, nccl().error_string(r__));   \
    } while (0)

}  // namespace

// =====================================================================================================
constexpr int MAX_WAVES = 4;
// One token wave of an expert-parallel forward: its own stream, communicator, plan and barrier payload.
struct EpWave {
    cudaStream_t stream;
    void* comm;
    route::RouteMeta* meta;
    int* mtile_slot;
    int* token;  // [2][MAX_RANKS] ints: payload of the two barrier all-gathers
    cudaEvent_t done;
    cudaEvent_t tl[8];  // timeline marks (timing enabled): scan, plan, dispatch, rows landed, gate|up, down, outputs ready, combine
};

struct prichs_moe {
    prichs_moe_config_t cfg;
    int d, f, E, k, Tmax, mode, device;
    int world, rank, El;   // expert-parallel group, local routed experts
    int n_slots;           // weight slots held locally: shared + El
    int K1, K2;            // K extent of the A operands (d, f; doubled in the fp32-fidelity mode)
    int Tcap;              // max_tokens rounded up to 128: row where the permuted region starts in H / Y
    int Rcap;              // rows of the permuted region (multiple of 128)
    int sm_count;
    bool weights_ready;
    int rt_nsplit;

    bf16 *w_gu, *w_dn, *w_rt;
    float *w_r8, *bias;
    bf16 *xs, *xp, *hbuf;
    void* xnorm;  // normalised activations of the block entry point: bf16 [Tmax,d] (fp32 in the fp32-fidelity mode)
    const float* norm_w;  // set while the block entry point runs with the pre-norm folded into the router's read
    float norm_eps;
    bool fuse_norm;
    int route_kernel;     // 0 choose, 1 single-pass route+place+dispatch kernel, 2 three launches
    int rd_stages[2];     // depth of the single-pass kernel's ring of tile buffers for 1 / 3 router-weight parts (0: does not fit)
    int fuse_scan;  // single-GPU forward, scan + plan at the tail of the router launch: 1 always, 0 never, -1 for small batches
    int router_ctas_per_sm;  // router grid cap (-1: library default)
    int host_chunk;       // tokens per chunk of the host-buffer pipeline (0 = choose)
    int seg_stride;       // all experts local: rows of every expert's fixed-capacity segment (0: dense, expert parallel)
    int* mtile_row;       // all experts local: GEMM tile table, tile index inside the permuted region
    uint32_t* tile_state; // single-pass kernel: look-back words [tiles][8], zero between launches
    int* rd_ctl;          // single-pass kernel: ticket and exit counters, zero between launches
    long long rd_wait_cycles;  // budget of the single-pass kernel's bounded waits
    int rd_stall_tile;    // test knob (prichs_moe_debug_set): the tile that never publishes its counts, -1 none
    int rd_poll_sleep_ns; // pause between two polls of a look-back window
    void* ybuf;
    size_t y_bytes;  // bytes of the expert outputs inside the allocation (the flags follow)
    float *logits, *gates;
    int *sel, *pos, *tile_counts, *tile_prefix, *mtile_slot, *status;
    route::RouteMeta* meta;
    CUtensorMap tm_xp, tm_wgu, tm_h, tm_wdn;
    CUtensorMap tm_h_out, tm_y_out;  // 32-row store boxes of the GEMM epilogues
    CUtensorMap tm_wgu_half, tm_wdn_half;  // 128-row boxes: one CTA's half of a B tile in the CTA-pair kernel
    bool pair_gemm;  // use the CTA-pair (cta_group::2) GEMM kernel
    bool narrow_down;  // small batches: down projection on 128-column tiles
    bool pdl;  // launch the kernels of the single-GPU forward with programmatic dependent launch
    bool small_batch;  // this forward has so few rows that 128-row tiles on single CTAs spread better over the SMs

    // expert-parallel group: peers' receive / output buffers mapped into this process, and the token waves
    bool ep_ready;
    void* xp_peer[route::MAX_RANKS];
    void* y_peer[route::MAX_RANKS];
    int n_waves;  // token waves of an expert-parallel forward (1 when all experts are local)
    int Rw;       // rows of one wave's permuted region (multiple of 128); Rcap = n_waves * Rw
    EpWave wave[MAX_WAVES];
    int ep_reserve_sms;  // SMs the expert-parallel GEMM launches leave to the exchange kernels
    int ep_combine_mode; // which combine launches keep off the GEMM SMs: 0 all, 1 all but the last wave's, 2 none
    int ep_copy_smem;    // dynamic shared memory requested by dispatch/combine in expert-parallel mode: more than a
                         // GEMM CTA leaves free, so these kernels only run on the reserved SMs (0 = share SMs)
    int* ep_flags;             // readiness flags written by the peers (tail of the expert-output allocation)
    void* flag_peer[route::MAX_RANKS];  // the same array of every rank
    int ep_timeout_ms;         // host-side limit on waiting for an expert-parallel forward (prichs_moe_sync_status)
    bool ep_broken;            // the communicators were aborted after such a wait ran out: the group must be rebuilt
    int ep_seq;                // sequence number of the expert-parallel forward being enqueued
    int ep_skip_signal;        // test knob: 1 + kind * 4 + wave of a signal this rank does not send (0: none)
    int ep_barrier_mode;       // 0: readiness flags over NVLink; 1: NCCL all-gathers as barriers
    bool ep_bulk_dispatch;     // expert-parallel dispatch with bulk copies through shared memory
    int db_stages;             // ... depth of its ring
    int* ep_zero;              // a device int that stays zero (the "no permuted tiles" count of the shared launches)
    cudaStream_t side_stream;  // shared-expert GEMMs of the expert-parallel mode
    cudaEvent_t ev_router, ev_shared;
    cudaEvent_t tl_base, tl_side[2];  // timeline: router done; shared gate|up done, shared down done

    // host-buffer path
    float *stage_x, *stage_r, *stage_y;
    int* counts_acc;
    bool host_ready;  // staging buffers, streams and events of the host-buffer path exist
    cudaStream_t own_stream, in_stream, out_stream;
    cudaEvent_t* chunk_ev;

    // backward pass (allocated by the first prichs_moe_backward): recomputed pre-activations, gradient buffers in
    // the forward's row space, transposed copies for the weight-gradient products, un-transposed weight copies
    bool want_stash;  // the forward being enqueued keeps the [gate | up] pre-activations (training forward)
    bool gu_valid;    // bwd.gu holds the pre-activations of the last forward
    struct Bwd {
        bool ready, nat_valid;
        bf16 *gu, *dyall, *dh, *dgu, *dxall, *xT, *hT, *dyT, *dguT, *w_dn_nat, *w_gu_nat;
        float *scal, *dlog, *dwr_part, *stage_dn, *stage_gu, *dnorm, *rinv, *dgamma_part;
        CUtensorMap tm_dyall, tm_dgu, tm_gu_out, tm_dh_out, tm_dxall_out, tm_wdn_nat, tm_wgu_nat, tm_stage_dn, tm_stage_gu;
    } bwd;

    cudaStream_t last_stream;
    int last_T;
    bool last_chunked;  // the last forward went through the host-buffer pipeline in chunks: only its last chunk's rows remain
    const bf16* last_a_shared;  // bf16 rows the last single-GPU forward fed to the shared expert and the dispatch
    bool last_was_block;  // ... and it came through prichs_moe_block_forward
    int tok_base;  // see prichs_moe_forward
    int resid_dtype;  // element type of the residual when it differs from x (block entry point), else -1
    bool timing;
    cudaEvent_t ev[7];
    bool ev_valid;
    bool tl_valid;  // the expert-parallel timeline events of the last forward are recorded
};

namespace {

template <class T>
int dalloc(T** p, size_t n) {
    *p = nullptr;
    CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(p), n * sizeof(T)));
    return PRICHS_OK;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~DeviceGuard() {
        int cur = -1;
        cudaGetDevice(&cur);
        if (prev >= 0 && cur != prev) cudaSetDevice(prev);
    }
};

int translate_status(int s) {
    switch (s) {
        case 0: return PRICHS_OK;
        case -2: return fail(PRICHS_ERR_CAPACITY, "an expert received more rows than the permuted region holds");
        case -7: return fail(PRICHS_ERR_BOUNDS, "an index check of the checking build failed: a kernel computed a row outside its buffer (the access was skipped)");
        case -5: return fail(PRICHS_ERR_TIMEOUT, "a bounded device-side wait gave up (expert GEMM or single-pass routing kernel)");
        default: return fail(PRICHS_ERR_CUDA, "device status word %d", s);
    }
}

// ---- launch helpers shared by the single-GPU and the expert-parallel forward ---------------------------
// Router over T tokens starting at `x_dev`; routing arrays are the caller's (already offset) pointers.
int launch_router(prichs_moe* h, const void* x_dev, int x_dtype, const route::ConceptBias& cb, int T, float* logits, int* sel,
                  float* gates, int* tile_counts, cudaStream_t st, bool pdl = false, const route::ScanTail& tail = route::ScanTail{}) {
    const int d = h->d, E = h->E;
    const int ntiles_all = (T + route::TILE_TOKENS - 1) / route::TILE_TOKENS;
    // The router kernel strides over tiles, so its grid can be capped. With the scan at its tail every CTA ends on a
    // fence and a ticket, which is cheap for two persistent CTAs per SM and costly for one short-lived CTA per
    // tile; without the tail one CTA per tile balances best. PRICHS_ROUTER_CTAS_PER_SM overrides (0 = per tile).
    const int cap_per_sm = h->router_ctas_per_sm >= 0 ? h->router_ctas_per_sm : (tail.done != nullptr ? 2 : 0);
    const int ntiles = cap_per_sm > 0 && h->mode != PRICHS_MODE_F32 ? std::min(ntiles_all, cap_per_sm * h->sm_count) : ntiles_all;
    if (h->mode == PRICHS_MODE_F32) {
        route::router_f32_kernel<<<ntiles, 512, 0, st>>>(reinterpret_cast<const float*>(x_dev), h->xs, h->w_r8, h->bias, cb, T, d, E, h->k,
                                                        logits, sel, gates, tile_counts);
    } else {
        constexpr int RT = route::ROUTER_WARPS * 32;
        const bool xf32 = x_dtype == PRICHS_DTYPE_F32, norm = h->norm_w != nullptr;
        bf16* xs = (xf32 || norm) ? h->xs : nullptr;  // bf16 (and normalised) copy of the rows for the expert GEMMs
#define PRICHS_ROUTER_CASE(NS, XF, NM)                                                                                              \
    if (h->rt_nsplit == NS && xf32 == XF && norm == NM)                                                                             \
        LAUNCH_K(pdl, (route::router_mma_kernel<NS, XF, NM>), ntiles, RT, 0, st, (const void*)x_dev, xs, (const bf16*)h->w_rt,      \
                 (const float*)h->bias, cb, T, d, E, h->k, logits, sel, gates, tile_counts, h->norm_w, h->norm_eps, tail);
        PRICHS_ROUTER_CASE(1, false, false)
        PRICHS_ROUTER_CASE(1, true, false)
        PRICHS_ROUTER_CASE(3, false, false)
        PRICHS_ROUTER_CASE(3, true, false)
        PRICHS_ROUTER_CASE(1, false, true)
        PRICHS_ROUTER_CASE(1, true, true)
        PRICHS_ROUTER_CASE(3, false, true)
        PRICHS_ROUTER_CASE(3, true, true)
#undef PRICHS_ROUTER_CASE
    }
    LAUNCH_CHECK("router");
    return PRICHS_OK;
}

// Arguments of the two grouped GEMMs (gate|up + SwiGLU, then down) for T un-permuted tokens and the permuted
// region that starts `region_tile` 128-row tiles into the permuted buffers.
void gemm_args(prichs_moe* h, int T, int region_tile, const int* n_routed_mtiles, const int* mtile_slot, const int* mtile_row,
               egemm::Args* a1, egemm::Args* a2) {
    const bool f32mode = h->mode == PRICHS_MODE_F32;
    memset(a1, 0, sizeof(*a1));
    a1->nk = h->d / egemm::BK;
    a1->split3 = f32mode;
    a1->n_ntiles = h->f / 128;
    a1->shared_mtiles = (T + 127) / 128;
    a1->routed_base_tiles = h->Tcap / 128 + region_tile;
    a1->a_routed_tile_off = region_tile;
    a1->n_routed_mtiles = n_routed_mtiles;
    a1->mtile_slot = mtile_slot;
    a1->mtile_row = mtile_row;
    a1->w_rows = 2 * h->f;
    a1->b_nkt = h->K1 / egemm::BK;
    a1->out_split = f32mode;
    a1->out_lo_off = h->f;
    a1->out_f32 = 0;
    a1->status = h->status;
    *a2 = *a1;
    if (h->want_stash) {
        a1->stash_gu = h->bwd.gu;
        a1->stash_ld = 2 * h->f;
    }
    a2->nk = h->f / egemm::BK;
    a2->n_ntiles = h->d / egemm::BN;
    a2->a_routed_tile_off = h->Tcap / 128 + region_tile;
    a2->w_rows = h->d;
    a2->b_nkt = h->K2 / egemm::BK;
    a2->out_split = 0;
    a2->out_f32 = f32mode;
}

// One grouped-GEMM launch: epi 0 = gate|up + SwiGLU into H, epi 1 = down projection into Y.
int launch_expert_gemm(prichs_moe* h, int epi, const CUtensorMap& tm_a_shared, const CUtensorMap& tm_a_routed, const egemm::Args& a,
                       int grid, cudaStream_t st, bool pdl = false) {
    if (h->pair_gemm && !h->small_batch) {
        const int g2 = std::max(2, grid & ~1);  // whole CTA pairs
        if (epi == 0)
            LAUNCH_K(pdl, egemm::expert_gemm_pair_kernel<egemm::EPI_SWIGLU>, g2, egemm::NUM_THREADS, egemm::PAIR_SMEM_BYTES, st, tm_a_shared, tm_a_routed, h->tm_wgu_half, h->tm_h_out, a);
        else
            LAUNCH_K(pdl, egemm::expert_gemm_pair_kernel<egemm::EPI_PLAIN>, g2, egemm::NUM_THREADS, egemm::PAIR_SMEM_BYTES, st, tm_a_shared, tm_a_routed, h->tm_wdn_half, h->tm_y_out, a);
    } else if (epi == 1 && h->small_batch && h->narrow_down && !a.out_f32) {
        // small batch: 128-column tiles for the down projection, twice as many tiles to spread over the SMs
        egemm::Args a128 = a;
        a128.n_ntiles = a.n_ntiles * 2;
        LAUNCH_K(pdl, (egemm::expert_gemm_kernel<egemm::EPI_PLAIN, 128>), grid, egemm::NUM_THREADS, egemm::GemmShape<128>::SMEM_BYTES, st,
                 tm_a_shared, tm_a_routed, h->tm_wdn_half, h->tm_y_out, a128);
    } else {
        if (epi == 0)
            LAUNCH_K(pdl, egemm::expert_gemm_kernel<egemm::EPI_SWIGLU>, grid, egemm::NUM_THREADS, egemm::SMEM_BYTES, st, tm_a_shared, tm_a_routed, h->tm_wgu, h->tm_h_out, a);
        else
            LAUNCH_K(pdl, egemm::expert_gemm_kernel<egemm::EPI_PLAIN>, grid, egemm::NUM_THREADS, egemm::SMEM_BYTES, st, tm_a_shared, tm_a_routed, h->tm_wdn, h->tm_y_out, a);
    }
    LAUNCH_CHECK(epi == 0 ? "gate/up GEMM" : "down GEMM");
    return PRICHS_OK;
}

// Combine of T tokens whose shared-expert rows start at `y_shared` and whose routing arrays / residual / output
// are the caller's (already offset) pointers.
int launch_combine(prichs_moe* h, const void* y_shared, const route::PeerPtrs& y_peers, long long routed_base_rows, const int* sel,
                   const float* gates, const int* pos, const void* resid_dev, void* y_dev, int x_dtype, int y_dtype, int T,
                   cudaStream_t st, bool exclusive = false, bool pdl = false) {
    // expert-parallel: a capped, grid-striding launch; `exclusive` keeps it off the SMs that hold GEMM CTAs
    const int grid = h->world > 1 ? std::min((T + 7) / 8, 4 * h->sm_count) : (T + 7) / 8;
    const int dyn_smem = exclusive ? h->ep_copy_smem : 0;
    const int rdt = h->resid_dtype >= 0 ? h->resid_dtype : x_dtype;
    const int res = !resid_dev ? 0 : (rdt == PRICHS_DTYPE_BF16 ? 1 : 2);
    const bool of32 = y_dtype == PRICHS_DTYPE_F32;
#define COMBINE(YF, OF, RS) \
    LAUNCH_K(pdl, (route::combine_kernel<YF, OF, RS>), grid, 256, dyn_smem, st, y_shared, y_peers, routed_base_rows, sel, gates, pos, resid_dev, y_dev, T, h->d, h->El, h->Rcap, h->status)
    if (h->mode == PRICHS_MODE_F32) {
        if (of32) { if (res == 0) COMBINE(true, true, 0); else if (res == 1) COMBINE(true, true, 1); else COMBINE(true, true, 2); }
        else      { if (res == 0) COMBINE(true, false, 0); else if (res == 1) COMBINE(true, false, 1); else COMBINE(true, false, 2); }
    } else {
        if (of32) { if (res == 0) COMBINE(false, true, 0); else if (res == 1) COMBINE(false, true, 1); else COMBINE(false, true, 2); }
        else      { if (res == 0) COMBINE(false, false, 0); else if (res == 1) COMBINE(false, false, 1); else COMBINE(false, false, 2); }
    }
#undef COMBINE
    LAUNCH_CHECK("combine");
    return PRICHS_OK;
}

int forward_ep(prichs_moe* h, const void* x_dev, int x_dtype, const void* resid_dev, const route::ConceptBias& cb, void* y_dev,
               int y_dtype, int T, cudaStream_t st);

}  // namespace

namespace {

// Adds the per-expert counts of the chunk that just ran to `acc` (first chunk: overwrite): acc[0..8) this rank's
// counts, acc[8..16) the totals over all ranks.
__global__ void host_chunk_accumulate_kernel(const route::RouteMeta* __restrict__ meta, int* __restrict__ acc, int first) {
    const int e = threadIdx.x;
    if (e < route::MAX_E) {
        acc[e] = (first ? 0 : acc[e]) + meta->counts[e];
        acc[route::MAX_E + e] = (first ? 0 : acc[route::MAX_E + e]) + meta->total[e];
    }
}
// After the last chunk: the call's totals become the handle's "last forward" counts.
__global__ void host_chunk_finish_kernel(route::RouteMeta* __restrict__ meta, const int* __restrict__ acc, int rank) {
    const int e = threadIdx.x;
    if (e < route::MAX_E) {
        meta->counts[e] = acc[e];
        meta->total[e] = acc[route::MAX_E + e];
        meta->cmat[rank * route::MAX_E + e] = acc[e];
    }
}

// Sums the waves' routing summaries into the handle's "last forward" summary (counts, totals, received rows,
// counts matrix); segment bases and source offsets are those of wave 0.
struct WaveMetas {
    const route::RouteMeta* m[MAX_WAVES];
};
__global__ void ep_totals_kernel(const WaveMetas wm, int n_waves, route::RouteMeta* __restrict__ out) {
    const int i = threadIdx.x;
    if (i < route::MAX_E) {
        int c = 0, t = 0;
        for (int w = 0; w < n_waves; ++w) {
            c += wm.m[w]->counts[i];
            t += wm.m[w]->total[i];
        }
        out->counts[i] = c;
        out->total[i] = t;
        out->seg_base[i] = wm.m[0]->seg_base[i];
        out->src_off[i] = wm.m[0]->src_off[i];
    }
    if (i < route::MAX_RANKS * route::MAX_E) {
        int c = 0;
        for (int w = 0; w < n_waves; ++w) c += wm.m[w]->cmat[i];
        out->cmat[i] = c;
    }
    if (i == 0) {
        int rows = 0, tiles = 0, over = 0;
        for (int w = 0; w < n_waves; ++w) {
            rows += wm.m[w]->recv_rows;
            tiles += wm.m[w]->n_routed_mtiles;
            over |= wm.m[w]->overflow;
        }
        out->recv_rows = rows;
        out->n_routed_mtiles = tiles;
        out->overflow = over;
    }
}

// Readiness flags (route::ep_signal_kernel / ep_wait_kernel) of wave `w`: `signal` tells every rank that this rank's
// part of `kind` is done (enqueued after the kernel that produced it), `wait` holds the stream until every rank has
// said so. Sequence number = the forward's.
int ep_signal_and_wait(prichs_moe* h, int kind, int w, cudaStream_t ws, bool signal, bool wait) {
    if (signal && h->ep_skip_signal != 1 + kind * 4 + w) {
        route::PeerPtrs fl;
        for (int i = 0; i < route::MAX_RANKS; ++i) fl.p[i] = h->flag_peer[i];
        route::ep_signal_kernel<<<1, 32, 0, ws>>>(fl, kind, w, h->rank, h->world, h->ep_seq);
        LAUNCH_CHECK("readiness signal");
    }
    if (wait) {
        route::ep_wait_kernel<<<1, 32, 0, ws>>>(h->ep_flags, kind, w, h->world, h->ep_seq, h->rd_wait_cycles, h->status);
        LAUNCH_CHECK("readiness wait");
    }
    return PRICHS_OK;
}

// Expert-parallel forward. Buffer-reuse hazards between consecutive forwards are closed by stream order plus
// the collectives: a peer writes this rank's receive region of wave w only after the counts all-gather of
// its next forward's wave w, which this rank joins after every wave of the current forward has been joined
// into `st`; a peer reads this rank's expert outputs of wave w in its combine, and this rank overwrites them
// only after the "rows landed" barrier of the next forward's wave w, which that peer enters after its combine.
int forward_ep(prichs_moe* h, const void* x_dev, int x_dtype, const void* resid_dev, const route::ConceptBias& cb, void* y_dev,
               int y_dtype, int T, cudaStream_t st) {
    const int E = h->E, W = h->n_waves;
    const bool f32mode = h->mode == PRICHS_MODE_F32;
    const bf16* a_shared = f32mode || x_dtype == PRICHS_DTYPE_F32 || h->norm_w ? h->xs : reinterpret_cast<const bf16*>(x_dev);
    CUtensorMap tm_x;
    int rc = make_tmap(&tm_x, a_shared, (size_t)T, (size_t)h->K1, egemm::BM);
    if (rc != PRICHS_OK) return rc;
    h->ev_valid = false;
    h->ep_seq += 1;
    // A few SMs stay free of the persistent GEMM CTAs so that the small kernels of the other streams (scans,
    // plans, NCCL) are never queued behind a whole GEMM.
    const int gemm_grid = std::max(2, h->sm_count - h->ep_reserve_sms);
    const size_t xsz = (h->resid_dtype >= 0 ? h->resid_dtype : x_dtype) == PRICHS_DTYPE_F32 ? 4 : 2, osz = y_dtype == PRICHS_DTYPE_F32 ? 4 : 2, ysz = f32mode ? 4 : 2;

    // 1. router over the whole batch
    // routing results of this call start at token `tok_base` of the stash arrays (non-zero only while the host-buffer
    // entry point feeds a batch through in chunks)
    float* const logits0 = h->logits + (size_t)h->tok_base * route::MAX_E;
    int* const sel0 = h->sel + (size_t)h->tok_base * 2;
    float* const gates0 = h->gates + (size_t)h->tok_base * 2;
    int* const pos0 = h->pos + (size_t)h->tok_base * 2;
    rc = launch_router(h, x_dev, x_dtype, cb, T, logits0, sel0, gates0, h->tile_counts, st);
    if (rc != PRICHS_OK) return rc;
    CUDA_TRY(cudaEventRecord(h->ev_router, st));
    const bool tl = h->timing;
    if (tl) CUDA_TRY(cudaEventRecord(h->tl_base, st));

    // 2. the shared expert needs no exchange: both of its GEMMs run on the side stream
    {
        egemm::Args s1, s2;
        gemm_args(h, T, 0, h->ep_zero, h->wave[0].mtile_slot, nullptr, &s1, &s2);
        CUDA_TRY(cudaStreamWaitEvent(h->side_stream, h->ev_router, 0));
        rc = launch_expert_gemm(h, 0, tm_x, h->tm_xp, s1, gemm_grid, h->side_stream);
        if (rc != PRICHS_OK) return rc;
        if (tl) cudaEventRecord(h->tl_side[0], h->side_stream);
        rc = launch_expert_gemm(h, 1, h->tm_h, h->tm_h, s2, gemm_grid, h->side_stream);
        if (rc != PRICHS_OK) return rc;
        if (tl) cudaEventRecord(h->tl_side[1], h->side_stream);
        CUDA_TRY(cudaEventRecord(h->ev_shared, h->side_stream));
    }

    // 3. token waves
    WaveMetas wm;
    for (int w = 0; w < MAX_WAVES; ++w) wm.m[w] = h->wave[w < W ? w : 0].meta;
    for (int w = 0; w < W; ++w) {
        EpWave& wv = h->wave[w];
        cudaStream_t ws = wv.stream;
        const int t0 = wave_begin(T, W, w), tn = wave_begin(T, W, w + 1) - t0;
        const int tile0 = t0 / route::TILE_TOKENS, ntl = (tn + route::TILE_TOKENS - 1) / route::TILE_TOKENS;
        const int region_tile = w * (h->Rw / 128);
        int* sel = sel0 + (size_t)t0 * 2;
        float* gates = gates0 + (size_t)t0 * 2;
        int* pos = pos0 + (size_t)t0 * 2;
        int* tprefix = h->tile_prefix + (size_t)tile0 * route::MAX_E;
        CUDA_TRY(cudaStreamWaitEvent(ws, h->ev_router, 0));
        // counts of this rank's wave -> all-gather (row `rank` of the matrix, in place) -> the same plan everywhere
        route::scan_kernel<<<1, 1024, 0, ws>>>(h->tile_counts + (size_t)tile0 * route::MAX_E, tprefix, ntl, wv.meta, wv.mtile_slot, nullptr, E, h->El,
                                               h->world, h->rank, h->Rw, 0, SEG_PAD, 0, h->status);
        LAUNCH_CHECK("scan");
        if (tl) cudaEventRecord(wv.tl[0], ws);
        NCCL_TRY(nccl().all_gather(wv.meta->cmat + h->rank * route::MAX_E, wv.meta->cmat, route::MAX_E, NCCL_INT32, wv.comm, ws));
        route::plan_kernel<<<1, 256, 0, ws>>>(wv.meta, wv.mtile_slot, E, h->El, h->world, h->rank, h->Rw, SEG_PAD, h->status);
        LAUNCH_CHECK("plan");
        if (tl) cudaEventRecord(wv.tl[1], ws);
        // dispatch: rows go straight into the owners' receive regions of this wave (peer memory over NVLink)
        route::PeerPtrs xp_peers, y_peers;
        for (int i = 0; i < route::MAX_RANKS; ++i) {
            xp_peers.p[i] = static_cast<bf16*>(h->xp_peer[i]) + (size_t)w * h->Rw * h->K1;
            y_peers.p[i] = h->y_peer[i];
        }
        if (tn > 0 && h->ep_bulk_dispatch) {
            // bulk copies through shared memory on the SMs the GEMMs leave free (its ring does not fit beside a GEMM CTA)
            const int grid = std::max(1, std::min((tn + route::TILE_TOKENS - 1) / route::TILE_TOKENS, std::max(2, h->ep_reserve_sms)));
            route::dispatch_bulk_kernel<<<grid, route::DB_THREADS, route::db_smem_bytes(h->K1 * 2, h->db_stages), ws>>>(
                a_shared + (size_t)t0 * h->K1, h->K1, tn, sel, tprefix, wv.meta, xp_peers, h->El, pos, h->Rw, h->db_stages, h->rd_wait_cycles, h->status);
            LAUNCH_CHECK("dispatch");
        } else if (tn > 0) {
            route::dispatch_kernel<<<std::min((tn + 7) / 8, 2 * h->sm_count), 256, h->ep_copy_smem, ws>>>(a_shared + (size_t)t0 * h->K1, h->K1, tn, sel, tprefix, wv.meta, xp_peers, h->El, pos, h->Rw, h->status);
            LAUNCH_CHECK("dispatch");
        }
        if (tl) cudaEventRecord(wv.tl[2], ws);
        // every rank's rows of this wave have landed before an expert GEMM reads them
        if (h->ep_barrier_mode == 1) {
            NCCL_TRY(nccl().all_gather(wv.token + h->rank, wv.token, 1, NCCL_INT32, wv.comm, ws));
        } else {
            rc = ep_signal_and_wait(h, 0, w, ws, true, true);
            if (rc != PRICHS_OK) return rc;
        }
        if (tl) cudaEventRecord(wv.tl[3], ws);
        egemm::Args a1, a2;
        gemm_args(h, 0, region_tile, &wv.meta->n_routed_mtiles, wv.mtile_slot, nullptr, &a1, &a2);
        rc = launch_expert_gemm(h, 0, tm_x, h->tm_xp, a1, gemm_grid, ws);
        if (rc != PRICHS_OK) return rc;
        if (tl) cudaEventRecord(wv.tl[4], ws);
        rc = launch_expert_gemm(h, 1, h->tm_h, h->tm_h, a2, gemm_grid, ws);
        if (rc != PRICHS_OK) return rc;
        if (tl) cudaEventRecord(wv.tl[5], ws);
        // every owner's outputs of this wave are complete before the combine gathers them over NVLink: the peers learn
        // of this rank's outputs as soon as its down projection ends, without waiting for its shared expert
        if (h->ep_barrier_mode != 1) {
            rc = ep_signal_and_wait(h, 1, w, ws, true, false);
            if (rc != PRICHS_OK) return rc;
        }
        CUDA_TRY(cudaStreamWaitEvent(ws, h->ev_shared, 0));  // the shared expert's rows are complete
        if (h->ep_barrier_mode == 1) {
            NCCL_TRY(nccl().all_gather(wv.token + route::MAX_RANKS + h->rank, wv.token + route::MAX_RANKS, 1, NCCL_INT32, wv.comm, ws));
        } else {
            rc = ep_signal_and_wait(h, 1, w, ws, false, true);
            if (rc != PRICHS_OK) return rc;
        }
        if (tl) cudaEventRecord(wv.tl[6], ws);
        if (tn > 0) {
            const char* resid_w = resid_dev ? static_cast<const char*>(resid_dev) + (size_t)t0 * h->d * xsz : nullptr;
            rc = launch_combine(h, static_cast<const char*>(h->ybuf) + (size_t)t0 * h->d * ysz, y_peers, (long long)h->Tcap + (long long)w * h->Rw,
                                sel, gates, pos, resid_w, static_cast<char*>(y_dev) + (size_t)t0 * h->d * osz, x_dtype, y_dtype, tn, ws,
                                h->ep_combine_mode == 0 || (h->ep_combine_mode == 1 && w + 1 < W));
            if (rc != PRICHS_OK) return rc;
        }
        if (tl) cudaEventRecord(wv.tl[7], ws);
        CUDA_TRY(cudaEventRecord(wv.done, ws));
    }
    h->tl_valid = tl;
    // 4. join the waves and publish the call's totals
    for (int w = 0; w < W; ++w) CUDA_TRY(cudaStreamWaitEvent(st, h->wave[w].done, 0));
    ep_totals_kernel<<<1, 64, 0, st>>>(wm, W, h->meta);
    LAUNCH_CHECK("wave totals");
    return PRICHS_OK;
}

}  // namespace

extern "C" {

const char* prichs_last_error(void) { return g_err; }
int prichs_bounds_checking(void) {
#ifdef PRICHS_BOUNDS_CHECK
    return 1;
#else
    return 0;
#endif
}
int64_t prichs_kernel_launches(void) { return (int64_t)g_launches.load(); }

int prichs_moe_create(const prichs_moe_config_t* cfg, prichs_moe_t** out_handle) {
    if (!cfg || !out_handle) return fail(PRICHS_ERR_BAD_ARG, "null config or handle pointer");
    *out_handle = nullptr;
    const int d = cfg->hidden_dim, f = cfg->intermediate_dim, E = cfg->num_experts, k = cfg->top_k;
    if (d <= 0 || f <= 0 || d % 256 != 0 || f % 128 != 0)
        return fail(PRICHS_ERR_BAD_SHAPE, "hidden_dim must be a multiple of 256 and intermediate_dim of 128 (got %d, %d)", d, f);
    if (E < 1 || E > route::MAX_E) return fail(PRICHS_ERR_BAD_SHAPE, "num_experts must be in 1..8 (got %d)", E);
    if (k < 1 || k > 2 || k > E) return fail(PRICHS_ERR_BAD_SHAPE, "k must be <= logits length and at most 2 (got %d)", k);
    if (cfg->max_tokens < 1) return fail(PRICHS_ERR_BAD_SHAPE, "max_tokens must be positive");
    if (cfg->mode != PRICHS_MODE_BF16 && cfg->mode != PRICHS_MODE_F32) return fail(PRICHS_ERR_BAD_ARG, "unknown mode %d", cfg->mode);
    const int world = cfg->ep_world <= 0 ? 1 : cfg->ep_world;
    if (world > route::MAX_RANKS || E % world != 0 || cfg->ep_rank < 0 || cfg->ep_rank >= world)
        return fail(PRICHS_ERR_BAD_ARG, "ep_world must divide num_experts and ep_rank lie in [0, ep_world)");

    int dev = cfg->device;
    if (dev < 0) CUDA_TRY(cudaGetDevice(&dev));
    int ndev = 0;
    CUDA_TRY(cudaGetDeviceCount(&ndev));
    if (dev >= ndev) return fail(PRICHS_ERR_CUDA, "device %d does not exist", dev);
    DeviceGuard guard(dev);
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10) return fail(PRICHS_ERR_CUDA, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major, prop.minor);

    prichs_moe* h = new prichs_moe();
    memset(h, 0, sizeof(*h));
    h->cfg = *cfg;
    h->d = d; h->f = f; h->E = E; h->k = k; h->Tmax = cfg->max_tokens; h->mode = cfg->mode; h->device = dev;
    h->world = world; h->rank = cfg->ep_rank; h->El = E / world; h->n_slots = 1 + h->El;
    const int mul = h->mode == PRICHS_MODE_F32 ? 2 : 1;
    h->K1 = d * mul; h->K2 = f * mul;
    h->Tcap = round_up(h->Tmax, SEG_PAD);
    h->resid_dtype = -1;
    h->fuse_norm = cfg->separate_prenorm == 0;
    h->fuse_scan = cfg->scan_placement == 1 ? 1 : (cfg->scan_placement == 2 ? 0 : -1);
    h->route_kernel = cfg->route_kernel;
    h->router_ctas_per_sm = cfg->router_ctas_per_sm == 0 ? -1 : std::max(0, cfg->router_ctas_per_sm);
    h->host_chunk = cfg->host_chunk_tokens > 0 ? std::max(256, cfg->host_chunk_tokens / 16 * 16) : 0;
    h->rd_stall_tile = -1;
    h->rd_poll_sleep_ns = 100;  // measured on B200: 46.2 against 47.2 us for the routing stage at 16384 tokens without the pause
    h->rd_wait_cycles = 4000000000LL;  // ~2 s, like the GEMM's waits
    h->n_waves = 1;
    if (world > 1) {
        const int want = cfg->ep_waves > 0 ? cfg->ep_waves : h->Tmax / 8192;
        h->n_waves = std::max(1, std::min(MAX_WAVES, want));
    }
    // worst case per wave: every token of the wave, from every rank, picks experts of this rank
    // the first wave is the largest
    const long long tw_max = wave_begin(h->Tmax, h->n_waves, 1) + route::TILE_TOKENS;
    // all experts local: every expert owns a segment of Tcap rows (a token picks an expert at most once), so a row's
    // place never depends on the totals
    h->seg_stride = world == 1 ? h->Tcap : 0;
    long long recv = world == 1 ? (long long)h->El * h->Tcap
                                : (cfg->ep_max_recv_rows > 0 ? (long long)cfg->ep_max_recv_rows * tw_max / h->Tmax + 1
                                                             : (long long)world * tw_max * k);
    const long long rw = world == 1 ? recv : (recv + (long long)h->El * (SEG_PAD - 1) + SEG_PAD - 1) / SEG_PAD * SEG_PAD;
    const long long rcap = rw * h->n_waves;
    if ((rcap + h->Tcap) * (long long)std::max(h->K1, h->K2) >= (1LL << 40) || rcap > (1LL << 30)) {
        const int tmax = h->Tmax;
        delete h;
        return fail(PRICHS_ERR_CAPACITY, "workspace for max_tokens=%d is too large", tmax);
    }
    h->Rcap = (int)rcap;
    h->Rw = (int)rw;
    h->sm_count = prop.multiProcessorCount;

    int rc = PRICHS_OK;
    auto A = [&](int r) { if (rc == PRICHS_OK) rc = r; };
    const size_t rows_all = (size_t)h->Tcap + h->Rcap;
    const size_t ntiles = ((size_t)h->Tmax + route::TILE_TOKENS - 1) / route::TILE_TOKENS;
    A(dalloc(&h->w_gu, (size_t)h->n_slots * 2 * f * h->K1));
    A(dalloc(&h->w_dn, (size_t)h->n_slots * d * h->K2));
    A(dalloc(&h->w_rt, (size_t)3 * route::MAX_E * d));
    A(dalloc(&h->w_r8, (size_t)d * route::MAX_E));
    A(dalloc(&h->bias, route::MAX_E));
    A(dalloc(&h->xs, (size_t)h->Tmax * h->K1));
    A(dalloc(&h->xp, (size_t)h->Rcap * h->K1));
    {
        void* p = nullptr;
        if (rc == PRICHS_OK && cudaMalloc(&p, (size_t)h->Tmax * d * (h->mode == PRICHS_MODE_F32 ? 4 : 2)) != cudaSuccess)
            rc = fail(PRICHS_ERR_CUDA, "cudaMalloc of the normalised-activation buffer failed");
        h->xnorm = p;
    }
    A(dalloc(&h->hbuf, rows_all * h->K2));
    {
        void* p = nullptr;
        // (+ the readiness flags of the expert-parallel exchange at its tail, so that one IPC handle maps both)
        const size_t ybytes = rows_all * d * (h->mode == PRICHS_MODE_F32 ? 4 : 2);
        if (rc == PRICHS_OK && cudaMalloc(&p, ybytes + 1024) != cudaSuccess)
            rc = fail(PRICHS_ERR_CUDA, "cudaMalloc of the expert-output buffer failed");
        h->ybuf = p;
        h->y_bytes = ybytes;
        if (p) {
            h->ep_flags = reinterpret_cast<int*>(static_cast<char*>(p) + ybytes);
            cudaMemset(h->ep_flags, 0, 1024);
        }
    }
    A(dalloc(&h->logits, (size_t)h->Tmax * route::MAX_E));
    A(dalloc(&h->gates, (size_t)h->Tmax * 2));
    A(dalloc(&h->sel, (size_t)h->Tmax * 2));
    A(dalloc(&h->pos, (size_t)h->Tmax * 2));
    A(dalloc(&h->tile_counts, ntiles * route::MAX_E));
    A(dalloc(&h->tile_prefix, ntiles * route::MAX_E));
    A(dalloc(&h->mtile_slot, (size_t)h->Rcap / 128 + 1));
    A(dalloc(&h->mtile_row, (size_t)h->Rcap / 128 + 1));
    A(dalloc(&h->tile_state, ntiles * route::MAX_E + 4));
    A(dalloc(&h->rd_ctl, 4));
    A(dalloc(&h->status, 2));  // [0] status word, [1] finished-CTA counter of the router's scan tail
    A(dalloc(&h->meta, 1));
    A(dalloc(&h->ep_zero, 8));
    for (int w = 0; w < h->n_waves && world > 1; ++w) {
        A(dalloc(&h->wave[w].meta, 1));
        A(dalloc(&h->wave[w].mtile_slot, (size_t)h->Rw / 128 + 1));
        A(dalloc(&h->wave[w].token, 2 * route::MAX_RANKS));
    }
    if (rc != PRICHS_OK) {
        prichs_moe_destroy(h);
        return rc;
    }
    cudaMemset(h->bias, 0, route::MAX_E * sizeof(float));
    cudaMemset(h->status, 0, 2 * sizeof(int));
    cudaMemset(h->tile_state, 0, (ntiles * route::MAX_E + 4) * sizeof(uint32_t));
    cudaMemset(h->rd_ctl, 0, 4 * sizeof(int));
    cudaMemset(h->mtile_row, 0, ((size_t)h->Rcap / 128 + 1) * sizeof(int));
    cudaMemset(h->pos, 0, (size_t)h->Tmax * 2 * sizeof(int));  // stale row maps always stay inside the buffers
    cudaMemset(h->meta, 0, sizeof(route::RouteMeta));
    cudaMemset(h->ep_zero, 0, 8 * sizeof(int));
    for (int w = 0; w < h->n_waves && world > 1; ++w) {
        cudaMemset(h->wave[w].meta, 0, sizeof(route::RouteMeta));
        cudaMemset(h->wave[w].token, 0, 2 * route::MAX_RANKS * sizeof(int));
    }
    for (int i = 0; i < route::MAX_RANKS; ++i) {
        h->xp_peer[i] = h->xp;
        h->y_peer[i] = h->ybuf;
        h->flag_peer[i] = h->ep_flags;
    }
    cudaMemset(h->xp, 0, (size_t)h->Rcap * h->K1 * sizeof(bf16));
    cudaMemset(h->hbuf, 0, rows_all * h->K2 * sizeof(bf16));

    A(make_tmap(&h->tm_xp, h->xp, h->Rcap, h->K1, egemm::BM));
    // weights: the matrix of 256 x 64 boxes (see repack_gate_up_kernel)
    A(make_tmap(&h->tm_wgu, h->w_gu, (size_t)h->n_slots * 2 * f * (h->K1 / 64), 64, egemm::BN));
    A(make_tmap(&h->tm_h, h->hbuf, rows_all, h->K2, egemm::BM));
    A(make_tmap(&h->tm_wdn, h->w_dn, (size_t)h->n_slots * d * (h->K2 / 64), 64, egemm::BN));
    A(make_tmap(&h->tm_wgu_half, h->w_gu, (size_t)h->n_slots * 2 * f * (h->K1 / 64), 64, 128));
    A(make_tmap(&h->tm_wdn_half, h->w_dn, (size_t)h->n_slots * d * (h->K2 / 64), 64, 128));
    A(make_tmap(&h->tm_h_out, h->hbuf, rows_all, h->K2, 32));
    A(make_tmap(&h->tm_y_out, h->ybuf, rows_all, d, 32, h->mode == PRICHS_MODE_F32));
    if (rc == PRICHS_OK) {
        if (cudaFuncSetAttribute(egemm::expert_gemm_kernel<egemm::EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, egemm::SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(egemm::expert_gemm_kernel<egemm::EPI_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, egemm::SMEM_BYTES) != cudaSuccess)
            rc = fail(PRICHS_ERR_CUDA, "cannot reserve %d bytes of shared memory for the expert GEMM", egemm::SMEM_BYTES);
        if (cudaFuncSetAttribute(egemm::expert_gemm_kernel<egemm::EPI_PLAIN, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, egemm::GemmShape<128>::SMEM_BYTES) != cudaSuccess)
            rc = fail(PRICHS_ERR_CUDA, "cannot reserve %d bytes of shared memory for the narrow expert GEMM", egemm::GemmShape<128>::SMEM_BYTES);
        if (cudaFuncSetAttribute(egemm::expert_gemm_pair_kernel<egemm::EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, egemm::PAIR_SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(egemm::expert_gemm_pair_kernel<egemm::EPI_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, egemm::PAIR_SMEM_BYTES) != cudaSuccess)
            rc = fail(PRICHS_ERR_CUDA, "cannot reserve %d bytes of shared memory for the CTA-pair expert GEMM", egemm::PAIR_SMEM_BYTES);
    }
    {
        // The CTA-pair kernel (256 x 256 tiles over two SMs) is the default; gemm_kernel = 1 selects the one-CTA
        // kernel (128 x 256 tiles), kept for comparison.
        h->pair_gemm = cfg->gemm_kernel != 1;
        // gemm_kernel = 2: 128-column tiles for the down projection of small batches. Measured on B200 (decode, 24 layers of
        // 64 tokens): 1.075 against 1.125 ms with the layers back to back on one stream, but 0.535 against 0.500 ms on eight
        // streams, where the SMs are busy anyway and narrower tiles only read the rows more often -- hence opt-in.
        h->narrow_down = cfg->gemm_kernel == 2 && h->mode == PRICHS_MODE_BF16;
        h->ep_reserve_sms = cfg->ep_reserve_sms < 0 ? 0 : (cfg->ep_reserve_sms == 0 ? 20 : std::min(64, cfg->ep_reserve_sms) & ~1);
        h->ep_copy_smem = cfg->ep_shared_copy_sms ? 0 : 8192;
        h->pdl = cfg->pdl != 2;
        h->ep_combine_mode = cfg->ep_combine_mode == 1 ? 0 : (cfg->ep_combine_mode == 2 ? 2 : 1);
        h->ep_barrier_mode = cfg->ep_nccl_barriers ? 1 : 0;
        h->ep_timeout_ms = cfg->ep_timeout_ms > 0 ? cfg->ep_timeout_ms : 60000;
        h->db_stages = std::min(route::DB_MAX_STAGES, (200 * 1024) / (route::TILE_TOKENS * h->K1 * 2));
        h->ep_bulk_dispatch = world > 1 && cfg->ep_dispatch_kernel != 1 && h->db_stages >= 2 && h->ep_reserve_sms >= 2;
        if (h->ep_bulk_dispatch && rc == PRICHS_OK &&
            cudaFuncSetAttribute(route::dispatch_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 route::db_smem_bytes(h->K1 * 2, h->db_stages)) != cudaSuccess)
            rc = fail(PRICHS_ERR_CUDA, "cannot reserve shared memory for the bulk dispatch kernel");
        // single-pass route + place + dispatch kernel: as many ring stages as fit next to the router weights (one
        // bf16 part when the weights are bf16 values, three when they are fp32 values; known at upload)
        if (h->mode != PRICHS_MODE_F32 && world == 1) {
            h->rd_stages[0] = rd_stages_for(d, 1);
            h->rd_stages[1] = rd_stages_for(d, 3);
            if (rc == PRICHS_OK && h->rd_stages[0] > 0 &&
                cudaFuncSetAttribute(route::route_dispatch_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     route::rd_smem_bytes(d, 1, h->rd_stages[0])) != cudaSuccess)
                rc = fail(PRICHS_ERR_CUDA, "cannot reserve shared memory for the single-pass routing kernel");
            if (rc == PRICHS_OK && h->rd_stages[1] > 0 &&
                cudaFuncSetAttribute(route::route_dispatch_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     route::rd_smem_bytes(d, 3, h->rd_stages[1])) != cudaSuccess)
                rc = fail(PRICHS_ERR_CUDA, "cannot reserve shared memory for the single-pass routing kernel");
        }
    }
    for (int i = 0; i < 7 && rc == PRICHS_OK; ++i)
        if (cudaEventCreate(&h->ev[i]) != cudaSuccess) rc = fail(PRICHS_ERR_CUDA, "cudaEventCreate failed");
    if (rc == PRICHS_OK && cudaDeviceSynchronize() != cudaSuccess) rc = fail(PRICHS_ERR_CUDA, "device set-up failed");
    if (rc != PRICHS_OK) {
        prichs_moe_destroy(h);
        return rc;
    }
    *out_handle = h;
    return PRICHS_OK;
}

int prichs_moe_destroy(prichs_moe_t* h) {
    if (!h) return PRICHS_OK;
    DeviceGuard guard(h->device);
    cudaDeviceSynchronize();
    // expert-parallel resources: released one by one, so that a set-up that stopped half way leaks nothing
    for (int r = 0; r < route::MAX_RANKS; ++r) {
        if (h->xp_peer[r] && h->xp_peer[r] != h->xp) cudaIpcCloseMemHandle(h->xp_peer[r]);
        if (h->y_peer[r] && h->y_peer[r] != h->ybuf) cudaIpcCloseMemHandle(h->y_peer[r]);
    }
    if (h->side_stream) cudaStreamDestroy(h->side_stream);
    if (h->ev_router) cudaEventDestroy(h->ev_router);
    if (h->ev_shared) cudaEventDestroy(h->ev_shared);
    if (h->tl_base) cudaEventDestroy(h->tl_base);
    if (h->tl_side[0]) cudaEventDestroy(h->tl_side[0]);
    if (h->tl_side[1]) cudaEventDestroy(h->tl_side[1]);
    for (int w = 0; w < MAX_WAVES; ++w) {
        EpWave& wv = h->wave[w];
        if (wv.comm && nccl().ok) nccl().comm_destroy(wv.comm);
        if (wv.stream) cudaStreamDestroy(wv.stream);
        if (wv.done) cudaEventDestroy(wv.done);
        for (int i = 0; i < 8; ++i)
            if (wv.tl[i]) cudaEventDestroy(wv.tl[i]);
        if (wv.meta) cudaFree(wv.meta);
        if (wv.mtile_slot) cudaFree(wv.mtile_slot);
        if (wv.token) cudaFree(wv.token);
    }
    void* ptrs[] = {h->mtile_row, h->tile_state, h->rd_ctl, h->xnorm, h->ep_zero, h->w_gu, h->w_dn, h->w_rt, h->w_r8, h->bias, h->xs, h->xp, h->hbuf, h->ybuf, h->logits, h->gates,
                    h->sel, h->pos, h->tile_counts, h->tile_prefix, h->mtile_slot, h->status, h->meta, h->stage_x,
                    h->stage_r, h->stage_y};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    for (int i = 0; i < 7; ++i)
        if (h->ev[i]) cudaEventDestroy(h->ev[i]);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
    if (h->in_stream) cudaStreamDestroy(h->in_stream);
    if (h->out_stream) cudaStreamDestroy(h->out_stream);
    if (h->chunk_ev) {
        for (int i = 0; i < 128; ++i)
            if (h->chunk_ev[i]) cudaEventDestroy(h->chunk_ev[i]);
        delete[] h->chunk_ev;
    }
    if (h->counts_acc) cudaFree(h->counts_acc);
    {
        void* bp[] = {h->bwd.gu, h->bwd.dyall, h->bwd.dh, h->bwd.dgu, h->bwd.dxall, h->bwd.xT, h->bwd.hT, h->bwd.dyT, h->bwd.dguT,
                      h->bwd.w_dn_nat, h->bwd.w_gu_nat, h->bwd.scal, h->bwd.dlog, h->bwd.dwr_part, h->bwd.stage_dn, h->bwd.stage_gu,
                      h->bwd.dnorm, h->bwd.rinv, h->bwd.dgamma_part};
        for (void* q : bp)
            if (q) cudaFree(q);
    }
    delete h;
    return PRICHS_OK;
}

int prichs_moe_upload_weights(prichs_moe_t* h, const float* const* host_ptrs, int n_ptrs) {
    if (!h || !host_ptrs) return fail(PRICHS_ERR_BAD_ARG, "null handle or pointer array");
    if (n_ptrs != 1 + 3 * (1 + h->E))
        return fail(PRICHS_ERR_BAD_SHAPE, "expected %d weight arrays (router, shared g/u/d, then g/u/d per expert), got %d",
                    1 + 3 * (1 + h->E), n_ptrs);
    DeviceGuard guard(h->device);
    const int d = h->d, f = h->f, E = h->E;
    const int split = h->mode == PRICHS_MODE_F32;
    const size_t nmat = (size_t)d * f;
    float* stage = nullptr;
    CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&stage), 3 * nmat * sizeof(float)));
    int rc = PRICHS_OK;
    auto bail = [&](int r) { cudaFree(stage); return r; };

    // router
    if (!host_ptrs[0]) return bail(fail(PRICHS_ERR_BAD_ARG, "router weights are null"));
    {
        const float* wr = host_ptrs[0];
        bool exact = true;
        for (size_t i = 0; i < (size_t)d * E && exact; ++i) {
            uint32_t bits;
            memcpy(&bits, &wr[i], 4);
            exact = (bits & 0xffffu) == 0;
        }
        h->rt_nsplit = exact ? 1 : 3;
        if (cudaMemcpy(stage, wr, (size_t)d * E * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
            return bail(fail(PRICHS_ERR_CUDA, "copy of the router weights failed"));
        repack_router_kernel<<<64, 256>>>(stage, h->w_rt, h->w_r8, d, E);
        g_launches.fetch_add(1);
    }
    for (int slot = 0; slot < h->n_slots && rc == PRICHS_OK; ++slot) {
        // slot 0 = shared expert, slot 1 + le = routed expert rank*El + le
        const int base = slot == 0 ? 1 : 4 + 3 * (h->rank * h->El + (slot - 1));
        const float *wg = host_ptrs[base], *wu = host_ptrs[base + 1], *wd = host_ptrs[base + 2];
        if (!wg || !wu || !wd) return bail(fail(PRICHS_ERR_BAD_ARG, "weights of a locally owned expert are null (slot %d)", slot));
        if (cudaMemcpy(stage, wg, nmat * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(stage + nmat, wu, nmat * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(stage + 2 * nmat, wd, nmat * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
            return bail(fail(PRICHS_ERR_CUDA, "copy of expert weights failed (slot %d)", slot));
        repack_gate_up_kernel<<<1024, 256>>>(stage, stage + nmat, h->w_gu + (size_t)slot * 2 * f * h->K1, d, f, split);
        repack_down_kernel<<<1024, 256>>>(stage + 2 * nmat, h->w_dn + (size_t)slot * d * h->K2, d, f, split);
        g_launches.fetch_add(2);
        if (cudaDeviceSynchronize() != cudaSuccess) rc = fail(PRICHS_ERR_CUDA, "weight repack failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    cudaFree(stage);
    if (rc == PRICHS_OK) h->weights_ready = true;
    h->bwd.nat_valid = false;
    return rc;
}

int prichs_moe_set_bias(prichs_moe_t* h, const float* host_bias, int n) {
    if (!h || !host_bias) return fail(PRICHS_ERR_BAD_ARG, "null handle or bias");
    if (n != h->E) return fail(PRICHS_ERR_BAD_SHAPE, "router_bias has %d entries, the layer has %d experts", n, h->E);
    DeviceGuard guard(h->device);
    float tmp[route::MAX_E] = {0};
    memcpy(tmp, host_bias, n * sizeof(float));
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));  // a forward or a bias update may still be using the old values
    CUDA_TRY(cudaMemcpy(h->bias, tmp, sizeof(tmp), cudaMemcpyHostToDevice));
    return PRICHS_OK;
}

int prichs_moe_get_bias(prichs_moe_t* h, float* host_bias, int n) {
    if (!h || !host_bias) return fail(PRICHS_ERR_BAD_ARG, "null handle or bias");
    if (n != h->E) return fail(PRICHS_ERR_BAD_SHAPE, "router_bias has %d entries, the layer has %d experts", n, h->E);
    DeviceGuard guard(h->device);
    float tmp[route::MAX_E];
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));  // bias updates are enqueued on the forward's stream
    CUDA_TRY(cudaMemcpy(tmp, h->bias, sizeof(tmp), cudaMemcpyDeviceToHost));
    memcpy(host_bias, tmp, n * sizeof(float));
    return PRICHS_OK;
}

int prichs_moe_forward(prichs_moe_t* h, const void* x_dev, int x_dtype, const void* resid_dev, const float* concept_bias,
                       int n_concept, void* y_dev, int y_dtype, int T, void* stream_) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if (!h->weights_ready) return fail(PRICHS_ERR_BAD_ARG, "weights have not been uploaded");
    if (T < 0) return fail(PRICHS_ERR_BAD_SHAPE, "negative token count");
    if (T > h->Tmax - h->tok_base) return fail(PRICHS_ERR_CAPACITY, "T=%d exceeds max_tokens=%d of this handle", T, h->Tmax);
    if ((x_dtype != PRICHS_DTYPE_F32 && x_dtype != PRICHS_DTYPE_BF16) || (y_dtype != PRICHS_DTYPE_F32 && y_dtype != PRICHS_DTYPE_BF16))
        return fail(PRICHS_ERR_BAD_ARG, "unknown element type");
    if (h->mode == PRICHS_MODE_F32 && x_dtype != PRICHS_DTYPE_F32)
        return fail(PRICHS_ERR_BAD_ARG, "the fp32-fidelity mode takes fp32 activations");
    if (n_concept < 0 || (n_concept > 0 && !concept_bias)) return fail(PRICHS_ERR_BAD_ARG, "concept bias length without data");
    if (h->world > 1 && !h->ep_ready) return fail(PRICHS_ERR_COMM, "expert-parallel exchange is not initialised");
    if (h->ep_broken) return fail(PRICHS_ERR_COMM, "the expert-parallel group was aborted after a peer stopped answering: destroy the handles and connect again");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
    h->last_stream = st;
    h->last_T = T;
    h->last_chunked = false;
    h->last_was_block = false;
    h->last_a_shared = nullptr;
    h->gu_valid = false;
    if (T == 0) {
        if (h->world > 1) return fail(PRICHS_ERR_BAD_SHAPE, "in expert-parallel mode every rank must pass at least one token");
        return PRICHS_OK;
    }
    if (!x_dev || !y_dev) return fail(PRICHS_ERR_BAD_ARG, "null activation pointer");
    if ((reinterpret_cast<uintptr_t>(x_dev) & 15) || (reinterpret_cast<uintptr_t>(y_dev) & 15) ||
        (resid_dev && (reinterpret_cast<uintptr_t>(resid_dev) & 15)))
        return fail(PRICHS_ERR_BAD_ARG, "activation pointers must be 16-byte aligned");
    DeviceGuard guard(h->device);

    const int E = h->E;
    // routing results of this call start at token `tok_base` of the stash arrays (non-zero only while the
    // host-buffer entry point feeds a batch through in chunks)
    float* logits = h->logits + (size_t)h->tok_base * route::MAX_E;
    int* sel = h->sel + (size_t)h->tok_base * 2;
    float* gates = h->gates + (size_t)h->tok_base * 2;
    int* pos = h->pos + (size_t)h->tok_base * 2;
    route::ConceptBias cb;
    for (int e = 0; e < route::MAX_E; ++e) cb.v[e] = (e < n_concept && e < E) ? concept_bias[e] : 0.0f;

    h->small_batch = T < 1024;
    if (h->world > 1) return forward_ep(h, x_dev, x_dtype, resid_dev, cb, y_dev, y_dtype, T, st);

    const bool f32mode = h->mode == PRICHS_MODE_F32;
    const bf16* a_shared = f32mode || x_dtype == PRICHS_DTYPE_F32 || h->norm_w ? h->xs : reinterpret_cast<const bf16*>(x_dev);
    CUtensorMap tm_x;
    int rc = make_tmap(&tm_x, a_shared, (size_t)T, (size_t)h->K1, egemm::BM);
    if (rc != PRICHS_OK) return rc;
    h->last_a_shared = a_shared;

    const bool timing = h->timing;
    int evi = 0;
    auto mark = [&]() { if (timing) cudaEventRecord(h->ev[evi++], st); };
    h->ev_valid = false;

    const int ntiles = (T + route::TILE_TOKENS - 1) / route::TILE_TOKENS;
    mark();
    const bool pdl = h->pdl;
    // Granularity of the GEMM tile table. The CTA-pair kernel walks 256-row tile pairs, so a segment's rows are
    // rounded up to 256. A small batch runs on the one-CTA kernel (128-row tiles): rounding to 128 leaves no tile of
    // padding rows in the table, so the few tiles of a decode step spread evenly over the SMs (with 256 a CTA that
    // draws a padding tile idles while another works through two real ones).
    const int tile_pad = (h->pair_gemm && !h->small_batch) ? SEG_PAD : 128;
    // Routing stage. Single pass (one kernel routes, places and dispatches) when the rows are bf16 as they arrive:
    // from 1024 tokens up by default, always / never with route_kernel = 1 / 2. Otherwise three launches.
    const int rd_stages = h->rd_stages[h->rt_nsplit == 1 ? 0 : 1];
    const bool rd_possible = !f32mode && x_dtype == PRICHS_DTYPE_BF16 && !h->norm_w && rd_stages > 0;
    const bool single_pass = rd_possible && (h->route_kernel == 1 || (h->route_kernel == 0 && !h->small_batch));
    if (single_pass) {
        route::RouteDispatchArgs ra;
        memset(&ra, 0, sizeof(ra));
        ra.x = reinterpret_cast<const bf16*>(x_dev);
        ra.wrt = h->w_rt;
        ra.bias = h->bias;
        ra.T = T; ra.d = h->d; ra.E = E; ra.top_k = h->k; ra.stages = rd_stages;
        ra.logits = logits; ra.sel = sel; ra.gates = gates; ra.pos = pos;
        ra.tile_counts = h->tile_counts; ra.tile_prefix = h->tile_prefix;
        ra.tile_state = h->tile_state; ra.ctl = h->rd_ctl;
        ra.xp = h->xp; ra.seg_stride = h->seg_stride; ra.pad_rows = tile_pad;
        ra.meta = h->meta; ra.mtile_slot = h->mtile_slot; ra.mtile_row = h->mtile_row;
        ra.status = h->status;
        ra.wait_cycles = h->rd_wait_cycles;
        ra.stall_tile = h->rd_stall_tile;
        ra.poll_sleep_ns = h->rd_poll_sleep_ns;
        const int grid = std::min(ntiles, h->sm_count);
        if (h->rt_nsplit == 1)
            LAUNCH_K(pdl, route::route_dispatch_kernel<1>, grid, route::RD_THREADS, route::rd_smem_bytes(h->d, 1, rd_stages), st, ra, cb);
        else
            LAUNCH_K(pdl, route::route_dispatch_kernel<3>, grid, route::RD_THREADS, route::rd_smem_bytes(h->d, 3, rd_stages), st, ra, cb);
        LAUNCH_CHECK("route + dispatch");
        mark();
        mark();  // (no separate scan and dispatch stages: their time reads as zero)
        mark();
    } else {
    // 1. router
    // 2. prefix sums + placement plan: by the last CTA of the router launch for small batches (decode), where a
    //    launch costs more than the work; as a launch of their own for large ones, where the tail would keep the
    //    whole router grid waiting on one CTA's latency chain for no gain (measured on B200: 2 us of 500 at
    //    T = 16384) and the fp32-fidelity router. The config's scan_placement forces one or the other.
    const bool scan_in_router = !f32mode && (h->fuse_scan < 0 ? h->small_batch : h->fuse_scan != 0);
    route::ScanTail tail{};
    if (scan_in_router) {
        tail.done = h->status + 1;
        tail.tile_prefix = h->tile_prefix;
        tail.meta = h->meta;
        tail.mtile_slot = h->mtile_slot;
        tail.mtile_row = h->mtile_row;
        tail.El = h->El;
        tail.cap_rows = h->Rcap;
        tail.pad_rows = tile_pad;
        tail.seg_stride = h->seg_stride;
        tail.status = h->status;
    }
    rc = launch_router(h, x_dev, x_dtype, cb, T, logits, sel, gates, h->tile_counts, st, pdl, tail);
    if (rc != PRICHS_OK) return rc;
    mark();
    if (!scan_in_router) {
        LAUNCH_K(pdl, route::scan_kernel, 1, 1024, 0, st, (const int*)h->tile_counts, h->tile_prefix, ntiles, h->meta, h->mtile_slot, h->mtile_row,
                 E, h->El, 1, 0, h->Rcap, 1, tile_pad, h->seg_stride, h->status);
        LAUNCH_CHECK("scan");
    }
    mark();
    // 3. dispatch
    route::PeerPtrs xp_peers;
    for (int i = 0; i < route::MAX_RANKS; ++i) xp_peers.p[i] = h->xp;
    LAUNCH_K(pdl, route::dispatch_kernel, (T + 7) / 8, 256, 0, st, a_shared, h->K1, T, (const int*)sel, (const int*)h->tile_prefix,
             (const route::RouteMeta*)h->meta, xp_peers, h->El, pos, h->Rcap, h->status);
    LAUNCH_CHECK("dispatch");
    mark();
    }
    route::PeerPtrs y_peers;
    for (int i = 0; i < route::MAX_RANKS; ++i) y_peers.p[i] = h->ybuf;
    // 4. gate|up GEMM + SwiGLU for the shared and all routed experts, 5. down GEMM
    egemm::Args a1, a2;
    gemm_args(h, T, 0, &h->meta->n_routed_mtiles, h->mtile_slot, h->mtile_row, &a1, &a2);
    rc = launch_expert_gemm(h, 0, tm_x, h->tm_xp, a1, h->sm_count, st, pdl);
    if (rc != PRICHS_OK) return rc;
    mark();
    rc = launch_expert_gemm(h, 1, h->tm_h, h->tm_h, a2, h->sm_count, st, pdl);
    if (rc != PRICHS_OK) return rc;
    mark();
    // 6. combine (+ residual)
    rc = launch_combine(h, h->ybuf, y_peers, h->Tcap, sel, gates, pos, resid_dev, y_dev, x_dtype, y_dtype, T, st, false, pdl);
    if (rc != PRICHS_OK) return rc;
    mark();
    h->ev_valid = timing;
    h->gu_valid = h->want_stash;
    return PRICHS_OK;
}

// Allocates the buffer of the [gate | up] pre-activations (rows of the forward's row space, 2f bf16 columns in the
// column order of the first GEMM's B operand).
static int stash_alloc(prichs_moe* h) {
    if (h->bwd.gu) return PRICHS_OK;
    const size_t R = (size_t)h->Tcap + h->Rcap;
    int rc = dalloc(&h->bwd.gu, R * 2 * h->f);
    if (rc != PRICHS_OK) return rc;
    CUDA_TRY(cudaMemset(h->bwd.gu, 0, R * 2 * h->f * sizeof(bf16)));
    return PRICHS_OK;
}

int prichs_moe_forward_train(prichs_moe_t* h, const void* x_dev, int x_dtype, const void* resid_dev, const float* concept_bias,
                             int n_concept, void* y_dev, int y_dtype, int T, void* stream) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if (h->world > 1 || h->mode != PRICHS_MODE_BF16)
        return fail(PRICHS_ERR_BAD_ARG, "the training forward (activation stash) runs with all experts local in the bf16 mode");
    {
        DeviceGuard guard(h->device);
        int rc = stash_alloc(h);
        if (rc != PRICHS_OK) return rc;
    }
    h->want_stash = true;
    const int rc = prichs_moe_forward(h, x_dev, x_dtype, resid_dev, concept_bias, n_concept, y_dev, y_dtype, T, stream);
    h->want_stash = false;
    return rc;
}

int prichs_moe_block_forward(prichs_moe_t* h, const void* x_res_dev, int x_dtype, const float* norm_weight_dev, float eps,
                             const float* concept_bias, int n_concept, void* y_dev, int y_dtype, int T, void* stream_) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if (!x_res_dev || !norm_weight_dev || !y_dev) return fail(PRICHS_ERR_BAD_ARG, "null device pointer");
    if (x_dtype != PRICHS_DTYPE_F32 && x_dtype != PRICHS_DTYPE_BF16) return fail(PRICHS_ERR_BAD_ARG, "unknown element type");
    if (T < 0 || T > h->Tmax) return fail(PRICHS_ERR_CAPACITY, "T=%d exceeds max_tokens=%d of this handle", T, h->Tmax);
    if (h->d > 2048) return fail(PRICHS_ERR_BAD_SHAPE, "the fused pre-norm supports hidden_dim up to 2048");
    if (h->mode == PRICHS_MODE_F32 && x_dtype != PRICHS_DTYPE_F32) return fail(PRICHS_ERR_BAD_ARG, "the fp32-fidelity mode takes fp32 activations");
    if ((reinterpret_cast<uintptr_t>(x_res_dev) & 15) || (reinterpret_cast<uintptr_t>(norm_weight_dev) & 15))
        return fail(PRICHS_ERR_BAD_ARG, "activation and weight pointers must be 16-byte aligned");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
    const bool of32 = h->mode == PRICHS_MODE_F32;
    // bf16 mode, whole row in one router pass: the norm is folded into the router kernel's read of the rows, which
    // then also writes the normalised bf16 rows the dispatch and the shared expert consume
    const bool fused = h->fuse_norm && !of32 && h->d <= route::ROUTER_KB * route::ROUTER_WARPS * 32 && h->d % 256 == 0;
    if (T > 0 && !fused) {
        DeviceGuard guard(h->device);
        const int grid = (T + 7) / 8;
        if (x_dtype == PRICHS_DTYPE_F32) {
            if (of32) route::rmsnorm_rows_kernel<true, true, 8><<<grid, 256, 0, st>>>(x_res_dev, norm_weight_dev, eps, h->xnorm, T, h->d);
            else route::rmsnorm_rows_kernel<true, false, 8><<<grid, 256, 0, st>>>(x_res_dev, norm_weight_dev, eps, h->xnorm, T, h->d);
        } else {
            route::rmsnorm_rows_kernel<false, false, 8><<<grid, 256, 0, st>>>(x_res_dev, norm_weight_dev, eps, h->xnorm, T, h->d);
        }
        LAUNCH_CHECK("pre-norm");
    }
    // the normalised rows are the layer's input, the un-normalised ones its fused residual (block.rs:64-67)
    h->resid_dtype = x_dtype;  // the residual keeps the caller's element type even when the normalised input is bf16
    int rc;
    if (fused) {
        h->norm_w = norm_weight_dev;
        h->norm_eps = eps;
        rc = prichs_moe_forward(h, x_res_dev, x_dtype, x_res_dev, concept_bias, n_concept, y_dev, y_dtype, T, stream_);
        h->norm_w = nullptr;
    } else {
        rc = prichs_moe_forward(h, h->xnorm, of32 ? PRICHS_DTYPE_F32 : PRICHS_DTYPE_BF16, x_res_dev, concept_bias, n_concept, y_dev,
                                y_dtype, T, stream_);
    }
    h->resid_dtype = -1;
    h->last_was_block = rc == PRICHS_OK;
    return rc;
}

}  // extern "C"

namespace {
int ep_query_stream(void* ctx);   // watchdog callbacks, defined next to prichs_moe_sync_status
void ep_abort_comms(void* ctx);
constexpr int HOST_MAX_CHUNKS = 64;
// Staging buffers, streams and events of the entry points that take host buffers; every resource is created only
// if it is still missing, so a call that failed half way can be repeated.
int host_path_setup(prichs_moe* h) {
    if (h->host_ready) return PRICHS_OK;
    const size_t n = (size_t)h->Tmax * h->d;
    int rc = PRICHS_OK;
    if (!h->stage_x) rc = dalloc(&h->stage_x, n);
    if (rc == PRICHS_OK && !h->stage_y) rc = dalloc(&h->stage_y, n);
    if (rc == PRICHS_OK && !h->counts_acc) rc = dalloc(&h->counts_acc, 2 * route::MAX_E);
    if (rc != PRICHS_OK) return rc;
    if (!h->own_stream) CUDA_TRY(cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking));
    if (!h->in_stream) CUDA_TRY(cudaStreamCreateWithFlags(&h->in_stream, cudaStreamNonBlocking));
    if (!h->out_stream) CUDA_TRY(cudaStreamCreateWithFlags(&h->out_stream, cudaStreamNonBlocking));
    if (!h->chunk_ev) h->chunk_ev = new cudaEvent_t[2 * HOST_MAX_CHUNKS]();
    for (int i = 0; i < 2 * HOST_MAX_CHUNKS; ++i)
        if (!h->chunk_ev[i]) CUDA_TRY(cudaEventCreateWithFlags(&h->chunk_ev[i], cudaEventDisableTiming));
    h->host_ready = true;
    return PRICHS_OK;
}
}  // namespace

extern "C" {

int prichs_moe_forward_host(prichs_moe_t* h, const float* x_host, const float* resid_host, const float* concept_bias,
                            int n_concept, float* y_host, int T) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if (T < 0) return fail(PRICHS_ERR_BAD_SHAPE, "negative token count");
    if (T > h->Tmax) return fail(PRICHS_ERR_CAPACITY, "T=%d exceeds max_tokens=%d of this handle", T, h->Tmax);
    if (T == 0) return PRICHS_OK;
    if (!x_host || !y_host) return fail(PRICHS_ERR_BAD_ARG, "null host buffer");
    DeviceGuard guard(h->device);
    const size_t n = (size_t)h->Tmax * h->d;
    constexpr int MAX_CHUNKS = HOST_MAX_CHUNKS;
    {
        const int rc0 = host_path_setup(h);
        if (rc0 != PRICHS_OK) return rc0;
    }
    if (resid_host && !h->stage_r) {
        int rc = dalloc(&h->stage_r, n);
        if (rc != PRICHS_OK) return rc;
    }
    // Tokens are independent, so a large batch is fed through in chunks: the upload of chunk i+1 and the
    // download of chunk i-1 overlap the kernels of chunk i (three streams). Results are bit-identical to one
    // pass; counts are summed over the chunks.
    // Chunk boundaries. All experts local: chunks of 1024 (2048) tokens. Expert parallel: every forward is a collective,
    // so all ranks must run the SAME number of chunks; that number depends only on max_tokens (equal on all ranks by
    // contract) and every rank cuts its own T into that many pieces.
    std::vector<int> bounds;  // chunk c covers tokens [bounds[c], bounds[c + 1])
    bounds.push_back(0);
    if (h->world == 1 && T >= 4096) {
        // Chunks of 1024 (2048) tokens; the config's host_chunk_tokens overrides. (Measured on B200: smaller first and
        // last chunks do not help, 2.76 against 2.72 ms per 16384 tokens; the copies run at 0.8 of their stand-alone
        // duplex rate while the GEMMs of other chunks run beside them.)
        int chunk = h->host_chunk > 0 ? h->host_chunk : (T >= 8192 ? 1024 : 2048);
        while ((T + chunk - 1) / chunk > MAX_CHUNKS) chunk *= 2;
        for (int t = 0; t < T;) bounds.push_back(t += std::min(chunk, T - t));
    } else if (h->world > 1) {
        const int n = std::max(1, std::min(8, h->Tmax / (h->host_chunk > 0 ? h->host_chunk : 8192)));
        if (n > 1 && T < 16 * n)
            return fail(PRICHS_ERR_BAD_SHAPE, "in expert-parallel mode the host-buffer entry point cuts every rank's batch into %d chunks: pass at least %d tokens", n, 16 * n);
        for (int c = 1; c < n; ++c) bounds.push_back((int)((long long)T * c / n / 16 * 16));
        bounds.push_back(T);
    } else {
        bounds.push_back(T);
    }
    const int nchunks = (int)bounds.size() - 1;
    auto bound = [&](int c) -> int { return bounds[c]; };
    cudaStream_t st = h->own_stream;
    const size_t row = (size_t)h->d;
    int rc = PRICHS_OK;
    // Chunk forwards are short and interleaved with copies on two other streams; measured on B200, kernels that are
    // launched early (programmatic dependent launch) and then wait on the SMs slow this pipeline down by a tenth,
    // while they gain a little on the device-resident path. So the chunks are launched without it.
    struct PdlOff {
        prichs_moe* h;
        bool saved;
        explicit PdlOff(prichs_moe* hh) : h(hh), saved(hh->pdl) { h->pdl = false; }
        ~PdlOff() { h->pdl = saved; }
    } pdl_off(h);
    // All uploads are enqueued first: the copy engine then never waits for the host thread, which needs about as long to
    // enqueue a chunk's kernels as the link needs to move a chunk.
    for (int c = 0; c < nchunks; ++c) {
        const int t0 = bound(c), tc = bound(c + 1) - t0;
        const size_t off = (size_t)t0 * row, bytes = (size_t)tc * row * sizeof(float);
        CUDA_TRY(cudaMemcpyAsync(h->stage_x + off, x_host + off, bytes, cudaMemcpyHostToDevice, h->in_stream));
        if (resid_host) CUDA_TRY(cudaMemcpyAsync(h->stage_r + off, resid_host + off, bytes, cudaMemcpyHostToDevice, h->in_stream));
        CUDA_TRY(cudaEventRecord(h->chunk_ev[2 * c], h->in_stream));
    }
    for (int c = 0; c < nchunks && rc == PRICHS_OK; ++c) {
        const int t0 = bound(c), tc = bound(c + 1) - t0;
        const size_t off = (size_t)t0 * row, bytes = (size_t)tc * row * sizeof(float);
        cudaEvent_t ev_in = h->chunk_ev[2 * c], ev_done = h->chunk_ev[2 * c + 1];
        CUDA_TRY(cudaStreamWaitEvent(st, ev_in, 0));
        h->tok_base = t0;
        rc = prichs_moe_forward(h, h->stage_x + off, PRICHS_DTYPE_F32, resid_host ? h->stage_r + off : nullptr, concept_bias,
                                n_concept, h->stage_y + off, PRICHS_DTYPE_F32, tc, st);
        h->tok_base = 0;
        if (rc != PRICHS_OK) break;
        if (nchunks > 1) {
            host_chunk_accumulate_kernel<<<1, 32, 0, st>>>(h->meta, h->counts_acc, c == 0);
            LAUNCH_CHECK("count accumulation");
        }
        CUDA_TRY(cudaEventRecord(ev_done, st));
        CUDA_TRY(cudaStreamWaitEvent(h->out_stream, ev_done, 0));
        CUDA_TRY(cudaMemcpyAsync(y_host + off, h->stage_y + off, bytes, cudaMemcpyDeviceToHost, h->out_stream));
    }
    if (rc == PRICHS_OK && nchunks > 1) {
        host_chunk_finish_kernel<<<1, 32, 0, st>>>(h->meta, h->counts_acc, h->rank);
        LAUNCH_CHECK("count totals");
    }
    h->last_T = T;
    h->last_stream = st;
    h->last_chunked = nchunks > 1;
    if (rc == PRICHS_OK && h->world > 1) {
        // the forwards hold collectives: wait for them under the watchdog, not for ever (see prichs_moe_sync_status)
        const int wrc = prichs_ep_wait_or_abort(ep_query_stream, ep_abort_comms, h, h->ep_timeout_ms, 50);
        if (wrc != PRICHS_OK) return wrc;
    }
    cudaError_t e1 = cudaStreamSynchronize(h->in_stream), e2 = cudaStreamSynchronize(st), e3 = cudaStreamSynchronize(h->out_stream);
    if (rc != PRICHS_OK) return rc;
    if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess)
        return fail(PRICHS_ERR_CUDA, "host-buffer forward failed: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3)));
    int sdev = 0;
    CUDA_TRY(cudaMemcpy(&sdev, h->status, sizeof(int), cudaMemcpyDeviceToHost));
    return translate_status(sdev);
}

// Host-side watchdog of the control plane. `query` says whether the awaited work has finished (0 = done, 1 = still
// running, anything else = failed); it is polled every poll_us microseconds for at most timeout_ms milliseconds.
// When the time runs out `abort_fn` (may be null) is called once -- the library passes a function that aborts its
// NCCL communicators, which releases a collective that a peer never joined -- and PRICHS_ERR_COMM is returned.
// Exported so that the policy can be exercised without a GPU (the tests drive it with gloo ranks one of which
// never posts its counts).
int prichs_ep_wait_or_abort(int (*query)(void*), void (*abort_fn)(void*), void* ctx, int timeout_ms, int poll_us) {
    if (!query || timeout_ms < 0) return fail(PRICHS_ERR_BAD_ARG, "null query function or negative timeout");
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const int q = query(ctx);
        if (q == 0) return PRICHS_OK;
        if (q != 1) return fail(PRICHS_ERR_COMM, "the awaited work failed (query returned %d)", q);
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms >= timeout_ms) {
            if (abort_fn) abort_fn(ctx);
            return fail(PRICHS_ERR_COMM, "no answer from the expert-parallel group within %d ms: a peer never joined a collective; the communicators were aborted", timeout_ms);
        }
        if (poll_us > 0) std::this_thread::sleep_for(std::chrono::microseconds(poll_us));
    }
}

}  // extern "C"

namespace {
int ep_query_stream(void* ctx) {
    prichs_moe* h = static_cast<prichs_moe*>(ctx);
    const cudaError_t e = cudaStreamQuery(h->last_stream);
    if (e == cudaSuccess) return 0;
    if (e != cudaErrorNotReady) return 2;
    for (int w = 0; w < h->n_waves; ++w) {  // a communicator that reports an asynchronous error will not finish either
        int st = 0;
        if (h->wave[w].comm && nccl().comm_async_error && nccl().comm_async_error(h->wave[w].comm, &st) == 0 && st != 0) return 3;
    }
    return 1;
}
void ep_abort_comms(void* ctx) {
    prichs_moe* h = static_cast<prichs_moe*>(ctx);
    for (int w = 0; w < MAX_WAVES; ++w)
        if (h->wave[w].comm && nccl().comm_abort) {
            nccl().comm_abort(h->wave[w].comm);
            h->wave[w].comm = nullptr;
        }
    h->ep_broken = true;
}
}  // namespace

extern "C" {

int prichs_moe_sync_status(prichs_moe_t* h) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    DeviceGuard guard(h->device);
    if (h->world > 1 && h->ep_ready) {
        // an expert-parallel forward holds collectives: wait with a limit instead of blocking for ever on a lost peer
        const int rc = prichs_ep_wait_or_abort(ep_query_stream, ep_abort_comms, h, h->ep_timeout_ms, 50);
        if (rc != PRICHS_OK) return rc;
    }
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    int s = 0;
    CUDA_TRY(cudaMemcpy(&s, h->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (s != 0) {
        // reported once, then the handle goes on: the scratch state of the kernels that may have given up starts clean
        CUDA_TRY(cudaMemset(h->status, 0, 2 * sizeof(int)));
        const size_t ntiles = ((size_t)h->Tmax + route::TILE_TOKENS - 1) / route::TILE_TOKENS;
        CUDA_TRY(cudaMemset(h->tile_state, 0, (ntiles * route::MAX_E + 4) * sizeof(uint32_t)));
        CUDA_TRY(cudaMemset(h->rd_ctl, 0, 4 * sizeof(int)));
    }
    return translate_status(s);
}

int prichs_moe_get_counts(prichs_moe_t* h, int64_t* counts_host, int n) {
    if (!h || !counts_host) return fail(PRICHS_ERR_BAD_ARG, "null handle or output");
    if (n != h->E) return fail(PRICHS_ERR_BAD_SHAPE, "counts has %d entries, the layer has %d experts", n, h->E);
    DeviceGuard guard(h->device);
    if (h->last_T == 0) {
        for (int i = 0; i < n; ++i) counts_host[i] = 0;
        return PRICHS_OK;
    }
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    route::RouteMeta m;
    CUDA_TRY(cudaMemcpy(&m, h->meta, sizeof(m), cudaMemcpyDeviceToHost));
    for (int i = 0; i < n; ++i) counts_host[i] = m.counts[i];
    return PRICHS_OK;
}

int prichs_moe_get_routing(prichs_moe_t* h, float* logits_host, int32_t* selected_host, float* gating_host, int T) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if (T != h->last_T) return fail(PRICHS_ERR_BAD_SHAPE, "T=%d differs from the last forward's T=%d", T, h->last_T);
    if (T == 0) return PRICHS_OK;
    DeviceGuard guard(h->device);
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    const int E = h->E, k = h->k;
    if (logits_host) {
        std::vector<float> tmp((size_t)T * route::MAX_E);
        CUDA_TRY(cudaMemcpy(tmp.data(), h->logits, tmp.size() * sizeof(float), cudaMemcpyDeviceToHost));
        for (int t = 0; t < T; ++t)
            for (int e = 0; e < E; ++e) logits_host[(size_t)t * E + e] = tmp[(size_t)t * route::MAX_E + e];
    }
    if (selected_host) {
        std::vector<int> tmp((size_t)T * 2);
        CUDA_TRY(cudaMemcpy(tmp.data(), h->sel, tmp.size() * sizeof(int), cudaMemcpyDeviceToHost));
        for (int t = 0; t < T; ++t)
            for (int j = 0; j < k; ++j) selected_host[(size_t)t * k + j] = tmp[(size_t)t * 2 + j] & 0xff;
    }
    if (gating_host) {
        std::vector<float> tmp((size_t)T * 2);
        CUDA_TRY(cudaMemcpy(tmp.data(), h->gates, tmp.size() * sizeof(float), cudaMemcpyDeviceToHost));
        for (int t = 0; t < T; ++t)
            for (int j = 0; j < k; ++j) gating_host[(size_t)t * k + j] = tmp[(size_t)t * 2 + j];
    }
    return PRICHS_OK;
}

int prichs_moe_update_aux_free_bias(prichs_moe_t* h, const size_t* expert_token_counts, int n, size_t total_tokens, float gamma) {
    if (!h || !expert_token_counts) return fail(PRICHS_ERR_BAD_ARG, "null handle or counts");
    if (n != h->E) return fail(PRICHS_ERR_BAD_SHAPE, "counts has %d entries, the layer has %d experts", n, h->E);
    if (total_tokens == 0) return PRICHS_OK;  // the reference returns early (moe.rs:233-235)
    DeviceGuard guard(h->device);
    // Host-supplied counts travel as kernel arguments: no allocation, no copy, no device-wide synchronisation. The
    // launch goes to the stream of the handle's last forward, so it is ordered after the router that read the bias
    // and before the next forward on that stream.
    route::ExpertCounts hc;
    for (int i = 0; i < route::MAX_E; ++i) hc.c[i] = i < n ? (unsigned long long)expert_token_counts[i] : 0ull;
    route::bias_update_kernel<<<1, 32, 0, h->last_stream>>>(h->bias, nullptr, hc, h->E, h->k, gamma, (unsigned long long)total_tokens);
    LAUNCH_CHECK("bias update");
    return PRICHS_OK;
}

int prichs_moe_update_bias_from_last(prichs_moe_t* h, float gamma, size_t total_tokens, void* stream_) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    DeviceGuard guard(h->device);
    unsigned long long tot = total_tokens ? (unsigned long long)total_tokens : (unsigned long long)h->last_T * h->world;
    if (tot == 0) return PRICHS_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
    if (st != h->last_stream && h->last_T > 0) {
        // another stream than the forward's: order the update after the forward that wrote the counts and read the bias
        cudaEvent_t ev;
        CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        cudaEventRecord(ev, h->last_stream);
        cudaStreamWaitEvent(st, ev, 0);
        cudaEventDestroy(ev);
    }
    route::bias_update_kernel<<<1, 32, 0, st>>>(h->bias, h->meta, route::ExpertCounts{}, h->E, h->k, gamma, tot);
    LAUNCH_CHECK("bias update");
    return PRICHS_OK;
}

int prichs_moe_ep_unique_id(void* id128) {
    if (!id128) return fail(PRICHS_ERR_BAD_ARG, "null id buffer");
    if (!nccl().ok) return fail(PRICHS_ERR_COMM, "libnccl.so.2 could not be loaded");
    memset(id128, 0, PRICHS_EP_ID_BYTES);
    for (int w = 0; w < MAX_WAVES; ++w) NCCL_TRY(nccl().get_unique_id(static_cast<char*>(id128) + 128 * w));
    return PRICHS_OK;
}

int prichs_moe_ep_export(prichs_moe_t* h, void* blob128) {
    if (!h || !blob128) return fail(PRICHS_ERR_BAD_ARG, "null handle or blob");
    static_assert(2 * sizeof(cudaIpcMemHandle_t) <= PRICHS_EP_BLOB_BYTES, "two IPC handles must fit the blob");
    DeviceGuard guard(h->device);
    cudaIpcMemHandle_t hs[2];
    CUDA_TRY(cudaIpcGetMemHandle(&hs[0], h->xp));
    CUDA_TRY(cudaIpcGetMemHandle(&hs[1], h->ybuf));
    memset(blob128, 0, PRICHS_EP_BLOB_BYTES);
    memcpy(blob128, hs, sizeof(hs));
    return PRICHS_OK;
}

int prichs_moe_ep_init(prichs_moe_t* h, const void* id128, const void* all_blobs) {
    if (!h || !id128 || !all_blobs) return fail(PRICHS_ERR_BAD_ARG, "null handle, id or blobs");
    if (h->world < 2) return fail(PRICHS_ERR_BAD_ARG, "the handle was created with ep_world = 1");
    if (h->ep_ready) return fail(PRICHS_ERR_BAD_ARG, "expert-parallel group is already initialised");
    if (!nccl().ok) return fail(PRICHS_ERR_COMM, "libnccl.so.2 could not be loaded");
    DeviceGuard guard(h->device);
    for (int r = 0; r < h->world; ++r) {
        if (r == h->rank) continue;
        cudaIpcMemHandle_t hs[2];
        memcpy(hs, static_cast<const char*>(all_blobs) + (size_t)r * PRICHS_EP_BLOB_BYTES, sizeof(hs));
        void *pxp = nullptr, *py = nullptr;
        CUDA_TRY(cudaIpcOpenMemHandle(&pxp, hs[0], cudaIpcMemLazyEnablePeerAccess));
        CUDA_TRY(cudaIpcOpenMemHandle(&py, hs[1], cudaIpcMemLazyEnablePeerAccess));
        h->xp_peer[r] = pxp;
        h->y_peer[r] = py;
        h->flag_peer[r] = static_cast<char*>(py) + h->y_bytes;  // every rank has the same sizes
    }
    static_assert(MAX_WAVES * 128 <= PRICHS_EP_ID_BYTES, "one 128-byte communicator id per wave");
    // Stream priorities order the work of a forward when several kernels compete for SMs: the shared expert
    // first (every wave's combine needs it), then wave 0, wave 1, ... so that an earlier wave's exchange and
    // combine are never queued behind a later wave's GEMM.
    int prio_lo = 0, prio_hi = 0;
    CUDA_TRY(cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi));  // hi is the numerically smallest
    auto prio = [&](int rank_from_top) { return std::min(prio_lo, prio_hi + rank_from_top); };
    for (int w = 0; w < h->n_waves; ++w) {
        NcclApi::Id128 id;
        memcpy(&id, static_cast<const char*>(id128) + 128 * w, sizeof(id));
        NCCL_TRY(nccl().comm_init_rank(&h->wave[w].comm, h->world, id, h->rank));
        CUDA_TRY(cudaStreamCreateWithPriority(&h->wave[w].stream, cudaStreamNonBlocking, prio(1 + w)));
        CUDA_TRY(cudaEventCreateWithFlags(&h->wave[w].done, cudaEventDisableTiming));
        for (int i = 0; i < 8; ++i) CUDA_TRY(cudaEventCreate(&h->wave[w].tl[i]));
    }
    CUDA_TRY(cudaEventCreate(&h->tl_base));
    CUDA_TRY(cudaEventCreate(&h->tl_side[0]));
    CUDA_TRY(cudaEventCreate(&h->tl_side[1]));
    CUDA_TRY(cudaStreamCreateWithPriority(&h->side_stream, cudaStreamNonBlocking, prio(0)));
    CUDA_TRY(cudaEventCreateWithFlags(&h->ev_router, cudaEventDisableTiming));
    CUDA_TRY(cudaEventCreateWithFlags(&h->ev_shared, cudaEventDisableTiming));
    h->ep_ready = true;
    return PRICHS_OK;
}

int prichs_moe_ep_recv_rows(prichs_moe_t* h, int64_t* rows) {
    if (!h || !rows) return fail(PRICHS_ERR_BAD_ARG, "null handle or output");
    DeviceGuard guard(h->device);
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    route::RouteMeta m;
    CUDA_TRY(cudaMemcpy(&m, h->meta, sizeof(m), cudaMemcpyDeviceToHost));
    *rows = m.recv_rows;
    return PRICHS_OK;
}

// ---- backward pass ---------------------------------------------------------------------------------------
namespace {

int bwd_alloc(prichs_moe* h) {
    prichs_moe::Bwd& b = h->bwd;
    if (b.ready) return PRICHS_OK;
    const size_t R = (size_t)h->Tcap + h->Rcap, d = h->d, f = h->f;
    int rc = PRICHS_OK;
    auto A = [&](int r) { if (rc == PRICHS_OK) rc = r; };
    if (!b.gu) A(stash_alloc(h));
    if (!b.dyall) A(dalloc(&b.dyall, R * d));
    if (!b.dh) A(dalloc(&b.dh, R * f));
    if (!b.dgu) A(dalloc(&b.dgu, R * 2 * f));
    if (!b.dxall) A(dalloc(&b.dxall, R * d));
    if (!b.xT) A(dalloc(&b.xT, d * R));
    if (!b.hT) A(dalloc(&b.hT, f * R));
    if (!b.dyT) A(dalloc(&b.dyT, d * R));
    if (!b.dguT) A(dalloc(&b.dguT, 2 * f * R));
    if (!b.w_dn_nat) A(dalloc(&b.w_dn_nat, (size_t)h->n_slots * f * d));
    if (!b.w_gu_nat) A(dalloc(&b.w_gu_nat, (size_t)h->n_slots * d * 2 * f));
    if (!b.scal) A(dalloc(&b.scal, (size_t)h->Tmax * 2));
    if (!b.dlog) A(dalloc(&b.dlog, (size_t)h->Tmax * route::MAX_E));
    if (!b.dwr_part) A(dalloc(&b.dwr_part, (size_t)bwd::DWR_SPLITS * d * route::MAX_E));
    if (!b.stage_dn) A(dalloc(&b.stage_dn, f * d));
    if (!b.stage_gu) A(dalloc(&b.stage_gu, d * 2 * f));
    if (!b.dnorm) A(dalloc(&b.dnorm, (size_t)h->Tmax * d));
    if (!b.rinv) A(dalloc(&b.rinv, (size_t)h->Tmax));
    if (!b.dgamma_part) A(dalloc(&b.dgamma_part, (size_t)bwd::DWR_SPLITS * d));
    if (rc != PRICHS_OK) return rc;
    // rows that no kernel of a backward pass writes (padding of the permuted region) must stay finite
    CUDA_TRY(cudaMemset(b.dyall, 0, R * d * sizeof(bf16)));
    CUDA_TRY(cudaMemset(b.dh, 0, R * f * sizeof(bf16)));
    CUDA_TRY(cudaMemset(b.dgu, 0, R * 2 * f * sizeof(bf16)));
    CUDA_TRY(cudaMemset(b.dxall, 0, R * d * sizeof(bf16)));
    A(make_tmap(&b.tm_dyall, b.dyall, R, d, egemm::BM));
    A(make_tmap(&b.tm_dgu, b.dgu, R, 2 * f, egemm::BM));
    A(make_tmap(&b.tm_gu_out, b.gu, R, 2 * f, 32));
    A(make_tmap(&b.tm_dh_out, b.dh, R, f, 32));
    A(make_tmap(&b.tm_dxall_out, b.dxall, R, d, 32));
    A(make_tmap(&b.tm_wdn_nat, b.w_dn_nat, (size_t)h->n_slots * f, d, egemm::BN));
    A(make_tmap(&b.tm_wgu_nat, b.w_gu_nat, (size_t)h->n_slots * d, 2 * f, egemm::BN));
    A(make_tmap(&b.tm_stage_dn, b.stage_dn, f, d, 32, true));
    A(make_tmap(&b.tm_stage_gu, b.stage_gu, d, 2 * f, 32, true));
    if (rc == PRICHS_OK) b.ready = true;
    return rc;
}

int bwd_transpose(const bf16* src, bf16* dst, long long rows, int cols, long long src_pitch, long long dst_pitch, cudaStream_t st,
                  int src_nkt = 0) {
    if (rows <= 0) return PRICHS_OK;
    const dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
    bwd::transpose_bf16_kernel<<<grid, 256, 0, st>>>(src, dst, rows, cols, src_pitch, dst_pitch, src_nkt);
    LAUNCH_CHECK("transpose");
    return PRICHS_OK;
}

// One launch of the one-CTA grouped GEMM with a plain epilogue.
int bwd_gemm(prichs_moe* h, const CUtensorMap& tm_a_shared, const CUtensorMap& tm_a_routed, const CUtensorMap& tm_b,
             const CUtensorMap& tm_out, const egemm::Args& a, cudaStream_t st, const char* what) {
    LAUNCH_K(false, egemm::expert_gemm_kernel<egemm::EPI_PLAIN>, h->sm_count, egemm::NUM_THREADS, egemm::SMEM_BYTES, st, tm_a_shared,
             tm_a_routed, tm_b, tm_out, a);
    LAUNCH_CHECK(what);
    return PRICHS_OK;
}

}  // namespace

namespace {

// Checks shared by the two backward entry points; returns the T of the forward to differentiate through *T_out.
int bwd_check(prichs_moe* h, const void* dy_dev, int dy_dtype, const void* dx_dev, float* const* grads_dev, int n_grads, int* T_out) {
    if (h->world > 1) return fail(PRICHS_ERR_BAD_ARG, "the backward pass runs with all experts local (ep_world = 1)");
    if (h->mode != PRICHS_MODE_BF16) return fail(PRICHS_ERR_BAD_ARG, "the backward pass runs in the bf16 mode");
    if (h->f % 256 != 0) return fail(PRICHS_ERR_BAD_SHAPE, "the backward pass needs intermediate_dim to be a multiple of 256 (got %d)", h->f);
    if (!dy_dev || !dx_dev) return fail(PRICHS_ERR_BAD_ARG, "null gradient pointer");
    if (dy_dtype != PRICHS_DTYPE_F32 && dy_dtype != PRICHS_DTYPE_BF16) return fail(PRICHS_ERR_BAD_ARG, "unknown element type");
    if (grads_dev && n_grads != 1 + 3 * (1 + h->E))
        return fail(PRICHS_ERR_BAD_SHAPE, "expected %d gradient buffers (router, shared g/u/d, then g/u/d per expert), got %d", 1 + 3 * (1 + h->E), n_grads);
    if ((reinterpret_cast<uintptr_t>(dy_dev) & 15) || (reinterpret_cast<uintptr_t>(dx_dev) & 15))
        return fail(PRICHS_ERR_BAD_ARG, "gradient pointers must be 16-byte aligned");
    if (h->last_T <= 0 || !h->last_a_shared) return fail(PRICHS_ERR_BAD_ARG, "no forward pass to differentiate: call prichs_moe_forward first");
    if (h->last_chunked) return fail(PRICHS_ERR_BAD_ARG, "the last forward went through host buffers in chunks; run prichs_moe_forward on device buffers before the backward pass");
    *T_out = h->last_T;
    return PRICHS_OK;
}

int backward_impl(prichs_moe* h, const bf16* a_shared, const void* dy_dev, int dy_dtype, float* dx_dev, float* const* grads_dev,
                  cudaStream_t st);

}  // namespace

int prichs_moe_backward(prichs_moe_t* h, const void* x_dev, int x_dtype, const void* dy_dev, int dy_dtype, float* dx_dev,
                        float* const* grads_dev, int n_grads, void* stream_) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if (!x_dev) return fail(PRICHS_ERR_BAD_ARG, "null activation pointer");
    if (x_dtype != PRICHS_DTYPE_F32 && x_dtype != PRICHS_DTYPE_BF16) return fail(PRICHS_ERR_BAD_ARG, "unknown element type");
    int T = 0;
    int rc = bwd_check(h, dy_dev, dy_dtype, dx_dev, grads_dev, n_grads, &T);
    if (rc != PRICHS_OK) return rc;
    if (h->last_was_block) return fail(PRICHS_ERR_BAD_ARG, "the last forward was prichs_moe_block_forward: use prichs_moe_block_backward");
    // the layer input as the forward used it: the caller's bf16 rows, or the bf16 copy the router wrote
    const bf16* a_shared = x_dtype == PRICHS_DTYPE_F32 ? h->xs : reinterpret_cast<const bf16*>(x_dev);
    if (a_shared != h->last_a_shared) return fail(PRICHS_ERR_BAD_ARG, "x_dev is not the input of the last forward on this handle");
    DeviceGuard guard(h->device);
    return backward_impl(h, a_shared, dy_dev, dy_dtype, dx_dev, grads_dev, reinterpret_cast<cudaStream_t>(stream_));
}

int prichs_moe_block_backward(prichs_moe_t* h, const void* x_res_dev, int x_dtype, const float* norm_weight_dev, float eps,
                              const void* dy_dev, int dy_dtype, float* dx_res_dev, float* d_norm_weight_dev,
                              float* const* grads_dev, int n_grads, void* stream_) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    if (!x_res_dev || !norm_weight_dev) return fail(PRICHS_ERR_BAD_ARG, "null activation or norm-weight pointer");
    if (x_dtype != PRICHS_DTYPE_F32 && x_dtype != PRICHS_DTYPE_BF16) return fail(PRICHS_ERR_BAD_ARG, "unknown element type");
    if ((reinterpret_cast<uintptr_t>(x_res_dev) & 15) || (reinterpret_cast<uintptr_t>(norm_weight_dev) & 15))
        return fail(PRICHS_ERR_BAD_ARG, "activation and weight pointers must be 16-byte aligned");
    if (h->d > 2048) return fail(PRICHS_ERR_BAD_SHAPE, "the block entry points support hidden_dim up to 2048");
    int T = 0;
    int rc = bwd_check(h, dy_dev, dy_dtype, dx_res_dev, grads_dev, n_grads, &T);
    if (rc != PRICHS_OK) return rc;
    if (!h->last_was_block) return fail(PRICHS_ERR_BAD_ARG, "the last forward was not prichs_moe_block_forward");
    DeviceGuard guard(h->device);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
    rc = bwd_alloc(h);
    if (rc != PRICHS_OK) return rc;
    prichs_moe::Bwd& b = h->bwd;
    // gradient of the normalised rows (the MoE layer's input) ...
    rc = backward_impl(h, h->last_a_shared, dy_dev, dy_dtype, b.dnorm, grads_dev, st);
    if (rc != PRICHS_OK) return rc;
    // ... through the pre-norm, seeded with the gradient that bypasses the sub-layer on the residual connection
    const int d = h->d, grid = (T + 7) / 8;
    const bool xf = x_dtype == PRICHS_DTYPE_F32, df = dy_dtype == PRICHS_DTYPE_F32;
    if (xf && df) bwd::rmsnorm_bwd_rows_kernel<true, true, 8><<<grid, 256, 0, st>>>(x_res_dev, b.dnorm, norm_weight_dev, dy_dev, eps, dx_res_dev, b.rinv, T, d);
    else if (xf) bwd::rmsnorm_bwd_rows_kernel<true, false, 8><<<grid, 256, 0, st>>>(x_res_dev, b.dnorm, norm_weight_dev, dy_dev, eps, dx_res_dev, b.rinv, T, d);
    else if (df) bwd::rmsnorm_bwd_rows_kernel<false, true, 8><<<grid, 256, 0, st>>>(x_res_dev, b.dnorm, norm_weight_dev, dy_dev, eps, dx_res_dev, b.rinv, T, d);
    else bwd::rmsnorm_bwd_rows_kernel<false, false, 8><<<grid, 256, 0, st>>>(x_res_dev, b.dnorm, norm_weight_dev, dy_dev, eps, dx_res_dev, b.rinv, T, d);
    LAUNCH_CHECK("pre-norm backward");
    if (d_norm_weight_dev) {
        if (xf) bwd::dgamma_partial_kernel<true><<<dim3(d / 256, bwd::DWR_SPLITS), 256, 0, st>>>(x_res_dev, b.dnorm, b.rinv, b.dgamma_part, T, d);
        else bwd::dgamma_partial_kernel<false><<<dim3(d / 256, bwd::DWR_SPLITS), 256, 0, st>>>(x_res_dev, b.dnorm, b.rinv, b.dgamma_part, T, d);
        LAUNCH_CHECK("norm weight gradient (partial sums)");
        bwd::dgamma_reduce_kernel<<<(d + 255) / 256, 256, 0, st>>>(b.dgamma_part, d_norm_weight_dev, d);
        LAUNCH_CHECK("norm weight gradient");
    }
    CUDA_TRY(cudaStreamSynchronize(st));
    return prichs_moe_sync_status(h);
}

namespace {

int backward_impl(prichs_moe* h, const bf16* a_shared, const void* dy_dev, int dy_dtype, float* dx_dev, float* const* grads_dev,
                  cudaStream_t st) {
    const int T = h->last_T;
    int rc = bwd_alloc(h);
    if (rc != PRICHS_OK) return rc;
    prichs_moe::Bwd& b = h->bwd;
    const int d = h->d, f = h->f, E = h->E;
    const long long tcap = h->Tcap;
    const size_t R = (size_t)h->Tcap + h->Rcap;

    // The forward's routing decides every size below: wait for it and read the placement.
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    if (st != h->last_stream) CUDA_TRY(cudaStreamSynchronize(st));
    route::RouteMeta meta;
    CUDA_TRY(cudaMemcpy(&meta, h->meta, sizeof(meta), cudaMemcpyDeviceToHost));
    if (meta.overflow) return fail(PRICHS_ERR_CAPACITY, "the forward pass overflowed its permuted region");

    // un-transposed weight copies ([f,d] and [d,2f] per slot, K-major for the input-gradient products)
    if (!b.nat_valid) {
        for (int s = 0; s < h->n_slots; ++s) {
            rc = bwd_transpose(h->w_dn + (size_t)s * d * h->K2, b.w_dn_nat + (size_t)s * f * d, d, f, h->K2, d, st, h->K2 / 64);
            if (rc != PRICHS_OK) return rc;
            rc = bwd_transpose(h->w_gu + (size_t)s * 2 * f * h->K1, b.w_gu_nat + (size_t)s * d * 2 * f, 2 * f, d, h->K1, 2 * f, st, h->K1 / 64);
            if (rc != PRICHS_OK) return rc;
        }
        b.nat_valid = true;
    }

    CUtensorMap tm_x;
    rc = make_tmap(&tm_x, a_shared, (size_t)T, (size_t)d, egemm::BM);
    if (rc != PRICHS_OK) return rc;

    // 1. d_out into the forward's row space (gate-weighted for routed rows) + the router's scalars
    if (dy_dtype == PRICHS_DTYPE_F32)
        bwd::dy_prepare_kernel<true><<<(T + 7) / 8, 256, 0, st>>>(dy_dev, reinterpret_cast<const bf16*>(h->ybuf), h->sel, h->gates, h->pos, b.dyall, b.scal, T, d, tcap);
    else
        bwd::dy_prepare_kernel<false><<<(T + 7) / 8, 256, 0, st>>>(dy_dev, reinterpret_cast<const bf16*>(h->ybuf), h->sel, h->gates, h->pos, b.dyall, b.scal, T, d, tcap);
    LAUNCH_CHECK("d_out preparation");

    egemm::Args base;
    memset(&base, 0, sizeof(base));
    base.shared_mtiles = (T + 127) / 128;
    base.routed_base_tiles = h->Tcap / 128;
    base.n_routed_mtiles = &h->meta->n_routed_mtiles;
    base.mtile_slot = h->mtile_slot;
    base.mtile_row = h->mtile_row;
    base.status = h->status;

    // 2. pre-activations: kept by a training forward; after a plain forward (which keeps only silu(gate) * up) they
    //    are computed again, [gate | up] = x . W_gu
    if (!h->gu_valid) {
        egemm::Args a = base;
        a.nk = d / egemm::BK;
        a.n_ntiles = 2 * f / egemm::BN;
        a.a_routed_tile_off = 0;
        a.w_rows = 2 * f;
        a.b_nkt = d / egemm::BK;  // the forward's weights are stored tile by tile
        rc = bwd_gemm(h, tm_x, h->tm_xp, h->tm_wgu, b.tm_gu_out, a, st, "pre-activation GEMM");
        if (rc != PRICHS_OK) return rc;
    }
    // 3. d_act = dY . W_down^T   (model.rs:580-588, 672-680)
    {
        egemm::Args a = base;
        a.nk = d / egemm::BK;
        a.n_ntiles = f / egemm::BN;
        a.a_routed_tile_off = h->Tcap / 128;
        a.w_rows = f;
        rc = bwd_gemm(h, b.tm_dyall, b.tm_dyall, b.tm_wdn_nat, b.tm_dh_out, a, st, "d_act GEMM");
        if (rc != PRICHS_OK) return rc;
    }
    // 4. SwiGLU backward
    bwd::swiglu_bwd_kernel<<<4 * h->sm_count, 256, 0, st>>>(b.dh, b.gu, b.dgu, T, f, tcap, &h->meta->n_routed_mtiles, h->mtile_row);
    LAUNCH_CHECK("SwiGLU backward");
    // 5. dX = d_gate . W_gate^T + d_up . W_up^T as one product over K = 2f   (model.rs:612-631, 702-722)
    {
        egemm::Args a = base;
        a.nk = 2 * f / egemm::BK;
        a.n_ntiles = d / egemm::BN;
        a.a_routed_tile_off = h->Tcap / 128;
        a.w_rows = d;
        rc = bwd_gemm(h, b.tm_dgu, b.tm_dgu, b.tm_wgu_nat, b.tm_dxall_out, a, st, "dX GEMM");
        if (rc != PRICHS_OK) return rc;
    }
    // 6. router VJP, 7. d_x
    bwd::router_vjp_kernel<<<(T + 255) / 256, 256, 0, st>>>(h->sel, h->gates, b.scal, b.dlog, T);
    LAUNCH_CHECK("router VJP");
    bwd::dx_combine_kernel<<<(T + 7) / 8, 256, 0, st>>>(b.dxall, h->sel, h->gates, h->pos, b.dlog, h->w_r8, dx_dev, T, d, tcap);
    LAUNCH_CHECK("d_x combine");
    if (!grads_dev) {
        CUDA_TRY(cudaStreamSynchronize(st));
        return prichs_moe_sync_status(h);
    }

    // 8. dW_router += X^T d_logits
    if (grads_dev[0]) {
        bwd::dwr_partial_kernel<<<dim3(d / 64, bwd::DWR_SPLITS), 512, 0, st>>>(a_shared, b.dlog, b.dwr_part, T, d);
        LAUNCH_CHECK("router weight gradient (partial sums)");
        bwd::dwr_reduce_kernel<<<(d * route::MAX_E + 255) / 256, 256, 0, st>>>(b.dwr_part, grads_dev[0], d, E);
        LAUNCH_CHECK("router weight gradient");
    }

    // 9. transposed copies: the weight-gradient products contract over rows. The shared expert's rows, then every
    //    expert's segment of the permuted region (its rows rounded up to whole tile pairs)
    rc = bwd_transpose(a_shared, b.xT, T, d, d, R, st);
    if (rc == PRICHS_OK) rc = bwd_transpose(h->hbuf, b.hT, T, f, h->K2, R, st);
    if (rc == PRICHS_OK) rc = bwd_transpose(b.dyall, b.dyT, T, d, d, R, st);
    if (rc == PRICHS_OK) rc = bwd_transpose(b.dgu, b.dguT, T, 2 * f, 2 * f, R, st);
    for (int e = 0; e < h->El && rc == PRICHS_OK; ++e) {
        const long long n = round_up(meta.counts[e], SEG_PAD), r0 = meta.seg_base[e], k0 = tcap + r0;
        if (n == 0) continue;
        rc = bwd_transpose(h->xp + (size_t)r0 * h->K1, b.xT + k0, n, d, h->K1, R, st);
        if (rc == PRICHS_OK) rc = bwd_transpose(h->hbuf + (size_t)k0 * h->K2, b.hT + k0, n, f, h->K2, R, st);
        if (rc == PRICHS_OK) rc = bwd_transpose(b.dyall + (size_t)k0 * d, b.dyT + k0, n, d, d, R, st);
        if (rc == PRICHS_OK) rc = bwd_transpose(b.dgu + (size_t)k0 * 2 * f, b.dguT + k0, n, 2 * f, 2 * f, R, st);
    }
    if (rc != PRICHS_OK) return rc;

    // 10. weight gradients, one expert at a time: its rows are the K window [k0, k0 + n) of the transposed copies
    //     (columns beyond n read as zero through the tensor map's bounds)
    for (int slot = 0; slot < h->n_slots; ++slot) {
        const int e = slot - 1;
        const long long k0 = slot == 0 ? 0 : tcap + meta.seg_base[e];
        const int n = slot == 0 ? T : meta.counts[e];
        float* gg = grads_dev[1 + 3 * slot];
        float* gu_ = grads_dev[2 + 3 * slot];
        float* gd = grads_dev[3 + 3 * slot];
        if (n <= 0 || (!gg && !gu_ && !gd)) continue;  // an expert without tokens gets no gradient (model.rs:641-643)
        egemm::Args a;
        memset(&a, 0, sizeof(a));
        a.nk = (n + egemm::BK - 1) / egemm::BK;
        a.n_routed_mtiles = h->ep_zero;
        a.mtile_slot = h->mtile_slot;
        a.out_f32 = 1;
        a.status = h->status;
        CUtensorMap tm_a, tm_b;
        if (gd) {
            // dW_down [f, d] = act^T . dY   (model.rs:572-579, 662-670)
            rc = make_tmap(&tm_a, b.hT + k0, f, (size_t)n, egemm::BM, false, R);
            if (rc == PRICHS_OK) rc = make_tmap(&tm_b, b.dyT + k0, d, (size_t)n, egemm::BN, false, R);
            if (rc != PRICHS_OK) return rc;
            a.shared_mtiles = f / egemm::BM;
            a.n_ntiles = d / egemm::BN;
            rc = bwd_gemm(h, tm_a, tm_a, tm_b, b.tm_stage_dn, a, st, "down-projection weight gradient");
            if (rc != PRICHS_OK) return rc;
            bwd::grad_accumulate_kernel<<<2 * h->sm_count, 256, 0, st>>>(b.stage_dn, gd, (size_t)f * d);
            LAUNCH_CHECK("down-projection gradient accumulation");
        }
        if (gg || gu_) {
            // dW_gate, dW_up [d, f] = x^T . d_gate, x^T . d_up as one product with N = 2f   (model.rs:600-611, 690-700)
            rc = make_tmap(&tm_a, b.xT + k0, d, (size_t)n, egemm::BM, false, R);
            if (rc == PRICHS_OK) rc = make_tmap(&tm_b, b.dguT + k0, 2 * f, (size_t)n, egemm::BN, false, R);
            if (rc != PRICHS_OK) return rc;
            a.shared_mtiles = d / egemm::BM;
            a.n_ntiles = 2 * f / egemm::BN;
            rc = bwd_gemm(h, tm_a, tm_a, tm_b, b.tm_stage_gu, a, st, "gate/up weight gradient");
            if (rc != PRICHS_OK) return rc;
            bwd::grad_unpack_gate_up_kernel<<<4 * h->sm_count, 256, 0, st>>>(b.stage_gu, gg, gu_, d, f);
            LAUNCH_CHECK("gate/up gradient accumulation");
        }
    }
    CUDA_TRY(cudaStreamSynchronize(st));
    h->last_stream = st;
    return prichs_moe_sync_status(h);
}

}  // namespace

int prichs_moe_debug_copy(prichs_moe_t* h, int which, size_t offset_bytes, void* host_dst, size_t bytes) {
    if (!h || !host_dst) return fail(PRICHS_ERR_BAD_ARG, "null handle or destination");
    DeviceGuard guard(h->device);
    const size_t rows_all = (size_t)h->Tcap + h->Rcap;
    const size_t ntiles = ((size_t)h->Tmax + route::TILE_TOKENS - 1) / route::TILE_TOKENS;
    const void* base = nullptr;
    size_t size = 0;
    switch (which) {
        case 0: base = h->xs; size = (size_t)h->Tmax * h->K1 * 2; break;
        case 1: base = h->xp; size = (size_t)h->Rcap * h->K1 * 2; break;
        case 2: base = h->hbuf; size = rows_all * h->K2 * 2; break;
        case 3: base = h->ybuf; size = rows_all * h->d * (h->mode == PRICHS_MODE_F32 ? 4 : 2); break;
        case 4: base = h->pos; size = (size_t)h->Tmax * 2 * 4; break;
        case 5: base = h->meta; size = sizeof(route::RouteMeta); break;
        case 6: base = h->tile_counts; size = ntiles * route::MAX_E * 4; break;
        case 7: base = h->tile_prefix; size = ntiles * route::MAX_E * 4; break;
        case 8: base = h->mtile_slot; size = ((size_t)h->Rcap / 128 + 1) * 4; break;
        // intermediates of the last backward pass (null until prichs_moe_backward has run)
        case 9: base = h->bwd.gu; size = rows_all * 2 * h->f * 2; break;
        case 10: base = h->bwd.dyall; size = rows_all * h->d * 2; break;
        case 11: base = h->bwd.dh; size = rows_all * h->f * 2; break;
        case 12: base = h->bwd.dgu; size = rows_all * 2 * h->f * 2; break;
        case 13: base = h->bwd.dxall; size = rows_all * h->d * 2; break;
        case 14: base = h->bwd.scal; size = (size_t)h->Tmax * 2 * 4; break;
        case 15: base = h->bwd.dlog; size = (size_t)h->Tmax * route::MAX_E * 4; break;
        case 16: base = h->mtile_row; size = ((size_t)h->Rcap / 128 + 1) * 4; break;
        default: return fail(PRICHS_ERR_BAD_ARG, "unknown buffer id %d", which);
    }
    if (!base) return fail(PRICHS_ERR_BAD_ARG, "buffer %d does not exist yet (no backward pass has run)", which);
    if (offset_bytes > size || bytes > size - offset_bytes) return fail(PRICHS_ERR_BAD_SHAPE, "range exceeds the buffer (%zu bytes)", size);
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    CUDA_TRY(cudaMemcpy(host_dst, static_cast<const char*>(base) + offset_bytes, bytes, cudaMemcpyDeviceToHost));
    return PRICHS_OK;
}

int prichs_moe_debug_set(prichs_moe_t* h, int key, long long value) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    switch (key) {
        case 0: h->rd_stall_tile = (int)value; return PRICHS_OK;
        case 1:
            if (value < 1000) return fail(PRICHS_ERR_BAD_ARG, "wait budget must be at least 1000 cycles");
            h->rd_wait_cycles = value;
            return PRICHS_OK;
        case 2: h->ep_skip_signal = (int)value; return PRICHS_OK;
        case 3: h->rd_poll_sleep_ns = (int)std::max<long long>(0, std::min<long long>(value, 10000)); return PRICHS_OK;
        default: return fail(PRICHS_ERR_BAD_ARG, "unknown debug key %d", key);
    }
}

int prichs_moe_enable_timing(prichs_moe_t* h, int on) {
    if (!h) return fail(PRICHS_ERR_BAD_ARG, "null handle");
    h->timing = on != 0;
    return PRICHS_OK;
}

int prichs_moe_get_ep_timeline(prichs_moe_t* h, float* ms, int n) {
    if (!h || !ms) return fail(PRICHS_ERR_BAD_ARG, "null handle or output");
    if (!h->tl_valid) return fail(PRICHS_ERR_BAD_ARG, "no expert-parallel timeline: enable timing before the forward");
    if (n < 2 + 8 * h->n_waves) return fail(PRICHS_ERR_BAD_SHAPE, "the timeline needs %d floats", 2 + 8 * h->n_waves);
    DeviceGuard guard(h->device);
    CUDA_TRY(cudaStreamSynchronize(h->last_stream));
    CUDA_TRY(cudaEventElapsedTime(&ms[0], h->tl_base, h->tl_side[0]));
    CUDA_TRY(cudaEventElapsedTime(&ms[1], h->tl_base, h->tl_side[1]));
    for (int w = 0; w < h->n_waves; ++w)
        for (int i = 0; i < 8; ++i) CUDA_TRY(cudaEventElapsedTime(&ms[2 + 8 * w + i], h->tl_base, h->wave[w].tl[i]));
    return PRICHS_OK;
}

int prichs_moe_get_stage_ms(prichs_moe_t* h, float* ms6) {
    if (!h || !ms6) return fail(PRICHS_ERR_BAD_ARG, "null handle or output");
    if (!h->ev_valid) return fail(PRICHS_ERR_BAD_ARG, "timing was not enabled for the last forward");
    DeviceGuard guard(h->device);
    CUDA_TRY(cudaEventSynchronize(h->ev[6]));
    for (int i = 0; i < 6; ++i) CUDA_TRY(cudaEventElapsedTime(&ms6[i], h->ev[i], h->ev[i + 1]));
    return PRICHS_OK;
}

void launch_moe_gather(const float* dev_in, const int* dev_token_indices, float* dev_out, size_t n_tokens, size_t hidden_dim, void* stream) {
    if (n_tokens * hidden_dim == 0) return;
    const size_t blocks = (n_tokens * 32 + 255) / 256;
    compat_gather_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dev_in, dev_token_indices, dev_out, n_tokens, hidden_dim);
    g_launches.fetch_add(1);
}

void launch_moe_scatter_add(const float* dev_exp_out, const int* dev_token_indices, const float* dev_weights, float* dev_accum_out,
                            size_t n_tokens, size_t hidden_dim, void* stream) {
    if (n_tokens * hidden_dim == 0) return;
    const size_t blocks = (n_tokens * 32 + 255) / 256;
    compat_scatter_add_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dev_exp_out, dev_token_indices, dev_weights,
                                                                                                   dev_accum_out, n_tokens, hidden_dim);
    g_launches.fetch_add(1);
}

void launch_swiglu_forward(const float* dev_gate, const float* dev_up, float* dev_out, size_t total_elements, void* stream) {
    if (total_elements == 0) return;
    size_t blocks = (total_elements + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    compat_swiglu_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dev_gate, dev_up, dev_out, total_elements);
    g_launches.fetch_add(1);
}

}  // extern "C"

// =====================================================================================================
// Routing without allocation (prichs_moe_route_static). Scratch lives in a file-scope device array; host
// code never uses the symbol as a pointer -- it asks the runtime for the device address once per device.
namespace {

constexpr size_t RS_MAX_T = PRICHS_ROUTE_STATIC_MAX_TOKENS;
constexpr size_t RS_MAX_D = PRICHS_ROUTE_STATIC_MAX_HIDDEN;
constexpr size_t RS_MAX_TILES = RS_MAX_T / route::TILE_TOKENS;
// byte offsets inside the scratch array (all multiples of 256)
constexpr size_t RS_OFF_WRT = 0;                                                   // [3][8][d] bf16
constexpr size_t RS_OFF_WR8 = RS_OFF_WRT + 3 * route::MAX_E * RS_MAX_D * 2;        // [d][8] fp32
constexpr size_t RS_OFF_BIAS0 = RS_OFF_WR8 + RS_MAX_D * route::MAX_E * 4;          // 8 zeros
constexpr size_t RS_OFF_LOGITS = RS_OFF_BIAS0 + 256;                               // [T][8] fp32
constexpr size_t RS_OFF_SEL = RS_OFF_LOGITS + RS_MAX_T * route::MAX_E * 4;         // [T][2] packed int32
constexpr size_t RS_OFF_GATES = RS_OFF_SEL + RS_MAX_T * 2 * 4;                     // [T][2] fp32
constexpr size_t RS_OFF_TCOUNT = RS_OFF_GATES + RS_MAX_T * 2 * 4;                  // [tiles][8] int32
constexpr size_t RS_OFF_TPREFIX = RS_OFF_TCOUNT + RS_MAX_TILES * route::MAX_E * 4; // [tiles][8] int32
constexpr size_t RS_OFF_META = RS_OFF_TPREFIX + RS_MAX_TILES * route::MAX_E * 4;   // RouteMeta
constexpr size_t RS_OFF_SLOTS = RS_OFF_META + 512;                                 // m-tile table
constexpr size_t RS_OFF_STATUS = RS_OFF_SLOTS + 2048;                              // status word
constexpr size_t RS_BYTES = 1u << 20;
static_assert(RS_OFF_STATUS + 256 <= RS_BYTES, "scratch layout exceeds the static array");
static_assert(sizeof(route::RouteMeta) <= 512, "RouteMeta outgrew its slot");
static_assert((RS_MAX_T * 2 + route::MAX_E * 128) / 128 + 1 <= 2048 / 4, "m-tile table outgrew its slot");

static __device__ __align__(256) unsigned char g_route_scratch[RS_BYTES];

// Unpacks the router's internal layouts into the caller's arrays.
__global__ void route_static_export_kernel(const float* __restrict__ logits8, const int* __restrict__ sel2,
                                           const float* __restrict__ gates2, const route::RouteMeta* __restrict__ meta,
                                           int T, int E, int top_k, float* __restrict__ logits, int32_t* __restrict__ selected,
                                           float* __restrict__ gating, int32_t* __restrict__ counts) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < E) counts[t] = meta->counts[t];
    if (t >= T) return;
    for (int e = 0; e < E; ++e) logits[(size_t)t * E + e] = logits8[(size_t)t * route::MAX_E + e];
    for (int j = 0; j < top_k; ++j) {
        selected[(size_t)t * top_k + j] = sel2[(size_t)t * 2 + j] & 0xff;
        gating[(size_t)t * top_k + j] = gates2[(size_t)t * 2 + j];
    }
}

// Device address of the scratch array on the current device, resolved once per device (std::call_once: two host
// threads that make the first call on a device at the same time both get the finished address).
int route_scratch_base(unsigned char** out) {
    constexpr int MAX_DEV = 64;
    static unsigned char* base[MAX_DEV] = {nullptr};
    static cudaError_t err[MAX_DEV];
    static std::once_flag once[MAX_DEV];
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEV) return fail(PRICHS_ERR_BAD_ARG, "device ordinal %d is out of range", dev);
    std::call_once(once[dev], [dev] {
        unsigned char* p = nullptr;
        err[dev] = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_route_scratch);
        base[dev] = p;
    });
    if (err[dev] != cudaSuccess || base[dev] == nullptr)
        return fail(PRICHS_ERR_CUDA, "cudaGetSymbolAddress of the routing scratch failed: %s", cudaGetErrorString(err[dev]));
    *out = base[dev];
    return PRICHS_OK;
}

}  // namespace

extern "C" int prichs_moe_route_static(const void* x_dev, const float* router_dev, const float* bias_dev, int T, int d,
                                       int E, int top_k, float* logits_dev, int32_t* selected_dev, float* gating_dev,
                                       int32_t* counts_dev, void* stream_) {
    if (!x_dev || !router_dev || !logits_dev || !selected_dev || !gating_dev || !counts_dev)
        return fail(PRICHS_ERR_BAD_ARG, "null device pointer");
    if (T < 1 || d < 256 || d % 256 != 0) return fail(PRICHS_ERR_BAD_SHAPE, "T must be positive and d a positive multiple of 256");
    if (E < 1 || E > route::MAX_E || top_k < 1 || top_k > 2 || top_k > E)
        return fail(PRICHS_ERR_BAD_SHAPE, "num_experts must be in 1..8 and top_k in 1..min(2, num_experts)");
    if ((size_t)T > RS_MAX_T || (size_t)d > RS_MAX_D)
        return fail(PRICHS_ERR_CAPACITY, "T=%d, d=%d exceed the static scratch limits (T <= %zu, d <= %zu)", T, d, RS_MAX_T, RS_MAX_D);
    if (reinterpret_cast<uintptr_t>(x_dev) & 15) return fail(PRICHS_ERR_BAD_ARG, "x must be 16-byte aligned");
    unsigned char* sc = nullptr;
    int rc = route_scratch_base(&sc);
    if (rc != PRICHS_OK) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);

    bf16* wrt = reinterpret_cast<bf16*>(sc + RS_OFF_WRT);
    float* wr8 = reinterpret_cast<float*>(sc + RS_OFF_WR8);
    float* bias0 = reinterpret_cast<float*>(sc + RS_OFF_BIAS0);
    float* logits8 = reinterpret_cast<float*>(sc + RS_OFF_LOGITS);
    int* sel2 = reinterpret_cast<int*>(sc + RS_OFF_SEL);
    float* gates2 = reinterpret_cast<float*>(sc + RS_OFF_GATES);
    int* tcount = reinterpret_cast<int*>(sc + RS_OFF_TCOUNT);
    int* tprefix = reinterpret_cast<int*>(sc + RS_OFF_TPREFIX);
    route::RouteMeta* meta = reinterpret_cast<route::RouteMeta*>(sc + RS_OFF_META);
    int* slots = reinterpret_cast<int*>(sc + RS_OFF_SLOTS);
    int* status = reinterpret_cast<int*>(sc + RS_OFF_STATUS);

    // the zero-bias block and the status word must start at zero; everything else is overwritten before use
    CUDA_TRY(cudaMemsetAsync(bias0, 0, 256, st));
    CUDA_TRY(cudaMemsetAsync(status, 0, 256, st));
    if (bias_dev) CUDA_TRY(cudaMemcpyAsync(bias0, bias_dev, (size_t)E * sizeof(float), cudaMemcpyDeviceToDevice, st));

    repack_router_kernel<<<64, 256, 0, st>>>(router_dev, wrt, wr8, d, E);
    LAUNCH_CHECK("router repack");
    route::ConceptBias cb;
    for (int e = 0; e < route::MAX_E; ++e) cb.v[e] = 0.0f;
    const int ntiles = (T + route::TILE_TOKENS - 1) / route::TILE_TOKENS;
    route::router_mma_kernel<3, false, false><<<ntiles, route::ROUTER_WARPS * 32, 0, st>>>(x_dev, nullptr, wrt, bias0, cb, T, d, E, top_k, logits8,
                                                                                         sel2, gates2, tcount, nullptr, 0.0f, route::ScanTail{});
    LAUNCH_CHECK("router");
    const int cap_rows = (int)((RS_MAX_T * 2 + route::MAX_E * 128) / 128 * 128);
    route::scan_kernel<<<1, 1024, 0, st>>>(tcount, tprefix, ntiles, meta, slots, nullptr, E, E, 1, 0, cap_rows, 1, 128, 0, status);
    LAUNCH_CHECK("scan");
    route_static_export_kernel<<<(T + 255) / 256, 256, 0, st>>>(logits8, sel2, gates2, meta, T, E, top_k, logits_dev, selected_dev,
                                                               gating_dev, counts_dev);
    LAUNCH_CHECK("export");
    return PRICHS_OK;
}

#include "engine_compat.cuh"
