// Grouped expert GEMM for sm_100a: one persistent, warp-specialised kernel serves the shared expert and
// all routed experts of a layer in a single launch (the reference runs one cuBLAS TF32 Sgemm per expert
// and per projection, crates/prichs-cuda/src/engine.rs:1957-2017,2112-2171, model.rs:1153-1174).
//
//   out[rows of m-tile, n-tile] = A[m-tile rows, :] . B_w[n-tile rows, :]^T        (bf16 in, fp32 accumulate)
//
// A is [rows, K] row-major (K-major), B is the stack of the experts' transposed weights [slot * w_rows + n, K]
// (also K-major), so both operands stream through TMA in 64-element (128-byte) K slices with the 128-byte
// swizzle and feed tcgen05.mma directly from shared memory. The 128 x 256 fp32 accumulator lives in tensor
// memory, double buffered (2 x 256 of the SM's 512 columns) so the epilogue of tile i overlaps the MMAs of
// tile i+1.
//
// Roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = TMEM owner + MMA issuer (one lane),
// warps 2..5 = epilogue (each owns the 32 TMEM lanes of quarter warp_idx % 4).
//
// Row space: m-tile i < shared_mtiles covers rows [128 i, 128 i + 128) of the un-permuted tokens (shared
// expert, weight slot 0); m-tile i >= shared_mtiles covers rows of the permuted buffer, where every
// expert's segment starts on a multiple of 128 rows, so a tile never straddles two experts; its weight slot
// is 1 + mtile_slot[i - shared_mtiles] (negative entries mark tiles made of padding rows only: skipped). Output rows: shared tiles at [128 i, ...), permuted tiles at
// 128 * (routed_base_tiles + j), a base that does not depend on T (peers of an expert-parallel group
// address each other's buffers with it).
//
// Epilogue data path: TMEM -> registers (tcgen05.ld, 32 columns at a time) -> a per-warp 32-row x 128-byte
// staging box in shared memory (128-byte swizzle, conflict-free 16-byte stores) -> TMA tiled store. Each warp
// owns two boxes and alternates, so the store of one box overlaps the conversion of the next; global memory
// sees full 128-byte row segments instead of 16-byte pieces.
//
// Epilogues:
//   EPI_SWIGLU  B rows of a tile are [128 gate columns | 128 up columns] of the same 128 hidden units, so one
//               thread owns matching g and u: h = silu(g) * u, written as bf16 (optionally as a bf16 hi/lo
//               pair in two column blocks for the fp32-fidelity mode).
//   EPI_PLAIN   accumulator written as bf16 or fp32.
//
// fp32-fidelity mode ("split3"): A and B each hold [hi | lo] bf16 halves side by side along K; the K loop
// runs three passes hi.hi + lo.hi + hi.lo over the same accumulator.
#pragma once

#include <cuda_bf16.h>

#include "ptx_sm100.cuh"

namespace egemm {

constexpr int BM = 128;
constexpr int BN = 256;  // default tile width (the kernels' template parameter of the same name shadows it)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int EPI_WARPS = 4;
constexpr int BOX_BYTES = 32 * 128;                      // one staging box: 32 rows x 128 bytes
constexpr int STAGING_BYTES = EPI_WARPS * 2 * BOX_BYTES;  // two boxes per epilogue warp
// dynamic shared memory: stages (1024-byte aligned) + staging boxes + barriers + TMEM base + abort flag
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 + 256;
// Every wait gives up after this many clock cycles (~2 s at 1.9 GHz) and the kernel reports a timeout.
constexpr long long WAIT_CYCLES = 4000000000LL;

enum { EPI_SWIGLU = 0, EPI_PLAIN = 1 };

struct Args {
    int nk;                    // 64-wide K blocks per pass (K / 64)
    int split3;                // 0: one pass; 1: three passes over [hi | lo] operands
    int n_ntiles;              // tiles along the output columns (B rows per weight / 256)
    int shared_mtiles;         // m-tiles of the shared expert (ceil(T / 128)); 0 when it is absent
    int routed_base_tiles;     // output row (in tiles) where the permuted region starts; fixed per handle
    int a_routed_tile_off;     // A row (in tiles) of permuted m-tile 0: 0 for the permuted-token buffer,
                               // routed_base_tiles when A is the previous GEMM's output
    const int* n_routed_mtiles;  // device scalar: m-tiles in the permuted region
    const int* mtile_slot;     // device: permuted m-tile -> routed weight slot (0-based)
    const int* mtile_row;      // device: permuted m-tile -> its 128-row tile index inside the permuted region; null when
                               // the region is dense (tile i sits at tile index i)
    int w_rows;                // B rows per weight slot
    int b_nkt;                 // 0: B is row-major [slot * w_rows + n, K]. > 0: B is stored tile by tile -- the 256 x 64
                               // block (n-tile, k-block) of a slot is one contiguous 32 KB box, b_nkt k-blocks per
                               // n-tile -- and its tensor map is the [all blocks x 256, 64] matrix of those boxes. A
                               // CTA then streams its weights from DRAM in 32 KB runs instead of 128-byte pieces
                               // 2 K bytes apart, which is what a small batch (weights read once) is bound by
    int out_split;             // SwiGLU only: also write the bf16 residual (lo) at column offset `out_lo_off`
    int out_lo_off;
    int out_f32;               // plain only: the output tensor map is fp32 (32-column boxes) instead of bf16
    int* status;               // device status word; set to -5 on a bounded-wait timeout
    __nv_bfloat16* stash_gu;   // SwiGLU only, training forward: when non-null the pre-activations are also written,
                               // as bf16 rows [., stash_ld] in the column order of B (128 gate | 128 up per block)
    int stash_ld;
};

// Training forward: the 32 gate and 32 up pre-activations one epilogue lane holds for its output row go to the stash
// as two 64-byte runs (full 32-byte sectors, so plain vector stores lose nothing against a staged TMA store).
__device__ __forceinline__ void stash_gate_up(__nv_bfloat16* row_ptr, const uint32_t (&g)[32], const uint32_t (&u)[32]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t pg[4], pu[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 a = __floats2bfloat162_rn(__uint_as_float(g[8 * j + 2 * i]), __uint_as_float(g[8 * j + 2 * i + 1]));
            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(u[8 * j + 2 * i]), __uint_as_float(u[8 * j + 2 * i + 1]));
            pg[i] = *reinterpret_cast<uint32_t*>(&a);
            pu[i] = *reinterpret_cast<uint32_t*>(&b);
        }
        reinterpret_cast<uint4*>(row_ptr)[j] = make_uint4(pg[0], pg[1], pg[2], pg[3]);
        reinterpret_cast<uint4*>(row_ptr + 128)[j] = make_uint4(pu[0], pu[1], pu[2], pu[3]);
    }
}

__device__ __forceinline__ float silu_mul(float g, float u) {
    // silu(g) * u with silu(g) = g / (1 + exp(-g))   (crates/prichs-core/src/ops.rs:137-140,142-159)
    return __fdividef(g, 1.0f + __expf(-g)) * u;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// BN: output columns of a tile. 256 everywhere but for the plain epilogue on small batches, where 128-column tiles
// (tiled B only: a tile then loads one 128-row half of a 256 x 64 weight block, a contiguous 16 KB run) double the number
// of tiles, so that a decode step's down projection (54 tiles of 256 columns for nine experts) spreads over the SMs.
template <int BN>
struct GemmShape {
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 + 256;
};

template <int EPI, int BN = 256>
__global__ void __launch_bounds__(NUM_THREADS, 1)
expert_gemm_kernel(const __grid_constant__ CUtensorMap tm_a_shared, const __grid_constant__ CUtensorMap tm_a_routed,
                   const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_out,
                   const Args args) {
    static_assert(BN == 256 || (BN == 128 && EPI == EPI_PLAIN), "128-column tiles exist for the plain epilogue only");
    constexpr int STAGES = GemmShape<BN>::STAGES;
    constexpr int STAGE_BYTES = GemmShape<BN>::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment is required by the 128-byte swizzle atoms.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = smem + STAGES * STAGE_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + STAGING_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full = empty_bar + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    ptx::grid_dep_launch();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_base_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    // set-up above touched no global memory; everything below may depend on the previous kernel of the stream
    ptx::grid_dep_wait();

    const int total_mtiles = args.shared_mtiles + *args.n_routed_mtiles;
    const int total_tiles = total_mtiles * args.n_ntiles;
    const int npass = args.split3 ? 3 : 1;
    const int k_elems = args.nk * BK;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            ptx::prefetch_tmap(&tm_a_shared);
            ptx::prefetch_tmap(&tm_a_routed);
            ptx::prefetch_tmap(&tm_b);
            int stage = 0;
            uint32_t phase = 0;
            long long issued = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int mt = tile / args.n_ntiles;
                const int nt = tile - mt * args.n_ntiles;
                const bool is_shared = mt < args.shared_mtiles;
                if (!is_shared && args.mtile_slot[mt - args.shared_mtiles] < 0) continue;  // padding-only tile
                const CUtensorMap* tm_a = is_shared ? &tm_a_shared : &tm_a_routed;
                const int rt = is_shared ? 0 : (args.mtile_row ? args.mtile_row[mt - args.shared_mtiles] : mt - args.shared_mtiles);
                const int a_row = (is_shared ? mt : args.a_routed_tile_off + rt) * BM;
                const int slot = is_shared ? 0 : 1 + args.mtile_slot[mt - args.shared_mtiles];
                const int b_row = slot * args.w_rows + nt * BN;
                // tiled B: first 256 x 64 block of this n-tile's K run, and the tile's row offset inside such a block
                const int b_blk0 = (slot * (args.w_rows / 256) + (nt * BN) / 256) * args.b_nkt;
                const int b_half = (nt * BN) % 256;
                for (int pass = 0; ok && pass < npass; ++pass) {
                    // pass 0: hi.hi, pass 1: lo.hi, pass 2: hi.lo
                    const int a_col0 = (pass == 1) ? k_elems : 0;
                    const int b_col0 = (pass == 2) ? k_elems : 0;
                    for (int kb = 0; kb < args.nk; ++kb) {
                        if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, WAIT_CYCLES)) {
                            ok = false;
                            break;
                        }
                        uint8_t* sa = smem + stage * STAGE_BYTES;
                        uint8_t* sb = sa + A_BYTES;
                        ptx::mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
                        ptx::tma_load_2d(sa, tm_a, a_col0 + kb * BK, a_row, &full_bar[stage]);
                        if (args.b_nkt > 0)
                            ptx::tma_load_2d(sb, &tm_b, 0, (b_blk0 + b_col0 / BK + kb) * 256 + b_half, &full_bar[stage]);
                        else
                            ptx::tma_load_2d(sb, &tm_b, b_col0 + kb * BK, b_row, &full_bar[stage]);
                        ++issued;
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
            if (!ok) {
                // Leaving early: let the copies already in flight land before the CTA's shared memory goes away.
                const long long first = issued > STAGES ? issued - STAGES : 0;
                for (long long i = first; i < issued; ++i) {
                    const int s = (int)(i % STAGES);
                    const uint32_t par = (uint32_t)((i / STAGES) & 1);
                    const long long t0 = clock64();
                    while (!ptx::mbar_try_wait(&full_bar[s], par) && clock64() - t0 < WAIT_CYCLES / 16) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const int iters = npass * args.nk;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int mt_ = tile / args.n_ntiles;
                if (mt_ >= args.shared_mtiles && args.mtile_slot[mt_ - args.shared_mtiles] < 0) continue;
                if (!ptx::mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1, abort_flag, WAIT_CYCLES)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int it = 0; it < iters; ++it) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag, WAIT_CYCLES)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t da = ptx::umma_desc_sw128(sa);
                    const uint64_t db = ptx::umma_desc_sw128(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advancing K by 16 elements = 32 bytes inside the swizzle atom: +2 in the address field
                        ptx::umma_bf16(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                       (uint32_t)((it | k) != 0));
                    }
                    ptx::umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                ptx::umma_commit(&tmem_full[acc]);  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps
        const int quarter = warp & 3;  // TMEM lanes [32 q, 32 q + 32) are the ones this warp may read
        uint8_t* box0 = staging + (warp - 2) * 2 * BOX_BYTES;
        uint8_t* my_row = box0 + lane * 128;      // this lane's row inside box 0 (box 1 is BOX_BYTES further)
        const int sw = lane & 7;                  // 128-byte swizzle: 16-byte chunk j of row r sits at j ^ (r & 7)
        if (lane == 0) ptx::prefetch_tmap(&tm_out);
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int mt = tile / args.n_ntiles;
            const int nt = tile - mt * args.n_ntiles;
            if (mt >= args.shared_mtiles && args.mtile_slot[mt - args.shared_mtiles] < 0) continue;
            // The vote keeps the warp converged for the .sync.aligned TMEM loads below.
            const bool ready = ptx::mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag, WAIT_CYCLES);
            if (!__all_sync(0xffffffffu, ready)) break;
            ptx::tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
            const int ut = mt < args.shared_mtiles
                               ? mt
                               : args.routed_base_tiles + (args.mtile_row ? args.mtile_row[mt - args.shared_mtiles] : mt - args.shared_mtiles);
            const int row0 = ut * BM + quarter * 32;  // first output row of this warp's boxes
            if constexpr (EPI == EPI_SWIGLU) {
#pragma unroll 1
                for (int c = 0; c < 128; c += 32) {
                    uint32_t g[32], u[32];
                    ptx::tmem_ld_32x32b_x32(taddr + c, g);
                    ptx::tmem_ld_32x32b_x32(taddr + 128 + c, u);
                    ptx::tmem_ld_wait();
                    if (c == 96) {
                        // all TMEM reads of this tile are done: hand the accumulator back to the MMA warp
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&tmem_empty[acc]);
                    }
                    if (args.stash_gu != nullptr)
                        stash_gate_up(args.stash_gu + (size_t)(row0 + lane) * args.stash_ld + nt * 256 + c, g, u);
                    const int sub = (c >> 5) & 1;                      // which half of the 64-column box
                    const int buf = args.out_split ? 0 : (c >> 6) & 1; // split mode: box 0 = hi, box 1 = lo
                    if (sub == 0) {
                        // the box is free once the store that last read it has fetched its data
                        if (lane == 0) {
                            if (args.out_split) ptx::bulk_wait_read<0>(); else ptx::bulk_wait_read<1>();
                        }
                        __syncwarp();
                    }
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float h0 = silu_mul(__uint_as_float(g[2 * j]), __uint_as_float(u[2 * j]));
                        const float h1 = silu_mul(__uint_as_float(g[2 * j + 1]), __uint_as_float(u[2 * j + 1]));
                        const __nv_bfloat162 hb = __floats2bfloat162_rn(h0, h1);
                        hi[j] = *reinterpret_cast<const uint32_t*>(&hb);
                        if (args.out_split) lo[j] = pack_bf16(h0 - __low2float(hb), h1 - __high2float(hb));
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int chunk = ((sub * 4 + j) ^ sw) << 4;
                        *reinterpret_cast<uint4*>(my_row + buf * BOX_BYTES + chunk) =
                            make_uint4(hi[4 * j], hi[4 * j + 1], hi[4 * j + 2], hi[4 * j + 3]);
                        if (args.out_split)
                            *reinterpret_cast<uint4*>(my_row + BOX_BYTES + chunk) =
                                make_uint4(lo[4 * j], lo[4 * j + 1], lo[4 * j + 2], lo[4 * j + 3]);
                    }
                    if (sub == 1) {
                        ptx::fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            const int col = nt * 128 + (c >> 6) * 64;
                            ptx::tma_store_2d(&tm_out, col, row0, box0 + buf * BOX_BYTES);
                            if (args.out_split) ptx::tma_store_2d(&tm_out, args.out_lo_off + col, row0, box0 + BOX_BYTES);
                            ptx::bulk_commit();
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(taddr + c, v);
                    ptx::tmem_ld_wait();
                    if (c == BN - 32) {
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&tmem_empty[acc]);
                    }
                    if (args.out_f32) {
                        // 32 fp32 columns fill one 128-byte box row
                        const int buf = (c >> 5) & 1;
                        if (lane == 0) ptx::bulk_wait_read<1>();
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *reinterpret_cast<uint4*>(my_row + buf * BOX_BYTES + ((j ^ sw) << 4)) =
                                make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        ptx::fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            ptx::tma_store_2d(&tm_out, nt * BN + c, row0, box0 + buf * BOX_BYTES);
                            ptx::bulk_commit();
                        }
                    } else {
                        const int sub = (c >> 5) & 1, buf = (c >> 6) & 1;
                        if (sub == 0) {
                            if (lane == 0) ptx::bulk_wait_read<1>();
                            __syncwarp();
                        }
                        uint32_t p[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            p[j] = pack_bf16(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<uint4*>(my_row + buf * BOX_BYTES + (((sub * 4 + j) ^ sw) << 4)) =
                                make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
                        if (sub == 1) {
                            ptx::fence_proxy_async();
                            __syncwarp();
                            if (lane == 0) {
                                ptx::tma_store_2d(&tm_out, nt * BN + (c >> 6) * 64, row0, box0 + buf * BOX_BYTES);
                                ptx::bulk_commit();
                            }
                        }
                    }
                }
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        // the stores read shared memory of this CTA and write global memory: both must be finished before exit
        if (lane == 0) ptx::bulk_wait_all();
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(args.status, -5);
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace egemm
