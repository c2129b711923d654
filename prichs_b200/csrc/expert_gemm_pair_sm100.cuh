// CTA-pair version of the grouped expert GEMM (see expert_gemm_sm100.cuh for the single-CTA kernel, whose
// tile table, row space, epilogues and Args it shares).
//
// Two CTAs of a cluster (two SMs of one TPC) work on one 256 x 256 output tile with tcgen05.mma.cta_group::2:
// CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and rows [128 r, 128 r + 128) of the B tile
// (half of the 256 output columns) into ITS OWN shared memory -- every TMA load is a plain per-CTA box load --
// and the tensor cores of both SMs read the two B halves from both shared memories. Per SM that is 32 KB of
// operands per 64-wide K block instead of 48 KB for the same MMA work, which lifts the L2 -> SM feed limit
// of the single-CTA kernel; the 128 x 256 fp32 accumulator of each CTA still lives double buffered in its own
// tensor memory, so epilogue and MMA overlap as before.
//
// Protocol (leader = CTA 0 of the pair):
//   full[s]    (leader)  one arrive.expect_tx of the leader's producer for the bytes of BOTH CTAs; each CTA's
//                        TMA loads complete_tx on it
//   empty[s]   (each)    the leader's MMA thread commits to both CTAs' barriers when the MMAs reading stage s
//                        have completed
//   tmem_full  (each)    committed by the leader for both CTAs when a tile's accumulator is complete
//   tmem_empty (leader)  8 arrivals: the four epilogue warps of both CTAs
// Every wait is bounded; a timeout is reported through Args::status and both CTAs still meet at the cluster
// barrier before tensor memory is released.
//
// Rows: every expert's segment of the permuted region is padded to 256 rows and the region of the un-permuted
// tokens is a multiple of 256 rows, so a 256-row tile never straddles two experts or two regions.
#pragma once

#include "expert_gemm_sm100.cuh"

namespace egemm {

constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_BYTES = 128 * BK * 2;                // this CTA's half of the B tile
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;  // 32 KB
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + STAGING_BYTES + 1024 + 256;

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
expert_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a_shared, const __grid_constant__ CUtensorMap tm_a_routed,
                        const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_out,
                        const Args args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = smem + PAIR_STAGES * PAIR_STAGE_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + STAGING_BYTES);
    uint64_t* empty_bar = full_bar + PAIR_STAGES;
    uint64_t* tmem_full = empty_bar + PAIR_STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    ptx::grid_dep_launch();
    const uint32_t cta_rank = ptx::cluster_ctarank();  // 0 = leader
    const bool leader = cta_rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 8);  // four epilogue warps of each CTA of the pair
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(tmem_base_slot, TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // the peer's barriers are initialised before anything signals them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    // set-up above touched no global memory; everything below may depend on the previous kernel of the stream
    ptx::grid_dep_wait();

    // tiles are enumerated in 256-row pairs: pair p covers 128-row tiles 2p and 2p+1 of the same kind
    const int shared_pairs = (args.shared_mtiles + 1) / 2;
    const int total_pairs = shared_pairs + *args.n_routed_mtiles / 2;
    const int total_tiles = total_pairs * args.n_ntiles;
    const int npass = args.split3 ? 3 : 1;
    const int k_elems = args.nk * BK;
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            ptx::prefetch_tmap(&tm_a_shared);
            ptx::prefetch_tmap(&tm_a_routed);
            ptx::prefetch_tmap(&tm_b);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; ok && tile < total_tiles; tile += n_clusters) {
                const int mp = tile / args.n_ntiles;
                const int nt = tile - mp * args.n_ntiles;
                const bool is_shared = mp < shared_pairs;
                const CUtensorMap* tm_a = is_shared ? &tm_a_shared : &tm_a_routed;
                const int rp = mp - shared_pairs;  // pair index inside the permuted region
                if (!is_shared && args.mtile_slot[2 * rp] < 0) continue;  // a pair of padding rows only
                const int rt = is_shared ? 0 : (args.mtile_row ? args.mtile_row[2 * rp] : 2 * rp);  // first tile of the pair
                const int a_row = (is_shared ? 2 * mp : args.a_routed_tile_off + rt) * BM + (int)cta_rank * BM;
                const int slot = is_shared ? 0 : 1 + args.mtile_slot[2 * rp];
                const int b_row = slot * args.w_rows + nt * BN + (int)cta_rank * 128;
                const int b_blk0 = (slot * (args.w_rows / BN) + nt) * args.b_nkt;  // first box of this n-tile (tiled B)
                for (int pass = 0; ok && pass < npass; ++pass) {
                    const int a_col0 = (pass == 1) ? k_elems : 0;
                    const int b_col0 = (pass == 2) ? k_elems : 0;
                    for (int kb = 0; kb < args.nk; ++kb) {
                        if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, WAIT_CYCLES)) {
                            ok = false;
                            break;
                        }
                        uint8_t* sa = smem + stage * PAIR_STAGE_BYTES;
                        uint8_t* sb = sa + A_BYTES;
                        const uint32_t full_leader = ptx::mapa_u32(ptx::smem_u32(&full_bar[stage]), 0);
                        if (leader) ptx::mbar_expect_tx(&full_bar[stage], 2 * PAIR_STAGE_BYTES);
                        ptx::tma_load_2d_pair(sa, tm_a, a_col0 + kb * BK, a_row, full_leader);
                        if (args.b_nkt > 0)  // this CTA's 128 rows of the contiguous 256 x 64 box
                            ptx::tma_load_2d_pair(sb, &tm_b, 0, (b_blk0 + b_col0 / BK + kb) * BN + (int)cta_rank * 128, full_leader);
                        else
                            ptx::tma_load_2d_pair(sb, &tm_b, b_col0 + kb * BK, b_row, full_leader);
                        if (++stage == PAIR_STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
            if (!ok) {
                // leaving early: give the copies already in flight time to land in this CTA's shared memory
                const long long t0 = clock64();
                while (clock64() - t0 < 4000000LL) {
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(2 * BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const int iters = npass * args.nk;
            for (int tile = cluster_id; ok && tile < total_tiles; tile += n_clusters) {
                const int mp_ = tile / args.n_ntiles;
                if (mp_ >= shared_pairs && args.mtile_slot[2 * (mp_ - shared_pairs)] < 0) continue;
                if (!ptx::mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1, abort_flag, WAIT_CYCLES)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int it = 0; it < iters; ++it) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag, WAIT_CYCLES)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + stage * PAIR_STAGE_BYTES);
                    const uint64_t da = ptx::umma_desc_sw128(sa);
                    const uint64_t db = ptx::umma_desc_sw128(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        ptx::umma_bf16_pair(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                            (uint32_t)((it | k) != 0));
                    }
                    // the stage is free in BOTH CTAs once these MMAs have read it
                    const uint32_t e_own = ptx::smem_u32(&empty_bar[stage]);
                    ptx::umma_commit_pair(ptx::mapa_u32(e_own, 0));
                    ptx::umma_commit_pair(ptx::mapa_u32(e_own, 1));
                    if (++stage == PAIR_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                const uint32_t f_own = ptx::smem_u32(&tmem_full[acc]);
                ptx::umma_commit_pair(ptx::mapa_u32(f_own, 0));
                ptx::umma_commit_pair(ptx::mapa_u32(f_own, 1));
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
        const uint32_t te_leader0 = ptx::mapa_u32(ptx::smem_u32(&tmem_empty[0]), 0);
        const uint32_t te_leader1 = ptx::mapa_u32(ptx::smem_u32(&tmem_empty[1]), 0);
        for (int tile = cluster_id; tile < total_tiles; tile += n_clusters) {
            const int mp = tile / args.n_ntiles;
            const int nt = tile - mp * args.n_ntiles;
            if (mp >= shared_pairs && args.mtile_slot[2 * (mp - shared_pairs)] < 0) continue;
            // The vote keeps the warp converged for the .sync.aligned TMEM loads below.
            const bool ready = ptx::mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag, WAIT_CYCLES);
            if (!__all_sync(0xffffffffu, ready)) break;
            ptx::tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
            // this CTA's 128-row half of the pair, as a tile index of the output row space
            const int rp_ = mp - shared_pairs;
            const int ut = (mp < shared_pairs ? 2 * mp : args.routed_base_tiles + (args.mtile_row ? args.mtile_row[2 * rp_] : 2 * rp_)) + (int)cta_rank;
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
                        if (lane == 0) ptx::mbar_arrive_cluster(acc ? te_leader1 : te_leader0);
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
                        if (lane == 0) ptx::mbar_arrive_cluster(acc ? te_leader1 : te_leader0);
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
    // Both CTAs are done with each other's shared memory and tensor memory only after this point.
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

}  // namespace egemm
