// The persistent per-block INT8 GEMM kernel (included by gemm.cu inside namespace jf, after the helpers it uses).
//
// CG = column groups of the consumer side: 4*CG consumer warps, each thread owns one row and 128/CG columns.
//
// Accumulators are handed over in GROUPS of two K blocks: the issuer waits for a free group, issues the two MMAs of the pair
// (one per 128-column accumulator) and signals the pair with ONE tcgen05.commit.  Measured on B200: with one commit per
// 128x128x32 MMA, the MMA -> commit -> mbarrier hand-over -- not the tensor core, the TMEM reads or TMA -- set a floor of about
// 600 SM clocks per K block (clock-stamped timeline: ~1600 clocks from the commit to the consumer seeing it with four
// accumulators in flight; the floor stayed when TMEM loads, arithmetic and even the TMA loads were removed).
#pragma once

// Tile rasterisation: tiles are numbered in groups of RASTER_GM tile-rows, M-fastest inside a group, so the ~148 tiles that
// are in flight together cover about 16 x 9 tiles: 16 A panels + 9 B panels (~26 MB at K = 8192) instead of a whole
// 64-row-panel column of A, which did not stay in L2 (ncu: 1.12 GB of DRAM traffic per 8192^3 launch against 0.2 GB algorithmic).
constexpr int RASTER_GM = 16;
__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t& tm, int64_t& tn) {
    const int64_t group_size = RASTER_GM * tiles_n;
    const int64_t group = tile / group_size, in_group = tile % group_size;
    const int64_t first_m = group * RASTER_GM;
    const int64_t gm = min((int64_t)RASTER_GM, tiles_m - first_m);
    tm = first_m + in_group % gm;
    tn = in_group / gm;
}

template <bool A_MN, bool B_MN, int CG, int CONV>
__global__ void __launch_bounds__((4 * CG + 2) * 32, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    constexpr int EPI_WARPS = 4 * CG;
    constexpr int WARP_TMA = EPI_WARPS, WARP_MMA = EPI_WARPS + 1;
    constexpr int NBLK = 4 / CG;          // 32-column blocks per thread (2 or 1)
    constexpr bool INT32ACC = (CONV == CONV_INT32);
    constexpr int NUM_GRP = 2, GRP_COLS = 2 * BN;   // two groups of two 128-column accumulators = all 512 TMEM columns
    static_assert(CG == 2 || CG == 4, "CG");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * STAGES * STAGE_BYTES);
    uint64_t* full_bar = bars;                            // [STAGES]   TMA -> MMA
    uint64_t* empty_bar = bars + STAGES;                  // [STAGES]   MMA -> TMA
    uint64_t* grp_full = bars + 2 * STAGES;               // [NUM_GRP]  MMA -> consumers
    uint64_t* grp_empty = bars + 2 * STAGES + NUM_GRP;    // [NUM_GRP]  consumers -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * NUM_GRP);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(&full_bar[s], 1); ptx::mbar_init(&empty_bar[s], 1); }
        for (int g = 0; g < NUM_GRP; ++g) { ptx::mbar_init(&grp_full[g], 1); ptx::mbar_init(&grp_empty[g], EPI_WARPS); }
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == WARP_MMA) {
        ptx::tmem_alloc(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    if (warp == WARP_TMA && lane == 0) {
        ptx::prefetch_tensormap(&map_a);
        ptx::prefetch_tensormap(&map_b);
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t num_tiles = p.tiles_m * p.tiles_n;
    const int64_t num_items = num_tiles * p.splits;

    if (warp == WARP_TMA) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t it = 0;   // running stage counter
            bool ok = true;
            for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                const int64_t tile = item % num_tiles, split = item / num_tiles;
                int64_t tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                const int64_t kb0 = split * p.kb_per_split;
                const int64_t kb1 = min(p.nkb, kb0 + p.kb_per_split);
                for (int64_t kb = kb0; kb < kb1; kb += KB_PER_STAGE, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!(ok = bounded_wait<true>(&empty_bar[s], ph ^ 1u, abort_flag, 1))) break;
                    ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
                    const int32_t k_off = (int32_t)(kb * QB);
                    if (A_MN) ptx::tma_load_2d(smem_a + s * STAGE_BYTES, &map_a, &full_bar[s], (int32_t)(tm * BM), k_off);
                    else      ptx::tma_load_2d(smem_a + s * STAGE_BYTES, &map_a, &full_bar[s], k_off, (int32_t)(tm * BM));
                    if (B_MN) ptx::tma_load_2d(smem_b + s * STAGE_BYTES, &map_b, &full_bar[s], (int32_t)(tn * BN), k_off);
                    else      ptx::tma_load_2d(smem_b + s * STAGE_BYTES, &map_b, &full_bar[s], k_off, (int32_t)(tn * BN));
                }
            }
        }
    } else if (warp == WARP_MMA) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_i8(BM, BN, A_MN, B_MN);
            uint32_t it = 0, gi = 0;   // running stage / accumulator-group counters
            bool ok = true;
            for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                const int64_t split = item / num_tiles;
                const int64_t kb0 = split * p.kb_per_split;
                const int64_t kb1 = min(p.nkb, kb0 + p.kb_per_split);
                for (int64_t kb = kb0; kb < kb1 && ok; kb += KB_PER_STAGE, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!(ok = bounded_wait<true>(&full_bar[s], ph, abort_flag, 2))) break;
                    ptx::tc_fence_after();
                    // descriptors of K block 0 of the stage; K block j is 32 bytes further along a K-major row and 32 K-rows
                    // (4096 B) further in an MN-major tile, i.e. +2 / +256 in the descriptor's 16-byte address units
                    const uint64_t da0 = ptx::make_smem_desc_sw128(ptx::smem_u32(smem_a + s * STAGE_BYTES), A_MN ? 128 * 128 : 16, 1024);
                    const uint64_t db0 = ptx::make_smem_desc_sw128(ptx::smem_u32(smem_b + s * STAGE_BYTES), B_MN ? 128 * 128 : 16, 1024);
                    const int nblk = (int)min((int64_t)KB_PER_STAGE, kb1 - kb);
                    if (INT32ACC) {
                        // diagnostic mode: the tensor core accumulates the whole K range in one accumulator of one group
                        const uint32_t g = gi % NUM_GRP;
                        for (int j = 0; j < nblk && ok; ++j) {
                            const bool first = (kb + j == kb0), last = (kb + j + 1 == kb1);
                            if (first) {
                                if (!(ok = bounded_wait<true>(&grp_empty[g], ((gi / NUM_GRP) & 1u) ^ 1u, abort_flag, 3))) break;
                                ptx::tc_fence_after();
                            }
                            ptx::umma_i8(tmem_base + g * GRP_COLS, da0 + (uint64_t)(A_MN ? j * 256 : j * 2),
                                         db0 + (uint64_t)(B_MN ? j * 256 : j * 2), idesc, first ? 0u : 1u);
                            if (last) { ptx::umma_commit(&grp_full[g]); ++gi; }
                        }
                    } else {
                        for (int j0 = 0; j0 < nblk && ok; j0 += 2, ++gi) {
                            const uint32_t g = gi % NUM_GRP;
                            if (!(ok = bounded_wait<true>(&grp_empty[g], ((gi / NUM_GRP) & 1u) ^ 1u, abort_flag, 3))) break;
                            ptx::tc_fence_after();
                            const int npair = min(2, nblk - j0);
                            for (int jj = 0; jj < npair; ++jj) {
                                const int j = j0 + jj;
                                ptx::umma_i8(tmem_base + g * GRP_COLS + jj * BN, da0 + (uint64_t)(A_MN ? j * 256 : j * 2),
                                             db0 + (uint64_t)(B_MN ? j * 256 : j * 2), idesc, 0u);
                            }
                            ptx::umma_commit(&grp_full[g]);
                        }
                    }
                    if (ok) ptx::umma_commit(&empty_bar[s]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ consumers
        const int quad = warp & 3, cgrp = warp >> 2;
        uint32_t gi = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            const int64_t tile = item % num_tiles, split = item / num_tiles;
            int64_t tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            const int64_t kb0 = split * p.kb_per_split;
            const int64_t kb1 = min(p.nkb, kb0 + p.kb_per_split);
            const int64_t rowblk = tm * (BM / QB) + quad;
            const int64_t colblk0 = tn * (BN / QB) + cgrp * NBLK;
            const bool row_ok = rowblk < p.M / QB;
            const bool col_ok0 = colblk0 < p.N / QB, col_ok1 = (NBLK > 1) && (colblk0 + 1 < p.N / QB);

            uint64_t acc2[NBLK][16];   // fp32 accumulators as packed pairs, one 32-column block per row of the array
#pragma unroll
            for (int b = 0; b < NBLK; ++b)
#pragma unroll
                for (int j = 0; j < 16; ++j) acc2[b][j] = 0ull;

            // lane-distributed scale fetch: lanes 0-7 hold sa for 8 consecutive K blocks, 8-15 sb of column block 0, 16-23 of block 1
            auto fetch_scales = [&](int64_t p0) -> float {
                const int which = lane >> 3;
                const int64_t pp = p0 + (lane & 7);
                float v = 0.f;
                if (pp < kb1) {
                    if (which == 0) { if (row_ok) v = __half2float(__ldg(p.sa + rowblk * p.sa_sm + pp * p.sa_sk)); }
                    else if (which == 1) { if (col_ok0) v = __half2float(__ldg(p.sb + colblk0 * p.sb_sn + pp * p.sb_sk)); }
                    else if (which == 2) { if (col_ok1) v = __half2float(__ldg(p.sb + (colblk0 + 1) * p.sb_sn + pp * p.sb_sk)); }
                }
                return v;
            };
            float sc_next = INT32ACC ? 0.f : fetch_scales(kb0);
            float sc_cur = 0.f;
            const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + cgrp * (32 * NBLK);
            const int64_t nloop = INT32ACC ? 1 : (kb1 - kb0);   // the int32 mode reads one accumulated tile

            // one accumulator (K block) of the current group: TMEM -> registers -> scale FMA
            auto consume = [&](uint32_t taddr, int64_t t, bool release_after, uint32_t g) {
                const int pi = (int)(t & 7);
                if (!INT32ACC && pi == 0) {
                    sc_cur = sc_next;
                    sc_next = fetch_scales(kb0 + t + 8);
                }
                const float sa_v = __shfl_sync(0xffffffffu, sc_cur, pi);
                const float s0 = __fmul_rn(sa_v, __shfl_sync(0xffffffffu, sc_cur, 8 + pi));
                const float s1 = (NBLK > 1) ? __fmul_rn(sa_v, __shfl_sync(0xffffffffu, sc_cur, 16 + pi)) : 0.f;
                uint32_t r0[32], r1[32];
                if (CONV == CONV_PROBE_NOLD) {   // timing probe: no TMEM read at all
#pragma unroll
                    for (int j = 0; j < 32; ++j) { r0[j] = (uint32_t)t; r1[j] = (uint32_t)t; }
                } else {
                    ptx::tmem_ld_32x32b_x32(taddr, r0);
                    if (NBLK > 1) ptx::tmem_ld_32x32b_x32(taddr + 32, r1);
                    ptx::tmem_wait_ld_regs(r0);
                    if (NBLK > 1) ptx::tmem_wait_ld_regs(r1);
                }
                if (release_after) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&grp_empty[g]);
                }
                scale_accumulate<CONV>(acc2[0], r0, s0);
                if (NBLK > 1) scale_accumulate<CONV>(acc2[NBLK - 1], r1, s1);
            };

            for (int64_t t = 0; t < nloop; t += 2, ++gi) {
                const uint32_t g = gi % NUM_GRP;
                if (!(ok = bounded_wait(&grp_full[g], (gi / NUM_GRP) & 1u, abort_flag, 4))) break;
                ptx::tc_fence_after();
                const bool two = (t + 1 < nloop);
                consume(lane_base + g * GRP_COLS, t, !two, g);
                if (two) consume(lane_base + g * GRP_COLS + BN, t + 1, true, g);
            }
            if (!ok) break;

            // ---------------------------------------------------------------- tile epilogue
            const int64_t row = tm * BM + quad * 32 + lane;
            if (!row_ok) continue;
#pragma unroll
            for (int b = 0; b < NBLK; ++b) {
                const bool col_ok = b == 0 ? col_ok0 : col_ok1;
                if (!col_ok) continue;   // warp-uniform
                float ab[32];
#pragma unroll
                for (int j = 0; j < 16; ++j) unpack2(acc2[b][j], ab[2 * j], ab[2 * j + 1]);
                store_block(p, ab, row, (colblk0 + b) * QB, rowblk, colblk0 + b, split, lane);
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}
