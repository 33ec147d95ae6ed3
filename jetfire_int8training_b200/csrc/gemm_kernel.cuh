// The persistent per-block INT8 GEMM kernel (included by gemm.cu inside namespace jf, after the helpers it uses).
//
// Warp roles (19 warps): 16 consumer warps, 1 TMA producer warp, 2 MMA-issuing warps (one lane each).
//
// Hand-over of the accumulators.  Tensor memory holds two GROUPS of two 128-column accumulators.  The four K blocks of a
// shared-memory stage form two pairs; pair 0 goes to group 0 and is issued by issuer 0, pair 1 to group 1 / issuer 1, each pair
// is signalled with ONE tcgen05.commit.  Two issuers because the cost of issuing is the issuing thread's, not the tensor pipe's:
// measured on B200 with a single-CTA microbenchmark, a thread that loops over [tcgen05.mma ; tcgen05.commit] needs ~457 SM clocks
// per iteration whatever the MMA's N (16..256), ~110 more per additional MMA before the commit -- and two such threads in
// different warps run at that rate EACH.  The shared-memory stage is released by a consumer warp once it has seen the stage's
// last pair complete, which saves the issuers a third commit per stage.
//
// Consumers.  Warp w owns TMEM lanes 32*(w%4).. (rows) and columns 32*(w/4).. of every accumulator: a thread is one row of one
// 32x32 quantisation block (32 fp32 accumulators in registers).  Every consumer warp has to walk through every K block, so the
// length of one warp's chain per pair (barrier test, fences, two tcgen05.ld round trips, release, 2 x 48 arithmetic
// instructions under four-way issue contention) is what bounds the kernel, not the tensor core (64 clocks per K block), the
// issuers or the operand stream.
//
// Abort path.  Every wait is bounded; when one expires the CTA's roles leave their loops.  Before the CTA frees its tensor
// memory the producer waits (bounded) for the bulk copies it has in flight and each issuer commits its outstanding MMAs to a
// scratch barrier and waits (bounded) for it, so that nothing writes into shared or tensor memory of an exited CTA.
#pragma once

// Tile rasterisation: tiles are numbered in groups of RASTER_GM tile-rows, M-fastest inside a group, so the ~148 tiles that
// are in flight together cover about 16 x 9 tiles: 16 A panels + 9 B panels (~26 MB at K = 8192) instead of a whole
// 64-row-panel column of A, which did not stay in L2 (ncu: 1.12 GB of DRAM traffic per 8192^3 launch against 0.2 GB algorithmic).
constexpr int RASTER_GM = 16;
constexpr int EPI_WARPS = 16;                      // consumer warps
constexpr int NUM_ISSUERS = 2;                     // MMA-issuing warps = accumulator groups
constexpr int GEMM_THREADS = (EPI_WARPS + 1 + NUM_ISSUERS) * 32;
// (32-bit arithmetic: the launcher refuses problems with 2^31 tiles or more, and 64-bit divisions cost ~40 instructions each)
__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t& tm, int64_t& tn) {
    const uint32_t t = (uint32_t)tile, tmx = (uint32_t)tiles_m, tnx = (uint32_t)tiles_n;
    const uint32_t group_size = RASTER_GM * tnx;
    const uint32_t group = t / group_size, in_group = t % group_size;
    const uint32_t first_m = group * RASTER_GM;
    const uint32_t gm = min((uint32_t)RASTER_GM, tmx - first_m);
    tm = (int64_t)(first_m + in_group % gm);
    tn = (int64_t)(in_group / gm);
}

template <bool A_MN, bool B_MN, int CONV>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    constexpr int WARP_TMA = EPI_WARPS, WARP_MMA = EPI_WARPS + 1;   // issuers: WARP_MMA, WARP_MMA + 1
    constexpr bool INT32ACC = (CONV == CONV_INT32);
    // F16OPS: the operands are fp16 copies of the int8 payloads (exact) and the MMAs are kind::f16 with fp32 accumulation, so
    // the accumulator already holds float(I_p) (|I_p| < 2^20: every partial sum is an integer below 2^24, exact in fp32) and the
    // consumers skip the int32 -> fp32 conversion.  A K block is 64 bytes of K instead of 32: a stage holds two 128 x 128 B
    // boxes per operand (K blocks 0-1 and 2-3) and there are three stages; a K block is two K = 16 MMAs.
    constexpr bool F16OPS = (CONV == CONV_F16OPS);
    constexpr int NST = F16OPS ? 3 : STAGES;                            // pipeline stages
    constexpr int OPER_STAGE = F16OPS ? 2 * STAGE_BYTES : STAGE_BYTES;  // bytes of one operand per stage
    constexpr int NUM_GRP = NUM_ISSUERS, GRP_COLS = 2 * BN;   // two groups of two 128-column accumulators = all 512 TMEM columns
    static_assert(NUM_GRP * GRP_COLS == TMEM_COLS && KB_PER_STAGE == 2 * NUM_GRP, "a stage = one pair of K blocks per group");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + NST * OPER_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * NST * OPER_STAGE);
    uint64_t* full_bar = bars;                            // [STAGES]   TMA -> MMA
    uint64_t* empty_bar = bars + NST;                  // [STAGES]   consumers (int32 mode: MMA) -> TMA
    uint64_t* grp_full = bars + 2 * NST;               // [NUM_GRP]  MMA -> consumers
    uint64_t* grp_empty = bars + 2 * NST + NUM_GRP;    // [NUM_GRP]  consumers -> MMA
    uint64_t* drain_bar = bars + 2 * NST + 2 * NUM_GRP;  // [NUM_ISSUERS]  abort path only: outstanding MMAs of an issuer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NST + 2 * NUM_GRP + NUM_ISSUERS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) { ptx::mbar_init(&full_bar[s], 1); ptx::mbar_init(&empty_bar[s], 1); }
        for (int g = 0; g < NUM_GRP; ++g) { ptx::mbar_init(&grp_full[g], 1); ptx::mbar_init(&grp_empty[g], EPI_WARPS); }
        for (int g = 0; g < NUM_ISSUERS; ++g) ptx::mbar_init(&drain_bar[g], 1);
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
                    const uint32_t s = it % NST, ph = (it / NST) & 1u;
                    if (!(ok = bounded_wait<true>(&empty_bar[s], ph ^ 1u, abort_flag, 1))) break;
                    ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * OPER_STAGE);
                    const int32_t k_off = (int32_t)(kb * QB);
                    if (F16OPS) {
                        // K-major fp16 operands: two boxes of 64 elements of K each (the second one may lie past K: zero fill)
                        ptx::tma_load_2d(smem_a + s * OPER_STAGE, &map_a, &full_bar[s], k_off, (int32_t)(tm * BM));
                        ptx::tma_load_2d(smem_a + s * OPER_STAGE + STAGE_BYTES, &map_a, &full_bar[s], k_off + 64, (int32_t)(tm * BM));
                        ptx::tma_load_2d(smem_b + s * OPER_STAGE, &map_b, &full_bar[s], k_off, (int32_t)(tn * BN));
                        ptx::tma_load_2d(smem_b + s * OPER_STAGE + STAGE_BYTES, &map_b, &full_bar[s], k_off + 64, (int32_t)(tn * BN));
                        continue;
                    }
                    if (A_MN) ptx::tma_load_2d(smem_a + s * STAGE_BYTES, &map_a, &full_bar[s], (int32_t)(tm * BM), k_off);
                    else      ptx::tma_load_2d(smem_a + s * STAGE_BYTES, &map_a, &full_bar[s], k_off, (int32_t)(tm * BM));
                    if (B_MN) ptx::tma_load_2d(smem_b + s * STAGE_BYTES, &map_b, &full_bar[s], (int32_t)(tn * BN), k_off);
                    else      ptx::tma_load_2d(smem_b + s * STAGE_BYTES, &map_b, &full_bar[s], k_off, (int32_t)(tn * BN));
                }
            }
            if (*abort_flag) {
                // abort: the copies of the last (up to STAGES) armed stages may still be landing in this CTA's shared memory
                for (uint32_t j = it > NST ? it - NST : 0u; j < it; ++j) drain_wait(&full_bar[j % NST], (j / NST) & 1u);
            }
        }
    } else if (warp >= WARP_MMA) {
        // ------------------------------------------------------------------ MMA issuers
        const uint32_t w = (uint32_t)(warp - WARP_MMA);   // issuer index = accumulator group it owns
        if (lane == 0 && !(INT32ACC && w != 0)) {
            constexpr uint32_t idesc = ptx::make_idesc_i8(BM, BN, A_MN, B_MN);
            uint32_t it = 0, gi = 0;   // running stage counter / uses of the accumulator group (int32 mode: tile counter)
            bool ok = true;
            for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                const int64_t split = item / num_tiles;
                const int64_t kb0 = split * p.kb_per_split;
                const int64_t kb1 = min(p.nkb, kb0 + p.kb_per_split);
                for (int64_t kb = kb0; kb < kb1 && ok; kb += KB_PER_STAGE, ++it) {
                    const uint32_t s = it % NST, ph = (it / NST) & 1u;
                    const int nblk = (int)min((int64_t)KB_PER_STAGE, kb1 - kb);
                    if (!INT32ACC && nblk <= 2 * (int)w) continue;   // the stage holds no K block of this issuer's pair
                    if (!(ok = bounded_wait<true>(&full_bar[s], ph, abort_flag, 2))) break;
                    ptx::tc_fence_after();
                    // descriptors of K block 0 of the stage; K block j is 32 bytes further along a K-major row and 32 K-rows
                    // (4096 B) further in an MN-major tile, i.e. +2 / +256 in the descriptor's 16-byte address units
                    const uint64_t da0 = ptx::make_smem_desc_sw128(ptx::smem_u32(smem_a + s * OPER_STAGE), A_MN ? 128 * 128 : 16, 1024);
                    const uint64_t db0 = ptx::make_smem_desc_sw128(ptx::smem_u32(smem_b + s * OPER_STAGE), B_MN ? 128 * 128 : 16, 1024);
                    if (INT32ACC) {
                        // diagnostic mode: one issuer; the tensor core accumulates the whole K range of a tile in one accumulator
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
                        if (ok) ptx::umma_commit(&empty_bar[s]);   // no consumer sees the stages of this mode: the issuer frees them
                    } else {
                        if (!(ok = bounded_wait<true>(&grp_empty[w], (gi & 1u) ^ 1u, abort_flag, 3))) break;
                        ptx::tc_fence_after();
                        const int npair = min(2, nblk - 2 * (int)w);
                        for (int jj = 0; jj < npair; ++jj) {
                            const int j = 2 * (int)w + jj;
                            if (F16OPS) {
                                // issuer w's pair lives in box w of the stage; K block jj of the pair starts 64 B into the 128-byte
                                // swizzle row, its two K = 16 halves are 32 B apart (descriptor address units of 16 B)
                                constexpr uint32_t idesc16 = ptx::make_idesc_f16(BM, BN);
                                const uint64_t off = (uint64_t)(w * (STAGE_BYTES / 16) + jj * 4);
                                ptx::umma_f16(tmem_base + w * GRP_COLS + jj * BN, da0 + off, db0 + off, idesc16, 0u);
                                ptx::umma_f16(tmem_base + w * GRP_COLS + jj * BN, da0 + off + 2, db0 + off + 2, idesc16, 1u);
                                continue;
                            }
                            ptx::umma_i8(tmem_base + w * GRP_COLS + jj * BN, da0 + (uint64_t)(A_MN ? j * 256 : j * 2),
                                         db0 + (uint64_t)(B_MN ? j * 256 : j * 2), idesc, 0u);
                        }
                        ptx::umma_commit(&grp_full[w]);
                        ++gi;
                    }
                }
            }
            if (*abort_flag) {
                // abort: wait until every MMA this thread has issued has completed (they read shared and write tensor memory)
                ptx::umma_commit(&drain_bar[w]);
                drain_wait(&drain_bar[w], 0u);
            }
        }
    } else {
        // ------------------------------------------------------------------ consumers
        const int quad = warp & 3, cgrp = warp >> 2;   // TMEM lane quadrant (rows) / 32-column group of every accumulator
        uint32_t use0 = 0, use1 = 0, sit = 0;   // uses of group 0 / 1 (int32 mode: use0 counts tiles) / running stage counter
        bool ok = true;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + cgrp * 32;
        for (int64_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            int tm32, tn32, split32;
            {
                const uint32_t tile = (uint32_t)item % (uint32_t)num_tiles;
                int64_t tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                tm32 = (int)tm; tn32 = (int)tn; split32 = (int)((uint32_t)item / (uint32_t)num_tiles);
            }
            const int kb0 = (int)(split32 * p.kb_per_split);
            const int kb1 = (int)min(p.nkb, (int64_t)kb0 + p.kb_per_split);
            const int rowblk = tm32 * (BM / QB) + quad;
            const int colblk = tn32 * (BN / QB) + cgrp;
            const bool blk_ok = rowblk < (int)(p.M / QB) && colblk < (int)(p.N / QB);   // warp-uniform

            uint64_t acc2[16];   // the thread's 32 fp32 accumulators as packed pairs
#pragma unroll
            for (int j = 0; j < 16; ++j) acc2[j] = 0ull;
            auto accumulate = [&](const uint32_t (&raw)[32], float sc) { scale_accumulate<CONV>(acc2, raw, sc); };

            // lanes 0-7 hold the scale products sa*sb of 8 consecutive K blocks
            const __half* sa_ptr = p.sa + (int64_t)rowblk * p.sa_sm + (int64_t)(kb0 + (lane & 7)) * p.sa_sk;
            const __half* sb_ptr = p.sb + (int64_t)colblk * p.sb_sn + (int64_t)(kb0 + (lane & 7)) * p.sb_sk;
            // The two loads are volatile asm so that they are ISSUED here, eight K blocks before their values are needed (a plain
            // __ldg is sunk by the compiler to its first use, which exposed the load latency once per eight K blocks).
            auto fetch_scales = [&](int t8) -> float {   // t8 = first K block (relative to kb0) of the group of 8
                unsigned short ha = 0, hb = 0;
                if (lane < 8 && kb0 + t8 + (lane & 7) < kb1 && blk_ok) {
                    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(ha) : "l"(sa_ptr + (int64_t)t8 * p.sa_sk));
                    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(hb) : "l"(sb_ptr + (int64_t)t8 * p.sb_sk));
                }
                return __fmul_rn(__half2float(__ushort_as_half(ha)), __half2float(__ushort_as_half(hb)));
            };
            float sc_next = INT32ACC ? 0.f : fetch_scales(0);
            float sc_cur = 0.f;
            const int nloop = INT32ACC ? (kb1 > kb0 ? 1 : 0) : (kb1 - kb0);   // the int32 mode reads one accumulated tile
            const uint32_t g32 = use0 % NUM_GRP;                               // int32 mode: the tile's group

            // One pair of K blocks (group g; `two` = the pair has its second K block; `stage_end` = last pair of its shared-memory
            // stage).  Returns false when a wait expired.
            // Registers (96 per thread with 19 warps) hold 32 accumulators + ONE accumulator's 32 raw columns: the pair's first
            // K block is converted and accumulated before the second one is read, and only then can the group be released.
            // Reading both first and releasing at once would shorten the hand-over (measured without arithmetic: 1.26 ms
            // instead of 1.43 ms at 8192^3) but needs 64 raw registers, and the spills cost far more than that.
            auto do_pair = [&](const uint32_t g, const bool two, const float s0, const float s1, const bool stage_end) -> bool {
                const uint32_t acc = lane_base + g * GRP_COLS;
                {
                    const uint32_t uses = INT32ACC ? use0 / NUM_GRP : (g ? use1 : use0);
                    const bool got = bounded_wait(&grp_full[g], uses & 1u, abort_flag, 4);
                    if (!__all_sync(0xffffffffu, got)) return false;   // warp-uniform exit
                    if (g && !INT32ACC) ++use1; else ++use0;
                    ptx::tc_fence_after();
                }
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(acc, r);
                ptx::tmem_wait_ld_regs(r);
                if (two) {
                    accumulate(r, s0);
                    ptx::tmem_ld_32x32b_x32(acc + BN, r);
                    ptx::tmem_wait_ld_regs(r);
                }
                // the group's accumulators have left tensor memory: hand the group back to its issuer
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&grp_empty[g]);
                if (!INT32ACC && stage_end) {
                    // the last pair of a shared-memory stage has completed (the earlier pair was seen before): hand the stage
                    // back to the TMA producer
                    if (warp == 0 && lane == 0) ptx::mbar_arrive(&empty_bar[sit % NST]);
                    ++sit;
                }
                accumulate(r, two ? s1 : s0);
                return true;
            };

            int t = 0;
            if (!INT32ACC) {
                // fast path: eight K blocks (two stages, groups 0 1 0 1) per iteration with everything about the pair a constant
                for (; t + 8 <= nloop && ok; t += 8) {
                    sc_cur = sc_next;
                    sc_next = fetch_scales(t + 8);
#pragma unroll
                    for (int pp = 0; pp < 4; ++pp) {
                        if (!ok) break;
                        ok = do_pair((uint32_t)(pp & 1), true, __shfl_sync(0xffffffffu, sc_cur, 2 * pp),
                                     __shfl_sync(0xffffffffu, sc_cur, 2 * pp + 1), (pp & 1) == 1);
                    }
                }
            }
            for (; t < nloop && ok; t += 2) {
                // remaining pairs: pair t/2 of the tile lives in group (t/2)%2 (the int32 mode: one accumulator per tile)
                const uint32_t g = INT32ACC ? g32 : (uint32_t)((t >> 1) & 1);
                const int pi = (int)(t & 7);
                if (!INT32ACC && pi == 0) {
                    sc_cur = sc_next;
                    sc_next = fetch_scales(t + 8);
                }
                const float s0 = __shfl_sync(0xffffffffu, sc_cur, pi);
                const float s1 = __shfl_sync(0xffffffffu, sc_cur, pi + 1);
                ok = do_pair(g, t + 1 < nloop, s0, s1, g == 1 || t + 2 >= nloop);
            }
            if (!ok) break;

            // ---------------------------------------------------------------- tile epilogue
            if (!blk_ok) continue;
            float ab[32];
#pragma unroll
            for (int j = 0; j < 16; ++j) unpack2(acc2[j], ab[2 * j], ab[2 * j + 1]);
            store_block(p, ab, (int64_t)tm32 * BM + quad * 32 + lane, (int64_t)colblk * QB, rowblk, colblk, split32, lane);
        }
    }

    // ---------------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}
