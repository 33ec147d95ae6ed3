// INT8-in / INT8-out nonlinear operators of the Jetfire data flow, written for sm_100a.
//
// All kernels are streaming kernels built on one work decomposition:
//   * a warp owns a tile of 32 rows x TW columns (TW = 32 or 64, i.e. one or two 32x32 quantisation blocks);
//   * a lane owns a 16-column chunk: with LPR = TW/16 lanes per row, lane = (rg, cc), rg = lane / LPR (row group),
//     cc = lane % LPR (chunk); in pass i (0 .. LPR-1) the lane touches row i*(32/LPR) + rg, columns [16*cc, 16*cc + 16):
//     one 16-byte access per int8 row chunk, every access of a warp covers whole 32/64-byte row segments, and all loads of a
//     tile are issued before the first use;
//   * a quantisation block is held by lanes {cc in {2b, 2b+1}} x all rg; its absmax is a thread-local max plus __shfl_xor
//     steps over lane bit 0 and the rg bits;
//   * the re-quantising division is an exact IEEE quotient computed with a shared correctly-rounded reciprocal (fast path
//     chosen once per warp), rounding is an add of 1.5*2^23, bytes are gathered with prmt;
//   * int8 -> fp32 avoids the conversion unit (prmt into the mantissa of 2^23, one subtract).
// Tile widths: 32 columns (at most 80 registers, three 8-warp CTAs per SM) for the kernels with arithmetic per element --
// quantize, GELU forward / backward, LayerNorm forward, the residual adds -- which is what keeps enough loads in flight;
// 64 columns for the pure data movers (dequantize, transpose, quantize with the transposed copy).  LayerNorm backward and the
// residual add with row statistics work on the reference's 128-column slab: two warps of 64 columns, resp. one warp walking
// four 32-column tiles.
#include <mutex>
#include <type_traits>

#include "jf_common.cuh"

namespace jf {

thread_local int g_last_cuda_error = 0;

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;

template <int TW>
struct Geo {
    static constexpr int LPR = TW / 16;      // lanes per tile row
    static constexpr int RPP = 32 / LPR;     // rows per pass
    static constexpr int NP = LPR;           // passes (NP * RPP = 32 rows)
};

struct Tile {
    int64_t tm, tn;   // tile coordinates
    int64_t row0;     // first row of the tile
    int64_t col;      // first column of this lane's 16-column chunk
    int rg, cc, lane;
    bool active;      // the chunk lies inside the tensor (N may end inside the tile)
};

template <int TW>
__device__ __forceinline__ Tile make_tile(int64_t tile, int64_t tiles_n, int64_t N) {
    Tile t;
    t.lane = threadIdx.x & 31;
    // 32-bit division: the entry points refuse tensors with 2^31 blocks or more, and a 64-bit division costs ~40 instructions,
    // which is noticeable when a lane handles only 32-64 elements per tile
    t.tm = (int64_t)((uint32_t)tile / (uint32_t)tiles_n);
    t.tn = (int64_t)((uint32_t)tile % (uint32_t)tiles_n);
    t.rg = t.lane / Geo<TW>::LPR;
    t.cc = t.lane % Geo<TW>::LPR;
    t.row0 = t.tm * QB;
    t.col = t.tn * TW + t.cc * 16;
    t.active = t.col < N;
    return t;
}

// Persistent loop of one warp over its tiles (tile index = blockIdx.x*WARPS + warp, stride gridDim.x*WARPS).  The loads of the
// NEXT tile are issued before the current tile is processed, so every warp keeps memory requests in flight while it computes.
//   load(const Tile&, Raw&)  : issue the global loads of a tile into registers
//   proc(const Tile&, Raw&)  : compute and store the tile
template <int TW, class Raw, bool PREFETCH, class LoadF, class ProcF>
__device__ __forceinline__ void for_each_tile(int64_t M, int64_t N, LoadF&& load, ProcF&& proc) {
    const int64_t tiles_n = (N + TW - 1) / TW, total = (M / QB) * tiles_n;
    const int64_t stride = (int64_t)gridDim.x * WARPS;
    int64_t tile = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (tile >= total) return;
    Tile t = make_tile<TW>(tile, tiles_n, N);
    Raw cur;
    load(t, cur);
    for (;;) {
        const int64_t next = tile + stride;
        const bool has_next = next < total;
        Tile tn = t;
        Raw nxt;
        if (has_next) {
            tn = make_tile<TW>(next, tiles_n, N);
            if (PREFETCH) load(tn, nxt);
        }
        proc(t, cur);
        if (!has_next) break;
        if (PREFETCH) cur = nxt;
        else load(tn, cur);
        t = tn;
        tile = next;
    }
}

template <int TW>
__device__ __forceinline__ int64_t row_of(const Tile& t, int i) { return t.row0 + i * Geo<TW>::RPP + t.rg; }

// number of CTAs: all tiles if they fit in `max_ctas`, else a persistent grid
template <int TW>
static inline unsigned grid_for(int64_t M, int64_t N, int max_ctas = 0) {
    const int64_t tiles = (M / QB) * ((N + TW - 1) / TW);
    const int64_t ctas = (tiles + WARPS - 1) / WARPS;
    return (unsigned)((max_ctas > 0 && ctas > max_ctas) ? max_ctas : ctas);
}

// max over the 32x32 block this lane belongs to (lane bit 0 = the two chunks of the block, then every rg bit)
template <int TW>
__device__ __forceinline__ float block_max(float m) {
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
#pragma unroll
    for (int mask = Geo<TW>::LPR; mask < 32; mask <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, mask));
    return m;
}
// sum over the lanes of one tile row (the cc bits)
template <int TW>
__device__ __forceinline__ float row_sum(float a) {
#pragma unroll
    for (int mask = 1; mask < Geo<TW>::LPR; mask <<= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, mask));
    return a;
}
// sum over the row groups (the rg bits): afterwards every lane holds the column sum over the tile's 32 rows
template <int TW>
__device__ __forceinline__ float col_sum(float a) {
#pragma unroll
    for (int mask = Geo<TW>::LPR; mask < 32; mask <<= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, mask));
    return a;
}

struct SrCfg {
    const float* noise;
    uint64_t offset;
    PhiloxKeys keys;
};
static inline SrCfg make_sr(const float* noise, uint64_t seed, uint64_t offset) { return SrCfg{noise, offset, make_philox_keys(seed)}; }

// low bytes of four registers -> one word
__device__ __forceinline__ uint32_t gather_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// 4x4 byte transpose: in w[k] = row k (4 column bytes); out o[j] = column j (4 row bytes).
__device__ __forceinline__ void transpose4x4(const uint32_t w[4], uint32_t o[4]) {
    const uint32_t t0 = __byte_perm(w[0], w[1], 0x5140), t1 = __byte_perm(w[2], w[3], 0x5140);
    const uint32_t t2 = __byte_perm(w[0], w[1], 0x7362), t3 = __byte_perm(w[2], w[3], 0x7362);
    o[0] = __byte_perm(t0, t1, 0x5410);
    o[1] = __byte_perm(t0, t1, 0x7632);
    o[2] = __byte_perm(t2, t3, 0x5410);
    o[3] = __byte_perm(t2, t3, 0x7632);
}

// Write the warp's 32 x TW int8 tile, staged in shared memory (row-major, TW bytes per row), transposed to qt[N, M].
// TW/4 column groups of 4 columns; lane l owns column group l % (TW/4) and the row range 32/(128/TW) * (l / (TW/4)):
//   TW = 128: 32 groups x 32 rows (two 16-byte stores per column); TW = 64: 16 groups x 16 rows (one 16-byte store per column).
template <int TW>
__device__ __forceinline__ void store_tile_transposed(const uint32_t* tile_words, const Tile& t, int64_t M, int64_t N, int8_t* qt) {
    constexpr int WPR = TW / 4;             // words per tile row = column groups
    constexpr int ROWS = 32 * WPR / 32;     // rows handled per lane (32 or 16)
    const int cg = t.lane % WPR, r0 = (t.lane / WPR) * ROWS;
    uint32_t colw[4][ROWS / 4];
#pragma unroll
    for (int g = 0; g < ROWS / 4; ++g) {
        uint32_t w[4], o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = tile_words[(r0 + 4 * g + k) * WPR + cg];
        transpose4x4(w, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) colw[j][g] = o[j];
    }
    const int64_t c0 = t.tn * TW + 4 * cg;
    if (c0 < N) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int4* dst = reinterpret_cast<int4*>(qt + (c0 + j) * M + t.row0 + r0);
#pragma unroll
            for (int h = 0; h < ROWS / 16; ++h) dst[h] = make_int4(colw[j][4 * h], colw[j][4 * h + 1], colw[j][4 * h + 2], colw[j][4 * h + 3]);
        }
    }
}

// Quantise the lane's NP x 16 values (row i delivered by rowf(i, a)) with the block scale `scale32` (= block absmax (+adj) / 127, identical in the lanes of a
// block) and store payload + scale.  TRUNC selects the truncating conversion of the residual-add kernels; SR the stochastic
// pre-step sign(v) * min(|v| + noise, 127) of the reference (its lower clamp at -128 can never bind).
template <int TW, bool TRUNC, bool SR, bool TRANSPOSE, class RowF>
__device__ __forceinline__ void emit_quantized(RowF&& rowf, float scale32, const Tile& t, int64_t M, int64_t N,
                                               int8_t* q, __half* s, const SrCfg& sr, uint32_t* tile_words, int8_t* qt) {
    constexpr int NP = Geo<TW>::NP;
    const Divisor d = make_divisor(scale32);
    const bool zero = (scale32 == 0.f);
    // One decision per warp: the Markstein path is exact only inside its exponent window.  The two paths are separate
    // instantiations of the loop (a run-time flag inside the element loop keeps both alive for every element).
    const bool fast = __all_sync(0xffffffffu, d.fast || zero);
    const uint64_t inv2 = f2_pack(d.inv, d.inv), negb2 = f2_pack(-d.b, -d.b), magic2 = f2_pack(12582912.0f, 12582912.0f);
    auto rows = [&](auto fast_c) {
    constexpr bool FAST = decltype(fast_c)::value;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        const int64_t row = row_of<TW>(t, i);
        uint32_t words[4] = {0u, 0u, 0u, 0u};
        if (t.active) {
            float av[16];
            rowf(i, av);
            float nz[16];
            if (SR) {
                if (sr.noise) {
                    const float4* np4 = reinterpret_cast<const float4*>(sr.noise + row * N + t.col);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float4 n4 = __ldg(np4 + k);
                        nz[4 * k] = n4.x; nz[4 * k + 1] = n4.y; nz[4 * k + 2] = n4.z; nz[4 * k + 3] = n4.w;
                    }
                } else {
                    philox_noise8((uint64_t)(row * N + t.col), sr.keys, sr.offset, &nz[0]);
                    philox_noise8((uint64_t)(row * N + t.col) + 8, sr.keys, sr.offset, &nz[8]);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t b[4];
#pragma unroll
                for (int j = 0; j < 4; j += 2) {
                    float x0, x1;
                    if (FAST) {
                        const uint64_t x2 = f2_div_fast(f2_pack(av[4 * k + j], av[4 * k + j + 1]), inv2, negb2);
                        if (!SR && !TRUNC) {
                            f2_unpack(f2_add(x2, magic2), x0, x1);
                            b[j] = __float_as_uint(x0); b[j + 1] = __float_as_uint(x1);
                            continue;
                        }
                        f2_unpack(x2, x0, x1);
                    } else {
                        x0 = __fdiv_rn(av[4 * k + j], d.b); x1 = __fdiv_rn(av[4 * k + j + 1], d.b);
                    }
                    if (SR) {
                        const float m0 = fminf(__fadd_rn(fabsf(x0), nz[4 * k + j]), 127.f), m1 = fminf(__fadd_rn(fabsf(x1), nz[4 * k + j + 1]), 127.f);
                        x0 = __uint_as_float(__float_as_uint(m0) ^ (__float_as_uint(x0) & 0x80000000u));
                        x1 = __uint_as_float(__float_as_uint(m1) ^ (__float_as_uint(x1) & 0x80000000u));
                    }
                    b[j] = TRUNC ? (uint32_t)__float2int_rz(x0) : __float_as_uint(__fadd_rn(x0, 12582912.0f));
                    b[j + 1] = TRUNC ? (uint32_t)__float2int_rz(x1) : __float_as_uint(__fadd_rn(x1, 12582912.0f));
                }
                words[k] = zero ? 0u : gather_bytes(b[0], b[1], b[2], b[3]);
            }
            *reinterpret_cast<int4*>(q + row * N + t.col) = make_int4(words[0], words[1], words[2], words[3]);
        }
        if (TRANSPOSE) {
            uint32_t* dst = tile_words + (i * Geo<TW>::RPP + t.rg) * (TW / 4) + t.cc * 4;
            *reinterpret_cast<int4*>(dst) = make_int4(words[0], words[1], words[2], words[3]);
        }
    }
    };
    if (fast) rows(std::true_type{}); else rows(std::false_type{});
    if (t.active && t.rg == 0 && (t.cc & 1) == 0) s[t.tm * (N / QB) + (t.col >> 5)] = __float2half_rn(scale32);
    if (TRANSPOSE) {
        __syncwarp();
        store_tile_transposed<TW>(tile_words, t, M, N, qt);
        __syncwarp();   // the tile buffer is reused by the warp's next tile
    }
}

template <int NP>
__device__ __forceinline__ float absmax_tile(const float (&v)[NP][16]) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < NP; ++i)
#pragma unroll
        for (int j = 0; j < 16; ++j) m = fmaxf(m, fabsf(v[i][j]));
    return m;
}

__device__ __forceinline__ float load_scale(const __half* s, const Tile& t, int64_t N) {
    return t.active ? __half2float(__ldg(s + t.tm * (N / QB) + (t.col >> 5))) : 0.f;
}
// the 16 payload values of one row chunk as exact fp32
__device__ __forceinline__ void unpack16(const int4& r, float (&f)[16]) {
    const uint32_t w[4] = {(uint32_t)r.x ^ 0x80808080u, (uint32_t)r.y ^ 0x80808080u, (uint32_t)r.z ^ 0x80808080u, (uint32_t)r.w ^ 0x80808080u};
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int j = 0; j < 4; ++j) f[4 * k + j] = byte_to_float(w[k], j);
}
// The 16 payload values of one row chunk as exact fp16 pairs, without a conversion instruction: a byte u = q ^ 0x80 placed under
// the high byte 0x64 is the half 1024 + u, and (1024 + u) - 1152 = q exactly (two values per prmt and per sub.f16x2).
__device__ __forceinline__ void unpack16_h2(const int4& r, __half2 (&h)[8]) {
    const uint32_t w[4] = {(uint32_t)r.x ^ 0x80808080u, (uint32_t)r.y ^ 0x80808080u, (uint32_t)r.z ^ 0x80808080u, (uint32_t)r.w ^ 0x80808080u};
    const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = __byte_perm(w[k], 0x64646464u, 0x5140), hi = __byte_perm(w[k], 0x64646464u, 0x5342);
        h[2 * k] = __hsub2_rn(*reinterpret_cast<const __half2*>(&lo), bias);
        h[2 * k + 1] = __hsub2_rn(*reinterpret_cast<const __half2*>(&hi), bias);
    }
}
// fp16-rounded dequantisation fp32(fp16(q) * s) of one row chunk (the reference's int8 * fp16 product), two values at a time
__device__ __forceinline__ void dequant16_h(const int4& r, __half2 s2, float (&f)[16]) {
    __half2 q2[8];
    unpack16_h2(r, q2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float2 p = __half22float2(__hmul2_rn(q2[j], s2));
        f[2 * j] = p.x; f[2 * j + 1] = p.y;
    }
}

__device__ __forceinline__ __half2 load_scale_h2(const __half* s, const Tile& t, int64_t N) {
    return t.active ? __half2half2(__ldg(s + t.tm * (N / QB) + (t.col >> 5))) : __half2half2(__float2half_rn(0.f));
}

// Raw (still packed) register images of a tile's inputs, as the loads deliver them.
template <int NP>
struct RawQ {          // one int8 tensor + its block scale
    int4 d[NP];
    __half sc;
};
template <int NP>
struct RawQ2 {         // two int8 tensors + their block scales
    int4 a[NP], b[NP];
    __half sa, sb;
};
template <typename T, int NP>
struct RawX {          // one tensor of T: 16 elements = sizeof(T) 16-byte words per row chunk
    uint4 d[NP][sizeof(T)];
};

template <int TW>
__device__ __forceinline__ void load_rows(const int8_t* q, const Tile& t, int64_t N, int4 (&raw)[Geo<TW>::NP]) {
#pragma unroll
    for (int i = 0; i < Geo<TW>::NP; ++i)
        raw[i] = t.active ? __ldg(reinterpret_cast<const int4*>(q + row_of<TW>(t, i) * N + t.col)) : make_int4(0, 0, 0, 0);
}
__device__ __forceinline__ __half load_scale16(const __half* s, const Tile& t, int64_t N) {
    return t.active ? __ldg(s + t.tm * (N / QB) + (t.col >> 5)) : __float2half_rn(0.f);
}
template <typename T, int TW>
__device__ __forceinline__ void load_x(const T* x, const Tile& t, int64_t N, RawX<T, Geo<TW>::NP>& r) {
#pragma unroll
    for (int i = 0; i < Geo<TW>::NP; ++i) {
        const uint4* p4 = reinterpret_cast<const uint4*>(x + row_of<TW>(t, i) * N + t.col);
#pragma unroll
        for (int k = 0; k < (int)sizeof(T); ++k) r.d[i][k] = t.active ? __ldg(p4 + k) : make_uint4(0, 0, 0, 0);
    }
}
// 16 values of T (held as sizeof(T) 16-byte words) -> fp32
__device__ __forceinline__ void widen16(const uint4 (&d)[4], float (&v)[16], float) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        v[4 * k] = __uint_as_float(d[k].x); v[4 * k + 1] = __uint_as_float(d[k].y);
        v[4 * k + 2] = __uint_as_float(d[k].z); v[4 * k + 3] = __uint_as_float(d[k].w);
    }
}
__device__ __forceinline__ void widen16(const uint4 (&d)[2], float (&v)[16], __half) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const uint32_t w[4] = {d[k].x, d[k].y, d[k].z, d[k].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            v[8 * k + 2 * j] = f.x; v[8 * k + 2 * j + 1] = f.y;
        }
    }
}
__device__ __forceinline__ void widen16(const uint4 (&d)[2], float (&v)[16], __nv_bfloat16) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const uint32_t w[4] = {d[k].x, d[k].y, d[k].z, d[k].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[8 * k + 2 * j] = __uint_as_float(w[j] << 16);
            v[8 * k + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    }
}

// =========================================================================================================
// quantize / quantize_transpose.  The tile stays packed in registers; it is widened once for the block absmax and once more
// for the quantisation, which is cheaper than holding 64 fp32 values next to the prefetched next tile.
// =========================================================================================================
template <typename T, int TW, bool SR, bool TRANSPOSE>
__global__ void __launch_bounds__(THREADS, TW == 32 ? 3 : 2)
quantize_kernel(const T* __restrict__ x, int64_t M, int64_t N, int8_t* __restrict__ q, __half* __restrict__ s,
                int8_t* __restrict__ qt, SrCfg sr) {
    constexpr int NP = Geo<TW>::NP;
    using Raw = RawX<T, NP>;
    __shared__ __align__(16) uint32_t smem_tiles[TRANSPOSE ? WARPS * 8 * TW : 1];
    uint32_t* tile_words = TRANSPOSE ? smem_tiles + (threadIdx.x >> 5) * 8 * TW : nullptr;
    // fp32 input: the packed tile is already 64 registers, prefetching a second one would spill
    for_each_tile<TW, Raw, sizeof(T) != 4>(
        M, N, [&](const Tile& t, Raw& r) { load_x<T, TW>(x, t, N, r); },
        [&](const Tile& t, Raw& r) {
            float m = 0.f;
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                float a[16];
                widen16(r.d[i], a, T());
#pragma unroll
                for (int j = 0; j < 16; ++j) m = fmaxf(m, fabsf(a[j]));
            }
            const float scale32 = __fdiv_rn(block_max<TW>(m), 127.0f);
            emit_quantized<TW, false, SR, TRANSPOSE>([&](int i, float (&a)[16]) { widen16(r.d[i], a, T()); }, scale32, t, M, N, q, s, sr,
                                                     tile_words, qt);
        });
}

// =========================================================================================================
// dequantize: y = fp32(fp16(q) * s).  Pure data movement with a 1 : 4 size ratio between input and output, so the lane mapping
// is chosen for the fp32 side: a thread owns one 4-byte word of payload (4 elements) per row and writes one float4; a CTA of 128
// threads covers 32 rows x 512 columns = one row of 16 quantisation blocks, so the scale is loaded once per thread and every
// warp access is a whole contiguous segment (128 B of payload, 512 B of output).  All 32 rows are in flight per thread.
// =========================================================================================================
constexpr int DQ_THREADS = 128;

__global__ void __launch_bounds__(DQ_THREADS)
dequantize_kernel(const int8_t* __restrict__ q, const __half* __restrict__ s, int64_t M, int64_t N, float* __restrict__ y) {
    const int64_t col = ((int64_t)blockIdx.x * DQ_THREADS + threadIdx.x) * 4;
    if (col >= N) return;
    const int64_t row0 = (int64_t)blockIdx.y * QB;
    const __half2 s2 = __half2half2(__ldg(s + blockIdx.y * (N / QB) + (col >> 5)));
    const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
    const int8_t* src = q + row0 * N + col;
    float* dst = y + row0 * N + col;
    // all 32 rows of the thread's column word are requested before the first one is used (128 bytes in flight per thread: a CTA
    // covers only 16 KB of payload, and small tensors put few CTAs on an SM)
    uint32_t w[QB];
#pragma unroll
    for (int r = 0; r < QB; ++r)       // (volatile asm: the compiler otherwise sinks each load to its use and keeps few in flight)
        asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(w[r]) : "l"(src + (int64_t)r * N));
#pragma unroll
    for (int r = 0; r < QB; ++r) {
        const uint32_t wx = w[r] ^ 0x80808080u;
        const uint32_t lo = __byte_perm(wx, 0x64646464u, 0x5140), hi = __byte_perm(wx, 0x64646464u, 0x5342);
        const float2 a = __half22float2(__hmul2_rn(__hsub2_rn(*reinterpret_cast<const __half2*>(&lo), bias), s2));
        const float2 b = __half22float2(__hmul2_rn(__hsub2_rn(*reinterpret_cast<const __half2*>(&hi), bias), s2));
        __stcs(reinterpret_cast<float4*>(dst + (int64_t)r * N), make_float4(a.x, a.y, b.x, b.y));   // written once, read by a later kernel
    }
}

// =========================================================================================================
// transpose: y[N, M] = x[M, N]^T (int8).  A CTA moves a 128 x 128 tile through 16 KB of shared memory so that BOTH sides of
// the copy are whole 128-byte lines: rows of x are loaded as 16-byte chunks (8 threads per row), the 16-byte chunks of a row are
// permuted in shared memory by an XOR with the row's 16-row group, which makes the column reads below bank-conflict free; then a
// thread gathers a 16-row x 4-column patch (16 words), transposes it with byte permutes (4x4 at a time) and writes 16 bytes of
// each of 4 output rows -- 8 neighbouring threads complete one 128-byte line of y.
// =========================================================================================================
constexpr int TR_TILE = 128;

__global__ void __launch_bounds__(THREADS)
transpose_kernel(const int8_t* __restrict__ x, int64_t M, int64_t N, int8_t* __restrict__ y) {
    __shared__ __align__(16) uint32_t tile[TR_TILE * TR_TILE / 4];
    const int64_t R0 = (int64_t)blockIdx.y * TR_TILE, C0 = (int64_t)blockIdx.x * TR_TILE;
    const int t = threadIdx.x;
    {
        const int chunk = t & 7;
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int row = (t >> 3) + 32 * pass;
            int4 v = make_int4(0, 0, 0, 0);
            if (R0 + row < M && C0 + 16 * chunk < N) v = __ldg(reinterpret_cast<const int4*>(x + (R0 + row) * N + C0 + 16 * chunk));
            *reinterpret_cast<int4*>(tile + row * 32 + 4 * (chunk ^ ((row >> 4) & 7))) = v;
        }
    }
    __syncthreads();
    const int warp = t >> 5, lane = t & 31;
    const int i = lane & 7;                     // 16-row group of the tile: rows 16i .. 16i+15
    const int cg = 4 * warp + (lane >> 3);      // column group: tile columns 4cg .. 4cg+3
    if (R0 + 16 * i >= M || C0 + 4 * cg >= N) return;
    uint32_t colw[4][4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint32_t w[4], o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int row = 16 * i + 4 * g + k;
            w[k] = tile[row * 32 + 4 * ((cg >> 2) ^ i) + (cg & 3)];      // (row >> 4) & 7 == i
        }
        transpose4x4(w, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) colw[j][g] = o[j];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
        *reinterpret_cast<int4*>(y + (C0 + 4 * cg + j) * M + R0 + 16 * i) = make_int4(colw[j][0], colw[j][1], colw[j][2], colw[j][3]);
}

// =========================================================================================================
// GELU.  Both kernels go through per-block lookup tables: inside one 32x32 quantisation block the input is q * s with a single
// scale s, so it takes at most 256 different values, and so does any function of it.  The transcendental functions are
// evaluated CORRECTLY ROUNDED (in fp64, rounded once to fp32), which is what makes the payloads bit-identical to the CPU
// restatement of the reference on every input; the tables make that affordable (at most 256 evaluations per 1024 elements).
// =========================================================================================================
constexpr float SQRT2_F = 1.41421353816986083984375f;      // sqrt(2) rounded to fp32 (the reference divides by this value)
constexpr float SQRT2PI_F = 2.50662827491760253906250f;    // fp32 sqrt of fp32(2*pi)

// Forward table.  y(x) = x * Phi(x) is needed at x = fp16(q * s) for the 256 payloads q of a block with scale s, i.e. at
// +-x for x = fp16(a * s), a = 1..128, and each of the 32768 non-negative fp16 bit patterns of s.  The device table holds, per
// (s, a), the pair ( y(+x), y(-x) ) with the reference's fp32 roundings and a correctly rounded erf (fp64, rounded once):
//      er = RN(erf(RN(x / sqrt2)));   y(+x) = RN(RN(RN(1 + er) / 2) * x),   y(-x) = RN(RN(RN(1 - er) / 2) * -x).
// 32 MB, filled once per device by one kernel; a block reads its row of 1 KB (lane l the pairs a = 4l+1 .. 4l+4).
constexpr uint32_t GELU_ROWS = 32768u;
__device__ float2 g_gelu_fwd_table[GELU_ROWS * 128u];

__global__ void gelu_fwd_table_kernel() {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= GELU_ROWS * 128u) return;
    const __half x16 = __hmul_rn(__int2half_rn((int)(i & 127u) + 1), __ushort_as_half((unsigned short)(i >> 7)));   // the reference's fp16 product
    const float x = __half2float(x16);
    const float er = (float)erf((double)__fdiv_rn(x, SQRT2_F));          // erf is odd: RN(erf(-u)) = -RN(erf(u))
    g_gelu_fwd_table[i] = make_float2(__fmul_rn(__fmul_rn(__fadd_rn(1.0f, er), 0.5f), x),
                                      __fmul_rn(__fmul_rn(__fsub_rn(1.0f, er), 0.5f), -x));
}

// address of entry `byte k of w` of a 256-byte table that starts at the 256-byte-aligned shared address `base`
template <int K>
__device__ __forceinline__ uint32_t byte_entry_addr(uint32_t w, uint32_t base) {
    return __byte_perm(w, base, 0x7650 + K);
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// the four table bytes selected by the four payload bytes of w
__device__ __forceinline__ uint32_t translate4(uint32_t w, uint32_t base) {
    const uint32_t b0 = lds_u8(byte_entry_addr<0>(w, base)), b1 = lds_u8(byte_entry_addr<1>(w, base));
    const uint32_t b2 = lds_u8(byte_entry_addr<2>(w, base)), b3 = lds_u8(byte_entry_addr<3>(w, base));
    return gather_bytes(b0, b1, b2, b3);
}
// the 16 fp32 table values of one row chunk (payload bytes in r) from a 256-entry fp32 table
__device__ __forceinline__ void lookup16(const float* lut_b, const int4& r, float (&f)[16]) {
    const uint32_t w[4] = {(uint32_t)r.x, (uint32_t)r.y, (uint32_t)r.z, (uint32_t)r.w};
    const char* base = reinterpret_cast<const char*>(lut_b);
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t off = (j == 0) ? ((w[k] << 2) & 0x3FCu) : ((w[k] >> (8 * j - 2)) & 0x3FCu);
            f[4 * k + j] = *reinterpret_cast<const float*>(base + off);
        }
}

// A lane's share of a table row: the pairs a = 4l+1, 4l+2 | 4l+3, 4l+4 of the row selected by the block scale (a negative or NaN
// scale, never produced by a quantiser, indexes by its magnitude bits).
struct TableRow {
    float4 p01, p23;
};
__device__ __forceinline__ TableRow load_table_row(const float2* table, __half sc, int lane) {
    const float4* row = reinterpret_cast<const float4*>(table + ((uint32_t)(__half_as_ushort(sc) & 0x7FFFu) << 7)) + 2 * lane;
    TableRow r;
    r.p01 = __ldg(row); r.p23 = __ldg(row + 1);
    return r;
}

// forward: x = fp16(q*s); y = x * Phi(x); block quantise with amax + 5e-5.
// Per 32x32 block (= one warp tile) the kernel builds the table "input payload -> OUTPUT payload" (256 bytes) from the block's
// row of the device table and translates every element through it:
//   (1) block absmax: y is non-decreasing for x > 0 and |y| < 0.17 for x < 0, so when y(largest positive payload) >= 0.17 that
//       value IS the absmax -- one SIMD byte max per four elements, no per-element arithmetic;
//   (2) table entries: lane l divides its eight exact y values (a = 4l+1 .. 4l+4, both signs) by the block scale -- the exact
//       quotient is the Markstein sequence with the correctly rounded reciprocal, valid because scale32 >= 0.17/127;
//   (3) a block of small inputs (absmax below 0.17, rare) finds its absmax over the elements and divides with div.rn.
__global__ void __launch_bounds__(THREADS, 3)
gelu_fwd_kernel(const int8_t* __restrict__ qx, const __half* __restrict__ sx, int64_t M, int64_t N, int8_t* __restrict__ qy,
                __half* __restrict__ sy) {
    constexpr int TW = 32, NP = Geo<TW>::NP;
    using Raw = RawQ<NP>;
    __shared__ __align__(16) float ytab_all[WARPS][256];          // path (3) only
    __shared__ __align__(256) uint8_t btab_all[WARPS][256];
    const int warp = threadIdx.x >> 5;
    float* ytab = ytab_all[warp];
    uint8_t* btab_g = btab_all[warp];
    const uint32_t btab = (uint32_t)__cvta_generic_to_shared(btab_g);
    for_each_tile<TW, Raw, true>(
        M, N,
        [&](const Tile& t, Raw& r) {
            load_rows<TW>(qx, t, N, r.d);
            r.sc = load_scale16(sx, t, N);
        },
        [&](const Tile& t, Raw& r) {
            const int lane = t.lane;
            const TableRow tr = load_table_row(g_gelu_fwd_table, r.sc, lane);
            const float4 p01 = tr.p01, p23 = tr.p23;
            const float yp[4] = {p01.x, p01.z, p23.x, p23.z}, yn[4] = {p01.y, p01.w, p23.y, p23.w};   // y(+a s), y(-a s), a = 4l+1 ..
            // largest payload of the block
            uint32_t m4 = 0x80808080u;   // four int8 -128
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                m4 = __vmaxs4(m4, (uint32_t)r.d[i].x); m4 = __vmaxs4(m4, (uint32_t)r.d[i].y);
                m4 = __vmaxs4(m4, (uint32_t)r.d[i].z); m4 = __vmaxs4(m4, (uint32_t)r.d[i].w);
            }
            m4 = __vmaxs4(m4, m4 >> 16);
            m4 = __vmaxs4(m4, m4 >> 8);
            const int qmax = __reduce_max_sync(0xffffffffu, (int)(int8_t)(m4 & 0xFFu));
            const int im = (qmax > 0 ? qmax : 1) - 1, cm = im & 3;
            const float ym = __shfl_sync(0xffffffffu, cm == 0 ? yp[0] : cm == 1 ? yp[1] : cm == 2 ? yp[2] : yp[3], im >> 2);
            float amax = qmax > 0 ? ym : 0.f;
            const bool fast_tile = amax >= 0.17f;     // warp-uniform
            __syncwarp();                             // the previous tile's translation is done
            if (!fast_tile) {
                // (3) absmax over the elements, through the fp32 table of the block
                const int a = 4 * lane + 1;
                ytab[a] = yp[0]; ytab[a + 1] = yp[1]; ytab[a + 2] = yp[2];
                if (a + 3 < 128) ytab[a + 3] = yp[3];                  // +128 is not a payload: that byte is -128's
                ytab[256 - a] = yn[0]; ytab[255 - a] = yn[1]; ytab[254 - a] = yn[2]; ytab[253 - a] = yn[3];
                if (lane == 0) ytab[0] = 0.f;
                __syncwarp();
                float m = 0.f;
#pragma unroll
                for (int i = 0; i < NP; ++i) {
                    float f[16];
                    lookup16(ytab, r.d[i], f);
#pragma unroll
                    for (int j = 0; j < 16; ++j) m = fmaxf(m, fabsf(f[j]));
                }
                amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m)));
            }
            const float scale32 = __fdiv_rn(__fadd_rn(amax, 5e-5f), 127.0f);
            uint32_t bp[4], bn[4];
            if (fast_tile) {
                const float inv = __frcp_rn(scale32);
                const uint64_t inv2 = f2_pack(inv, inv), negb2 = f2_pack(-scale32, -scale32), magic2 = f2_pack(12582912.0f, 12582912.0f);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float rp, rn;
                    f2_unpack(f2_add(f2_div_fast(f2_pack(yp[j], yn[j]), inv2, negb2), magic2), rp, rn);
                    bp[j] = __float_as_uint(rp); bn[j] = __float_as_uint(rn);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    bp[j] = __float_as_uint(__fadd_rn(__fdiv_rn(yp[j], scale32), 12582912.0f));
                    bn[j] = __float_as_uint(__fadd_rn(__fdiv_rn(yn[j], scale32), 12582912.0f));
                }
            }
            // entries 4l+1 .. 4l+4 (the last lane's +128 does not exist: that byte is -128's) and 252-4l .. 255-4l
            if (lane < 31) {
                btab_g[4 * lane + 1] = (uint8_t)bp[0]; btab_g[4 * lane + 2] = (uint8_t)bp[1];
                btab_g[4 * lane + 3] = (uint8_t)bp[2]; btab_g[4 * lane + 4] = (uint8_t)bp[3];
            } else {
                btab_g[125] = (uint8_t)bp[0]; btab_g[126] = (uint8_t)bp[1]; btab_g[127] = (uint8_t)bp[2];
            }
            *reinterpret_cast<uint32_t*>(btab_g + 252 - 4 * lane) = gather_bytes(bn[3], bn[2], bn[1], bn[0]);
            if (lane == 0) btab_g[0] = 0;          // y(0) = 0
            __syncwarp();
            // translate and store
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int4 o = make_int4((int)translate4((uint32_t)r.d[i].x, btab), (int)translate4((uint32_t)r.d[i].y, btab),
                                         (int)translate4((uint32_t)r.d[i].z, btab), (int)translate4((uint32_t)r.d[i].w, btab));
                *reinterpret_cast<int4*>(qy + row_of<TW>(t, i) * N + t.col) = o;
            }
            if (lane == 0) sy[t.tm * (N / QB) + (t.col >> 5)] = __float2half_rn(scale32);
        });
}

// The derivative table.  d(x) = Phi(x) + x*phi(x) is needed at x = q*s for the 256 payloads q of a block with scale s, i.e. at
// |x| = a*s for a = 1..128 and each of the 32768 non-negative fp16 bit patterns of s: 4 M arguments in all.  The device table
// holds, per (s, a), the pair ( d(+a*s), d(-a*s) ) evaluated with the reference's fp32 roundings
//      er = RN(erf(u)), u = RN(x / sqrt2);   e = RN(exp(RN(-RN(x*x)/2)));   ex = RN(RN(x / sqrt(2 pi)) * e)
//      d(+x) = RN(RN(0.5*(1 + er)) + ex),    d(-x) = RN(RN(0.5*(1 - er)) - ex)
// where erf and exp are correctly rounded (fp64, rounded once).  32 MB, filled once per device by one kernel (a millisecond);
// a block reads its row of 1 KB (lane l the pairs a = 4l+1..4l+4), which replaces 128 fp64 erf + exp evaluations per block --
// the part that bound the kernel (instruction issue, not the fp64 pipe).  Rows in use cluster (scales of neighbouring blocks
// share their exponent), so the reads are served by L2.
__device__ float2 g_gelu_bwd_table[GELU_ROWS * 128u];

__global__ void gelu_bwd_table_kernel() {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= GELU_ROWS * 128u) return;
    const float scx = __half2float(__ushort_as_half((unsigned short)(i >> 7)));
    const float x = __fmul_rn((float)((i & 127u) + 1u), scx);                    // exact
    const float er = (float)erf((double)__fdiv_rn(x, SQRT2_F));
    const float e = (float)exp((double)__fmul_rn(__fmul_rn(x, x), -0.5f));
    const float ex = __fmul_rn(__fdiv_rn(x, SQRT2PI_F), e);
    g_gelu_bwd_table[i] = make_float2(__fadd_rn(__fmul_rn(0.5f, __fadd_rn(1.0f, er)), ex),
                                      __fsub_rn(__fmul_rn(0.5f, __fsub_rn(1.0f, er)), ex));
}

// backward: x = q*s, g = qg*sg in fp32; d = (Phi(x) + x*phi(x)) * g; block quantise (+SR).
// Per block the 256-entry table "payload -> d(q*s)" is copied from the block's row of the device table into shared memory.
template <bool SR>
__global__ void __launch_bounds__(THREADS, 3)
gelu_bwd_kernel(const int8_t* __restrict__ qx, const __half* __restrict__ sx, const int8_t* __restrict__ qg,
                const __half* __restrict__ sg, int64_t M, int64_t N, int8_t* __restrict__ qd, __half* __restrict__ sd, SrCfg sr) {
    constexpr int TW = 32, NP = Geo<TW>::NP;
    using Raw = RawQ2<NP>;
    __shared__ __align__(16) float lut_all[WARPS][256];
    float* lut = lut_all[threadIdx.x >> 5];
    for_each_tile<TW, Raw, true>(
        M, N,
        [&](const Tile& t, Raw& r) {
            load_rows<TW>(qx, t, N, r.a);
            load_rows<TW>(qg, t, N, r.b);
            r.sa = load_scale16(sx, t, N);
            r.sb = load_scale16(sg, t, N);
        },
        [&](const Tile& t, Raw& r) {
            const TableRow tr = load_table_row(g_gelu_bwd_table, r.sa, t.lane);
            const float4 p01 = tr.p01, p23 = tr.p23;       // pairs a = 4l+1, 4l+2 | 4l+3, 4l+4
            __syncwarp();   // the previous tile's lookups are done
            {
                const int a = 4 * t.lane + 1;
                lut[a] = p01.x; lut[a + 1] = p01.z; lut[a + 2] = p23.x;
                if (a + 3 < 128) lut[a + 3] = p23.z;                   // +128 is not a payload: that byte is -128's
                lut[256 - a] = p01.y; lut[255 - a] = p01.w; lut[254 - a] = p23.y; lut[253 - a] = p23.w;
            }
            if (t.lane == 0) lut[0] = 0.5f;
            __syncwarp();
            const float scg = __half2float(r.sb);
            const uint64_t scg2 = f2_pack(scg, scg);
            float v[NP][16];
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                float fd[16], fg[16];
                lookup16(lut, r.a[i], fd);
                unpack16(r.b[i], fg);
#pragma unroll
                for (int j = 0; j < 16; j += 2)
                    f2_unpack(f2_mul(f2_pack(fd[j], fd[j + 1]), f2_mul(f2_pack(fg[j], fg[j + 1]), scg2)), v[i][j], v[i][j + 1]);
            }
            const float scale32 = __fdiv_rn(block_max<TW>(absmax_tile<NP>(v)), 127.0f);
            emit_quantized<TW, false, SR, false>([&](int i, float (&a)[16]) {
#pragma unroll
                for (int j = 0; j < 16; ++j) a[j] = v[i][j];
            }, scale32, t, M, N, qd, sd, sr, nullptr, nullptr);
        });
}

// =========================================================================================================
// LayerNorm forward: y = ((fp16(q*s) - mean) * rstd) * gamma; statistics are inputs
// =========================================================================================================
template <int TW>
__global__ void __launch_bounds__(THREADS, TW == 32 ? 3 : 2)
ln_fwd_kernel(const int8_t* __restrict__ qx, const __half* __restrict__ sx, const float* __restrict__ gamma,
              const float* __restrict__ mean, const float* __restrict__ rstd, int64_t M, int64_t N, int8_t* __restrict__ qy,
              __half* __restrict__ sy) {
    constexpr int NP = Geo<TW>::NP;
    using Raw = RawQ<NP>;
    for_each_tile<TW, Raw, true>(
        M, N,
        [&](const Tile& t, Raw& r) {
            load_rows<TW>(qx, t, N, r.d);
            r.sc = load_scale16(sx, t, N);
        },
        [&](const Tile& t, Raw& r) {
            const __half2 s2 = __half2half2(r.sc);
            float gm[16];
            if (t.active) {
                Load16<float>::load(gamma + t.col, gm);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) gm[j] = 0.f;
            }
            uint64_t gm2[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) gm2[j] = f2_pack(gm[2 * j], gm[2 * j + 1]);
            float v[NP][16];
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int64_t row = row_of<TW>(t, i);
                const float mu = __ldg(mean + row), rs = __ldg(rstd + row);
                const uint64_t nmu2 = f2_pack(-mu, -mu), rs2 = f2_pack(rs, rs);
                float f[16];
                dequant16_h(r.d[i], s2, f);
#pragma unroll
                for (int j = 0; j < 8; ++j)        // ((f - mu) * rs) * gamma, two columns per instruction
                    f2_unpack(f2_mul(f2_mul(f2_add(f2_pack(f[2 * j], f[2 * j + 1]), nmu2), rs2), gm2[j]), v[i][2 * j], v[i][2 * j + 1]);
            }
            const float scale32 = __fdiv_rn(block_max<TW>(absmax_tile<NP>(v)), 127.0f);
            SrCfg sr{};
            emit_quantized<TW, false, false, false>([&](int i, float (&a)[16]) {
#pragma unroll
                for (int j = 0; j < 16; ++j) a[j] = v[i][j];
            }, scale32, t, M, N, qy, sy, sr, nullptr, nullptr);
        });
}

// =========================================================================================================
// LayerNorm backward (dx and per-32-row partial dgamma), row reductions over the tile's 128-column slab.
// Rounding points of the reference: mean, rstd, x, dy, xhat in fp16; c1, c2 and the dx expression in fp32; dx -> fp16.
// =========================================================================================================
// Two warps share one 32x128 slab tile, 64 columns each (64 values per lane instead of 128: 2 CTAs per SM instead of one
// at 242 registers).  The quantisation blocks and the dgamma columns are private to a warp; only the two row sums per row cross
// the warps, through shared memory and a 64-thread named barrier per row pass.  The sum order is the one of a single warp over
// 8 lanes: ((l0+l1)+(l2+l3)) + ((l4+l5)+(l6+l7)).
template <bool SR, int TW = 64>
__global__ void __launch_bounds__(THREADS, 2)
ln_bwd_kernel(const int8_t* __restrict__ qx, const __half* __restrict__ sx, const int8_t* __restrict__ qg,
              const __half* __restrict__ sg, const float* __restrict__ gamma, const float* __restrict__ mean,
              const float* __restrict__ rstd, int64_t M, int64_t N, int8_t* __restrict__ qd, __half* __restrict__ sd,
              float* __restrict__ dw_partial, SrCfg sr) {
    constexpr int NP = Geo<TW>::NP, WPS = 128 / TW, PAIRS = WARPS / WPS;   // WPS warps per slab tile, PAIRS slab tiles per CTA
    __shared__ float2 row_part[PAIRS][WPS][QB];        // [slab tile][part][row of the tile] = (sum xhat*wdy, sum wdy) over the part
    const int warp = threadIdx.x >> 5, pair = warp / WPS, half = warp % WPS;
    const int64_t slabs_n = (N + 127) / 128, tiles_n_ = (N + TW - 1) / TW;
    const int64_t slab_tile = (int64_t)blockIdx.x * PAIRS + pair;          // index of the 32 x 128 slab tile
    if (slab_tile >= (M / QB) * slabs_n) return;                           // both warps of a pair leave together
    const int64_t tm_ = (int64_t)((uint32_t)slab_tile / (uint32_t)slabs_n);                      // 32-bit division
    const int64_t tn_ = (int64_t)((uint32_t)slab_tile % (uint32_t)slabs_n) * WPS + half;
    // the right half of a short last slab may lie outside the tensor: such a warp loads zeros and only takes part in the sums
    Tile t = make_tile<TW>(tm_ * tiles_n_ + (tn_ < tiles_n_ ? tn_ : tiles_n_ - 1), tiles_n_, N);
    if (tn_ >= tiles_n_) t.active = false;
    int4 rx[NP], rgr[NP];
    load_rows<TW>(qx, t, N, rx);
    load_rows<TW>(qg, t, N, rgr);
    const __half2 sx2 = load_scale_h2(sx, t, N), sg2 = load_scale_h2(sg, t, N);
    float gm[16];
    if (t.active) {
        Load16<float>::load(gamma + t.col, gm);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) gm[j] = 0.f;
    }
    const float n_f = (float)N;
    float v[NP][16];    // dx, rounded to fp16 and widened
    float dwp[16];      // partial dgamma over this lane's rows
#pragma unroll
    for (int j = 0; j < 16; ++j) dwp[j] = 0.f;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        const int64_t row = row_of<TW>(t, i);
        const int row_in_tile = i * Geo<TW>::RPP + t.rg;
        const __half2 mu2 = __half2half2(__float2half_rn(__ldg(mean + row)));
        const __half rs16 = __float2half_rn(__ldg(rstd + row));
        const __half2 rs2 = __half2half2(rs16);
        const float rs = __half2float(rs16);
        float xh[16], wdy[16];
        __half2 hx[8], hg[8];
        unpack16_h2(rx[i], hx);
        unpack16_h2(rgr[i], hg);
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __half2 x16 = __hmul2_rn(hx[j], sx2);
            const __half2 dy16 = __hmul2_rn(hg[j], sg2);
            const __half2 xhat16 = __hmul2_rn(__hsub2_rn(x16, mu2), rs2);
            const float2 xf = __half22float2(xhat16), dyf = __half22float2(dy16), pr = __half22float2(__hmul2_rn(dy16, xhat16));
            xh[2 * j] = xf.x; xh[2 * j + 1] = xf.y;
            wdy[2 * j] = __fmul_rn(gm[2 * j], dyf.x); wdy[2 * j + 1] = __fmul_rn(gm[2 * j + 1], dyf.y);
            s1 = __fadd_rn(__fadd_rn(s1, __fmul_rn(xh[2 * j], wdy[2 * j])), __fmul_rn(xh[2 * j + 1], wdy[2 * j + 1]));
            s2 = __fadd_rn(__fadd_rn(s2, wdy[2 * j]), wdy[2 * j + 1]);
            dwp[2 * j] = __fadd_rn(dwp[2 * j], pr.x); dwp[2 * j + 1] = __fadd_rn(dwp[2 * j + 1], pr.y);
        }
        // sums over this warp's 64 columns, then the other warp's through shared memory (left + right)
        s1 = row_sum<TW>(s1);
        s2 = row_sum<TW>(s2);
        if (t.cc == 0) row_part[pair][half][row_in_tile] = make_float2(s1, s2);
        asm volatile("bar.sync %0, %1;" ::"r"(1 + pair), "n"(32 * WPS) : "memory");
        float2 tot;
        {
            const float2 lft = row_part[pair][0][row_in_tile], rgt = row_part[pair][1][row_in_tile];
            tot = make_float2(__fadd_rn(lft.x, rgt.x), __fadd_rn(lft.y, rgt.y));
            if (WPS == 4) {
                const float2 l2 = row_part[pair][2][row_in_tile], r2 = row_part[pair][3][row_in_tile];
                tot = make_float2(__fadd_rn(tot.x, __fadd_rn(l2.x, r2.x)), __fadd_rn(tot.y, __fadd_rn(l2.y, r2.y)));
            }
        }
        const float c1 = __fdiv_rn(tot.x, n_f), c2 = __fdiv_rn(tot.y, n_f);
        const uint64_t nc1 = f2_pack(-c1, -c1), nc2 = f2_pack(-c2, -c2), rs_2 = f2_pack(rs, rs);
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            // (wdy - (xhat * c1 + c2)) * rstd, each operation rounded:  -(a*b + c) == (a * -b) + -c  exactly
            const uint64_t ntt = f2_add(f2_mul(f2_pack(xh[j], xh[j + 1]), nc1), nc2);
            float d0, d1;
            f2_unpack(f2_mul(f2_add(f2_pack(wdy[j], wdy[j + 1]), ntt), rs_2), d0, d1);
            const float2 dd = __half22float2(__floats2half2_rn(d0, d1));
            v[i][j] = dd.x; v[i][j + 1] = dd.y;
        }
    }
    // partial dgamma: reduce the row groups, lanes with rg == 0 write 16 columns
#pragma unroll
    for (int j = 0; j < 16; ++j) dwp[j] = col_sum<TW>(dwp[j]);
    if (t.active && t.rg == 0) {
        float4* dst = reinterpret_cast<float4*>(dw_partial + t.tm * N + t.col);
#pragma unroll
        for (int k = 0; k < 4; ++k) dst[k] = make_float4(dwp[4 * k], dwp[4 * k + 1], dwp[4 * k + 2], dwp[4 * k + 3]);
    }
    const float amax = block_max<TW>(absmax_tile<NP>(v));   // exactly representable in fp16
    const float scale32 = __fdiv_rn(amax, 127.0f);
    emit_quantized<TW, false, SR, false>([&](int i, float (&a)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) a[j] = v[i][j];
    }, scale32, t, M, N, qd, sd, sr, nullptr, nullptr);
}

// dgamma[n] = sum over the M/32 partial rows: 8 interleaved row groups per column (thread (x, g) sums rows g, g+8, ...), then the
// 8 group sums in ascending order -- a fixed order, so the result is deterministic.  Block = 32 columns x 8 groups.
__global__ void __launch_bounds__(256) ln_bwd_dw_kernel(const float* __restrict__ partial, int64_t rows, int64_t N, float* __restrict__ dgamma) {
    __shared__ float red[8][32];
    const int tx = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int64_t n = (int64_t)blockIdx.x * 32 + tx;
    float a = 0.f;
    if (n < N)
        for (int64_t r = g; r < rows; r += 8) a = __fadd_rn(a, partial[r * N + n]);
    red[g][tx] = a;
    __syncthreads();
    if (g == 0 && n < N) {
        float s = red[0][tx];
#pragma unroll
        for (int k = 1; k < 8; ++k) s = __fadd_rn(s, red[k][tx]);
        dgamma[n] = s;
    }
}

__device__ __forceinline__ float4 widen4(const float4& v, float) { return v; }
__device__ __forceinline__ float4 widen4(const uint2& v, __half) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 widen4(const uint2& v, __nv_bfloat16) {
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xFFFF0000u));
}

// Quantise and store the 8 x 4 values a lane holds of one 32x32 block in the "4 columns per lane" mapping (rows 4i + r, columns
// 4c .. 4c+3; `base` = linear index of the lane's first element).  TRUNC: truncating conversion (residual add) instead of
// round-half-even.  Stochastic rounding: one Philox call yields the noise of 8 consecutive elements = two neighbouring lanes;
// the even lane generates the call of the even passes, the odd lane that of the odd passes, and they exchange the halves they
// owe each other with shuffles.
template <bool TRUNC, bool SR, class RowF>
__device__ __forceinline__ void emit_block4(RowF&& rowf /* i -> the lane's float4 of pass i */, float scale32, int64_t base, int64_t N, int c,
                                            int8_t* __restrict__ qy, const SrCfg& sr) {
    const Divisor d = make_divisor(scale32);
    const bool zero = (scale32 == 0.f);
    const bool fast = d.fast || zero;                      // identical in every lane: one divisor per block
    const uint64_t inv2 = f2_pack(d.inv, d.inv), negb2 = f2_pack(-d.b, -d.b), magic2 = f2_pack(12582912.0f, 12582912.0f);
    auto rows = [&](auto fast_c) {
        constexpr bool FAST = decltype(fast_c)::value;
#pragma unroll
        for (int i2 = 0; i2 < 8; i2 += 2) {
            float nz[2][4];
            if (SR) {
                if (sr.noise) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float4 n4 = __ldg(reinterpret_cast<const float4*>(sr.noise + base + (int64_t)(4 * (i2 + h)) * N));
                        nz[h][0] = n4.x; nz[h][1] = n4.y; nz[h][2] = n4.z; nz[h][3] = n4.w;
                    }
                } else {
                    // this lane generates the 8-element group of pass i2 (even c) or i2 + 1 (odd c); a group starts at the even
                    // lane's first column
                    const int odd = c & 1;
                    const uint64_t e = (uint64_t)(base + (int64_t)(4 * (i2 + odd)) * N - 4 * odd);
                    float g8[8];
                    philox_noise8(e, sr.keys, sr.offset, g8);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // keep the half over this lane's own columns; the other half is the neighbour's (even lane: high half of
                        // pass i2's group, odd lane: low half of pass i2+1's group)
                        const float got = __shfl_xor_sync(0xffffffffu, odd ? g8[k] : g8[4 + k], 1);
                        const float own = odd ? g8[4 + k] : g8[k];
                        nz[0][k] = odd ? got : own;       // (selects, not a run-time array index: that would put nz in local memory)
                        nz[1][k] = odd ? own : got;
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int i = i2 + h;
                const float4 vi = rowf(i);
                const float a[4] = {vi.x, vi.y, vi.z, vi.w};
                uint32_t bts[4];
#pragma unroll
                for (int k = 0; k < 4; k += 2) {
                    float x0, x1;
                    if (FAST) {
                        const uint64_t x2 = f2_div_fast(f2_pack(a[k], a[k + 1]), inv2, negb2);
                        if (!SR && !TRUNC) {
                            f2_unpack(f2_add(x2, magic2), x0, x1);
                            bts[k] = __float_as_uint(x0); bts[k + 1] = __float_as_uint(x1);
                            continue;
                        }
                        f2_unpack(x2, x0, x1);
                    } else {
                        x0 = __fdiv_rn(a[k], d.b); x1 = __fdiv_rn(a[k + 1], d.b);
                    }
                    if (SR) {
                        const float m0 = fminf(__fadd_rn(fabsf(x0), nz[h][k]), 127.f), m1 = fminf(__fadd_rn(fabsf(x1), nz[h][k + 1]), 127.f);
                        x0 = __uint_as_float(__float_as_uint(m0) ^ (__float_as_uint(x0) & 0x80000000u));
                        x1 = __uint_as_float(__float_as_uint(m1) ^ (__float_as_uint(x1) & 0x80000000u));
                    }
                    bts[k] = TRUNC ? (uint32_t)__float2int_rz(x0) : __float_as_uint(__fadd_rn(x0, 12582912.0f));
                    bts[k + 1] = TRUNC ? (uint32_t)__float2int_rz(x1) : __float_as_uint(__fadd_rn(x1, 12582912.0f));
                }
                const uint32_t word = zero ? 0u : gather_bytes(bts[0], bts[1], bts[2], bts[3]);
                *reinterpret_cast<uint32_t*>(qy + base + (int64_t)(4 * i) * N) = word;
            }
        }
    };
    if (fast) rows(std::true_type{}); else rows(std::false_type{});
}

// quantize without the transposed copy, in the same mapping: a warp owns one 32x32 block, persistent over the blocks with the
// next block's loads in flight.
template <typename T, bool SR>
__global__ void __launch_bounds__(THREADS, 3)
quantize4_kernel(const T* __restrict__ x, int64_t M, int64_t N, int8_t* __restrict__ q, __half* __restrict__ s, SrCfg sr) {
    const int64_t blocks_n = N / QB, total = (M / QB) * blocks_n;
    const int64_t stride = (int64_t)gridDim.x * WARPS;
    const int lane = threadIdx.x & 31, r = lane >> 3, c = lane & 7;
    int64_t blk = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (blk >= total) return;
    auto base_of = [&](int64_t b) {
        const int64_t tm = (int64_t)((uint32_t)b / (uint32_t)blocks_n), tn = (int64_t)((uint32_t)b % (uint32_t)blocks_n);
        return (tm * QB + r) * N + tn * QB + 4 * c;
    };
    using Raw = typename std::conditional<sizeof(T) == 4, float4, uint2>::type;
    constexpr bool PREFETCH = sizeof(T) != 4;      // fp32 input: a second packed block (32 more registers) would spill
    auto load = [&](int64_t base, Raw (&raw)[8]) {
#pragma unroll
        for (int i = 0; i < 8; ++i) raw[i] = __ldg(reinterpret_cast<const Raw*>(x + base + (int64_t)(4 * i) * N));
    };
    int64_t base = base_of(blk);
    Raw cur[8];
    load(base, cur);
    for (;;) {
        const int64_t next = blk + stride;
        const bool has_next = next < total;
        const int64_t nbase = has_next ? base_of(next) : base;
        Raw nxt[8];
        if (PREFETCH && has_next) load(nbase, nxt);
        // the block stays packed in registers and is widened twice (absmax, then quantisation): cheaper than holding 32 fp32 values
        // next to the prefetched next block
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 w = widen4(cur[i], T());
            m = fmaxf(fmaxf(m, fmaxf(fabsf(w.x), fabsf(w.y))), fmaxf(fabsf(w.z), fabsf(w.w)));
        }
        const float scale32 = __fdiv_rn(__uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m))), 127.0f);
        emit_block4<false, SR>([&](int i) { return widen4(cur[i], T()); }, scale32, base, N, c, q, sr);
        if (lane == 0) s[blk] = __float2half_rn(scale32);          // scales are [M/32, N/32] row-major = block index
        if (!has_next) break;
        if (PREFETCH) {
#pragma unroll
            for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
        } else {
            load(nbase, cur);
        }
        base = nbase;
        blk = next;
    }
}

// Round-to-nearest quantisation of up to 8 tensors of one dtype in ONE launch (the weight matrices of a transformer block, or of
// several blocks): the blocks of all tensors are numbered consecutively and a warp finds its tensor by comparing its block number
// with the running totals.  One block per warp per iteration, no prefetch (the tensors are small and many).
constexpr int QMULTI_MAX = 8;
struct QuantizeJobs {
    const void* x[QMULTI_MAX];
    int8_t* q[QMULTI_MAX];
    __half* s[QMULTI_MAX];
    int64_t N[QMULTI_MAX];             // columns
    int64_t first_block[QMULTI_MAX + 1];   // first global block number of tensor j; [count] = total
    int count;
};

template <typename T>
__global__ void __launch_bounds__(THREADS, 3) quantize_multi_kernel(const QuantizeJobs jobs) {
    const int64_t total = jobs.first_block[jobs.count];
    const int64_t stride = (int64_t)gridDim.x * WARPS;
    const int lane = threadIdx.x & 31, r = lane >> 3, c = lane & 7;
    using Raw = typename std::conditional<sizeof(T) == 4, float4, uint2>::type;
    SrCfg sr{};
    for (int64_t g = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5); g < total; g += stride) {
        int j = 0;
#pragma unroll
        for (int k = 1; k < QMULTI_MAX; ++k) j += (k < jobs.count && g >= jobs.first_block[k]) ? 1 : 0;
        const int64_t blk = g - jobs.first_block[j];
        const int64_t N = jobs.N[j], blocks_n = N / QB;
        const int64_t tm = (int64_t)((uint32_t)blk / (uint32_t)blocks_n), tn = (int64_t)((uint32_t)blk % (uint32_t)blocks_n);
        const int64_t base = (tm * QB + r) * N + tn * QB + 4 * c;
        const T* x = static_cast<const T*>(jobs.x[j]);
        Raw cur[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) cur[i] = __ldg(reinterpret_cast<const Raw*>(x + base + (int64_t)(4 * i) * N));
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 w = widen4(cur[i], T());
            m = fmaxf(fmaxf(m, fmaxf(fabsf(w.x), fabsf(w.y))), fmaxf(fabsf(w.z), fabsf(w.w)));
        }
        const float scale32 = __fdiv_rn(__uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m))), 127.0f);
        emit_block4<false, false>([&](int i) { return widen4(cur[i], T()); }, scale32, base, N, c, jobs.q[j], sr);
        if (lane == 0) jobs.s[j][blk] = __float2half_rn(scale32);
    }
}

// =========================================================================================================
// residual add (+ optional row statistics): y = x1 + q2*s2 (fp32); store y; block quantise y by truncation
// =========================================================================================================
// This operator moves 8-10 bytes per element, most of them fp32, so its lane mapping is chosen for the wide side: a warp owns
// one 32x32 block; lane = (r = lane / 8, c = lane % 8) owns columns 4c .. 4c+3 of rows 4i + r, i = 0 .. 7.  Every warp access
// is then made of whole segments: 128 B of fp32 per row (one float4 per lane, 8 lanes), 64 B of bf16, one 32-byte sector of
// int8.  (With the 16-columns-per-lane mapping of the other kernels a lane's four float4 accesses to one row landed in four
// different instructions, each of which touched 32 half-used sectors: 65.8 us for bf16 + stochastic rounding on [8192 x 3072].)
// The block absmax is a thread-local max + one redux.sync.  Stochastic rounding: one Philox call yields the noise of 8
// consecutive elements = two neighbouring lanes; the even lane generates the call of the even passes, the odd lane that of the
// odd passes, and they exchange the halves they owe each other with two shuffles per pair of passes.
// With MEANVAR a warp walks the four blocks of a 128-column slab and writes one partial sum / sum of squares per row and slab.
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
template <>
__device__ __forceinline__ float4 load4<__half>(const __half* p) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xFFFF0000u));
}

template <typename T, bool MEANVAR, bool SR>
__global__ void __launch_bounds__(THREADS, 3)
add_kernel(const T* __restrict__ x1, const int8_t* __restrict__ q2, const __half* __restrict__ s2, int64_t M, int64_t N,
           float* __restrict__ y1, int8_t* __restrict__ qy, __half* __restrict__ sy, float* __restrict__ part_sum,
           float* __restrict__ part_sq, SrCfg sr) {
    constexpr int SUBS = MEANVAR ? 4 : 1;                     // 32-column blocks per work item
    const int64_t blocks_n = N / QB;                          // blocks per row of blocks
    const int64_t groups_n = (blocks_n + SUBS - 1) / SUBS;    // work items per row of blocks (MEANVAR: 128-column slabs)
    const int64_t item = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (item >= (M / QB) * groups_n) return;
    const int64_t tm = (int64_t)((uint32_t)item / (uint32_t)groups_n), grp = (int64_t)((uint32_t)item % (uint32_t)groups_n);   // 32-bit division
    const int lane = threadIdx.x & 31, r = lane >> 3, c = lane & 7;
    float ps[8], pq[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) ps[i] = pq[i] = 0.f;
#pragma unroll 1
    for (int sub = 0; sub < SUBS; ++sub) {
        const int64_t tn = grp * SUBS + sub;
        if (tn >= blocks_n) break;                            // warp-uniform
        const int64_t base = (tm * QB + r) * N + tn * QB + 4 * c;      // element (row r of the block, this lane's columns)
        uint32_t qw[8];
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) qw[i] = __ldg(reinterpret_cast<const uint32_t*>(q2 + base + (int64_t)(4 * i) * N)) ^ 0x80808080u;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = load4<T>(x1 + base + (int64_t)(4 * i) * N);
        const float sc = __half2float(__ldg(s2 + tm * blocks_n + tn));
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i].x = __fadd_rn(v[i].x, __fmul_rn(byte_to_float(qw[i], 0), sc));
            v[i].y = __fadd_rn(v[i].y, __fmul_rn(byte_to_float(qw[i], 1), sc));
            v[i].z = __fadd_rn(v[i].z, __fmul_rn(byte_to_float(qw[i], 2), sc));
            v[i].w = __fadd_rn(v[i].w, __fmul_rn(byte_to_float(qw[i], 3), sc));
            *reinterpret_cast<float4*>(y1 + base + (int64_t)(4 * i) * N) = v[i];
            m = fmaxf(fmaxf(m, fmaxf(fabsf(v[i].x), fabsf(v[i].y))), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
            if (MEANVAR) {
                ps[i] = __fadd_rn(ps[i], __fadd_rn(__fadd_rn(v[i].x, v[i].y), __fadd_rn(v[i].z, v[i].w)));
                pq[i] = __fadd_rn(pq[i], __fadd_rn(__fadd_rn(__fmul_rn(v[i].x, v[i].x), __fmul_rn(v[i].y, v[i].y)),
                                                   __fadd_rn(__fmul_rn(v[i].z, v[i].z), __fmul_rn(v[i].w, v[i].w))));
            }
        }
        const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m)));
        const float scale32 = __fdiv_rn(amax, 127.0f);
        emit_block4<true, SR>([&](int i) { return v[i]; }, scale32, base, N, c, qy, sr);
        if (lane == 0) sy[tm * blocks_n + tn] = __float2half_rn(scale32);
    }
    if (MEANVAR) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float a = ps[i], b2 = pq[i];
#pragma unroll
            for (int mask = 1; mask < 8; mask <<= 1) {
                a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, mask));
                b2 = __fadd_rn(b2, __shfl_xor_sync(0xffffffffu, b2, mask));
            }
            if (c == 0) {
                const int64_t row = tm * QB + 4 * i + r;
                part_sum[row * groups_n + grp] = a;
                part_sq[row * groups_n + grp] = b2;
            }
        }
    }
}

// mean = sum/N; rstd = 1/sqrt(sumsq/N - mean^2)
__global__ void meanvar_finish_kernel(const float* __restrict__ part_sum, const float* __restrict__ part_sq, int64_t M, int64_t tiles_n,
                                      int64_t N, float* __restrict__ mean, float* __restrict__ rstd) {
    const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= M) return;
    float a = 0.f, b = 0.f;
    for (int64_t k = 0; k < tiles_n; ++k) {
        a = __fadd_rn(a, part_sum[row * tiles_n + k]);
        b = __fadd_rn(b, part_sq[row * tiles_n + k]);
    }
    const float n = (float)N;
    const float mu = __fdiv_rn(a, n);
    const float var = __fsub_rn(__fdiv_rn(b, n), __fmul_rn(mu, mu));
    mean[row] = mu;
    rstd[row] = __fdiv_rn(1.0f, __fsqrt_rn(var));
}



}  // namespace jf

// =========================================================================================================
// C ABI
// =========================================================================================================
using namespace jf;

#define JF_REQUIRE_PTR(p) \
    do {                  \
        if (!(p)) return JF_ERR_NULL; \
    } while (0)
#define JF_REQUIRE_ALIGNED(p) \
    do {                      \
        if (!aligned16(p)) return JF_ERR_ALIGN; \
    } while (0)

static inline int check_mn(int64_t M, int64_t N) {
    // blocks are indexed with 32-bit arithmetic inside the kernels
    return (mult32(M) && mult32(N) && (M / 32) * (N / 32) < (int64_t(1) << 31)) ? JF_OK : JF_ERR_SHAPE;
}

// CTAs of a persistent launch: `per_sm` 8-warp CTAs per SM (3 for the 32-column kernels at <= 80 registers, 2 otherwise).
static int persistent_ctas(int per_sm) {
    static const int sms = [] {
        int dev = 0, n = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        return n;
    }();
    return per_sm * sms;
}

// Tile widths (measured choices): 32 columns for the kernels with arithmetic per element (quantize without the transposed
// copy, GELU, LayerNorm forward, residual add), 64 for the pure data movers (dequantize, transpose, quantize + transposed copy).
template <typename T>
static void launch_quantize(const void* x, int64_t M, int64_t N, int8_t* q, __half* s, int8_t* qt, bool stochastic, SrCfg sr,
                            cudaStream_t st) {
    const T* xp = (const T*)x;
    if (qt) {
        const unsigned grid = grid_for<64>(M, N, persistent_ctas(2));
        if (stochastic) quantize_kernel<T, 64, true, true><<<grid, THREADS, 0, st>>>(xp, M, N, q, s, qt, sr);
        else quantize_kernel<T, 64, false, true><<<grid, THREADS, 0, st>>>(xp, M, N, q, s, qt, sr);
    } else {
        const unsigned grid = grid_for<32>(M, N, persistent_ctas(3));
        // round-to-nearest: the 4-columns-per-lane mapping (whole sectors per access); stochastic rounding: the 16-columns-per-lane
        // mapping, where a lane owns whole 8-element Philox groups (measured on [8192 x 3072] bf16: 31.1 us against 33.4 us)
        if (stochastic) quantize_kernel<T, 32, true, false><<<grid, THREADS, 0, st>>>(xp, M, N, q, s, nullptr, sr);
        else quantize4_kernel<T, false><<<grid, THREADS, 0, st>>>(xp, M, N, q, s, sr);
    }
}

// The GELU tables (32 MB each) of the current device: each filled by one kernel launch on the first call's stream; until that launch is
// known to have finished, calls on any stream wait for its event.
struct FwdTableState {
    cudaEvent_t ready = nullptr;
    bool launched = false, complete = false;
};
static FwdTableState g_fwd_table[64], g_bwd_table[64];
static std::mutex g_fwd_table_mutex;

static int ensure_gelu_table(cudaStream_t st, bool backward) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return JF_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_fwd_table_mutex);
    FwdTableState& ts = (backward ? g_bwd_table : g_fwd_table)[dev];
    if (ts.complete) return JF_OK;
    if (!ts.launched) {
        cudaStreamCaptureStatus cap0 = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cap0) != cudaSuccess) return JF_ERR_LAUNCH;
        if (cap0 != cudaStreamCaptureStatusNone) return JF_ERR_UNSUPPORTED;     // the fill must not become part of a graph
        if (cudaEventCreateWithFlags(&ts.ready, cudaEventDisableTiming) != cudaSuccess) return JF_ERR_LAUNCH;
        if (backward) gelu_bwd_table_kernel<<<GELU_ROWS * 128u / 256u, 256, 0, st>>>();
        else gelu_fwd_table_kernel<<<GELU_ROWS * 128u / 256u, 256, 0, st>>>();
        if (int e = check_launch()) return e;
        if (cudaEventRecord(ts.ready, st) != cudaSuccess) return JF_ERR_LAUNCH;
        ts.launched = true;
        return JF_OK;   // later work on `st` is ordered after the fill
    }
    // a stream that is being captured must not be queried: order the captured work after the fill instead
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) return JF_ERR_LAUNCH;
    if (cap == cudaStreamCaptureStatusNone && cudaEventQuery(ts.ready) == cudaSuccess) {
        ts.complete = true;
        return JF_OK;
    }
    return cudaStreamWaitEvent(st, ts.ready, 0) == cudaSuccess ? JF_OK : JF_ERR_LAUNCH;
}

template <typename T>
static void launch_add(const void* x1, const int8_t* q2, const __half* s2, int64_t M, int64_t N, float* y1, int8_t* qy, __half* sy,
                       float* ps, float* pq, bool meanvar, bool stochastic, SrCfg sr, cudaStream_t st) {
    // work items: 32x32 blocks, or (with row statistics) 128-column slabs of four blocks walked by one warp each
    const T* xp = (const T*)x1;
    const int64_t blocks = (M / QB) * (N / QB), slabs = (M / QB) * ((N + 127) / 128);
    const unsigned grid_b = (unsigned)((blocks + WARPS - 1) / WARPS), grid_s = (unsigned)((slabs + WARPS - 1) / WARPS);
    if (meanvar) add_kernel<T, true, false><<<grid_s, THREADS, 0, st>>>(xp, q2, s2, M, N, y1, qy, sy, ps, pq, sr);
    else if (stochastic) add_kernel<T, false, true><<<grid_b, THREADS, 0, st>>>(xp, q2, s2, M, N, y1, qy, sy, ps, pq, sr);
    else add_kernel<T, false, false><<<grid_b, THREADS, 0, st>>>(xp, q2, s2, M, N, y1, qy, sy, ps, pq, sr);
}

extern "C" {

const char* jf_status_string(int status) {
    switch (status) {
        case JF_OK: return "ok";
        case JF_ERR_NULL: return "a required pointer is NULL";
        case JF_ERR_SHAPE: return "dimensions must be positive multiples of 32 (and within documented limits)";
        case JF_ERR_ALIGN: return "pointers must be 16-byte aligned";
        case JF_ERR_DTYPE: return "unknown dtype code";
        case JF_ERR_LAUNCH: return "CUDA launch error";
        case JF_ERR_UNSUPPORTED: return "unsupported device or missing driver entry point";
        case JF_ERR_ARG: return "invalid argument";
        default: return "unknown status";
    }
}
int jf_last_cuda_error(void) { return g_last_cuda_error; }
int jf_abi_version(void) { return 1; }

int jf_int8_quantize(const void* x, int x_dtype, int64_t M, int64_t N, int8_t* q, void* s, int8_t* qt, int stochastic,
                     const float* noise, uint64_t seed, uint64_t offset, void* stream) {
    JF_REQUIRE_PTR(x); JF_REQUIRE_PTR(q); JF_REQUIRE_PTR(s);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(x); JF_REQUIRE_ALIGNED(q);
    if (qt) JF_REQUIRE_ALIGNED(qt);
    if (noise) JF_REQUIRE_ALIGNED(noise);
    cudaStream_t st = (cudaStream_t)stream;
    SrCfg sr = make_sr(noise, seed, offset);
    __half* sh = (__half*)s;
    const bool sto = stochastic != 0;
    switch (x_dtype) {
        case JF_F32: launch_quantize<float>(x, M, N, q, sh, qt, sto, sr, st); break;
        case JF_F16: launch_quantize<__half>(x, M, N, q, sh, qt, sto, sr, st); break;
        case JF_BF16: launch_quantize<__nv_bfloat16>(x, M, N, q, sh, qt, sto, sr, st); break;
        default: return JF_ERR_DTYPE;
    }
    return check_launch();
}

int jf_int8_quantize_multi(int count, const void* const* x, int x_dtype, const int64_t* M, const int64_t* N, int8_t* const* q,
                           void* const* s, void* stream) {
    if (count <= 0 || count > QMULTI_MAX) return JF_ERR_ARG;
    JF_REQUIRE_PTR(x); JF_REQUIRE_PTR(M); JF_REQUIRE_PTR(N); JF_REQUIRE_PTR(q); JF_REQUIRE_PTR(s);
    QuantizeJobs jobs{};
    jobs.count = count;
    int64_t total = 0;
    for (int j = 0; j < count; ++j) {
        JF_REQUIRE_PTR(x[j]); JF_REQUIRE_PTR(q[j]); JF_REQUIRE_PTR(s[j]);
        if (int e = check_mn(M[j], N[j])) return e;
        JF_REQUIRE_ALIGNED(x[j]); JF_REQUIRE_ALIGNED(q[j]);
        jobs.x[j] = x[j]; jobs.q[j] = q[j]; jobs.s[j] = (__half*)s[j]; jobs.N[j] = N[j];
        jobs.first_block[j] = total;
        total += (M[j] / QB) * (N[j] / QB);
    }
    jobs.first_block[count] = total;
    if (total >= (int64_t(1) << 31)) return JF_ERR_SHAPE;
    const int64_t ctas = (total + WARPS - 1) / WARPS;
    const int cap = persistent_ctas(3) * 4;
    const unsigned grid = (unsigned)(ctas > cap ? cap : ctas);
    cudaStream_t st = (cudaStream_t)stream;
    switch (x_dtype) {
        case JF_F32: quantize_multi_kernel<float><<<grid, THREADS, 0, st>>>(jobs); break;
        case JF_F16: quantize_multi_kernel<__half><<<grid, THREADS, 0, st>>>(jobs); break;
        case JF_BF16: quantize_multi_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(jobs); break;
        default: return JF_ERR_DTYPE;
    }
    return check_launch();
}

int jf_int8_dequantize(const int8_t* q, const void* s, int64_t M, int64_t N, float* y, void* stream) {
    JF_REQUIRE_PTR(q); JF_REQUIRE_PTR(s); JF_REQUIRE_PTR(y);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(q); JF_REQUIRE_ALIGNED(y);
    cudaStream_t st = (cudaStream_t)stream;
    if (M / QB > 65535) return JF_ERR_SHAPE;     // one grid row per row of blocks
    const dim3 grid((unsigned)((N / 4 + DQ_THREADS - 1) / DQ_THREADS), (unsigned)(M / QB));
    dequantize_kernel<<<grid, DQ_THREADS, 0, st>>>(q, (const __half*)s, M, N, y);
    return check_launch();
}

int jf_int8_transpose(const int8_t* x, int64_t M, int64_t N, int8_t* y, void* stream) {
    JF_REQUIRE_PTR(x); JF_REQUIRE_PTR(y);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(x); JF_REQUIRE_ALIGNED(y);
    cudaStream_t st = (cudaStream_t)stream;
    if ((M + TR_TILE - 1) / TR_TILE > 65535) return JF_ERR_SHAPE;     // one grid row per 128 rows
    const dim3 grid((unsigned)((N + TR_TILE - 1) / TR_TILE), (unsigned)((M + TR_TILE - 1) / TR_TILE));
    transpose_kernel<<<grid, THREADS, 0, st>>>(x, M, N, y);
    return check_launch();
}

int jf_int8_gelu_forward(const int8_t* qx, const void* sx, int64_t M, int64_t N, int8_t* qy, void* sy, void* stream) {
    JF_REQUIRE_PTR(qx); JF_REQUIRE_PTR(sx); JF_REQUIRE_PTR(qy); JF_REQUIRE_PTR(sy);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(qx); JF_REQUIRE_ALIGNED(qy);
    cudaStream_t st = (cudaStream_t)stream;
    if (int e = ensure_gelu_table(st, false)) return e;
    gelu_fwd_kernel<<<grid_for<32>(M, N, persistent_ctas(3)), THREADS, 0, st>>>(qx, (const __half*)sx, M, N, qy, (__half*)sy);
    return check_launch();
}

int jf_int8_gelu_backward(const int8_t* qx, const void* sx, const int8_t* qg, const void* sg, int64_t M, int64_t N, int8_t* qd,
                          void* sd, int stochastic, const float* noise, uint64_t seed, uint64_t offset, void* stream) {
    JF_REQUIRE_PTR(qx); JF_REQUIRE_PTR(sx); JF_REQUIRE_PTR(qg); JF_REQUIRE_PTR(sg); JF_REQUIRE_PTR(qd); JF_REQUIRE_PTR(sd);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(qx); JF_REQUIRE_ALIGNED(qg); JF_REQUIRE_ALIGNED(qd);
    if (noise) JF_REQUIRE_ALIGNED(noise);
    SrCfg sr = make_sr(noise, seed, offset);
    cudaStream_t st = (cudaStream_t)stream;
    const __half* sxh = (const __half*)sx; const __half* sgh = (const __half*)sg; __half* sdh = (__half*)sd;
    if (int e = ensure_gelu_table(st, true)) return e;
    const unsigned grid = grid_for<32>(M, N, persistent_ctas(3));
    if (stochastic) gelu_bwd_kernel<true><<<grid, THREADS, 0, st>>>(qx, sxh, qg, sgh, M, N, qd, sdh, sr);
    else gelu_bwd_kernel<false><<<grid, THREADS, 0, st>>>(qx, sxh, qg, sgh, M, N, qd, sdh, sr);
    return check_launch();
}

int jf_int8_layernorm_forward(const int8_t* qx, const void* sx, const float* gamma, const float* mean, const float* rstd, int64_t M,
                              int64_t N, int8_t* qy, void* sy, void* stream) {
    JF_REQUIRE_PTR(qx); JF_REQUIRE_PTR(sx); JF_REQUIRE_PTR(gamma); JF_REQUIRE_PTR(mean); JF_REQUIRE_PTR(rstd);
    JF_REQUIRE_PTR(qy); JF_REQUIRE_PTR(sy);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(qx); JF_REQUIRE_ALIGNED(qy); JF_REQUIRE_ALIGNED(gamma);
    cudaStream_t st = (cudaStream_t)stream;
    ln_fwd_kernel<32><<<grid_for<32>(M, N, persistent_ctas(3)), THREADS, 0, st>>>(qx, (const __half*)sx, gamma, mean, rstd, M, N, qy, (__half*)sy);
    return check_launch();
}

int jf_int8_layernorm_backward(const int8_t* qx, const void* sx, const int8_t* qg, const void* sg, const float* gamma,
                               const float* mean, const float* rstd, int64_t M, int64_t N, int slab, int8_t* qd, void* sd,
                               float* dgamma, float* scratch, int stochastic, const float* noise, uint64_t seed, uint64_t offset,
                               void* stream) {
    JF_REQUIRE_PTR(qx); JF_REQUIRE_PTR(sx); JF_REQUIRE_PTR(qg); JF_REQUIRE_PTR(sg); JF_REQUIRE_PTR(gamma);
    JF_REQUIRE_PTR(mean); JF_REQUIRE_PTR(rstd); JF_REQUIRE_PTR(qd); JF_REQUIRE_PTR(sd); JF_REQUIRE_PTR(dgamma);
    JF_REQUIRE_PTR(scratch);
    if (int e = check_mn(M, N)) return e;
    if (slab != 128) return JF_ERR_ARG;         // only the reference's 128-column slab is implemented
    JF_REQUIRE_ALIGNED(qx); JF_REQUIRE_ALIGNED(qg); JF_REQUIRE_ALIGNED(qd); JF_REQUIRE_ALIGNED(gamma); JF_REQUIRE_ALIGNED(scratch);
    if (noise) JF_REQUIRE_ALIGNED(noise);
    cudaStream_t st = (cudaStream_t)stream;
    SrCfg sr = make_sr(noise, seed, offset);
    const int64_t slab_tiles = (M / QB) * ((N + 127) / 128);
    const unsigned grid = (unsigned)((slab_tiles + WARPS / 2 - 1) / (WARPS / 2));   // two warps per 32 x 128 slab tile
    const __half* sxh = (const __half*)sx; const __half* sgh = (const __half*)sg; __half* sdh = (__half*)sd;
    if (stochastic) ln_bwd_kernel<true><<<grid, THREADS, 0, st>>>(qx, sxh, qg, sgh, gamma, mean, rstd, M, N, qd, sdh, scratch, sr);
    else ln_bwd_kernel<false><<<grid, THREADS, 0, st>>>(qx, sxh, qg, sgh, gamma, mean, rstd, M, N, qd, sdh, scratch, sr);
    if (int e = check_launch()) return e;
    ln_bwd_dw_kernel<<<(unsigned)((N + 31) / 32), 256, 0, st>>>(scratch, M / QB, N, dgamma);
    return check_launch();
}

static int add_impl(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N, float* y1, int8_t* qy,
                    void* sy, float* mean, float* rstd, float* scratch, bool meanvar, bool stochastic, SrCfg sr, cudaStream_t st) {
    JF_REQUIRE_PTR(x1); JF_REQUIRE_PTR(q2); JF_REQUIRE_PTR(s2); JF_REQUIRE_PTR(y1); JF_REQUIRE_PTR(qy); JF_REQUIRE_PTR(sy);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(x1); JF_REQUIRE_ALIGNED(q2); JF_REQUIRE_ALIGNED(y1); JF_REQUIRE_ALIGNED(qy);
    if (sr.noise) JF_REQUIRE_ALIGNED(sr.noise);
    const int64_t tiles_n = (N + 127) / 128;
    float* ps = nullptr;
    float* pq = nullptr;
    if (meanvar) {
        JF_REQUIRE_PTR(mean); JF_REQUIRE_PTR(rstd); JF_REQUIRE_PTR(scratch);
        ps = scratch;
        pq = scratch + M * tiles_n;
    }
    const __half* s2h = (const __half*)s2;
    __half* syh = (__half*)sy;
    switch (x1_dtype) {
        case JF_F32: launch_add<float>(x1, q2, s2h, M, N, y1, qy, syh, ps, pq, meanvar, stochastic, sr, st); break;
        case JF_F16: launch_add<__half>(x1, q2, s2h, M, N, y1, qy, syh, ps, pq, meanvar, stochastic, sr, st); break;
        case JF_BF16: launch_add<__nv_bfloat16>(x1, q2, s2h, M, N, y1, qy, syh, ps, pq, meanvar, stochastic, sr, st); break;
        default: return JF_ERR_DTYPE;
    }
    if (int e = check_launch()) return e;
    if (meanvar) {
        meanvar_finish_kernel<<<(unsigned)((M + 127) / 128), 128, 0, st>>>(ps, pq, M, tiles_n, N, mean, rstd);
        return check_launch();
    }
    return JF_OK;
}

int jf_int8_add(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N, float* y1, int8_t* qy, void* sy,
                int stochastic, const float* noise, uint64_t seed, uint64_t offset, void* stream) {
    SrCfg sr = make_sr(noise, seed, offset);
    return add_impl(x1, x1_dtype, q2, s2, M, N, y1, qy, sy, nullptr, nullptr, nullptr, false, stochastic != 0, sr, (cudaStream_t)stream);
}

int jf_int8_add_meanvar(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N, float* y1, int8_t* qy,
                        void* sy, float* mean, float* rstd, float* scratch, void* stream) {
    SrCfg sr{};
    return add_impl(x1, x1_dtype, q2, s2, M, N, y1, qy, sy, mean, rstd, scratch, true, false, sr, (cudaStream_t)stream);
}

}  // extern "C"

