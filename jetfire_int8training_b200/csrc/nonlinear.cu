// INT8-in / INT8-out nonlinear operators of the Jetfire data flow, written for sm_100a.
//
// All kernels are bandwidth-bound streaming kernels built on one work decomposition:
//   * a warp owns a tile of 32 rows x 128 columns = four 32x32 quantisation blocks;
//   * lane = (rg, cc) with rg = lane / 8 (row group) and cc = lane % 8 (16-column chunk); in pass i (0..7) the lane
//     touches row 4*i + rg, columns [16*cc, 16*cc + 16): one 16-byte access per int8 row chunk, so a warp-wide
//     access covers four full 128-byte lines and every thread keeps 8 independent 16-byte loads in flight;
//   * a quantisation block is held by the 8 lanes {cc in {2b, 2b+1}} x {rg 0..3}; its absmax is three
//     __shfl_xor steps (lane masks 1, 8, 16);
//   * the re-quantising division is an exact IEEE quotient computed with a shared correctly-rounded reciprocal.
// CTAs are 8 warps; consecutive warps take consecutive tiles (row-major over the tile grid).
#include "jf_common.cuh"

namespace jf {

thread_local int g_last_cuda_error = 0;

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int TILE_N = 128;

struct Tile {
    int64_t tm, tn;   // tile coordinates
    int64_t row0;     // first row of the tile
    int64_t col;      // first column of this lane's 16-column chunk
    int rg, cc, lane;
    bool active;      // the chunk lies inside the tensor (N may end inside the tile)
};

__device__ __forceinline__ bool tile_setup(int64_t M, int64_t N, Tile& t) {
    const int warp = threadIdx.x >> 5;
    t.lane = threadIdx.x & 31;
    const int64_t tiles_n = (N + TILE_N - 1) / TILE_N;
    const int64_t tile = (int64_t)blockIdx.x * WARPS + warp;
    if (tile >= (M / QB) * tiles_n) return false;
    t.tm = tile / tiles_n;
    t.tn = tile % tiles_n;
    t.rg = t.lane >> 3;
    t.cc = t.lane & 7;
    t.row0 = t.tm * QB;
    t.col = t.tn * TILE_N + t.cc * 16;
    t.active = t.col < N;
    return true;
}

static inline unsigned grid_for(int64_t M, int64_t N) {
    const int64_t tiles = (M / QB) * ((N + TILE_N - 1) / TILE_N);
    return (unsigned)((tiles + WARPS - 1) / WARPS);
}

__device__ __forceinline__ float block_max(float m) {
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
    return m;
}

struct SrCfg {
    int stochastic;
    const float* noise;
    uint64_t seed, offset;
};

// 4x4 byte transpose: in w[k] = row k (4 column bytes); out o[j] = column j (4 row bytes).
__device__ __forceinline__ void transpose4x4(const uint32_t w[4], uint32_t o[4]) {
    const uint32_t t0 = __byte_perm(w[0], w[1], 0x5140), t1 = __byte_perm(w[2], w[3], 0x5140);
    const uint32_t t2 = __byte_perm(w[0], w[1], 0x7362), t3 = __byte_perm(w[2], w[3], 0x7362);
    o[0] = __byte_perm(t0, t1, 0x5410);
    o[1] = __byte_perm(t0, t1, 0x7632);
    o[2] = __byte_perm(t2, t3, 0x5410);
    o[3] = __byte_perm(t2, t3, 0x7632);
}

// Write the warp's 32x128 int8 tile, staged in shared memory (row-major, 128 B per row), transposed to qt[N, M].
// Lane l owns tile columns 4l..4l+3 and emits, per column, two 16-byte stores (rows 0-15 and 16-31).
__device__ __forceinline__ void store_tile_transposed(const uint32_t* tile_words, const Tile& t, int64_t M, int64_t N,
                                                      int8_t* qt) {
    uint32_t colw[4][8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        uint32_t w[4], o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = tile_words[(4 * g + k) * 32 + t.lane];
        transpose4x4(w, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) colw[j][g] = o[j];
    }
    const int64_t c0 = t.tn * TILE_N + 4 * t.lane;
    if (c0 < N) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int4* dst = reinterpret_cast<int4*>(qt + (c0 + j) * M + t.row0);
            dst[0] = make_int4(colw[j][0], colw[j][1], colw[j][2], colw[j][3]);
            dst[1] = make_int4(colw[j][4], colw[j][5], colw[j][6], colw[j][7]);
        }
    }
}

// Quantise the lane's 8x16 values with the block scale `scale32` (= block absmax (+adj) / 127, identical in the 8
// lanes of a block) and store payload + scale.  TRUNC selects the truncating conversion of the residual-add kernels.
template <bool TRUNC, bool TRANSPOSE>
__device__ __forceinline__ void emit_quantized(const float (&v)[8][16], float scale32, const Tile& t, int64_t M, int64_t N,
                                               int8_t* q, __half* s, const SrCfg& sr, uint32_t* tile_words, int8_t* qt) {
    const Divisor d = make_divisor(scale32);
    const bool zero = (scale32 == 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = t.row0 + 4 * i + t.rg;
        uint32_t words[4];
        if (t.active) {
            float nz[16];
            if (sr.stochastic) {
                if (sr.noise) {
                    const float4* np4 = reinterpret_cast<const float4*>(sr.noise + row * N + t.col);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float4 n4 = __ldg(np4 + k);
                        nz[4 * k] = n4.x; nz[4 * k + 1] = n4.y; nz[4 * k + 2] = n4.z; nz[4 * k + 3] = n4.w;
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k) philox_noise4((uint64_t)(row * N + t.col) + 4 * k, sr.seed, sr.offset, &nz[4 * k]);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float x = div_exact(v[i][4 * k + j], d);
                    if (sr.stochastic) x = sr_prestep(x, nz[4 * k + j]);
                    b[j] = TRUNC ? trunc_byte(x) : rne_byte(x);
                }
                words[k] = zero ? 0u : pack4(b[0], b[1], b[2], b[3]);
            }
            *reinterpret_cast<int4*>(q + row * N + t.col) = make_int4(words[0], words[1], words[2], words[3]);
        } else {
            words[0] = words[1] = words[2] = words[3] = 0u;
        }
        if (TRANSPOSE) {
            uint32_t* dst = tile_words + (4 * i + t.rg) * 32 + t.cc * 4;
            *reinterpret_cast<int4*>(dst) = make_int4(words[0], words[1], words[2], words[3]);
        }
    }
    if (t.active && t.rg == 0 && (t.cc & 1) == 0) s[t.tm * (N / QB) + (t.col >> 5)] = __float2half_rn(scale32);
    if (TRANSPOSE) {
        __syncwarp();
        store_tile_transposed(tile_words, t, M, N, qt);
    }
}

__device__ __forceinline__ float absmax_8x16(const float (&v)[8][16]) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 16; ++j) m = fmaxf(m, fabsf(v[i][j]));
    return m;
}

// Load the lane's 8 int8 row chunks (16 B each); inactive lanes get zeros.
__device__ __forceinline__ void load_q(const int8_t* q, const Tile& t, int64_t N, int4 (&raw)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        raw[i] = t.active ? __ldg(reinterpret_cast<const int4*>(q + (t.row0 + 4 * i + t.rg) * N + t.col)) : make_int4(0, 0, 0, 0);
    }
}
__device__ __forceinline__ float load_scale(const __half* s, const Tile& t, int64_t N) {
    return t.active ? __half2float(__ldg(s + t.tm * (N / QB) + (t.col >> 5))) : 0.f;
}
__device__ __forceinline__ int q_at(const int4& r, int j) {
    const uint32_t w = (j < 4) ? (uint32_t)r.x : (j < 8) ? (uint32_t)r.y : (j < 12) ? (uint32_t)r.z : (uint32_t)r.w;
    return sbyte(w, j & 3);
}

// =========================================================================================================
// quantize / quantize_transpose
// =========================================================================================================
template <typename T, bool TRANSPOSE>
__global__ void __launch_bounds__(THREADS) quantize_kernel(const T* __restrict__ x, int64_t M, int64_t N, int8_t* __restrict__ q,
                                                           __half* __restrict__ s, int8_t* __restrict__ qt, SrCfg sr) {
    __shared__ __align__(16) uint32_t smem_tiles[TRANSPOSE ? WARPS * 32 * 32 : 1];
    Tile t;
    if (!tile_setup(M, N, t)) return;
    float v[8][16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (t.active) {
            Load16<T>::load(x + (t.row0 + 4 * i + t.rg) * N + t.col, v[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[i][j] = 0.f;
        }
    }
    const float amax = block_max(absmax_8x16(v));
    const float scale32 = __fdiv_rn(amax, 127.0f);
    emit_quantized<false, TRANSPOSE>(v, scale32, t, M, N, q, s, sr, TRANSPOSE ? smem_tiles + (threadIdx.x >> 5) * 1024 : nullptr, qt);
}

// =========================================================================================================
// dequantize: y = fp32(fp16(q) * s)
// =========================================================================================================
__global__ void __launch_bounds__(THREADS) dequantize_kernel(const int8_t* __restrict__ q, const __half* __restrict__ s, int64_t M,
                                                             int64_t N, float* __restrict__ y) {
    Tile t;
    if (!tile_setup(M, N, t)) return;
    if (!t.active) return;
    int4 raw[8];
    load_q(q, t, N, raw);
    const float sc = load_scale(s, t, N);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float4* dst = reinterpret_cast<float4*>(y + (t.row0 + 4 * i + t.rg) * N + t.col);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float4 o;
            o.x = __half2float(deq16(q_at(raw[i], 4 * k + 0), sc));
            o.y = __half2float(deq16(q_at(raw[i], 4 * k + 1), sc));
            o.z = __half2float(deq16(q_at(raw[i], 4 * k + 2), sc));
            o.w = __half2float(deq16(q_at(raw[i], 4 * k + 3), sc));
            dst[k] = o;
        }
    }
}

// =========================================================================================================
// transpose: y[N, M] = x[M, N]^T (int8)
// =========================================================================================================
__global__ void __launch_bounds__(THREADS) transpose_kernel(const int8_t* __restrict__ x, int64_t M, int64_t N, int8_t* __restrict__ y) {
    __shared__ __align__(16) uint32_t smem_tiles[WARPS * 32 * 32];
    Tile t;
    if (!tile_setup(M, N, t)) return;
    uint32_t* tile_words = smem_tiles + (threadIdx.x >> 5) * 1024;
    int4 raw[8];
    load_q(x, t, N, raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) *reinterpret_cast<int4*>(tile_words + (4 * i + t.rg) * 32 + t.cc * 4) = raw[i];
    __syncwarp();
    store_tile_transposed(tile_words, t, M, N, y);
}

// =========================================================================================================
// GELU forward: x = fp16(q*s); y = x * (1 + erf(x / sqrt(2))) / 2; block quantise with amax + 5e-5
// =========================================================================================================
__device__ __forceinline__ float div_const(float a, float b, float inv_b) {
    // exact RN(a / b) for a compile-time divisor whose correctly rounded reciprocal is inv_b
    const float q0 = __fmul_rn(a, inv_b);
    const float r = __fmaf_rn(-b, q0, a);
    return __fmaf_rn(r, inv_b, q0);
}
#define JF_SQRT2 0x1.6a09e6p+0f        /* RN(sqrt(2)) in fp32        */
#define JF_INV_SQRT2 0x1.6a09e6p-1f    /* RN(1 / JF_SQRT2)           */
#define JF_SQRT2PI 0x1.40d932p+1f      /* RN(sqrt(RN(2*pi))) in fp32 */
#define JF_INV_SQRT2PI 0x1.988454p-2f  /* RN(1 / JF_SQRT2PI)         */

__global__ void __launch_bounds__(THREADS) gelu_fwd_kernel(const int8_t* __restrict__ qx, const __half* __restrict__ sx, int64_t M,
                                                           int64_t N, int8_t* __restrict__ qy, __half* __restrict__ sy) {
    Tile t;
    if (!tile_setup(M, N, t)) return;
    int4 raw[8];
    load_q(qx, t, N, raw);
    const float sc = load_scale(sx, t, N);
    float v[8][16];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float x = __half2float(deq16(q_at(raw[i], j), sc));
            const float e = erff(div_const(x, JF_SQRT2, JF_INV_SQRT2));
            const float cdf = __fmul_rn(__fadd_rn(1.0f, e), 0.5f);
            v[i][j] = __fmul_rn(cdf, x);
        }
    const float amax = __fadd_rn(block_max(absmax_8x16(v)), 5e-5f);
    const float scale32 = __fdiv_rn(amax, 127.0f);
    SrCfg sr{0, nullptr, 0, 0};
    emit_quantized<false, false>(v, scale32, t, M, N, qy, sy, sr, nullptr, nullptr);
}

// =========================================================================================================
// GELU backward: x = q*s, g = qg*sg in fp32; d = (Phi(x) + x*phi(x)) * g; block quantise (+SR)
// =========================================================================================================
__global__ void __launch_bounds__(THREADS) gelu_bwd_kernel(const int8_t* __restrict__ qx, const __half* __restrict__ sx,
                                                           const int8_t* __restrict__ qg, const __half* __restrict__ sg, int64_t M,
                                                           int64_t N, int8_t* __restrict__ qd, __half* __restrict__ sd, SrCfg sr) {
    Tile t;
    if (!tile_setup(M, N, t)) return;
    int4 rx[8], rg_[8];
    load_q(qx, t, N, rx);
    load_q(qg, t, N, rg_);
    const float scx = load_scale(sx, t, N), scg = load_scale(sg, t, N);
    float v[8][16];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float x = __fmul_rn((float)q_at(rx[i], j), scx);
            const float g = __fmul_rn((float)q_at(rg_[i], j), scg);
            const float cdf = __fmul_rn(0.5f, __fadd_rn(1.0f, erff(div_const(x, JF_SQRT2, JF_INV_SQRT2))));
            const float ex = expf(__fmul_rn(-__fmul_rn(x, x), 0.5f));
            const float pdf = __fmul_rn(div_const(x, JF_SQRT2PI, JF_INV_SQRT2PI), ex);
            v[i][j] = __fmul_rn(__fadd_rn(cdf, pdf), g);
        }
    const float amax = block_max(absmax_8x16(v));
    const float scale32 = __fdiv_rn(amax, 127.0f);
    emit_quantized<false, false>(v, scale32, t, M, N, qd, sd, sr, nullptr, nullptr);
}

// =========================================================================================================
// LayerNorm forward: y = ((fp16(q*s) - mean) * rstd) * gamma; statistics are inputs
// =========================================================================================================
__global__ void __launch_bounds__(THREADS) ln_fwd_kernel(const int8_t* __restrict__ qx, const __half* __restrict__ sx,
                                                         const float* __restrict__ gamma, const float* __restrict__ mean,
                                                         const float* __restrict__ rstd, int64_t M, int64_t N, int8_t* __restrict__ qy,
                                                         __half* __restrict__ sy) {
    Tile t;
    if (!tile_setup(M, N, t)) return;
    int4 raw[8];
    load_q(qx, t, N, raw);
    const float sc = load_scale(sx, t, N);
    float gm[16];
    if (t.active) {
        Load16<float>::load(gamma + t.col, gm);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) gm[j] = 0.f;
    }
    float v[8][16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = t.row0 + 4 * i + t.rg;
        const float mu = __ldg(mean + row), rs = __ldg(rstd + row);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float x = __half2float(deq16(q_at(raw[i], j), sc));
            const float xhat = __fmul_rn(__fsub_rn(x, mu), rs);
            v[i][j] = __fadd_rn(__fmul_rn(xhat, gm[j]), 0.0f);
        }
    }
    const float amax = block_max(absmax_8x16(v));
    const float scale32 = __fdiv_rn(amax, 127.0f);
    SrCfg sr{0, nullptr, 0, 0};
    emit_quantized<false, false>(v, scale32, t, M, N, qy, sy, sr, nullptr, nullptr);
}

// =========================================================================================================
// LayerNorm backward (dx and per-32-row partial dgamma), row reductions over the tile's 128-column slab
// =========================================================================================================
__global__ void __launch_bounds__(THREADS) ln_bwd_kernel(const int8_t* __restrict__ qx, const __half* __restrict__ sx,
                                                         const int8_t* __restrict__ qg, const __half* __restrict__ sg,
                                                         const float* __restrict__ gamma, const float* __restrict__ mean,
                                                         const float* __restrict__ rstd, int64_t M, int64_t N, int8_t* __restrict__ qd,
                                                         __half* __restrict__ sd, float* __restrict__ dw_partial, SrCfg sr) {
    Tile t;
    if (!tile_setup(M, N, t)) return;
    int4 rx[8], rgr[8];
    load_q(qx, t, N, rx);
    load_q(qg, t, N, rgr);
    const float scx = load_scale(sx, t, N), scg = load_scale(sg, t, N);
    float gm[16];
    if (t.active) {
        Load16<float>::load(gamma + t.col, gm);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) gm[j] = 0.f;
    }
    const float invN_den = (float)N;
    float v[8][16];     // dx, rounded to fp16 and widened
    float dwp[16];      // partial dgamma over this lane's 8 rows
#pragma unroll
    for (int j = 0; j < 16; ++j) dwp[j] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = t.row0 + 4 * i + t.rg;
        const __half mu16 = __float2half_rn(__ldg(mean + row));
        const __half rs16 = __float2half_rn(__ldg(rstd + row));
        const float rs = __half2float(rs16);
        float xh[16], wdy[16];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const __half x16 = deq16(q_at(rx[i], j), scx);
            const __half dy16 = deq16(q_at(rgr[i], j), scg);
            const __half xhat16 = __hmul(__hsub(x16, mu16), rs16);
            xh[j] = __half2float(xhat16);
            const float dy = __half2float(dy16);
            wdy[j] = __fmul_rn(gm[j], dy);
            s1 = __fadd_rn(s1, __fmul_rn(xh[j], wdy[j]));
            s2 = __fadd_rn(s2, wdy[j]);
            dwp[j] = __fadd_rn(dwp[j], __half2float(__hmul(dy16, xhat16)));
        }
        // row sums over the 128-column slab: the 8 lanes sharing rg
        s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, 1)); s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, 1));
        s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, 2)); s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, 2));
        s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, 4)); s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, 4));
        const float c1 = __fdiv_rn(s1, invN_den), c2 = __fdiv_rn(s2, invN_den);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float tt = __fadd_rn(__fmul_rn(xh[j], c1), c2);
            const float dx = __fmul_rn(__fsub_rn(wdy[j], tt), rs);
            v[i][j] = __half2float(__float2half_rn(dx));
        }
    }
    // partial dgamma: reduce the four row groups, lanes with rg == 0 write 16 columns
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float a = dwp[j];
        a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 8));
        a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 16));
        dwp[j] = a;
    }
    if (t.active && t.rg == 0) {
        float4* dst = reinterpret_cast<float4*>(dw_partial + t.tm * N + t.col);
#pragma unroll
        for (int k = 0; k < 4; ++k) dst[k] = make_float4(dwp[4 * k], dwp[4 * k + 1], dwp[4 * k + 2], dwp[4 * k + 3]);
    }
    const float amax = block_max(absmax_8x16(v));   // exactly representable in fp16
    const float scale32 = __fdiv_rn(amax, 127.0f);
    emit_quantized<false, false>(v, scale32, t, M, N, qd, sd, sr, nullptr, nullptr);
}

// dgamma[n] = sum over the M/32 partial rows, ascending
__global__ void ln_bwd_dw_kernel(const float* __restrict__ partial, int64_t rows, int64_t N, float* __restrict__ dgamma) {
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float a = 0.f;
    for (int64_t r = 0; r < rows; ++r) a = __fadd_rn(a, partial[r * N + n]);
    dgamma[n] = a;
}

// =========================================================================================================
// residual add (+ optional row statistics): y = x1 + q2*s2 (fp32); store y; block quantise y by truncation
// =========================================================================================================
template <typename T, bool MEANVAR>
__global__ void __launch_bounds__(THREADS) add_kernel(const T* __restrict__ x1, const int8_t* __restrict__ q2,
                                                      const __half* __restrict__ s2, int64_t M, int64_t N, float* __restrict__ y1,
                                                      int8_t* __restrict__ qy, __half* __restrict__ sy, float* __restrict__ part_sum,
                                                      float* __restrict__ part_sq, SrCfg sr) {
    Tile t;
    if (!tile_setup(M, N, t)) return;
    int4 raw[8];
    load_q(q2, t, N, raw);
    const float sc = load_scale(s2, t, N);
    const int64_t tiles_n = (N + TILE_N - 1) / TILE_N;
    float v[8][16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = t.row0 + 4 * i + t.rg;
        if (t.active) {
            Load16<T>::load(x1 + row * N + t.col, v[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[i][j] = 0.f;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = t.row0 + 4 * i + t.rg;
        float ps = 0.f, pq = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float y = __fadd_rn(v[i][j], __fmul_rn((float)q_at(raw[i], j), sc));
            v[i][j] = y;
            if (MEANVAR) {
                ps = __fadd_rn(ps, y);
                pq = __fadd_rn(pq, __fmul_rn(y, y));
            }
        }
        if (t.active) {
            float4* dst = reinterpret_cast<float4*>(y1 + row * N + t.col);
#pragma unroll
            for (int k = 0; k < 4; ++k) dst[k] = make_float4(v[i][4 * k], v[i][4 * k + 1], v[i][4 * k + 2], v[i][4 * k + 3]);
        }
        if (MEANVAR) {
            ps = __fadd_rn(ps, __shfl_xor_sync(0xffffffffu, ps, 1)); pq = __fadd_rn(pq, __shfl_xor_sync(0xffffffffu, pq, 1));
            ps = __fadd_rn(ps, __shfl_xor_sync(0xffffffffu, ps, 2)); pq = __fadd_rn(pq, __shfl_xor_sync(0xffffffffu, pq, 2));
            ps = __fadd_rn(ps, __shfl_xor_sync(0xffffffffu, ps, 4)); pq = __fadd_rn(pq, __shfl_xor_sync(0xffffffffu, pq, 4));
            if (t.cc == 0) {
                part_sum[row * tiles_n + t.tn] = ps;
                part_sq[row * tiles_n + t.tn] = pq;
            }
        }
    }
    const float amax = block_max(absmax_8x16(v));
    const float scale32 = __fdiv_rn(amax, 127.0f);
    emit_quantized<true, false>(v, scale32, t, M, N, qy, sy, sr, nullptr, nullptr);
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

static inline int check_mn(int64_t M, int64_t N) { return (mult32(M) && mult32(N)) ? JF_OK : JF_ERR_SHAPE; }

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
    SrCfg sr{stochastic, noise, seed, offset};
    const unsigned grid = grid_for(M, N);
    __half* sh = (__half*)s;
#define JF_LAUNCH_Q(T)                                                                                   \
    if (qt) quantize_kernel<T, true><<<grid, THREADS, 0, st>>>((const T*)x, M, N, q, sh, qt, sr);        \
    else quantize_kernel<T, false><<<grid, THREADS, 0, st>>>((const T*)x, M, N, q, sh, nullptr, sr);
    switch (x_dtype) {
        case JF_F32: JF_LAUNCH_Q(float) break;
        case JF_F16: JF_LAUNCH_Q(__half) break;
        case JF_BF16: JF_LAUNCH_Q(__nv_bfloat16) break;
        default: return JF_ERR_DTYPE;
    }
#undef JF_LAUNCH_Q
    return check_launch();
}

int jf_int8_dequantize(const int8_t* q, const void* s, int64_t M, int64_t N, float* y, void* stream) {
    JF_REQUIRE_PTR(q); JF_REQUIRE_PTR(s); JF_REQUIRE_PTR(y);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(q); JF_REQUIRE_ALIGNED(y);
    dequantize_kernel<<<grid_for(M, N), THREADS, 0, (cudaStream_t)stream>>>(q, (const __half*)s, M, N, y);
    return check_launch();
}

int jf_int8_transpose(const int8_t* x, int64_t M, int64_t N, int8_t* y, void* stream) {
    JF_REQUIRE_PTR(x); JF_REQUIRE_PTR(y);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(x); JF_REQUIRE_ALIGNED(y);
    transpose_kernel<<<grid_for(M, N), THREADS, 0, (cudaStream_t)stream>>>(x, M, N, y);
    return check_launch();
}

int jf_int8_gelu_forward(const int8_t* qx, const void* sx, int64_t M, int64_t N, int8_t* qy, void* sy, void* stream) {
    JF_REQUIRE_PTR(qx); JF_REQUIRE_PTR(sx); JF_REQUIRE_PTR(qy); JF_REQUIRE_PTR(sy);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(qx); JF_REQUIRE_ALIGNED(qy);
    gelu_fwd_kernel<<<grid_for(M, N), THREADS, 0, (cudaStream_t)stream>>>(qx, (const __half*)sx, M, N, qy, (__half*)sy);
    return check_launch();
}

int jf_int8_gelu_backward(const int8_t* qx, const void* sx, const int8_t* qg, const void* sg, int64_t M, int64_t N, int8_t* qd,
                          void* sd, int stochastic, const float* noise, uint64_t seed, uint64_t offset, void* stream) {
    JF_REQUIRE_PTR(qx); JF_REQUIRE_PTR(sx); JF_REQUIRE_PTR(qg); JF_REQUIRE_PTR(sg); JF_REQUIRE_PTR(qd); JF_REQUIRE_PTR(sd);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(qx); JF_REQUIRE_ALIGNED(qg); JF_REQUIRE_ALIGNED(qd);
    if (noise) JF_REQUIRE_ALIGNED(noise);
    SrCfg sr{stochastic, noise, seed, offset};
    gelu_bwd_kernel<<<grid_for(M, N), THREADS, 0, (cudaStream_t)stream>>>(qx, (const __half*)sx, qg, (const __half*)sg, M, N, qd,
                                                                          (__half*)sd, sr);
    return check_launch();
}

int jf_int8_layernorm_forward(const int8_t* qx, const void* sx, const float* gamma, const float* mean, const float* rstd, int64_t M,
                              int64_t N, int8_t* qy, void* sy, void* stream) {
    JF_REQUIRE_PTR(qx); JF_REQUIRE_PTR(sx); JF_REQUIRE_PTR(gamma); JF_REQUIRE_PTR(mean); JF_REQUIRE_PTR(rstd);
    JF_REQUIRE_PTR(qy); JF_REQUIRE_PTR(sy);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(qx); JF_REQUIRE_ALIGNED(qy); JF_REQUIRE_ALIGNED(gamma);
    ln_fwd_kernel<<<grid_for(M, N), THREADS, 0, (cudaStream_t)stream>>>(qx, (const __half*)sx, gamma, mean, rstd, M, N, qy,
                                                                        (__half*)sy);
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
    if (slab != TILE_N) return JF_ERR_ARG;         // only the reference's 128-column slab is implemented
    if (N % TILE_N != 0) return JF_ERR_SHAPE;
    JF_REQUIRE_ALIGNED(qx); JF_REQUIRE_ALIGNED(qg); JF_REQUIRE_ALIGNED(qd); JF_REQUIRE_ALIGNED(gamma); JF_REQUIRE_ALIGNED(scratch);
    if (noise) JF_REQUIRE_ALIGNED(noise);
    cudaStream_t st = (cudaStream_t)stream;
    SrCfg sr{stochastic, noise, seed, offset};
    ln_bwd_kernel<<<grid_for(M, N), THREADS, 0, st>>>(qx, (const __half*)sx, qg, (const __half*)sg, gamma, mean, rstd, M, N, qd,
                                                      (__half*)sd, scratch, sr);
    if (int e = check_launch()) return e;
    ln_bwd_dw_kernel<<<(unsigned)((N + 127) / 128), 128, 0, st>>>(scratch, M / QB, N, dgamma);
    return check_launch();
}

static int add_impl(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N, float* y1, int8_t* qy,
                    void* sy, float* mean, float* rstd, float* scratch, bool meanvar, SrCfg sr, cudaStream_t st) {
    JF_REQUIRE_PTR(x1); JF_REQUIRE_PTR(q2); JF_REQUIRE_PTR(s2); JF_REQUIRE_PTR(y1); JF_REQUIRE_PTR(qy); JF_REQUIRE_PTR(sy);
    if (int e = check_mn(M, N)) return e;
    JF_REQUIRE_ALIGNED(x1); JF_REQUIRE_ALIGNED(q2); JF_REQUIRE_ALIGNED(y1); JF_REQUIRE_ALIGNED(qy);
    if (sr.noise) JF_REQUIRE_ALIGNED(sr.noise);
    const int64_t tiles_n = (N + TILE_N - 1) / TILE_N;
    float* ps = nullptr;
    float* pq = nullptr;
    if (meanvar) {
        JF_REQUIRE_PTR(mean); JF_REQUIRE_PTR(rstd); JF_REQUIRE_PTR(scratch);
        ps = scratch;
        pq = scratch + M * tiles_n;
    }
    const unsigned grid = grid_for(M, N);
    const __half* s2h = (const __half*)s2;
    __half* syh = (__half*)sy;
#define JF_LAUNCH_ADD(T)                                                                                        \
    if (meanvar) add_kernel<T, true><<<grid, THREADS, 0, st>>>((const T*)x1, q2, s2h, M, N, y1, qy, syh, ps, pq, sr); \
    else add_kernel<T, false><<<grid, THREADS, 0, st>>>((const T*)x1, q2, s2h, M, N, y1, qy, syh, ps, pq, sr);
    switch (x1_dtype) {
        case JF_F32: JF_LAUNCH_ADD(float) break;
        case JF_F16: JF_LAUNCH_ADD(__half) break;
        case JF_BF16: JF_LAUNCH_ADD(__nv_bfloat16) break;
        default: return JF_ERR_DTYPE;
    }
#undef JF_LAUNCH_ADD
    if (int e = check_launch()) return e;
    if (meanvar) {
        meanvar_finish_kernel<<<(unsigned)((M + 127) / 128), 128, 0, st>>>(ps, pq, M, tiles_n, N, mean, rstd);
        return check_launch();
    }
    return JF_OK;
}

int jf_int8_add(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N, float* y1, int8_t* qy, void* sy,
                int stochastic, const float* noise, uint64_t seed, uint64_t offset, void* stream) {
    SrCfg sr{stochastic, noise, seed, offset};
    return add_impl(x1, x1_dtype, q2, s2, M, N, y1, qy, sy, nullptr, nullptr, nullptr, false, sr, (cudaStream_t)stream);
}

int jf_int8_add_meanvar(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N, float* y1, int8_t* qy,
                        void* sy, float* mean, float* rstd, float* scratch, void* stream) {
    SrCfg sr{0, nullptr, 0, 0};
    return add_impl(x1, x1_dtype, q2, s2, M, N, y1, qy, sy, mean, rstd, scratch, true, sr, (cudaStream_t)stream);
}

}  // extern "C"
