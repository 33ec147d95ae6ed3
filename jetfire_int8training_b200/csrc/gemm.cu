// Per-block (32x32) quantised INT8 GEMMs for sm_100a: forward Y = X W^T, input gradient dX = dY W and weight gradient
// dW = dY^T X, all from one persistent, warp-specialised kernel (gemm_kernel.cuh).
//
// Algorithm (fixed by the reference and its oracle): for every 32-wide K block p, in ascending order,
//     I_p = A_blk x B_blk^T  (exact int32),      acc = fma(sa[i,p] * sb[j,p], float(I_p), acc)   (fp32)
// followed by a per-32x32-block re-quantisation (or a dense fp16/fp32 store) of acc.
//
// Mapping to the hardware
//   * CTA tile 128 x 128, one CTA per SM, persistent over a static list of (tile, K-split) work items.
//   * 19 warps: 16 consumers, 1 TMA producer (one lane), 2 MMA issuers (one lane each).
//   * producer: a 128-byte-swizzled 128 x 128 B box per operand per stage = four K blocks; a 4-stage mbarrier ring (128 KB).
//   * issuers: tcgen05.mma kind::i8 has K = 32 = one quantisation block, so every K block is ONE 128x128x32 MMA with
//     accumulation disabled.  Tensor memory (512 columns) holds two groups of two 128-column accumulators; the four K blocks
//     of a stage form two pairs, pair g goes to group g and is issued by issuer g with one tcgen05.commit.
//   * consumers: warp w reads TMEM lanes 32*(w%4).. (rows) and columns 32*(w/4).. of every accumulator with tcgen05.ld (a
//     thread = one row of one quantisation block), converts int32 -> fp32 and does the scale FMA into 32 fp32 registers.  This
//     CUDA-core work, not the tensor core, bounds the kernel.  Scale products are fetched one per lane for 8 K blocks at a
//     time and broadcast by shuffle.
//   * operands are consumed in place in either orientation: K-major (row-major [rows, K]) or MN-major (row-major
//     [K, rows]) through the UMMA descriptor major bits, so no transposed copy of W, dY or X is ever materialised.
//   * epilogue: a 32x32 block = 32 lanes x 32 thread-local values; absmax is a local max + one redux.sync.
// Every mbarrier wait is bounded by a clock budget; on expiry the CTA raises an error flag (read with jf_igemm_error_flag),
// leaves its loops, waits (bounded) for its copies and MMAs in flight and frees its tensor memory.
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "jf_common.cuh"
#include "ptx_sm100.cuh"

namespace jf {

constexpr int BM = 128, BN = 128;
constexpr int KB_PER_STAGE = 4;                 // 32-wide K blocks per pipeline stage (128 bytes of K)
constexpr int STAGES = 4;
constexpr int STAGE_BYTES = 128 * 128;          // one operand tile
constexpr int TMEM_COLS = 512;
constexpr size_t GEMM_SMEM = 2 * STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr size_t GEMM_SMEM_F16OPS = 2 * 3 * 2 * STAGE_BYTES + 1024 + 256;   // three stages of two boxes per operand
constexpr long long DRAIN_BUDGET_CLOCKS = 20000000LL;   // ~10 ms: abort-path wait for copies / MMAs already in flight
constexpr long long WAIT_BUDGET_CLOCKS = 4000000000LL;  // ~2 s at 2 GHz

enum GemmMode : int {
    MODE_INT8 = 0,      // int8 payload + fp16 scales
    MODE_DEQ16 = 1,     // fp16(q) * scale
    MODE_F16 = 2,       // dense fp16(acc)
    MODE_F32 = 3,       // dense fp32 acc (also used for split-K partials)
    MODE_INT32 = 4      // plain int32 accumulation (diagnostic)
};

struct GemmParams {
    int64_t M, N, K;
    int64_t tiles_m, tiles_n;
    int64_t nkb;            // K / 32
    int64_t splits;         // number of K ranges
    int64_t kb_per_split;   // K blocks per range (last may be shorter)
    const __half* sa; int64_t sa_sm, sa_sk;   // sa(i,p) = sa[i*sa_sm + p*sa_sk]
    const __half* sb; int64_t sb_sn, sb_sk;   // sb(j,p) = sb[j*sb_sn + p*sb_sk]
    int mode;
    int8_t* out8; __half* out_scale; __half* out16; float* out32; int32_t* out_i32;
    int stochastic; const float* noise; uint64_t offset; PhiloxKeys keys;
};

__device__ int g_gemm_error = 0;   // 0 = ok; otherwise the code of the first wait that expired

// Wait for a barrier phase, giving up after WAIT_BUDGET_CLOCKS.  SUSPEND = true (producer and issuer warps): every try lets the
// hardware park the thread for up to 2 us; SUSPEND = false (consumers): plain try_wait polling.  (An additional __nanosleep of
// 40-250 ns between the tries of the producer / issuer warps measured 2-4 % slower.)
template <bool SUSPEND = false>
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if (SUSPEND ? ptx::mbar_try_wait_hint(bar, parity, 2000u) : ptx::mbar_try_wait(bar, parity)) return true;
        if ((it & (SUSPEND ? 31u : 255u)) == (SUSPEND ? 31u : 255u)) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_BUDGET_CLOCKS) {
                *abort_flag = code;
                atomicCAS(&g_gemm_error, 0, code);
                return false;
            }
        }
    }
}

// Abort path: wait for a barrier phase that operations already in flight will complete, without touching the abort state.
__device__ __forceinline__ void drain_wait(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!ptx::mbar_try_wait_hint(bar, parity, 2000u))
        if (clock64() - t0 > DRAIN_BUDGET_CLOCKS) break;
}

// ---------------------------------------------------------------------------------------------------------
// Consumer arithmetic.  acc is kept as packed pairs of fp32 so the scale FMA can use the two-wide fma.rn.f32x2.
// int32 -> fp32 (cvt.rn.f32.s32) is exact: |I| <= 32*127^2 < 2^22.  (Building the float with an integer add of 0x4B400000 and
// a subtraction of 1.5*2^23 instead, for all or for every other pair, measured slower: the add runs on the same pipe.)
// CONV_INT32 adds the raw integers instead: the plain int32 GEMM behind jf_igemm_int32.
// ---------------------------------------------------------------------------------------------------------
enum ConvMode : int { CONV_I2F = 0, CONV_INT32 = 1, CONV_F16OPS = 2 };

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// acc2[j] (16 packed pairs) += s * float(r[2j], r[2j+1]) for the 32 int32 values in r
template <int CONV>
__device__ __forceinline__ void scale_accumulate(uint64_t (&acc2)[16], const uint32_t (&r)[32], float s) {
    if (CONV == CONV_INT32) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t lo = (uint32_t)acc2[j] + r[2 * j], hi = (uint32_t)(acc2[j] >> 32) + r[2 * j + 1];
            acc2[j] = ((uint64_t)hi << 32) | lo;
        }
        return;
    }
    const uint64_t s2 = pack2(s, s);
    if constexpr (CONV == CONV_F16OPS) {      // the accumulator already holds float(I_p)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc2[j] = fma2(s2, pack2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), acc2[j]);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            acc2[j] = fma2(s2, pack2(__int2float_rn((int)r[2 * j]), __int2float_rn((int)r[2 * j + 1])), acc2[j]);
    }
}

// Re-quantise / convert one 32x32 block held as 32 lanes x 32 values and store it.
__device__ __forceinline__ void store_block(const GemmParams& p, const float (&ab)[32], int64_t row, int64_t col, int64_t rowblk,
                                            int64_t colblk, int64_t split, int lane) {
    if (p.mode == MODE_INT32) {
        int4* dst = reinterpret_cast<int4*>(p.out_i32 + row * p.N + col);
#pragma unroll
        for (int k = 0; k < 8; ++k)
            dst[k] = make_int4(__float_as_int(ab[4 * k]), __float_as_int(ab[4 * k + 1]), __float_as_int(ab[4 * k + 2]), __float_as_int(ab[4 * k + 3]));
    } else if (p.mode == MODE_F32) {
        float4* dst = reinterpret_cast<float4*>(p.out32 + (split * p.M + row) * p.N + col);
#pragma unroll
        for (int k = 0; k < 8; ++k) dst[k] = make_float4(ab[4 * k], ab[4 * k + 1], ab[4 * k + 2], ab[4 * k + 3]);
    } else if (p.mode == MODE_F16) {
        int4* dst = reinterpret_cast<int4*>(p.out16 + row * p.N + col);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __half2 h[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) h[u] = __floats2half2_rn(ab[8 * k + 2 * u], ab[8 * k + 2 * u + 1]);
            dst[k] = *reinterpret_cast<int4*>(h);
        }
    } else {
        float m = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) m = fmaxf(m, fabsf(ab[j]));
        const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m)));
        const __half sc16 = __float2half_rn(__fdiv_rn(amax, 127.0f));
        const Divisor d = make_divisor(amax);
        const bool zero = (amax == 0.f);
        uint32_t words[8];
        // One decision per warp each: the exact-quotient fast path is valid for the whole block (same divisor in every lane),
        // and only stochastic rounding can leave [-127, 127] (127 + noise -> 128), so only it needs the clamp.
        const bool fast = __all_sync(0xffffffffu, d.fast || zero);
        auto quantise_all = [&](auto fast_c, auto sr_c) {
            constexpr bool FAST = decltype(fast_c)::value, SRND = decltype(sr_c)::value;
#pragma unroll
            for (int k8 = 0; k8 < 4; ++k8) {      // 8 elements = one Philox call
                float nz[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (SRND) {
                    if (p.noise) {
                        const float4 n0 = __ldg(reinterpret_cast<const float4*>(p.noise + row * p.N + col + 8 * k8));
                        const float4 n1 = __ldg(reinterpret_cast<const float4*>(p.noise + row * p.N + col + 8 * k8 + 4));
                        nz[0] = n0.x; nz[1] = n0.y; nz[2] = n0.z; nz[3] = n0.w; nz[4] = n1.x; nz[5] = n1.y; nz[6] = n1.z; nz[7] = n1.w;
                    } else {
                        philox_noise8((uint64_t)(row * p.N + col + 8 * k8), p.keys, p.offset, nz);
                    }
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t bts[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float a127 = __fmul_rn(127.0f, ab[8 * k8 + 4 * h + u]);
                        float v;
                        if (FAST) {
                            const float q0 = __fmul_rn(a127, d.inv);
                            v = __fmaf_rn(__fmaf_rn(-d.b, q0, a127), d.inv, q0);
                        } else {
                            v = __fdiv_rn(a127, d.b);
                        }
                        if (SRND) v = fminf(fmaxf(__fadd_rn(v, nz[4 * h + u]), -127.f), 127.f);
                        bts[u] = __float_as_uint(__fadd_rn(v, 12582912.0f));     // round to nearest even; the low byte is the payload
                    }
                    words[2 * k8 + h] = zero ? 0u : __byte_perm(__byte_perm(bts[0], bts[1], 0x0040), __byte_perm(bts[2], bts[3], 0x0040), 0x5410);
                }
            }
        };
        using T_ = std::true_type; using F_ = std::false_type;
        if (fast) { if (p.stochastic) quantise_all(T_{}, T_{}); else quantise_all(T_{}, F_{}); }
        else      { if (p.stochastic) quantise_all(F_{}, T_{}); else quantise_all(F_{}, F_{}); }
        if (p.mode == MODE_INT8) {
            int4* dst = reinterpret_cast<int4*>(p.out8 + row * p.N + col);
            dst[0] = make_int4(words[0], words[1], words[2], words[3]);
            dst[1] = make_int4(words[4], words[5], words[6], words[7]);
            if (lane == 0) p.out_scale[rowblk * (p.N / QB) + colblk] = sc16;
        } else {   // MODE_DEQ16
            const float scf = __half2float(sc16);
            int4* dst = reinterpret_cast<int4*>(p.out16 + row * p.N + col);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                __half h[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) h[u] = deq16(sbyte(words[2 * k + (u >> 2)], u & 3), scf);
                dst[k] = *reinterpret_cast<int4*>(h);
            }
        }
    }
}

#include "gemm_kernel.cuh"

// out[i] = ((p0[i] + p1[i]) + p2[i]) + ...   then converted to the output type
template <typename OutT>
__global__ void splitk_reduce_kernel(const float* __restrict__ partials, int64_t splits, int64_t count, OutT* __restrict__ out) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= count) return;
    float4 a = *reinterpret_cast<const float4*>(partials + i);
    for (int64_t k = 1; k < splits; ++k) {
        const float4 b = *reinterpret_cast<const float4*>(partials + k * count + i);
        a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y); a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
    }
    if constexpr (sizeof(OutT) == 4) {
        *reinterpret_cast<float4*>(out + i) = a;
    } else {
        __half2 h[2] = {__floats2half2_rn(a.x, a.y), __floats2half2_rn(a.z, a.w)};
        *reinterpret_cast<uint2*>(out + i) = *reinterpret_cast<uint2*>(h);
    }
}

// ------------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// 2-D uint8 tensor [outer, inner] with row pitch `pitch` bytes; box 128 x 128, 128-byte swizzle, zero fill outside.
static int make_map(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t pitch) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return JF_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch};
    const cuuint32_t box[2] = {128, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return JF_ERR_LAUNCH;
    }
    return JF_OK;
}

// 2-D fp16 tensor [outer, inner]: box 64 elements (128 B) x 128 rows, 128-byte swizzle, zero fill outside.
static int make_map_f16(CUtensorMap* map, const void* base, int64_t inner, int64_t outer) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return JF_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    const cuuint64_t strides[1] = {(cuuint64_t)(inner * 2)};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return JF_ERR_LAUNCH;
    }
    return JF_OK;
}

// exact fp16 copy of an int8 tensor (16 elements per thread)
__global__ void int8_to_f16_kernel(const int8_t* __restrict__ q, int64_t count16, __half* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count16) return;
    const int4 v = __ldg(reinterpret_cast<const int4*>(q) + i);
    const uint32_t w[4] = {(uint32_t)v.x ^ 0x80808080u, (uint32_t)v.y ^ 0x80808080u, (uint32_t)v.z ^ 0x80808080u, (uint32_t)v.w ^ 0x80808080u};
    const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
    uint32_t o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = __byte_perm(w[k], 0x64646464u, 0x5140), hi = __byte_perm(w[k], 0x64646464u, 0x5342);
        const __half2 a = __hsub2_rn(*reinterpret_cast<const __half2*>(&lo), bias), b = __hsub2_rn(*reinterpret_cast<const __half2*>(&hi), bias);
        o[2 * k] = *reinterpret_cast<const uint32_t*>(&a); o[2 * k + 1] = *reinterpret_cast<const uint32_t*>(&b);
    }
    uint4* dst = reinterpret_cast<uint4*>(out) + 2 * i;
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// exact fp16 copy of the TRANSPOSE of an int8 tensor: q [R, C] row-major -> out [C, R] row-major.  A CTA moves a 128 x 128 tile
// through shared memory (16-byte chunks XOR-permuted per 16-row group, so that the column reads are bank-conflict free); a thread
// gathers a 16-row x 4-column patch, transposes it with byte permutes and writes 16 fp16 (32 bytes) of each of 4 output rows:
// 8 neighbouring threads complete 256 contiguous bytes.
__global__ void __launch_bounds__(256) int8_to_f16_transposed_kernel(const int8_t* __restrict__ q, int64_t R, int64_t C, __half* __restrict__ out) {
    __shared__ __align__(16) uint32_t tile[128 * 128 / 4];
    const int64_t R0 = (int64_t)blockIdx.y * 128, C0 = (int64_t)blockIdx.x * 128;
    const int t = threadIdx.x;
    {
        const int chunk = t & 7;
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int row = (t >> 3) + 32 * pass;
            int4 v = make_int4(0, 0, 0, 0);
            if (R0 + row < R && C0 + 16 * chunk < C) v = __ldg(reinterpret_cast<const int4*>(q + (R0 + row) * C + C0 + 16 * chunk));
            *reinterpret_cast<int4*>(tile + row * 32 + 4 * (chunk ^ ((row >> 4) & 7))) = v;
        }
    }
    __syncthreads();
    const int warp = t >> 5, lane = t & 31;
    const int i = lane & 7, cg = 4 * warp + (lane >> 3);
    if (R0 + 16 * i >= R || C0 + 4 * cg >= C) return;
    const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
    uint32_t colw[4][4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = tile[(16 * i + 4 * g + k) * 32 + 4 * ((cg >> 2) ^ i) + (cg & 3)];
        // 4x4 byte transpose: colw[j][g] = rows 4g..4g+3 of column j
        const uint32_t t0 = __byte_perm(w[0], w[1], 0x5140), t1 = __byte_perm(w[2], w[3], 0x5140);
        const uint32_t t2 = __byte_perm(w[0], w[1], 0x7362), t3 = __byte_perm(w[2], w[3], 0x7362);
        colw[0][g] = __byte_perm(t0, t1, 0x5410); colw[1][g] = __byte_perm(t0, t1, 0x7632);
        colw[2][g] = __byte_perm(t2, t3, 0x5410); colw[3][g] = __byte_perm(t2, t3, 0x7632);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t o[8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t wx = colw[j][g] ^ 0x80808080u;
            const uint32_t lo = __byte_perm(wx, 0x64646464u, 0x5140), hi = __byte_perm(wx, 0x64646464u, 0x5342);
            const __half2 a = __hsub2_rn(*reinterpret_cast<const __half2*>(&lo), bias), b = __hsub2_rn(*reinterpret_cast<const __half2*>(&hi), bias);
            o[2 * g] = *reinterpret_cast<const uint32_t*>(&a); o[2 * g + 1] = *reinterpret_cast<const uint32_t*>(&b);
        }
        uint4* dst = reinterpret_cast<uint4*>(out + (C0 + 4 * cg + j) * R + R0 + 16 * i);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

// Fill the fp16 operand copies of one GEMM: a16 [M,K] from a ([M,K], or [K,M] when a_transposed), b16 [N,K] likewise.
static int fill_f16_operands(const int8_t* a, bool a_transposed, const int8_t* b, bool b_transposed, int64_t M, int64_t N, int64_t K,
                             __half* a16, __half* b16, cudaStream_t st) {
    auto one = [&](const int8_t* src, bool transposed, int64_t rows, __half* dst) {     // dst [rows, K]
        if (transposed) {   // src is [K, rows]
            const dim3 grid((unsigned)((rows + 127) / 128), (unsigned)((K + 127) / 128));
            int8_to_f16_transposed_kernel<<<grid, 256, 0, st>>>(src, K, rows, dst);
        } else {
            const int64_t n16 = rows * K / 16;
            int8_to_f16_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, st>>>(src, n16, dst);
        }
    };
    if ((K + 127) / 128 > 65535) return JF_ERR_SHAPE;
    one(a, a_transposed, M, a16);
    one(b, b_transposed, N, b16);
    return check_launch();
}

struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    bool attr_set[32] = {};
};
static DeviceInfo g_dev[64];
static std::mutex g_dev_mutex;

static int device_info(DeviceInfo** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return JF_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if (d.sm_count == 0) {
        cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    }
    *out = &d;
    return d.cc_major == 10 ? JF_OK : JF_ERR_UNSUPPORTED;
}

#include "gemm_launch.inc"

static int plan_splits(int64_t M, int64_t N, int64_t K, int split_k, int sm_count, int64_t* per_out) {
    const int64_t nkb = K / QB;
    int64_t s = split_k;
    if (s <= 0) {
        const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
        s = sm_count / tiles;
        const int64_t cap = nkb / 16;   // keep at least 16 K blocks per range
        if (s > cap) s = cap;
        if (s < 1) s = 1;
    }
    if (s > nkb) s = nkb;
    const int64_t per = (nkb + s - 1) / s;
    if (per_out) *per_out = per;
    return (int)((nkb + per - 1) / per);
}

}  // namespace jf

using namespace jf;

// the fp16-operand path is taken when the caller handed in enough scratch for both operand copies
static inline bool use_op16(const void* op16, int64_t op16_bytes, int64_t M, int64_t N, int64_t K) {
    return op16 != nullptr && aligned16(op16) && op16_bytes >= 2 * (M * K + N * K);
}

static inline int check_gemm_dims(int64_t M, int64_t N, int64_t K) {
    if (!mult32(M) || !mult32(N) || !mult32(K)) return JF_ERR_SHAPE;
    if (M > (1LL << 30) || N > (1LL << 30) || K > (1LL << 30)) return JF_ERR_SHAPE;
    return JF_OK;
}

extern "C" {

int jf_igemm_forward(const int8_t* x, const int8_t* w, const void* sx, int64_t sx_stride_m, int64_t sx_stride_k, const void* sw,
                     int64_t sw_stride_n, int64_t sw_stride_k, int64_t M, int64_t N, int64_t K, int out_mode, int8_t* y8, void* sy,
                     void* y16, void* op16, int64_t op16_bytes, void* stream) {
    if (!x || !w || !sx || !sw) return JF_ERR_NULL;
    if (int e = check_gemm_dims(M, N, K)) return e;
    if (!aligned16(x) || !aligned16(w)) return JF_ERR_ALIGN;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.splits = 1; p.kb_per_split = K / QB;
    p.sa = (const __half*)sx; p.sa_sm = sx_stride_m; p.sa_sk = sx_stride_k;
    p.sb = (const __half*)sw; p.sb_sn = sw_stride_n; p.sb_sk = sw_stride_k;
    if (out_mode == JF_OUT_INT8) {
        if (!y8 || !sy) return JF_ERR_NULL;
        if (!aligned16(y8)) return JF_ERR_ALIGN;
        p.mode = MODE_INT8; p.out8 = y8; p.out_scale = (__half*)sy;
    } else if (out_mode == JF_OUT_DEQUANT_F16) {
        if (!y16) return JF_ERR_NULL;
        if (!aligned16(y16)) return JF_ERR_ALIGN;
        p.mode = MODE_DEQ16; p.out16 = (__half*)y16;
    } else {
        return JF_ERR_ARG;
    }
    if (use_op16(op16, op16_bytes, M, N, K)) {
        __half* a16 = (__half*)op16;
        __half* b16 = a16 + M * K;
        if (int e = fill_f16_operands(x, false, w, false, M, N, K, a16, b16, (cudaStream_t)stream)) return e;
        return launch_f16ops(a16, b16, p, (cudaStream_t)stream);
    }
    return launch_fwd(x, w, p, (cudaStream_t)stream);
}

/* Bytes of fp16 operand scratch a GEMM with these dimensions needs for the fp16-operand path (2 * (M*K + N*K)), or 0 when that
 * path is not expected to pay for its conversion passes.  Model: the kernel saves ~20 % of a GEMM that runs at ~630e12 ops/s; the
 * passes move 3 bytes per operand element at ~5e12 B/s plus two launches. */
int64_t jf_igemm_op16_bytes(int64_t M, int64_t N, int64_t K) {
    if (check_gemm_dims(M, N, K)) return 0;
    const double gain = 0.2 * 2.0 * (double)M * (double)N * (double)K / 630e12;
    const double cost = 3.0 * ((double)M * K + (double)N * K) / 5e12 + 4e-6;
    return gain > 1.5 * cost ? 2 * (M * K + N * K) : 0;
}

int jf_igemm_dgrad(const int8_t* g, const int8_t* w, const void* sg, int64_t sg_stride_m, int64_t sg_stride_k, const void* sw,
                   int64_t sw_stride_k, int64_t sw_stride_n, int64_t M, int64_t N, int64_t K, int out_mode, int8_t* dx8, void* sdx,
                   void* dx16, int stochastic, const float* noise, uint64_t seed, uint64_t offset, void* op16, int64_t op16_bytes,
                   void* stream) {
    if (!g || !w || !sg || !sw) return JF_ERR_NULL;
    if (int e = check_gemm_dims(M, N, K)) return e;
    if (!aligned16(g) || !aligned16(w) || (noise && !aligned16(noise))) return JF_ERR_ALIGN;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.splits = 1; p.kb_per_split = K / QB;
    p.sa = (const __half*)sg; p.sa_sm = sg_stride_m; p.sa_sk = sg_stride_k;
    p.sb = (const __half*)sw; p.sb_sn = sw_stride_n; p.sb_sk = sw_stride_k;
    p.stochastic = stochastic; p.noise = noise; p.keys = make_philox_keys(seed); p.offset = offset;
    if (out_mode == JF_OUT_INT8) {
        if (!dx8 || !sdx) return JF_ERR_NULL;
        if (!aligned16(dx8)) return JF_ERR_ALIGN;
        p.mode = MODE_INT8; p.out8 = dx8; p.out_scale = (__half*)sdx;
    } else if (out_mode == JF_OUT_DEQUANT_F16) {
        if (!dx16) return JF_ERR_NULL;
        if (!aligned16(dx16)) return JF_ERR_ALIGN;
        p.mode = MODE_DEQ16; p.out16 = (__half*)dx16;
    } else {
        return JF_ERR_ARG;
    }
    if (use_op16(op16, op16_bytes, M, N, K)) {
        __half* a16 = (__half*)op16;
        __half* b16 = a16 + M * K;
        if (int e = fill_f16_operands(g, false, w, true, M, N, K, a16, b16, (cudaStream_t)stream)) return e;
        return launch_f16ops(a16, b16, p, (cudaStream_t)stream);
    }
    return launch_dgrad_layout(g, w, p, (cudaStream_t)stream);
}

int jf_igemm_wgrad_plan(int64_t M, int64_t N, int64_t K, int split_k) {
    if (check_gemm_dims(M, N, K)) return JF_ERR_SHAPE;
    int sm = 148;
    DeviceInfo* di = nullptr;
    if (device_info(&di) == JF_OK) sm = di->sm_count;
    return plan_splits(M, N, K, split_k, sm, nullptr);
}

int jf_igemm_wgrad(const int8_t* g, int g_transposed, const int8_t* x, const void* sg, int64_t sg_stride_k, int64_t sg_stride_m,
                   const void* sx, int64_t sx_stride_k, int64_t sx_stride_n, int64_t M, int64_t N, int64_t K, int out_dtype, void* dw,
                   int split_k, float* scratch, void* op16, int64_t op16_bytes, void* stream) {
    if (!g || !x || !sg || !sx || !dw) return JF_ERR_NULL;
    if (int e = check_gemm_dims(M, N, K)) return e;
    if (!aligned16(g) || !aligned16(x) || !aligned16(dw)) return JF_ERR_ALIGN;
    if (out_dtype != JF_F16 && out_dtype != JF_F32) return JF_ERR_DTYPE;
    DeviceInfo* di = nullptr;
    if (int e = device_info(&di)) return e;
    int64_t per = 0;
    const int splits = plan_splits(M, N, K, split_k, di->sm_count, &per);
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.splits = splits; p.kb_per_split = per;
    p.sa = (const __half*)sg; p.sa_sm = sg_stride_m; p.sa_sk = sg_stride_k;
    p.sb = (const __half*)sx; p.sb_sn = sx_stride_n; p.sb_sk = sx_stride_k;
    cudaStream_t st = (cudaStream_t)stream;
    const bool f16 = use_op16(op16, op16_bytes, M, N, K);
    __half* a16 = (__half*)op16;
    __half* b16 = f16 ? a16 + M * K : nullptr;
    if (f16)
        if (int e = fill_f16_operands(g, !g_transposed, x, true, M, N, K, a16, b16, st)) return e;
    auto launch = [&]() { return f16 ? launch_f16ops(a16, b16, p, st) : (g_transposed ? launch_dgrad_layout(g, x, p, st) : launch_wgrad_layout(g, x, p, st)); };
    if (splits == 1) {
        if (out_dtype == JF_F16) { p.mode = MODE_F16; p.out16 = (__half*)dw; }
        else { p.mode = MODE_F32; p.out32 = (float*)dw; }
        return launch();
    }
    if (!scratch) return JF_ERR_NULL;
    if (!aligned16(scratch)) return JF_ERR_ALIGN;
    p.mode = MODE_F32; p.out32 = scratch;
    if (int e = launch()) return e;
    const int64_t count = M * N;
    const unsigned grid = (unsigned)((count / 4 + 255) / 256);
    if (out_dtype == JF_F16) splitk_reduce_kernel<__half><<<grid, 256, 0, st>>>(scratch, splits, count, (__half*)dw);
    else splitk_reduce_kernel<float><<<grid, 256, 0, st>>>(scratch, splits, count, (float*)dw);
    return check_launch();
}

int jf_igemm_int32(const int8_t* a, const int8_t* b, int64_t M, int64_t N, int64_t K, int32_t* c, void* stream) {
    if (!a || !b || !c) return JF_ERR_NULL;
    if (int e = check_gemm_dims(M, N, K)) return e;
    if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return JF_ERR_ALIGN;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.splits = 1; p.kb_per_split = K / QB;
    p.mode = MODE_INT32; p.out_i32 = c;
    return launch_int32(a, b, p, (cudaStream_t)stream);
}

/* Reads (and clears) the device-side error flag raised when a bounded wait inside the GEMM kernel expired.
 * Synchronises the device.  0 = no error. */
int jf_igemm_error_flag(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return JF_ERR_LAUNCH;
    if (v != 0) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

}  // extern "C"
