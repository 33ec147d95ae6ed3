/*
 * CPU oracle for the per-block (32x32) INT8 GEMM path.  TEST INFRASTRUCTURE ONLY: nothing in the
 * product package links or calls this file; it is the checker for the CUDA kernels and the timed
 * CPU baseline.
 *
 * It restates, in IEEE arithmetic (no fast-math), the algorithm of the reference's three GEMM kernels
 * (paths relative to the reference project root):
 *   main loop   JetfireGEMMKernel/BlockQuantize/cpp_extension/igemm/igemm_BlockSquare32OutputIntQuantizeBiasRowCol.cu:134-225
 *               per 32-wide K block p:  I_p = A_blk * B_blk^T in int32,  acc += (sa*sb) * I_p   (fp32, fused multiply-add)
 *   forward     ...BiasRowCol.cu:294-370   amax = max|acc| (+biasmax), q = clamp(rn(127*(acc+bias)/amax), -127, 127),
 *                                          scale = half(amax/127)
 *   dgrad       ...igemm_BlockSquare32OutputIntQuantizeStochastic.cu:311-365   q = rn(127*acc/amax + noise)
 *   wgrad       ...igemm_BlockSquare32OutputFp.cu:309-336                      out = half(acc)
 * and the naive CPU loop of JetfireGEMMKernel/cppsrc/igemm/igemm_BlockSquare32OutputFp/compute.cu:22-40.
 *
 * The reference draws its dgrad noise from curand seeded by libc rand(); that stream is not reproducible,
 * so the noise here is passed in by the caller (tests generate it with the oracle's Philox, which the CUDA
 * kernels implement identically).
 *
 * Operands are addressed with element strides so one routine covers the three layouts:
 *   A(m,k) = A[m*a_sm + k*a_sk],  B(n,k) = B[n*b_sn + k*b_sk],
 *   SA(i,p) = SA[i*sa_si + p*sa_sp],  SB(j,p) = SB[j*sb_sj + p*sb_sp]     (fp16 bit patterns)
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QB 32

static inline float h2f(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f2h(float f) {
    _Float16 v = (_Float16)f; /* round-to-nearest-even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

/* acc[M,N] (row-major fp32) = sum over K blocks p in [p_begin, p_end) in ascending order of
 * fmaf(sa*sb, (float)I_p, acc).  acc must be initialised by the caller (zeros for a fresh GEMM). */
void jf_oracle_gemm_accumulate(const int8_t* A, int64_t a_sm, int64_t a_sk,
                               const int8_t* B, int64_t b_sn, int64_t b_sk,
                               const uint16_t* SA, int64_t sa_si, int64_t sa_sp,
                               const uint16_t* SB, int64_t sb_sj, int64_t sb_sp,
                               float* acc, int64_t M, int64_t N, int64_t K,
                               int64_t p_begin, int64_t p_end) {
    const int64_t MB = M / QB, NB = N / QB;
    (void)K;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < MB; ++i) {
        for (int64_t j = 0; j < NB; ++j) {
            int16_t a16[QB][QB], b16[QB][QB];
            float tile[QB][QB];
            for (int r = 0; r < QB; ++r)
                for (int c = 0; c < QB; ++c) tile[r][c] = acc[(i * QB + r) * N + j * QB + c];
            for (int64_t p = p_begin; p < p_end; ++p) {
                for (int r = 0; r < QB; ++r)
                    for (int k = 0; k < QB; ++k) a16[r][k] = A[(i * QB + r) * a_sm + (p * QB + k) * a_sk];
                for (int c = 0; c < QB; ++c)
                    for (int k = 0; k < QB; ++k) b16[c][k] = B[(j * QB + c) * b_sn + (p * QB + k) * b_sk];
                /* product of two fp16 values is exact in fp32 */
                const float s = h2f(SA[i * sa_si + p * sa_sp]) * h2f(SB[j * sb_sj + p * sb_sp]);
                for (int r = 0; r < QB; ++r) {
                    for (int c = 0; c < QB; ++c) {
                        int32_t I = 0;
                        for (int k = 0; k < QB; ++k) I += (int32_t)a16[r][k] * (int32_t)b16[c][k];
                        tile[r][c] = fmaf(s, (float)I, tile[r][c]);
                    }
                }
            }
            for (int r = 0; r < QB; ++r)
                for (int c = 0; c < QB; ++c) acc[(i * QB + r) * N + j * QB + c] = tile[r][c];
        }
    }
}

/* Plain int32 block product C = A * B^T over the whole K (the reference's igemm_basic_int8_gemm,
 * .../igemm/igemm_BasicInt8Gemm.cu:14-110). */
void jf_oracle_gemm_int32(const int8_t* A, int64_t a_sm, int64_t a_sk,
                          const int8_t* B, int64_t b_sn, int64_t b_sk,
                          int32_t* C, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            int32_t s = 0;
            for (int64_t k = 0; k < K; ++k) s += (int32_t)A[m * a_sm + k * a_sk] * (int32_t)B[n * b_sn + k * b_sk];
            C[m * N + n] = s;
        }
}

/* Per-32x32-block re-quantisation of acc.
 *   noise == NULL : q = clamp(rint((127*acc)/amax), -127, 127)               (forward epilogue, bias = 0)
 *   noise != NULL : q = clamp(rint((127*acc)/amax + noise), -127, 127)       (dgrad epilogue)
 * scale = fp16(amax/127); an all-zero block gives q = 0, scale = 0.
 * If deq != NULL it additionally receives fp16(q) * scale evaluated in fp16 (the "output_quantized=False" /
 * "dgrad_quantize=False" path of Jetfire/Linear/linear_fwd.py:30 and linear_bwd.py:27). */
void jf_oracle_requant(const float* acc, int64_t M, int64_t N, const float* noise,
                       int8_t* q, uint16_t* scale, uint16_t* deq) {
    const int64_t MB = M / QB, NB = N / QB;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < MB; ++i)
        for (int64_t j = 0; j < NB; ++j) {
            float amax = 0.f;
            for (int r = 0; r < QB; ++r)
                for (int c = 0; c < QB; ++c) amax = fmaxf(amax, fabsf(acc[(i * QB + r) * N + j * QB + c]));
            const uint16_t sh = f2h(amax / 127.0f);
            scale[i * NB + j] = sh;
            for (int r = 0; r < QB; ++r)
                for (int c = 0; c < QB; ++c) {
                    const int64_t idx = (i * QB + r) * N + j * QB + c;
                    float v = (127.0f * acc[idx]) / amax;
                    if (noise) v = v + noise[idx];
                    float rr = rintf(v); /* round-half-even in the default rounding mode */
                    int qi = (rr != rr) ? 0 : (rr > 127.f ? 127 : (rr < -127.f ? -127 : (int)rr));
                    q[idx] = (int8_t)qi;
                    if (deq) deq[idx] = f2h((float)qi * h2f(sh));
                }
        }
}

/* fp32 -> fp16 dense output (wgrad epilogue). */
void jf_oracle_to_half(const float* acc, int64_t count, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) out[i] = f2h(acc[i]);
}

/* Fixed-order reduction of split-K partial accumulators: out = ((p0 + p1) + p2) + ... */
void jf_oracle_sum_partials(const float* partials, int64_t splits, int64_t count, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        float s = partials[i];
        for (int64_t k = 1; k < splits; ++k) s = s + partials[k * count + i];
        out[i] = s;
    }
}

/* Thread control for the timed CPU baseline: launchers such as torchrun export OMP_NUM_THREADS=1, which would silently turn the
 * "all host cores" baseline into a single-threaded one. */
void jf_oracle_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int jf_oracle_max_threads(void) { return omp_get_max_threads(); }

/* RN(a / b) by the sequence the CUDA kernels use for their re-quantising divisions (Markstein's correction step with the
 * correctly rounded reciprocal):  y = RN(1/b);  q0 = RN(a*y);  r = fma(-b, q0, a);  q = fma(r, y, q0).
 * Exposed so that a CPU test can compare it with the IEEE quotient on hard operands. */
float jf_oracle_markstein_div(float a, float b) {
    const float y = 1.0f / b;
    const float q0 = a * y;
    const float r = fmaf(-b, q0, a);
    return fmaf(r, y, q0);
}
/* Number of mismatches between the sequence above and a / b over `count` pairs (arrays a, b). */
int64_t jf_oracle_markstein_mismatches(const float* a, const float* b, int64_t count) {
    int64_t bad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        const float q = jf_oracle_markstein_div(a[i], b[i]);
        const float want = a[i] / b[i];
        uint32_t uq, uw;
        memcpy(&uq, &q, 4);
        memcpy(&uw, &want, 4);
        bad += (uq != uw);
    }
    return bad;
}
/* The same, for ONE divisor and every dividend mantissa: dividends m * 2^e for all 2^23 mantissas m in [2^23, 2^24). */
int64_t jf_oracle_markstein_sweep_mantissas(float b, int e) {
    int64_t bad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (int64_t m = (1 << 23); m < (1 << 24); ++m) {
        const float a = ldexpf((float)m, e);
        const float q = jf_oracle_markstein_div(a, b);
        const float want = a / b;
        uint32_t uq, uw;
        memcpy(&uq, &q, 4);
        memcpy(&uw, &want, 4);
        bad += (uq != uw);
    }
    return bad;
}
