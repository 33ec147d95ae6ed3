// Cross-entropy of the language-model head without an fp32 copy of the logits (sm_100a).
//
// The caller of the INT8 path ends in  logits = x W_vocab^T  (bf16, [tokens, vocab]) followed by a softmax cross-entropy
// (reference: INT8_GPT2/qmodel.py:433-439).  Done with framework operators that is a widening copy of the logits to fp32, a
// log-softmax pass that reads and writes them, a backward pass that does so again and a narrowing copy -- about 20 bytes per
// logit through HBM for a tensor of 0.6 G logits per step of GPT-2 124M.  Here:
//   forward : one read of the bf16 logits; per row an online (max, sum of exp) reduction, loss_row = logsumexp - logit[target];
//   backward: one read + one write, IN PLACE: logit <- (exp(logit - logsumexp) - [col == target]) * scale, as bf16,
// 2 + 4 bytes per logit.  One CTA per row; a thread owns 16-byte chunks (8 logits) at a stride of the CTA width.
// All arithmetic is fp32 on the bf16 values (exp via exp2f of a pre-scaled argument).
#include <cuda_bf16.h>

#include "jf_common.cuh"

namespace jf {

constexpr int LM_THREADS = 512;

__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        f[2 * j] = __uint_as_float(w[j] << 16);
        f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
}

// (m, s) <- merge of two partial (max, sum exp(x - max)) pairs
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
    const float mn = fmaxf(m, m2);
    s = s * exp2f((m - mn) * 1.4426950408889634f) + s2 * exp2f((m2 - mn) * 1.4426950408889634f);
    m = mn;
}

__device__ __forceinline__ void block_lse(float& m, float& s) {
    __shared__ float sm[LM_THREADS / 32], ss[LM_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lse_merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sm[warp] = m; ss[warp] = s; }
    __syncthreads();
    m = sm[0]; s = ss[0];
    for (int w = 1; w < LM_THREADS / 32; ++w) lse_merge(m, s, sm[w], ss[w]);
}

// per row: lse[row] = log sum exp(logits[row, :]);  loss[row] = lse - logits[row, target]   (0 for an ignored target < 0)
__global__ void __launch_bounds__(LM_THREADS) lm_loss_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                                int64_t V, float* __restrict__ lse, float* __restrict__ loss) {
    const int64_t row = blockIdx.x;
    const __nv_bfloat16* x = logits + row * V;
    float m = -INFINITY, s = 0.f;
    const int64_t chunks = V / 8;
    for (int64_t c = threadIdx.x; c < chunks; c += LM_THREADS) {
        float f[8];
        bf16x8_to_float(__ldg(reinterpret_cast<const uint4*>(x) + c), f);
        float cm = f[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
        const float mn = fmaxf(m, cm);
        float acc = s * exp2f((m - mn) * 1.4426950408889634f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += exp2f((f[j] - mn) * 1.4426950408889634f);
        m = mn; s = acc;
    }
    for (int64_t i = chunks * 8 + threadIdx.x; i < V; i += LM_THREADS) {      // tail when V is not a multiple of 8
        const float v = __bfloat162float(x[i]);
        lse_merge(m, s, v, 1.f);
    }
    if (m == -INFINITY) { m = -3.0e38f; s = 0.f; }     // a thread without any element
    block_lse(m, s);
    if (threadIdx.x == 0) {
        const float l = m + logf(s);
        lse[row] = l;
        const int64_t t = targets[row];
        loss[row] = (t >= 0 && t < V) ? l - __bfloat162float(x[t]) : 0.f;
    }
}

// in place: logits[row, c] <- (exp(logits[row, c] - lse[row]) - [c == target]) * (*grad_out) * inv_count   (0 for an ignored row)
__global__ void __launch_bounds__(LM_THREADS) lm_loss_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                                const float* __restrict__ lse, const float* __restrict__ grad_out,
                                                                float inv_count, int64_t V) {
    const int64_t row = blockIdx.x;
    __nv_bfloat16* x = logits + row * V;
    const int64_t t = targets[row];
    const bool live = t >= 0 && t < V;
    const float scale = live ? __ldg(grad_out) * inv_count : 0.f;
    const float l2 = lse[row] * 1.4426950408889634f;
    const int64_t chunks = V / 8;
    for (int64_t c = threadIdx.x; c < chunks; c += LM_THREADS) {
        float f[8];
        uint4* p = reinterpret_cast<uint4*>(x) + c;
        bf16x8_to_float(*p, f);
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float g = exp2f(__fmaf_rn(f[j], 1.4426950408889634f, -l2));
            if (c * 8 + j == t) g -= 1.f;
            f[j] = g * scale;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *p = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (int64_t i = chunks * 8 + threadIdx.x; i < V; i += LM_THREADS) {
        float g = exp2f(__fmaf_rn(__bfloat162float(x[i]), 1.4426950408889634f, -l2));
        if (i == t) g -= 1.f;
        x[i] = __float2bfloat16_rn(g * scale);
    }
}

}  // namespace jf

using namespace jf;

extern "C" {

int jf_lm_loss_forward(const void* logits_bf16, const int64_t* targets, int64_t rows, int64_t V, float* lse, float* loss_rows,
                       void* stream) {
    if (!logits_bf16 || !targets || !lse || !loss_rows) return JF_ERR_NULL;
    if (rows <= 0 || V <= 0 || rows >= (int64_t(1) << 31)) return JF_ERR_SHAPE;
    if (!aligned16(logits_bf16) || (V % 8 != 0 && rows > 1)) return JF_ERR_ALIGN;     // every row must start on a 16-byte boundary
    lm_loss_fwd_kernel<<<(unsigned)rows, LM_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits_bf16, targets, V, lse, loss_rows);
    return check_launch();
}

int jf_lm_loss_backward(void* logits_bf16, const int64_t* targets, const float* lse, const float* grad_out, float inv_count,
                        int64_t rows, int64_t V, void* stream) {
    if (!logits_bf16 || !targets || !lse || !grad_out) return JF_ERR_NULL;
    if (rows <= 0 || V <= 0 || rows >= (int64_t(1) << 31)) return JF_ERR_SHAPE;
    if (!aligned16(logits_bf16) || (V % 8 != 0 && rows > 1)) return JF_ERR_ALIGN;
    lm_loss_bwd_kernel<<<(unsigned)rows, LM_THREADS, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits_bf16, targets, lse, grad_out, inv_count, V);
    return check_launch();
}

}  // extern "C"
