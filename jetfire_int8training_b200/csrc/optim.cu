// Gradient clipping by global norm + AdamW in two passes over the gradients and one over the optimiser state (sm_100a).
//
// The caller of the INT8 path ends every step with  clip_grad_norm_(params, max_norm); AdamW.step()  (reference:
// INT8_GPT2/train.py:320-329).  With framework operators that is: one norm kernel per tensor, a norm of norms, a scaling pass that
// reads and writes every gradient, and the optimiser pass -- 36 bytes per parameter through HBM and a few hundred launches.  Here:
//   pass 1: sum of squares of every gradient (read 4 B / parameter), one partial per 4096-element chunk, reduced in a fixed order;
//   pass 2: p, m, v <- AdamW(p, m, v, g * coef) with coef = min(1, max_norm / (norm + 1e-6)) / loss scale, read from device memory
//           (read 16 B, write 12 B / parameter) -- the clipped gradient is never written.
// Parameters, first and second moments live in three flat fp32 buffers in which tensor t occupies elements
// [4096 * start_chunk[t], 4096 * start_chunk[t] + numel[t]); the gradients stay where autograd put them and are passed as a pointer
// per tensor.  The per-tensor tables travel in the kernel parameters (at most ADAMW_MAX_TENSORS per launch; the host entry point
// loops).  A CTA owns one chunk and finds its tensor by bisection over start_chunk.
//
// Loss scaling (the reference trains in fp16 with torch's GradScaler, init_scale 2^24: INT8_GPT2/train.py:216-217, 320-327): the
// gradients arrive multiplied by the loss scale.  Its state lives in device memory (`state`, 8 floats: [0] scale, [1] steps since
// the scale last changed, [2] optimiser steps taken, [3] norm of the unscaled gradients, [4] factor applied to the raw gradients =
// clip factor / scale, [5] 1 if this call found a non-finite gradient, [6] lr / (1 - beta1^t), [7] sqrt(1 - beta2^t)): the
// one-CTA kernel between the two passes unscales the norm, decides whether the step is skipped (non-finite gradients: scale *=
// backoff, nothing else changes) and grows the scale after `growth_interval` good steps, as GradScaler does -- without a host
// synchronisation.  scale = 1 with growth_interval = 0 is plain training without loss scaling.
//
// Arithmetic (fp32, the same expressions as torch.optim.AdamW, whose scalar factors are formed in double precision on the host and
// rounded to fp32 once): p *= 1 - lr * wd;  m += (g - m) * (1 - beta1);  v = beta2 * v + (1 - beta2) * g * g;
// p -= (lr / bc1) * (m / (sqrt(v) / sqrt(bc2) + eps)),  bc_i = 1 - beta_i^step.
#include "jf_common.cuh"

namespace jf {

constexpr int ADAMW_CHUNK = 4096;
constexpr int ADAMW_THREADS = 256;
constexpr int ADAMW_MAX_TENSORS = 160;

struct AdamwTensors {
    const float* grad[ADAMW_MAX_TENSORS];
    int32_t start_chunk[ADAMW_MAX_TENSORS + 1];   // relative to the launch's first chunk; [count] = number of chunks of the launch
    int32_t numel[ADAMW_MAX_TENSORS];
    float decay[ADAMW_MAX_TENSORS];               // 1 - lr * weight_decay of the tensor
    int32_t count;
};

__device__ __forceinline__ int find_tensor(const AdamwTensors& ts, int chunk) {
    int lo = 0, hi = ts.count;          // start_chunk[lo] <= chunk < start_chunk[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (ts.start_chunk[mid] <= chunk) lo = mid; else hi = mid;
    }
    return lo;
}

// partial[first_chunk + blockIdx.x] = sum of g^2 over the chunk: per thread four float4 in index order, then a shuffle tree, then
// the eight warp sums in order -- a fixed order, so the norm is deterministic.
__global__ void __launch_bounds__(ADAMW_THREADS) grad_sumsq_kernel(const AdamwTensors ts, int64_t first_chunk, float* __restrict__ partial) {
    __shared__ float warp_sum[ADAMW_THREADS / 32];
    const int t = find_tensor(ts, (int)blockIdx.x);
    const int off = ((int)blockIdx.x - ts.start_chunk[t]) * ADAMW_CHUNK;
    const int n = min(ADAMW_CHUNK, ts.numel[t] - off);
    const float4* g = reinterpret_cast<const float4*>(ts.grad[t] + off);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < ADAMW_CHUNK / 4 / ADAMW_THREADS; ++k) {
        const int i = k * ADAMW_THREADS + threadIdx.x;
        if (4 * i < n) {
            const float4 v = __ldg(g + i);
            s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = warp_sum[0];
#pragma unroll
        for (int w = 1; w < ADAMW_THREADS / 32; ++w) a += warp_sum[w];
        partial[first_chunk + blockIdx.x] = a;
    }
}

struct AdamwScalars {
    double lr, beta1, beta2, max_norm, growth_factor, backoff_factor;
    int64_t growth_interval;      // 0: the scale never grows
};

// One CTA: global norm from the partials, loss-scale bookkeeping, and the per-step scalars of the update (see `state` above).
__global__ void __launch_bounds__(1024) grad_norm_finish_kernel(const float* __restrict__ partial, int64_t count, const AdamwScalars h,
                                                               float* __restrict__ state) {
    __shared__ double red[1024];
    double a = 0.0;
    for (int64_t i = threadIdx.x; i < count; i += 1024) a += (double)partial[i];
    red[threadIdx.x] = a;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const double sumsq = red[0];
        const float scale = state[0];
        const bool bad = !isfinite(sumsq) || !(scale > 0.f);
        state[5] = bad ? 1.f : 0.f;
        if (bad) {
            state[0] = (float)((double)scale * h.backoff_factor);
            state[1] = 0.f;
            state[3] = (float)sqrt(sumsq) / scale;
            state[4] = 0.f;
            return;
        }
        const float norm = (float)(sqrt(sumsq) / (double)scale);
        const float clip = h.max_norm > 0.0 ? fminf(1.f, (float)h.max_norm / (norm + 1e-6f)) : 1.f;
        const double step = (double)state[2] + 1.0;
        state[2] = (float)step;
        state[3] = norm;
        state[4] = clip / scale;
        state[6] = (float)(h.lr / (1.0 - pow(h.beta1, step)));
        state[7] = (float)sqrt(1.0 - pow(h.beta2, step));
        float tracker = state[1] + 1.f;
        if (h.growth_interval > 0 && tracker >= (float)h.growth_interval) {
            state[0] = (float)((double)scale * h.growth_factor);
            tracker = 0.f;
        }
        state[1] = tracker;
    }
}

struct AdamwHyper {
    float one_minus_beta1, beta2, one_minus_beta2, eps;
};

__global__ void __launch_bounds__(ADAMW_THREADS) adamw_kernel(const AdamwTensors ts, int64_t first_chunk, float* __restrict__ p_flat,
                                                             float* __restrict__ m_flat, float* __restrict__ v_flat,
                                                             const float* __restrict__ state, const AdamwHyper h) {
    if (__ldg(state + 5) != 0.f) return;      // non-finite gradients: the step is skipped
    const int t = find_tensor(ts, (int)blockIdx.x);
    const int off = ((int)blockIdx.x - ts.start_chunk[t]) * ADAMW_CHUNK;
    const int n = min(ADAMW_CHUNK, ts.numel[t] - off);
    const float4* g4 = reinterpret_cast<const float4*>(ts.grad[t] + off);
    const int64_t base = (first_chunk + blockIdx.x) * ADAMW_CHUNK;
    float4* p4 = reinterpret_cast<float4*>(p_flat + base);
    float4* m4 = reinterpret_cast<float4*>(m_flat + base);
    float4* v4 = reinterpret_cast<float4*>(v_flat + base);
    const float coef = __ldg(state + 4), step_size = __ldg(state + 6), sqrt_bc2 = __ldg(state + 7);
    const float decay = ts.decay[t];
    const float omb1 = h.one_minus_beta1, omb2 = h.one_minus_beta2;
#pragma unroll
    for (int k = 0; k < ADAMW_CHUNK / 4 / ADAMW_THREADS; ++k) {
        const int i = k * ADAMW_THREADS + threadIdx.x;
        if (4 * i >= n) continue;
        const float4 gv = __ldg(g4 + i);
        float4 pv = p4[i], mv = m4[i], vv = v4[i];
        const float g[4] = {gv.x * coef, gv.y * coef, gv.z * coef, gv.w * coef};
        float p[4] = {pv.x, pv.y, pv.z, pv.w}, m[4] = {mv.x, mv.y, mv.z, mv.w}, v[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            p[j] *= decay;
            m[j] += (g[j] - m[j]) * omb1;
            v[j] = h.beta2 * v[j] + omb2 * g[j] * g[j];
            const float denom = __fdiv_rn(__fsqrt_rn(v[j]), sqrt_bc2) + h.eps;
            p[j] -= step_size * __fdiv_rn(m[j], denom);
        }
        p4[i] = make_float4(p[0], p[1], p[2], p[3]);
        m4[i] = make_float4(m[0], m[1], m[2], m[3]);
        v4[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

}  // namespace jf

using namespace jf;

extern "C" {

int64_t jf_adamw_chunk_elements(void) { return ADAMW_CHUNK; }

int jf_adamw_clip_step(int64_t n_tensors, const void* const* grads, const int64_t* numel, const int64_t* start_chunk,
                       const float* weight_decay, float* params_flat, float* m_flat, float* v_flat, int64_t total_chunks,
                       double lr, double beta1, double beta2, double eps, double max_norm, float* state, int64_t growth_interval,
                       double growth_factor, double backoff_factor, float* partial, void* stream) {
    if (!grads || !numel || !start_chunk || !weight_decay || !params_flat || !m_flat || !v_flat || !partial || !state) return JF_ERR_NULL;
    if (n_tensors <= 0 || total_chunks <= 0 || total_chunks >= (int64_t(1) << 31) || growth_interval < 0) return JF_ERR_SHAPE;
    if (!aligned16(params_flat) || !aligned16(m_flat) || !aligned16(v_flat)) return JF_ERR_ALIGN;
    for (int64_t t = 0; t < n_tensors; ++t) {
        if (!grads[t]) return JF_ERR_NULL;
        if (!aligned16(grads[t])) return JF_ERR_ALIGN;
        if (numel[t] <= 0 || numel[t] % 4 != 0 || numel[t] >= (int64_t(1) << 31)) return JF_ERR_SHAPE;
        const int64_t next = t + 1 < n_tensors ? start_chunk[t + 1] : total_chunks;
        if (start_chunk[t] < 0 || (next - start_chunk[t]) * ADAMW_CHUNK < numel[t]) return JF_ERR_SHAPE;   // segments must not overlap
    }
    cudaStream_t st = (cudaStream_t)stream;
    AdamwHyper h;
    h.one_minus_beta1 = (float)(1.0 - beta1); h.beta2 = (float)beta2; h.one_minus_beta2 = (float)(1.0 - beta2); h.eps = (float)eps;
    AdamwScalars sc;
    sc.lr = lr; sc.beta1 = beta1; sc.beta2 = beta2; sc.max_norm = max_norm; sc.growth_factor = growth_factor;
    sc.backoff_factor = backoff_factor; sc.growth_interval = growth_interval;
    // launches of at most ADAMW_MAX_TENSORS tensors; a launch covers exactly the chunks that hold numbers (the padding chunks
    // between two segments, if any, belong to no launch)
    auto for_groups = [&](auto&& launch) -> int {
        for (int64_t t0 = 0; t0 < n_tensors; t0 += ADAMW_MAX_TENSORS) {
            const int64_t cnt = n_tensors - t0 < ADAMW_MAX_TENSORS ? n_tensors - t0 : ADAMW_MAX_TENSORS;
            AdamwTensors ts{};
            ts.count = (int32_t)cnt;
            const int64_t first = start_chunk[t0];
            int64_t last = first;
            for (int64_t i = 0; i < cnt; ++i) {
                ts.grad[i] = (const float*)grads[t0 + i];
                ts.start_chunk[i] = (int32_t)(start_chunk[t0 + i] - first);
                ts.numel[i] = (int32_t)numel[t0 + i];
                ts.decay[i] = (float)(1.0 - lr * (double)weight_decay[t0 + i]);
                last = start_chunk[t0 + i] + (numel[t0 + i] + ADAMW_CHUNK - 1) / ADAMW_CHUNK;
            }
            ts.start_chunk[cnt] = (int32_t)(last - first);
            // the segments of one launch must be back to back (no padding chunk inside it)
            for (int64_t i = 0; i + 1 < cnt; ++i)
                if (start_chunk[t0 + i] + (numel[t0 + i] + ADAMW_CHUNK - 1) / ADAMW_CHUNK != start_chunk[t0 + i + 1]) return JF_ERR_SHAPE;
            launch(ts, first, (unsigned)(last - first));
            if (int e = check_launch()) return e;
        }
        return JF_OK;
    };
    if (cudaMemsetAsync(partial, 0, (size_t)total_chunks * sizeof(float), st) != cudaSuccess) return JF_ERR_LAUNCH;
    if (int e = for_groups([&](const AdamwTensors& ts, int64_t first, unsigned chunks) {
            grad_sumsq_kernel<<<chunks, ADAMW_THREADS, 0, st>>>(ts, first, partial);
        })) return e;
    grad_norm_finish_kernel<<<1, 1024, 0, st>>>(partial, total_chunks, sc, state);
    if (int e = check_launch()) return e;
    return for_groups([&](const AdamwTensors& ts, int64_t first, unsigned chunks) {
        adamw_kernel<<<chunks, ADAMW_THREADS, 0, st>>>(ts, first, params_flat, m_flat, v_flat, state, h);
    });
}

}  // extern "C"
