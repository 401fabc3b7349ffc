// Optimizer step on the lattice values: AdamW as the reference's training loops apply it to the
// table (examples/performance.py:161 -- torch.optim.AdamW(amsgrad=False, betas=(0.9, 0.99),
// eps=1e-15, weight_decay=0) -- and examples/train_toy_example.py:30), as ONE elementwise kernel
// over the [L, C, F] table instead of the chain of elementwise launches a generic optimizer makes.
//
// Per element, in fp32, in the order of torch's single-tensor AdamW:
//   p  <- p * (1 - lr * weight_decay)
//   m  <- m + (g - m) * (1 - beta1)
//   v  <- v * beta2 + (1 - beta2) * g * g
//   p  <- p - (lr / (1 - beta1^t)) * m / (sqrt(v) / sqrt(1 - beta2^t) + eps)
// The step-dependent scalars are computed on the host in double precision, like torch does.
//
// HBM-bound streaming: 4 loads + 3 stores of 4 bytes per element, moved as 16-byte vectors by a
// grid of (multiprocessors x resident blocks) blocks that strides over the table.  Two options
// trim the bytes: entries whose gradient and both moments are zero (slots no point has touched
// yet -- most of a fine level early in training) are left alone when there is no weight decay,
// which is exact; and the gradient can be cleared in the same pass, which replaces the separate
// clearing of the 50-134 MB gradient table before the next backward.
#include <cmath>
#include <cstdint>
#include <cuda_runtime.h>

#include "permuto_b200.h"
#include "permuto_internal.h"

namespace {

struct AdamScalars {
    float decay;        // 1 - lr * weight_decay
    float one_m_beta1;  // 1 - beta1
    float beta2;
    float one_m_beta2;  // 1 - beta2
    float step_size;    // lr / (1 - beta1^t)
    float inv_bc2_sqrt; // 1 / sqrt(1 - beta2^t)
    float eps;
};

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamScalars& s) {
    p = p * s.decay;
    m = fmaf(g - m, s.one_m_beta1, m);
    v = fmaf(s.one_m_beta2 * g, g, v * s.beta2);
    const float denom = sqrtf(v) * s.inv_bc2_sqrt + s.eps;
    p = p - s.step_size * (m / denom);
}

template <bool SKIP_UNTOUCHED, bool ZERO_GRAD>
__global__ void __launch_bounds__(256) adam_kernel(float* __restrict__ values, float* __restrict__ grad,
                                                   float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
                                                   int64_t n_vec4, int64_t n, AdamScalars s) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int64_t i = tid; i < n_vec4; i += stride) {
        const float4 g = reinterpret_cast<const float4*>(grad)[i];
        float4 m = reinterpret_cast<const float4*>(exp_avg)[i];
        float4 v = reinterpret_cast<const float4*>(exp_avg_sq)[i];
        if (SKIP_UNTOUCHED) {
            const bool untouched = g.x == 0.f && g.y == 0.f && g.z == 0.f && g.w == 0.f && m.x == 0.f && m.y == 0.f &&
                                   m.z == 0.f && m.w == 0.f && v.x == 0.f && v.y == 0.f && v.z == 0.f && v.w == 0.f;
            if (untouched) continue;  // update is exactly zero: nothing to read or write further
        }
        float4 p = reinterpret_cast<const float4*>(values)[i];
        adam_one(p.x, g.x, m.x, v.x, s);
        adam_one(p.y, g.y, m.y, v.y, s);
        adam_one(p.z, g.z, m.z, v.z, s);
        adam_one(p.w, g.w, m.w, v.w, s);
        reinterpret_cast<float4*>(values)[i] = p;
        reinterpret_cast<float4*>(exp_avg)[i] = m;
        reinterpret_cast<float4*>(exp_avg_sq)[i] = v;
        if (ZERO_GRAD) reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // the last n % 4 elements
    for (int64_t i = 4 * n_vec4 + tid; i < n; i += stride) {
        const float g = grad[i];
        float m = exp_avg[i], v = exp_avg_sq[i], p = values[i];
        if (!(SKIP_UNTOUCHED && g == 0.f && m == 0.f && v == 0.f)) {
            adam_one(p, g, m, v, s);
            values[i] = p;
            exp_avg[i] = m;
            exp_avg_sq[i] = v;
        }
        if (ZERO_GRAD) grad[i] = 0.f;
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int permuto_adam_step(float* values, float* grad, float* exp_avg, float* exp_avg_sq, int64_t n, double lr,
                                 double beta1, double beta2, double eps, double weight_decay, int64_t step,
                                 uint32_t flags, void* stream) {
    using permuto::set_error;
    if (!values || !grad || !exp_avg || !exp_avg_sq)
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "adam: values, grad, exp_avg and exp_avg_sq must not be NULL");
    if (n < 1) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "adam: n must be >= 1");
    if (step < 1) return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "adam: step counts from 1 (got %lld)", (long long)step);
    if (!(beta1 >= 0.0 && beta1 < 1.0) || !(beta2 >= 0.0 && beta2 < 1.0))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "adam: betas must be in [0, 1)");
    if (!(lr >= 0.0) || !(eps >= 0.0) || !(weight_decay >= 0.0))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "adam: lr, eps and weight_decay must be >= 0");
    if (!aligned16(values) || !aligned16(grad) || !aligned16(exp_avg) || !aligned16(exp_avg_sq))
        return set_error(PERMUTO_ERR_INVALID_ARGUMENT, "adam: all four arrays must be 16-byte aligned");
    AdamScalars s;
    // hyper-parameters arrive as doubles and are combined in double before the one rounding to
    // fp32, as torch does with its Python scalars (1 - 0.999 must not be taken from fp32 0.999)
    const double bc1 = 1.0 - std::pow(beta1, (double)step);
    const double bc2 = 1.0 - std::pow(beta2, (double)step);
    s.decay = (float)(1.0 - lr * weight_decay);
    s.one_m_beta1 = (float)(1.0 - beta1);
    s.beta2 = (float)beta2;
    s.one_m_beta2 = (float)(1.0 - beta2);
    s.step_size = (float)(lr / bc1);
    s.inv_bc2_sqrt = (float)(1.0 / std::sqrt(bc2));
    s.eps = (float)eps;
    const int sms = permuto::sm_count();
    if (sms <= 0) return set_error(PERMUTO_ERR_CUDA, "adam: cannot query the device");
    const int64_t n_vec4 = n / 4;
    int64_t blocks = (n_vec4 + 255) / 256;
    const int64_t cap = (int64_t)sms * 8;  // 8 resident blocks of 256 threads per multiprocessor
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool skip = (flags & PERMUTO_ADAM_SKIP_UNTOUCHED) && weight_decay == 0.0;
    const bool zero = (flags & PERMUTO_ADAM_ZERO_GRAD) != 0;
    const dim3 g((unsigned)blocks);
    if (skip && zero)
        adam_kernel<true, true><<<g, 256, 0, st>>>(values, grad, exp_avg, exp_avg_sq, n_vec4, n, s);
    else if (skip)
        adam_kernel<true, false><<<g, 256, 0, st>>>(values, grad, exp_avg, exp_avg_sq, n_vec4, n, s);
    else if (zero)
        adam_kernel<false, true><<<g, 256, 0, st>>>(values, grad, exp_avg, exp_avg_sq, n_vec4, n, s);
    else
        adam_kernel<false, false><<<g, 256, 0, st>>>(values, grad, exp_avg, exp_avg_sq, n_vec4, n, s);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? PERMUTO_OK : set_error(PERMUTO_ERR_CUDA, "permuto_adam_step launch: %s", cudaGetErrorString(e));
}
