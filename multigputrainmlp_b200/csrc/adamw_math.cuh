// AdamW update of one parameter, shared by the stand-alone optimizer kernel and by the fused
// allreduce + AdamW kernels. Arithmetic follows native/cuda/adamw.cu:8-23 operation by operation
// (fp32, bias corrections from powf, L2-style decay folded into the gradient).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mgt {

struct AdamWScalars {
    float lr, beta1, beta2, eps, wd, one_minus_b1, one_minus_b2, bias1, bias2;
};

__device__ __forceinline__ AdamWScalars MakeAdamWScalars(uint64_t step, float lr, float beta1, float beta2, float eps, float wd) {
    AdamWScalars s;
    s.lr = lr;
    s.beta1 = beta1;
    s.beta2 = beta2;
    s.eps = eps;
    s.wd = wd;
    s.one_minus_b1 = 1.0f - beta1;
    s.one_minus_b2 = 1.0f - beta2;
    s.bias1 = 1.0f - powf(beta1, static_cast<float>(step));
    s.bias2 = 1.0f - powf(beta2, static_cast<float>(step));
    return s;
}

// Correctly rounded division and square root take a slow path in the compiler's expansion when an operand is zero, and a
// warp pays for it when any lane does. Exact zeros are common here: gradients, and with them both moments, of units whose
// ReLU never opens and of padding columns (the p888 update ran 0.115 ms with them against 0.080 ms on all-normal data). A
// zero numerator is therefore replaced by 1 before the operation and the zero (with its sign: x / b for b > 0 and sqrt(x)
// return x itself when x is +-0) selected afterwards - the same bits, checked against the plain operations on normal,
// zero, negative-zero and denormal data.
__device__ __forceinline__ float DivByPositiveExact(float a, float b) {
    const bool zero = a == 0.0f;
    const float q = __fdiv_rn(zero ? 1.0f : a, b);
    return zero ? a : q;
}

__device__ __forceinline__ float SqrtExact(float a) {
    const bool zero = a == 0.0f;
    const float q = __fsqrt_rn(zero ? 1.0f : a);
    return zero ? a : q;
}

// Every operation is an explicitly rounded IEEE fp32 operation (no FMA contraction), so that all
// call sites - and therefore all data-parallel replicas - produce bit-identical weights, and so that
// the result equals the plain C expression of the reference evaluated operation by operation.
// The three divisors are positive: the bias corrections lie in (0, 1], and sqrt(.) + eps >= eps > 0.
__device__ __forceinline__ float AdamWUpdateOne(const AdamWScalars& s, float weight, float grad, float* m, float* v) {
    const float decayed = __fadd_rn(grad, __fmul_rn(s.wd, weight));
    const float next_m = __fadd_rn(__fmul_rn(s.beta1, *m), __fmul_rn(s.one_minus_b1, decayed));
    const float next_v = __fadd_rn(__fmul_rn(s.beta2, *v), __fmul_rn(__fmul_rn(s.one_minus_b2, decayed), decayed));
    *m = next_m;
    *v = next_v;
    const float m_hat = DivByPositiveExact(next_m, s.bias1);
    const float v_hat = DivByPositiveExact(next_v, s.bias2);
    return __fsub_rn(weight, DivByPositiveExact(__fmul_rn(s.lr, m_hat), __fadd_rn(SqrtExact(v_hat), s.eps)));
}

}  // namespace mgt
