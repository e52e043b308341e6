// Device helpers shared by the element-wise kernels and the exchange's sum kernels: 16-byte packs of fp32 / fp16 values
// to and from float accumulators, and one element of Math::AdamUpdate.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace d8k {

template <typename T>
__device__ __forceinline__ void accumulate16(float* acc, const uint4& v);
template <>
__device__ __forceinline__ void accumulate16<float>(float* acc, const uint4& v) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void accumulate16<__half>(float* acc, const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 f = __half22float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
    }
}
template <typename T>
__device__ __forceinline__ uint4 round16(const float* acc);
template <>
__device__ __forceinline__ uint4 round16<float>(const float* acc) {
    return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
}
template <>
__device__ __forceinline__ uint4 round16<__half>(const float* acc) {
    uint4 o;
    __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2half2_rn(acc[2 * k], acc[2 * k + 1]);
    return o;
}

template <typename T>
__device__ __forceinline__ float widen(T v);
template <>
__device__ __forceinline__ float widen<float>(float v) { return v; }
template <>
__device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T narrow(float v);
template <>
__device__ __forceinline__ float narrow<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }

// ---- Math::AdamUpdate (deep8/src/math/AdamUpdate.cpp:24-41), one element, statement by statement, each operation
// rounded in fp32 (no fused multiply-add: the reference is built without -m flags):
//   gradient += value * weightDecay;  m = m * beta1 + gradient * (1 - beta1);  v = v * beta2 + gradient^2 * (1 - beta2);
//   value -= m / (sqrt(v) + epsilon) * ratio,   ratio = learningRate * sqrt(1 - beta2^steps) / (1 - beta1^steps)
struct AdamCoeff {
    float beta1, beta2, one_minus_beta1, one_minus_beta2, epsilon, weight_decay, ratio;
};
__device__ __forceinline__ void adam_element(float& w, float& g, float& m, float& v, const AdamCoeff& c) {
    g = __fadd_rn(g, __fmul_rn(w, c.weight_decay));
    m = __fadd_rn(__fmul_rn(m, c.beta1), __fmul_rn(g, c.one_minus_beta1));
    v = __fadd_rn(__fmul_rn(v, c.beta2), __fmul_rn(__fmul_rn(g, g), c.one_minus_beta2));
    w = __fsub_rn(w, __fmul_rn(__fdiv_rn(m, __fadd_rn(__fsqrt_rn(v), c.epsilon)), c.ratio));
}

}  // namespace d8k
