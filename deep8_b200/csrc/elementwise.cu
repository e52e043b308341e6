// extern "C" layer, part three (include/d8k.h): the element-wise neighbours of the contractions that are not ReLU -
// Math::Linear and its gradient, Math::AdamUpdate - as HBM-bound kernels (16 bytes per thread per step, a grid of a few
// CTAs per SM).  fp32 arithmetic follows the reference's CPU expressions operation by operation (separate roundings, no
// fused multiply-add: the reference is built without -m flags), so results equal the CPU oracle bit for bit wherever
// the oracle itself is exact.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <string>

#include "../../include/d8k.h"
#include "elementwise.cuh"
#include "gemm_host.h"

struct d8k_ctx : public d8k::Ctx {};

namespace d8k {
namespace {

#define D8K_CUDA(call)                                                                                          \
    do {                                                                                                        \
        cudaError_t e__ = (call);                                                                               \
        if (e__ != cudaSuccess) return fail(D8K_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__)); \
    } while (0)

int grid_for(const d8k_ctx* ctx, size_t n, int per_thread) {
    size_t blocks = (n / per_thread + 255) / 256;
    size_t cap = static_cast<size_t>(ctx->num_sms) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

// ---- Math::Linear: y = x * a + b (deep8/src/math/Linear.cpp:46-54; GPU form deep8/src/math/Linear.cu:11-23)
__device__ __forceinline__ float linear_op(float x, float a, float b) { return __fadd_rn(__fmul_rn(x, a), b); }
// the reference's half kernel computes a * x + b in half arithmetic with a and b converted to half (Linear.cu:46-52)
__device__ __forceinline__ __half linear_op(__half x, __half a, __half b) { return __hadd(__hmul(a, x), b); }
// ---- Math::LinearGrad: dx += dy * a (deep8/src/math/Linear.cpp:72-80; Linear.cu:60-72 with the += of GPUUnaryElementWise.h:31)
__device__ __forceinline__ float linear_grad_op(float dx, float dy, float a) { return __fadd_rn(dx, __fmul_rn(dy, a)); }
__device__ __forceinline__ __half linear_grad_op(__half dx, __half dy, __half a) { return __hadd(dx, __hmul(a, dy)); }

template <typename T>
__global__ void linear_forward_kernel(const T* __restrict__ x, T* __restrict__ y, T a, T b, size_t n, bool vec) {
    constexpr int V = 16 / sizeof(T);
    const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = gridDim.x * static_cast<size_t>(blockDim.x);
    const size_t nv = vec ? n / V : 0;
    size_t i = tid;
    // four independent 16-byte loads in flight per thread before the first store: a lone load per iteration left the
    // kernel at 5.1 TB/s where the gradient kernel, with two loads per iteration, reached 5.8
    for (; i + 3 * stride < nv; i += 4 * stride) {
        uint4 in[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) in[u] = __ldcs(reinterpret_cast<const uint4*>(x) + i + u * stride);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            T* e = reinterpret_cast<T*>(&in[u]);
#pragma unroll
            for (int k = 0; k < V; ++k) e[k] = linear_op(e[k], a, b);
            reinterpret_cast<uint4*>(y)[i + u * stride] = in[u];
        }
    }
    for (; i < nv; i += stride) {
        uint4 in = __ldcs(reinterpret_cast<const uint4*>(x) + i);
        T* e = reinterpret_cast<T*>(&in);
#pragma unroll
        for (int k = 0; k < V; ++k) e[k] = linear_op(e[k], a, b);
        reinterpret_cast<uint4*>(y)[i] = in;
    }
    for (size_t j = nv * V + tid; j < n; j += stride) y[j] = linear_op(x[j], a, b);
}

template <typename T>
__global__ void linear_grad_kernel(T* __restrict__ dx, const T* __restrict__ dy, T a, size_t n, bool vec) {
    constexpr int V = 16 / sizeof(T);
    const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = gridDim.x * static_cast<size_t>(blockDim.x);
    const size_t nv = vec ? n / V : 0;
    for (size_t i = tid; i < nv; i += stride) {
        uint4 g = __ldcs(reinterpret_cast<const uint4*>(dy) + i);
        uint4 acc = reinterpret_cast<const uint4*>(dx)[i];
        const T* ge = reinterpret_cast<const T*>(&g);
        T* ae = reinterpret_cast<T*>(&acc);
#pragma unroll
        for (int k = 0; k < V; ++k) ae[k] = linear_grad_op(ae[k], ge[k], a);
        reinterpret_cast<uint4*>(dx)[i] = acc;
    }
    for (size_t i = nv * V + tid; i < n; i += stride) dx[i] = linear_grad_op(dx[i], dy[i], a);
}

// fp16 tensors are widened, updated in fp32 and each array is rounded once on the way out.
template <typename T>
__global__ void adam_update_kernel(T* __restrict__ value, T* __restrict__ gradient, T* __restrict__ m, T* __restrict__ v, AdamCoeff c,
                                   size_t n, bool vec) {
    constexpr int V = 16 / sizeof(T);
    const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = gridDim.x * static_cast<size_t>(blockDim.x);
    const size_t nv = vec ? n / V : 0;
    for (size_t i = tid; i < nv; i += stride) {
        uint4 w4 = reinterpret_cast<const uint4*>(value)[i], g4 = reinterpret_cast<const uint4*>(gradient)[i];
        uint4 m4 = reinterpret_cast<const uint4*>(m)[i], v4 = reinterpret_cast<const uint4*>(v)[i];
        T* we = reinterpret_cast<T*>(&w4);
        T* ge = reinterpret_cast<T*>(&g4);
        T* me = reinterpret_cast<T*>(&m4);
        T* ve = reinterpret_cast<T*>(&v4);
#pragma unroll
        for (int k = 0; k < V; ++k) {
            float w = widen(we[k]), g = widen(ge[k]), mm = widen(me[k]), vv = widen(ve[k]);
            adam_element(w, g, mm, vv, c);
            we[k] = narrow<T>(w); ge[k] = narrow<T>(g); me[k] = narrow<T>(mm); ve[k] = narrow<T>(vv);
        }
        reinterpret_cast<uint4*>(value)[i] = w4;
        reinterpret_cast<uint4*>(gradient)[i] = g4;
        reinterpret_cast<uint4*>(m)[i] = m4;
        reinterpret_cast<uint4*>(v)[i] = v4;
    }
    for (size_t i = nv * V + tid; i < n; i += stride) {
        float w = widen(value[i]), g = widen(gradient[i]), mm = widen(m[i]), vv = widen(v[i]);
        adam_element(w, g, mm, vv, c);
        value[i] = narrow<T>(w); gradient[i] = narrow<T>(g); m[i] = narrow<T>(mm); v[i] = narrow<T>(vv);
    }
}

bool all_aligned16(std::initializer_list<const void*> ptrs) {
    uintptr_t bits = 0;
    for (const void* p : ptrs) bits |= reinterpret_cast<uintptr_t>(p);
    return (bits & 15) == 0;
}

int check(const d8k_ctx* ctx, int dtype) {
    if (!ctx) return fail(D8K_ERR_ARGUMENT, "null context");
    if (dtype != D8K_F16 && dtype != D8K_F32) return fail(D8K_ERR_ARGUMENT, "type is not support: dtype must be D8K_F16 or D8K_F32");
    return 0;
}

}  // namespace
}  // namespace d8k

using namespace d8k;

extern "C" {

int d8k_linear_forward(d8k_ctx* ctx, int dtype, const void* x, float a, float b, void* y, size_t n) {
    if (int rc = check(ctx, dtype)) return rc;
    if (n == 0) return 0;
    if (!x || !y) return fail(D8K_ERR_ARGUMENT, "linear: null pointer");
    const bool vec = all_aligned16({x, y});
    if (dtype == D8K_F32)
        linear_forward_kernel<float><<<grid_for(ctx, n, 4), 256, 0, ctx->stream>>>(static_cast<const float*>(x), static_cast<float*>(y), a, b, n, vec);
    else
        linear_forward_kernel<__half><<<grid_for(ctx, n, 8), 256, 0, ctx->stream>>>(static_cast<const __half*>(x), static_cast<__half*>(y),
                                                                                    __float2half(a), __float2half(b), n, vec);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

int d8k_linear_grad(d8k_ctx* ctx, int dtype, void* dx, float a, const void* dy, size_t n) {
    if (int rc = check(ctx, dtype)) return rc;
    if (n == 0) return 0;
    if (!dx || !dy) return fail(D8K_ERR_ARGUMENT, "linear: null pointer");
    const bool vec = all_aligned16({dx, dy});
    if (dtype == D8K_F32)
        linear_grad_kernel<float><<<grid_for(ctx, n, 4), 256, 0, ctx->stream>>>(static_cast<float*>(dx), static_cast<const float*>(dy), a, n, vec);
    else
        linear_grad_kernel<__half><<<grid_for(ctx, n, 8), 256, 0, ctx->stream>>>(static_cast<__half*>(dx), static_cast<const __half*>(dy),
                                                                                 __float2half(a), n, vec);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

float d8k_adam_ratio(float learning_rate, float beta1, float beta2, long long steps) {
    if (steps <= 0) steps = 1;  // deep8/src/math/AdamUpdate.cpp:11-14
    // deep8/src/math/AdamUpdate.cpp:38 with T = float
    return learning_rate * std::sqrt(1 - std::pow(beta2, static_cast<float>(steps))) / (1 - std::pow(beta1, static_cast<float>(steps)));
}

int d8k_adam_update(d8k_ctx* ctx, int dtype, void* value, void* gradient, void* m, void* v, float beta1, float beta2, float epsilon,
                    float learning_rate, float weight_decay, long long steps, size_t n) {
    if (int rc = check(ctx, dtype)) return rc;
    if (n == 0) return 0;
    if (!value || !gradient || !m || !v) return fail(D8K_ERR_ARGUMENT, "adam_update: null pointer");
    AdamCoeff c = {beta1, beta2, 1.0f - beta1, 1.0f - beta2, epsilon, weight_decay, d8k_adam_ratio(learning_rate, beta1, beta2, steps)};
    const bool vec = all_aligned16({value, gradient, m, v});
    if (dtype == D8K_F32)
        adam_update_kernel<float><<<grid_for(ctx, n, 4), 256, 0, ctx->stream>>>(static_cast<float*>(value), static_cast<float*>(gradient),
                                                                                static_cast<float*>(m), static_cast<float*>(v), c, n, vec);
    else
        adam_update_kernel<__half><<<grid_for(ctx, n, 8), 256, 0, ctx->stream>>>(static_cast<__half*>(value), static_cast<__half*>(gradient),
                                                                                 static_cast<__half*>(m), static_cast<__half*>(v), c, n, vec);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

}  // extern "C"
