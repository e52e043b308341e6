// extern "C" layer, part two (include/d8k.h, "Exchange of replicated-operand gradients"): memory that the other
// processes of the box map through CUDA IPC, stream-ordered flags between processes, copy-engine transfers and the
// fixed-order sum of partial gradients.  The transfers use no SM, and the three small kernels here (signal, wait, sum)
// need no shared memory and few registers, so they share SMs with a running contraction kernel instead of waiting for
// one to drain - which is what a library all-reduce kernel, with its large register footprint, has to do.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/d8k.h"
#include "elementwise.cuh"
#include "gemm_host.h"

struct d8k_ctx : public d8k::Ctx {};

namespace d8k {
namespace {

constexpr int kMaxPeers = 16;
constexpr int kRoleExchange = 5;  // role field of the status word for a wait that expired here

#define D8K_CUDA(call)                                                                                          \
    do {                                                                                                        \
        cudaError_t e__ = (call);                                                                               \
        if (e__ != cudaSuccess) return fail(D8K_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__)); \
    } while (0)

struct FlagList {
    unsigned* p[kMaxPeers];
};
struct SrcList {
    const void* p[kMaxPeers];
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// One warp; lane i publishes to flag i.  The fence orders every earlier write of this GPU (kernels and copies that
// completed before this kernel started, in stream order) before the flag for an observer on any GPU.
__global__ void peer_signal_kernel(FlagList flags, int n, unsigned value) {
    int i = threadIdx.x;
    if (i < n) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[i]), "r"(value) : "memory");
    }
}

// One warp; lane i polls flag i until it reaches `value` or the time limit passes.  The first lane that gives up
// records (role << 8 | i) in the status word; the kernel then ends either way, so the stream always moves on.
__global__ void peer_wait_kernel(FlagList flags, int n, unsigned value, unsigned long long limit_ns, int* status) {
    int i = threadIdx.x;
    if (i >= n) return;
    const unsigned long long t0 = global_ns();
    unsigned seen;
    for (;;) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags.p[i]) : "memory");
        if (static_cast<int>(seen - value) >= 0) break;  // counters wrap: compare as a signed distance
        if (global_ns() - t0 > limit_ns) {
            atomicCAS(status, 0, (kRoleExchange << 8) | i);
            break;
        }
        __nanosleep(256);
    }
}

// w = g * alpha + w * beta for 16 bytes of weights, g in fp32: two products and one sum, each rounded (no fused
// multiply-add), then - for fp16 weights - one rounding to T.  For fp32 this is the reference's CPU arithmetic bit for bit.
template <typename T>
__device__ __forceinline__ uint4 sgd16(const float* g, const uint4& w_in, float alpha, float beta) {
    constexpr int V = 16 / sizeof(T);
    float w[V];
#pragma unroll
    for (int k = 0; k < V; ++k) w[k] = 0.f;
    accumulate16<T>(w, w_in);
#pragma unroll
    for (int k = 0; k < V; ++k) w[k] = __fadd_rn(__fmul_rn(g[k], alpha), __fmul_rn(w[k], beta));
    return round16<T>(w);
}

// out = srcs[0] + srcs[1] + ... in that order, fp32 accumulation, 16 bytes per thread per step; NSRC > 0 unrolls the
// source loop so that all loads of a step are in flight together.
// With `weights` the trainer's step follows on the same elements (sgd16).
template <typename T, int NSRC>
__global__ void __launch_bounds__(256) sum_shards_kernel(T* out, SrcList srcs, int nsrc, size_t count, bool vec, T* weights, float alpha,
                                                         float beta, FlagList copies, int ncopies) {
    constexpr int V = 16 / sizeof(T);
    const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = gridDim.x * static_cast<size_t>(blockDim.x);
    const size_t nv = vec ? count / V : 0;
    for (size_t i = tid; i < nv; i += stride) {
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = 0.f;
        if constexpr (NSRC > 0) {
            uint4 v[NSRC];
#pragma unroll
            for (int s = 0; s < NSRC; ++s) v[s] = __ldcs(reinterpret_cast<const uint4*>(srcs.p[s]) + i);
#pragma unroll
            for (int s = 0; s < NSRC; ++s) accumulate16<T>(acc, v[s]);
        } else {
            for (int s = 0; s < nsrc; ++s) accumulate16<T>(acc, __ldcs(reinterpret_cast<const uint4*>(srcs.p[s]) + i));
        }
        const uint4 g = round16<T>(acc);
        if (out) reinterpret_cast<uint4*>(out)[i] = g;
        if (weights) {  // the trainer's step on the gradient as stored (rounded to T), like a separate pass would see it
            float gs[V];
#pragma unroll
            for (int k = 0; k < V; ++k) gs[k] = 0.f;
            accumulate16<T>(gs, g);
            const uint4 w = sgd16<T>(gs, reinterpret_cast<const uint4*>(weights)[i], alpha, beta);
            reinterpret_cast<uint4*>(weights)[i] = w;
            for (int c = 0; c < ncopies; ++c) reinterpret_cast<uint4*>(copies.p[c])[i] = w;  // the all-gather: peers' copies of the weights
        } else {
            for (int c = 0; c < ncopies; ++c) reinterpret_cast<uint4*>(copies.p[c])[i] = g;  // the all-gather: peers' copies of the sum
        }
    }
    for (size_t i = nv * V + tid; i < count; i += stride) {
        float a = 0.f;
        for (int s = 0; s < nsrc; ++s) {
            if constexpr (sizeof(T) == 4) a += reinterpret_cast<const float*>(srcs.p[s])[i];
            else a += __half2float(reinterpret_cast<const __half*>(srcs.p[s])[i]);
        }
        T gt;
        if constexpr (sizeof(T) == 4) gt = a;
        else gt = __float2half_rn(a);
        if (out) out[i] = gt;
        if (weights) {
            float gs, ws;
            if constexpr (sizeof(T) == 4) { gs = gt; ws = weights[i]; }
            else { gs = __half2float(gt); ws = __half2float(weights[i]); }
            float r = __fadd_rn(__fmul_rn(gs, alpha), __fmul_rn(ws, beta));
            if constexpr (sizeof(T) == 4) gt = r;
            else gt = __float2half_rn(r);
            weights[i] = gt;
        }
        for (int c = 0; c < ncopies; ++c) reinterpret_cast<T*>(copies.p[c])[i] = gt;
    }
    // the copies may sit in peers' memory: order this thread's stores before whatever the host enqueues next
    if (ncopies) __threadfence_system();
}

// The sum with Adam behind it (Math::AdamUpdate on the shard a GPU owns): g = srcs[0] + ... rounded to T as the separate
// sum would store it, then gradient += value * decay, m, v and value are updated on the same elements; the updated
// weights also go to `copies` (the peers' buffers).  m and v exist only for the owned shard: each GPU keeps 1 / N of
// the optimiser's state.
template <typename T>
__global__ void __launch_bounds__(256) sum_shards_adam_kernel(T* grad_out, SrcList srcs, int nsrc, size_t count, bool vec, T* weights, T* m,
                                                              T* v, AdamCoeff c, FlagList copies, int ncopies) {
    constexpr int V = 16 / sizeof(T);
    const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = gridDim.x * static_cast<size_t>(blockDim.x);
    const size_t nv = vec ? count / V : 0;
    for (size_t i = tid; i < nv; i += stride) {
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = 0.f;
        for (int s = 0; s < nsrc; ++s) accumulate16<T>(acc, __ldcs(reinterpret_cast<const uint4*>(srcs.p[s]) + i));
        uint4 g4 = round16<T>(acc), w4 = reinterpret_cast<const uint4*>(weights)[i];
        uint4 m4 = reinterpret_cast<const uint4*>(m)[i], v4 = reinterpret_cast<const uint4*>(v)[i];
        T* ge = reinterpret_cast<T*>(&g4);
        T* we = reinterpret_cast<T*>(&w4);
        T* me = reinterpret_cast<T*>(&m4);
        T* ve = reinterpret_cast<T*>(&v4);
#pragma unroll
        for (int k = 0; k < V; ++k) {
            float w = widen(we[k]), g = widen(ge[k]), mm = widen(me[k]), vv = widen(ve[k]);
            adam_element(w, g, mm, vv, c);
            we[k] = narrow<T>(w); ge[k] = narrow<T>(g); me[k] = narrow<T>(mm); ve[k] = narrow<T>(vv);
        }
        if (grad_out) reinterpret_cast<uint4*>(grad_out)[i] = g4;
        reinterpret_cast<uint4*>(weights)[i] = w4;
        reinterpret_cast<uint4*>(m)[i] = m4;
        reinterpret_cast<uint4*>(v)[i] = v4;
        for (int q = 0; q < ncopies; ++q) reinterpret_cast<uint4*>(copies.p[q])[i] = w4;
    }
    for (size_t i = nv * V + tid; i < count; i += stride) {
        float a = 0.f;
        for (int s = 0; s < nsrc; ++s) a += widen(reinterpret_cast<const T*>(srcs.p[s])[i]);
        float g = widen(narrow<T>(a)), w = widen(weights[i]), mm = widen(m[i]), vv = widen(v[i]);
        adam_element(w, g, mm, vv, c);
        if (grad_out) grad_out[i] = narrow<T>(g);
        weights[i] = narrow<T>(w);
        m[i] = narrow<T>(mm);
        v[i] = narrow<T>(vv);
        for (int q = 0; q < ncopies; ++q) reinterpret_cast<T*>(copies.p[q])[i] = narrow<T>(w);
    }
    if (ncopies) __threadfence_system();
}

template <typename T>
void launch_sum(const Ctx* ctx, void* out, const SrcList& srcs, int nsrc, size_t count, bool vec, void* weights, float alpha, float beta,
                const FlagList& copies, int ncopies) {
    constexpr int V = 16 / sizeof(T);
    size_t blocks = (count / V + 255) / 256;
    // One CTA of 256 threads per SM.  The sum runs beside a persistent contraction kernel and shares its SMs' issue slots:
    // with 8 CTAs per SM (2048 extra threads) the contractions of a 2-GPU step took 5.40 ms, with one they took 5.22 ms -
    // what they take with no exchange at all - and the sum (nsrc + 1 16-byte accesses in flight per thread) still ends
    // long before the contractions behind it.  D8K_SUM_BLOCKS_PER_SM overrides.
    static const int forced = [] { const char* v = std::getenv("D8K_SUM_BLOCKS_PER_SM"); return v ? std::atoi(v) : 0; }();
    size_t cap = static_cast<size_t>(ctx->num_sms) * (forced > 0 ? forced : 1);
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    dim3 grid(static_cast<unsigned>(blocks));
    T* o = static_cast<T*>(out);
    T* w = static_cast<T*>(weights);
    switch (nsrc) {
        case 1: sum_shards_kernel<T, 1><<<grid, 256, 0, ctx->stream>>>(o, srcs, nsrc, count, vec, w, alpha, beta, copies, ncopies); break;
        case 2: sum_shards_kernel<T, 2><<<grid, 256, 0, ctx->stream>>>(o, srcs, nsrc, count, vec, w, alpha, beta, copies, ncopies); break;
        case 4: sum_shards_kernel<T, 4><<<grid, 256, 0, ctx->stream>>>(o, srcs, nsrc, count, vec, w, alpha, beta, copies, ncopies); break;
        case 8: sum_shards_kernel<T, 8><<<grid, 256, 0, ctx->stream>>>(o, srcs, nsrc, count, vec, w, alpha, beta, copies, ncopies); break;
        default: sum_shards_kernel<T, 0><<<grid, 256, 0, ctx->stream>>>(o, srcs, nsrc, count, vec, w, alpha, beta, copies, ncopies); break;
    }
}

int check_ctx(const d8k_ctx* ctx) {
    if (!ctx) return fail(D8K_ERR_ARGUMENT, "null context");
    return 0;
}

}  // namespace
}  // namespace d8k

using namespace d8k;

extern "C" {

int d8k_peer_alloc(d8k_ctx* ctx, size_t bytes, void** ptr, unsigned char handle[D8K_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == D8K_IPC_HANDLE_BYTES, "IPC handle size");
    if (int rc = check_ctx(ctx)) return rc;
    if (!ptr || !handle || bytes == 0) return fail(D8K_ERR_ARGUMENT, "peer_alloc: null pointer or zero size");
    D8K_CUDA(cudaSetDevice(ctx->device));
    void* p = nullptr;
    D8K_CUDA(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(D8K_ERR_CUDA, std::string("peer_alloc: ") + cudaGetErrorString(e));
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return 0;
}

int d8k_peer_free(d8k_ctx* ctx, void* ptr) {
    if (int rc = check_ctx(ctx)) return rc;
    if (!ptr) return 0;
    D8K_CUDA(cudaSetDevice(ctx->device));
    D8K_CUDA(cudaFree(ptr));
    return 0;
}

int d8k_peer_open(d8k_ctx* ctx, const unsigned char handle[D8K_IPC_HANDLE_BYTES], void** ptr) {
    if (int rc = check_ctx(ctx)) return rc;
    if (!ptr || !handle) return fail(D8K_ERR_ARGUMENT, "peer_open: null pointer");
    D8K_CUDA(cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    D8K_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return 0;
}

int d8k_peer_close(d8k_ctx* ctx, void* ptr) {
    if (int rc = check_ctx(ctx)) return rc;
    if (!ptr) return 0;
    D8K_CUDA(cudaSetDevice(ctx->device));
    D8K_CUDA(cudaIpcCloseMemHandle(ptr));
    return 0;
}

int d8k_peer_signal(d8k_ctx* ctx, void* const* flags, int n, unsigned value) {
    if (int rc = check_ctx(ctx)) return rc;
    if (n == 0) return 0;
    if (!flags || n < 0 || n > kMaxPeers) return fail(D8K_ERR_ARGUMENT, "peer_signal: 1 to 16 flags");
    FlagList f = {};
    for (int i = 0; i < n; ++i) {
        if (!flags[i] || (reinterpret_cast<uintptr_t>(flags[i]) & 3)) return fail(D8K_ERR_ARGUMENT, "peer_signal: null or unaligned flag");
        f.p[i] = static_cast<unsigned*>(flags[i]);
    }
    peer_signal_kernel<<<1, 32, 0, ctx->stream>>>(f, n, value);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

int d8k_peer_wait(d8k_ctx* ctx, const void* const* flags, int n, unsigned value, double timeout_ms) {
    if (int rc = check_ctx(ctx)) return rc;
    if (n == 0) return 0;
    if (!flags || n < 0 || n > kMaxPeers) return fail(D8K_ERR_ARGUMENT, "peer_wait: 1 to 16 flags");
    if (!(timeout_ms > 0.0) || timeout_ms > 60000.0) return fail(D8K_ERR_ARGUMENT, "peer_wait: the time limit must be in (0, 60000] ms");
    FlagList f = {};
    for (int i = 0; i < n; ++i) {
        if (!flags[i] || (reinterpret_cast<uintptr_t>(flags[i]) & 3)) return fail(D8K_ERR_ARGUMENT, "peer_wait: null or unaligned flag");
        f.p[i] = const_cast<unsigned*>(static_cast<const unsigned*>(flags[i]));
    }
    peer_wait_kernel<<<1, 32, 0, ctx->stream>>>(f, n, value, static_cast<unsigned long long>(timeout_ms * 1e6), ctx->status);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

int d8k_peer_copy(d8k_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (int rc = check_ctx(ctx)) return rc;
    if (bytes == 0) return 0;
    if (!dst || !src) return fail(D8K_ERR_ARGUMENT, "peer_copy: null pointer");
    D8K_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, ctx->stream));
    return 0;
}

static int sum_shards_impl(d8k_ctx* ctx, int dtype, void* out, const void* const* srcs, int nsrc, size_t count, void* weights, float alpha,
                           float beta, void* const* copies = nullptr, int ncopies = 0) {
    if (int rc = check_ctx(ctx)) return rc;
    if (dtype != D8K_F16 && dtype != D8K_F32) return fail(D8K_ERR_ARGUMENT, "type is not support: dtype must be D8K_F16 or D8K_F32");
    if (count == 0) return 0;
    if ((!out && !weights) || !srcs || nsrc < 1 || nsrc > kMaxPeers) return fail(D8K_ERR_ARGUMENT, "sum_shards: 1 to 16 sources");
    SrcList s = {};
    uintptr_t bits = reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(weights);
    for (int i = 0; i < nsrc; ++i) {
        if (!srcs[i]) return fail(D8K_ERR_ARGUMENT, "sum_shards: null source");
        s.p[i] = srcs[i];
        bits |= reinterpret_cast<uintptr_t>(srcs[i]);
    }
    FlagList cp = {};
    if (ncopies < 0 || ncopies > kMaxPeers || (ncopies > 0 && !copies)) return fail(D8K_ERR_ARGUMENT, "sum_shards: 0 to 16 copies");
    for (int i = 0; i < ncopies; ++i) {
        if (!copies[i]) return fail(D8K_ERR_ARGUMENT, "sum_shards: null copy");
        cp.p[i] = static_cast<unsigned*>(copies[i]);
        bits |= reinterpret_cast<uintptr_t>(copies[i]);
    }
    bool vec = (bits & 15) == 0;
    if (dtype == D8K_F32) launch_sum<float>(ctx, out, s, nsrc, count, vec, weights, alpha, beta, cp, ncopies);
    else launch_sum<__half>(ctx, out, s, nsrc, count, vec, weights, alpha, beta, cp, ncopies);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

int d8k_sum_shards(d8k_ctx* ctx, int dtype, void* out, const void* const* srcs, int nsrc, size_t count) {
    if (!out) return fail(D8K_ERR_ARGUMENT, "sum_shards: null output");
    return sum_shards_impl(ctx, dtype, out, srcs, nsrc, count, nullptr, 0.f, 0.f);
}

int d8k_sum_shards_sgd(d8k_ctx* ctx, int dtype, void* grad_out, const void* const* srcs, int nsrc, size_t count, void* weights, float alpha,
                       float beta) {
    if (!weights) return fail(D8K_ERR_ARGUMENT, "sum_shards_sgd: null weights");
    return sum_shards_impl(ctx, dtype, grad_out, srcs, nsrc, count, weights, alpha, beta);
}

int d8k_sum_shards_gather(d8k_ctx* ctx, int dtype, void* out, const void* const* srcs, int nsrc, size_t count, void* weights, float alpha,
                          float beta, void* const* copies, int ncopies) {
    if (!out && !weights) return fail(D8K_ERR_ARGUMENT, "sum_shards_gather: null output");
    return sum_shards_impl(ctx, dtype, out, srcs, nsrc, count, weights, alpha, beta, copies, ncopies);
}

int d8k_sum_shards_adam(d8k_ctx* ctx, int dtype, void* grad_out, const void* const* srcs, int nsrc, size_t count, void* weights, void* m, void* v,
                        float beta1, float beta2, float epsilon, float learning_rate, float weight_decay, long long steps, void* const* copies,
                        int ncopies) {
    if (int rc = check_ctx(ctx)) return rc;
    if (dtype != D8K_F16 && dtype != D8K_F32) return fail(D8K_ERR_ARGUMENT, "type is not support: dtype must be D8K_F16 or D8K_F32");
    if (count == 0) return 0;
    if (!weights || !m || !v || !srcs || nsrc < 1 || nsrc > kMaxPeers) return fail(D8K_ERR_ARGUMENT, "sum_shards_adam: null pointer, or not 1 to 16 sources");
    if (ncopies < 0 || ncopies > kMaxPeers || (ncopies > 0 && !copies)) return fail(D8K_ERR_ARGUMENT, "sum_shards_adam: 0 to 16 copies");
    SrcList sl = {};
    FlagList cp = {};
    uintptr_t bits = reinterpret_cast<uintptr_t>(grad_out) | reinterpret_cast<uintptr_t>(weights) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v);
    for (int i = 0; i < nsrc; ++i) {
        if (!srcs[i]) return fail(D8K_ERR_ARGUMENT, "sum_shards_adam: null source");
        sl.p[i] = srcs[i];
        bits |= reinterpret_cast<uintptr_t>(srcs[i]);
    }
    for (int i = 0; i < ncopies; ++i) {
        if (!copies[i]) return fail(D8K_ERR_ARGUMENT, "sum_shards_adam: null copy");
        cp.p[i] = static_cast<unsigned*>(copies[i]);
        bits |= reinterpret_cast<uintptr_t>(copies[i]);
    }
    const bool vec = (bits & 15) == 0;
    AdamCoeff c = {beta1, beta2, 1.0f - beta1, 1.0f - beta2, epsilon, weight_decay, d8k_adam_ratio(learning_rate, beta1, beta2, steps)};
    const int per = dtype == D8K_F32 ? 4 : 8;
    size_t blocks = (count / per + 255) / 256;
    if (blocks > static_cast<size_t>(ctx->num_sms)) blocks = ctx->num_sms;  // one CTA per SM, like the plain sum
    if (blocks < 1) blocks = 1;
    if (dtype == D8K_F32)
        sum_shards_adam_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(
            static_cast<float*>(grad_out), sl, nsrc, count, vec, static_cast<float*>(weights), static_cast<float*>(m), static_cast<float*>(v), c, cp,
            ncopies);
    else
        sum_shards_adam_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(
            static_cast<__half*>(grad_out), sl, nsrc, count, vec, static_cast<__half*>(weights), static_cast<__half*>(m), static_cast<__half*>(v), c,
            cp, ncopies);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

int d8k_axpby(d8k_ctx* ctx, int dtype, const void* x, float alpha, void* y, float beta, size_t n) {
    if (!x || !y) return n == 0 ? 0 : fail(D8K_ERR_ARGUMENT, "axpby: null pointer");
    const void* src[1] = {x};
    return sum_shards_impl(ctx, dtype, nullptr, src, 1, n, y, alpha, beta);
}

}  // extern "C"
