// d8k_gemm_static: the split-K contraction for callers that must not allocate device memory.
//
// Who that is: code that runs after a framework has handed all of the GPU's memory to its own pool (Deep8's
// GPUMemoryPool takes it in 512 MiB blocks and nothing else is expected to call cudaMalloc behind its back), code
// inside a latency-critical loop where cudaMalloc's implicit device-wide synchronisation is not acceptable, and
// plug-in callbacks that are forbidden to create a d8k context (whose constructor allocates).  For them the split-K
// scratch - partial tiles, tile tickets and the status word - lives in one file-scope device array that every GPU
// loading this library holds from load to exit: kStaticScratchBytes + 20 KiB, about 16 MiB.
//
// The array's name is only a host-side handle in host code; the device address comes from cudaGetSymbolAddress, asked
// once per device with that device current (the first call on a device does it: make that call before any stream
// capture).  The entry point calls no cudaMalloc, cudaFree or allocating library routine.
//
// All calls on a device share the array and it keeps the previous call's contents: tile tickets carry the number of the launch
// that drew them (stale ones count as zero), partial tiles are always written before they are read, and two calls whose kernels
// overlap on the GPU (different streams, or different host threads) race on it - serialise them.
#include <mutex>
#include <string>

#include "../../include/d8k.h"
#include "gemm_host.h"

namespace d8k {
namespace {

constexpr size_t kStaticScratchBytes = static_cast<size_t>(16) << 20;        // partial tiles
constexpr size_t kStaticTailBytes = (kMaxCounters + 1) * sizeof(int) + 4092;  // tickets + status word, padded
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes + kStaticTailBytes];

struct DeviceSlot {
    unsigned char* base = nullptr;  // device address of g_static_scratch on this device
    int num_sms = 0;
    unsigned epoch = 0;             // split launches made on this device's array so far (Ctx::epoch_counter between calls)
};
DeviceSlot g_slots[64];
std::mutex g_slots_mutex;

// Once per device, with that device current: resolve the array's device address.
int device_slot(DeviceSlot* out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(D8K_ERR_CUDA, std::string("d8k_gemm_static: cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(D8K_ERR_ARGUMENT, "d8k_gemm_static: device index out of range");
    std::lock_guard<std::mutex> lock(g_slots_mutex);
    if (!g_slots[dev].base) {
        int major = 0, sms = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(D8K_ERR_CUDA, std::string("d8k_gemm_static: cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        if (major != 10) return fail(D8K_ERR_CUDA, "d8k_gemm_static: these kernels are built for sm_100a (B200) only");
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(D8K_ERR_CUDA, std::string("d8k_gemm_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        g_slots[dev].base = ptr;
        g_slots[dev].num_sms = sms;
    }
    *out = g_slots[dev];
    return 0;
}

}  // namespace
}  // namespace d8k

using namespace d8k;

extern "C" int d8k_gemm_static(int dtype, int transA, int transB, int M, int N, int K, const void* A, long long lda, const void* B,
                               long long ldb, void* C, long long ldc, int beta, void* stream) {
    if (dtype != D8K_F16 && dtype != D8K_F32) return fail(D8K_ERR_ARGUMENT, "d8k_gemm_static: dtype must be D8K_F16 or D8K_F32");
    DeviceSlot slot;
    if (int rc = device_slot(&slot)) return rc;

    // a context on the stack that points into the static array: nothing is allocated and nothing outlives the call
    Ctx ctx;
    cudaGetDevice(&ctx.device);
    ctx.num_sms = slot.num_sms;
    ctx.stream = static_cast<cudaStream_t>(stream);
    ctx.scratch = reinterpret_cast<float*>(slot.base);
    ctx.scratch_bytes = kStaticScratchBytes;
    ctx.counters = reinterpret_cast<int*>(slot.base + kStaticScratchBytes);
    ctx.status = ctx.counters + kMaxCounters;

    GemmProblem g;
    g.dtype = dtype;
    g.M = M; g.N = N; g.K = K;
    g.a.ptr = A; g.a.mn = transA != 0; g.a.ld = lda;
    g.b.ptr = B; g.b.mn = transB == 0; g.b.ld = ldb;
    g.C = C; g.ldc = ldc;
    g.beta = beta;

    size_t need = gemm_scratch_need(&ctx, g);
    if (need > kStaticScratchBytes)
        return fail(D8K_ERR_ARGUMENT, "d8k_gemm_static: this contraction needs " + std::to_string(need) +
                                          " bytes of split-K scratch, the static maximum is " + std::to_string(kStaticScratchBytes) +
                                          "; use d8k_gemm with a context");
    // ticket words carry the epoch of the launch that wrote them, so whatever an earlier call left behind counts as zero; the
    // epoch lives with the device's slot between calls (calls on one device are serialised by contract)
    ctx.epoch_counter = slot.epoch;
    const int rc = run_gemm(&ctx, g);
    {
        std::lock_guard<std::mutex> lock(g_slots_mutex);
        g_slots[ctx.device].epoch = ctx.epoch_counter;
    }
    return rc;
}
