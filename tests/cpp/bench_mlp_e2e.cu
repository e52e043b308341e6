// The benchmark's MLP step through the C++ interface, end to end: every step feeds X from pinned host memory (Variable::feed),
// builds H = X W1, A = ReLu(H), Y = A W2 on the executor (fused launches), runs backward from a host gradient dY, and
// fetches Y back (Variable::fetch).  feed and fetch are synchronous copies, as in the reference (deep8/src/nodes/Variable.cpp),
// so nothing overlaps: this is what a user of the reference's interface gets without touching streams.
// Prints one JSON object.   usage: bench_mlp_e2e [steps] [rows]
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/deep8/Deep8.h"

using namespace Deep8;

static void fill(half_t* p, size_t n, float scale, unsigned seed) {
    unsigned s = seed * 2654435761u + 1u;
    for (size_t i = 0; i < n; ++i) {
        s = s * 1664525u + 1013904223u;
        const float u = (static_cast<float>(s >> 8) / 16777216.0f - 0.5f) * 2.0f * scale;
        __half h = __float2half(u);
        p[i].bits = *reinterpret_cast<uint16_t*>(&h);
    }
}

int main(int argc, char** argv) {
    const int steps = argc > 1 ? std::atoi(argv[1]) : 10;
    const size_t rows = argc > 2 ? std::atoi(argv[2]) : 8192, din = 4096, dhid = 16384;
    try {
        EagerExecutor executor(DeviceType::GPU);
        Variable& x = parameter(&executor, {rows, din}, true, DType::Float16);
        Variable& w1 = parameter(&executor, {din, dhid}, true, DType::Float16);
        Variable& w2 = parameter(&executor, {dhid, din}, true, DType::Float16);
        half_t *hx, *hdy, *hy, *hw;
        cudaHostAlloc(&hx, rows * din * 2, cudaHostAllocDefault);
        cudaHostAlloc(&hdy, rows * din * 2, cudaHostAllocDefault);
        cudaHostAlloc(&hy, rows * din * 2, cudaHostAllocDefault);
        cudaHostAlloc(&hw, din * dhid * 2, cudaHostAllocDefault);
        fill(hx, rows * din, 1.0f, 1);
        fill(hdy, rows * din, 0.01f, 2);
        fill(hw, din * dhid, 0.03f, 3);
        w1.feed(hw);
        fill(hw, din * dhid, 0.03f, 4);
        w2.feed(hw);
        auto step = [&] {
            x.feed(hx);
            Variable& h = x * w1;
            Variable& a = relu(h);
            Variable& y = matrixMultiply(a, w2);
            executor.backward(&y, hdy, false);
            y.fetch(hy);
            executor.clearInterimNodes();
        };
        for (int i = 0; i < 3; ++i) step();
        const unsigned long long l0 = d8k_launch_count();
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < steps; ++i) step();
        static_cast<GPUDevice*>(executor.getDevice())->synchronize();
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / steps;
        const double flop = 6.0 * 2.0 * rows * din * dhid;
        std::printf("{\"ms_per_step\": %.4f, \"tflops\": %.2f, \"steps\": %d, \"rows\": %zu, \"kernel_launches_per_step\": %.1f, "
                    "\"h2d_bytes_per_step\": %zu, \"d2h_bytes_per_step\": %zu, "
                    "\"path\": \"Deep8::Variable::feed -> EagerExecutor (fused launches, first-touch gradients) -> backward(host gradient) -> fetch; "
                    "synchronous copies, nothing overlapped\"}\n",
                    ms, flop / ms / 1e9, steps, rows, static_cast<double>(d8k_launch_count() - l0) / steps, 2 * rows * din * 2, rows * din * 2);
        return 0;
    } catch (const std::exception& e) {
        std::printf("{\"error\": \"%s\"}\n", e.what());
        return 1;
    }
}
