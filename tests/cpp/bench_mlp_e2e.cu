// The benchmark's MLP step through the C++ interface, end to end: every step feeds X from pinned host memory (Variable::feed),
// builds H = X W1, A = ReLu(H), Y = A W2 on the executor (fused launches), runs backward from a host gradient dY, and
// fetches Y back (Variable::fetch).  feed and fetch are synchronous copies, as in the reference (deep8/src/nodes/Variable.cpp),
// so nothing overlaps: this is what a user of the reference's interface gets without touching streams.
// With a third argument `overlap` the same step runs with its copies on two Deep8::CopyStream objects: the inputs of step
// i + 1 travel while step i computes, Y of step i travels while step i + 1 computes (double-buffered X, dY and Y).
// Prints one JSON object.   usage: bench_mlp_e2e [steps] [rows] [overlap]
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>
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
        if (argc > 3 && std::string(argv[3]) == "overlap") {
            auto dev = static_cast<GPUDevice*>(executor.getDevice());
            Variable* xs[2] = {&x, &parameter(&executor, {rows, din}, true, DType::Float16)};
            Variable* dys[2] = {&parameter(&executor, {rows, din}, false, DType::Float16), &parameter(&executor, {rows, din}, false, DType::Float16)};
            Variable* ys[2] = {&parameter(&executor, {rows, din}, false, DType::Float16), &parameter(&executor, {rows, din}, false, DType::Float16)};
            half_t* hys[2] = {hy, nullptr};
            cudaHostAlloc(&hys[1], rows * din * 2, cudaHostAllocDefault);
            CopyStream in(dev), out(dev);
            void* fed[2] = {nullptr, nullptr};     // inputs of parity p are on the device
            void* fetched[2] = {nullptr, nullptr};  // Y of parity p has reached the host
            void* done = nullptr;                   // the previous step is enqueued up to here
            in.toDevice(hx, xs[0]->value);
            in.toDevice(hdy, dys[0]->value);
            fed[0] = in.mark();
            auto ostep = [&](int i) {
                const int p = i & 1;
                // the next step's inputs: their buffers were last read by step i - 1
                if (done) in.waitFor(done);
                in.toDevice(hx, xs[p ^ 1]->value);
                in.toDevice(hdy, dys[p ^ 1]->value);
                fed[p ^ 1] = in.mark();
                in.executorWaitsFor(fed[p]);
                Variable& h = *xs[p] * w1;
                Variable& a = relu(h);
                Variable& y = matrixMultiply(a, w2);
                executor.backward(&y, dys[p]->value, false);
                if (fetched[p]) out.executorWaitsFor(fetched[p]);  // Y of step i - 2 has left this buffer
                copyOnExecutorStream(y.value, ys[p]->value);
                executor.clearInterimNodes();
                done = in.markExecutor();
                out.waitFor(done);
                out.toHost(ys[p]->value, hys[p]);
                fetched[p] = out.mark();
            };
            for (int i = 0; i < 4; ++i) ostep(i);
            out.synchronize();
            dev->synchronize();
            const unsigned long long l0 = d8k_launch_count();
            const auto t0 = std::chrono::steady_clock::now();
            for (int i = 0; i < steps; ++i) ostep(i);
            out.synchronize();
            in.synchronize();
            dev->synchronize();
            const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / steps;
            const double flop = 6.0 * 2.0 * rows * din * dhid;
            // the same Y must come out of every step (same inputs): compare the two host buffers
            size_t differ = 0;
            for (size_t k = 0; k < rows * din; ++k) differ += hys[0][k].bits != hys[1][k].bits;
            std::printf("{\"ms_per_step\": %.4f, \"tflops\": %.2f, \"steps\": %d, \"rows\": %zu, \"kernel_launches_per_step\": %.1f, "
                        "\"h2d_bytes_per_step\": %zu, \"d2h_bytes_per_step\": %zu, \"y_buffers_differ\": %zu, "
                        "\"path\": \"Deep8::CopyStream (inputs of the next step and Y of the previous one travel beside the kernels) -> EagerExecutor "
                        "(fused launches, first-touch gradients) -> backward(device gradient)\"}\n",
                        ms, flop / ms / 1e9, steps, rows, static_cast<double>(d8k_launch_count() - l0) / steps, 2 * rows * din * 2, rows * din * 2, differ);
            return differ == 0 ? 0 : 2;
        }
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
