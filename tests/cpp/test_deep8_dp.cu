// Two (or more) processes, one GPU each: a batch-sharded x * w + b step through the C++ interface, the gradients of w and b
// summed over the ranks with Deep8::PeerGradientSum, then one SGDTrainer step.  Every rank rebuilds every rank's inputs from
// seeds and checks the summed gradients and the updated weights against the CPU oracle for equality (integer-valued data:
// any order of summation gives the same bits).   usage: test_deep8_dp <rendezvous dir> <rank> <world>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/deep8/Deep8.h"

extern "C" {
void d8o_matmul_grad_y_f32(const float* x, size_t xb, size_t xr, size_t xc, float* dy, size_t yb, size_t yc, const float* dz);
void d8o_add_bias_grad_f32(float* dbias, const float* dz, size_t rows, size_t cols);
void d8o_axpby_f32(const float* x, float alpha, const float* y, float beta, float* z, size_t n);
}

using namespace Deep8;

static std::vector<float> ints(unsigned seed, size_t n, int hi) {
    std::vector<float> v(n);
    unsigned s = seed * 2654435761u + 12345u;
    for (auto& e : v) {
        s = s * 1664525u + 1013904223u;
        e = static_cast<float>((s >> 16) % hi);
    }
    return v;
}

int main(int argc, char** argv) {
    if (argc != 4) {
        std::printf("usage: %s <dir> <rank> <world>\n", argv[0]);
        return 2;
    }
    const int rank = std::atoi(argv[2]), world = std::atoi(argv[3]);
    const size_t rows = 48, din = 40, dout = 72;
    try {
        EagerExecutor executor(DeviceType::GPU, rank);
        FileRendezvous rv(argv[1], rank, world, 60.0);
        Variable& x = parameter(&executor, {rows, din}, false);
        Variable& w = parameter(&executor, {din, dout});
        Variable& b = parameter(&executor, {dout});
        auto hw = ints(7, din * dout, 5), hb = ints(8, dout, 5);
        w.feed(hw.data());
        b.feed(hb.data());
        PeerGradientSum dp(&executor, &rv, {&w, &b}, 20000.0);
        ConstantLearningRateIterator lr(0.125f);
        SGDTrainer trainer(&lr, 0.5f);
        std::vector<float> rw = hw, rb = hb;
        int failed = 0;
        for (int step = 0; step < 3; ++step) {
            auto hx = ints(100 * step + rank, rows * din, 5), hdz = ints(1000 * step + rank, rows * dout, 5);
            x.feed(hx.data());
            Variable& z = x * w + b;
            executor.backward(&z, hdz.data(), true);
            dp.sum();
            dp.synchronize();
            // what every rank must now hold: the sum over the ranks of each rank's gradients
            std::vector<float> rdw(din * dout, 0.f), rdb(dout, 0.f);
            for (int q = 0; q < world; ++q) {
                auto qx = ints(100 * step + q, rows * din, 5), qdz = ints(1000 * step + q, rows * dout, 5);
                d8o_matmul_grad_y_f32(qx.data(), 1, rows, din, rdw.data(), 1, dout, qdz.data());
                d8o_add_bias_grad_f32(rdb.data(), qdz.data(), rows, dout);
            }
            std::vector<float> gdw(din * dout), gdb(dout);
            w.fetchGradient(gdw.data());
            b.fetchGradient(gdb.data());
            if (0 != std::memcmp(gdw.data(), rdw.data(), gdw.size() * 4) || 0 != std::memcmp(gdb.data(), rdb.data(), gdb.size() * 4)) {
                std::printf("rank %d step %d: summed gradients differ from the oracle\n", rank, step);
                ++failed;
            }
            trainer.train(&executor);
            float alpha = -1 * 0.125f, beta = (1.0 - 0.125f * 0.5f);
            d8o_axpby_f32(rdw.data(), alpha, rw.data(), beta, rw.data(), rw.size());
            d8o_axpby_f32(rdb.data(), alpha, rb.data(), beta, rb.data(), rb.size());
            std::vector<float> gw(hw.size()), gb(hb.size());
            w.fetch(gw.data());
            b.fetch(gb.data());
            if (0 != std::memcmp(gw.data(), rw.data(), gw.size() * 4) || 0 != std::memcmp(gb.data(), rb.data(), gb.size() * 4)) {
                std::printf("rank %d step %d: weights after the trainer step differ from the oracle\n", rank, step);
                ++failed;
            }
        }
        std::printf("rank %d: %s\n", rank, failed ? "FAILED" : "OK");
        return failed ? 1 : 0;
    } catch (const std::exception& e) {
        std::printf("rank %d: EXCEPTION %s\n", rank, e.what());
        return 1;
    }
}
