// GPU tests of the C++ host interface (include/deep8/Deep8.h) in the style of the reference's own node tests
// (test/MatrixMultiplyTest.h, test/Conv2dTest.h, test/DeConv2dTest.h): tensors of small integers ("rand() % 50"), the
// operator run through the node / executor interface, results compared for equality with the CPU oracle
// (oracle/d8_oracle.c, linked as a checker).  Prints one line per test; exits non-zero on the first failure.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "../../include/deep8/Deep8.h"

extern "C" {
void d8o_matmul_forward_f32(const float* x, size_t xb, size_t xr, size_t xc, const float* y, size_t yb, size_t yc, float* z);
void d8o_matmul_grad_x_f32(float* dx, size_t xb, size_t xr, size_t xc, const float* y, size_t yb, size_t yc, const float* dz);
void d8o_matmul_grad_y_f32(const float* x, size_t xb, size_t xr, size_t xc, float* dy, size_t yb, size_t yc, const float* dz);
void d8o_conv2d_forward_f32(const float* x, int b, int ih, int iw, int ic, const float* y, int oc, int fh, int fw, float* z, int oh, int ow,
                            int sy, int sx, int dy, int dx);
void d8o_conv2d_grad_x_f32(float* dx, int b, int ih, int iw, int ic, const float* y, int oc, int fh, int fw, const float* dz, int oh, int ow,
                           int sy, int sx, int dy, int dxx);
void d8o_conv2d_grad_y_f32(const float* x, int b, int ih, int iw, int ic, float* dy, int oc, int fh, int fw, const float* dz, int oh, int ow,
                           int sy, int sx, int dyy, int dx);
void d8o_deconv2d_forward_f32(const float* x, int b, int ih, int iw, int ic, const float* y, int oc, int fh, int fw, float* z, int oh, int ow,
                              int sy, int sx);
void d8o_deconv2d_grad_x_f32(float* dx, int b, int ih, int iw, int ic, const float* y, int oc, int fh, int fw, const float* dz, int oh, int ow,
                             int sy, int sx);
void d8o_deconv2d_grad_y_f32(const float* x, int b, int ih, int iw, int ic, float* dy, int oc, int fh, int fw, const float* dz, int oh, int ow,
                             int sy, int sx);
void d8o_add_bias_f32(const float* x, const float* bias, float* z, size_t rows, size_t cols);
void d8o_add_bias_grad_f32(float* dbias, const float* dz, size_t rows, size_t cols);
void d8o_axpby_f32(const float* x, float alpha, const float* y, float beta, float* z, size_t n);
void d8o_linear_f32(const float* x, float a, float b, float* y, size_t n);
void d8o_linear_grad_f32(float* dx, float a, const float* dy, size_t n);
void d8o_adam_update_f32(float* value, float* gradient, float* m, float* v, float beta1, float beta2, float epsilon, float weight_decay,
                         float ratio, size_t n);
}

using namespace Deep8;

static int g_failed = 0;
#define EXPECT(cond)                                                         \
    do {                                                                     \
        if (!(cond)) {                                                       \
            std::printf("  FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);  \
            ++g_failed;                                                      \
            return;                                                          \
        }                                                                    \
    } while (0)

static std::vector<float> ints(size_t n, int hi = 50) {
    std::vector<float> v(n);
    for (auto& e : v) e = static_cast<float>(std::rand() % hi);
    return v;
}

static bool same(const std::vector<float>& a, const std::vector<float>& b) {
    return a.size() == b.size() && 0 == std::memcmp(a.data(), b.data(), a.size() * sizeof(float));
}

// a tensor on `device` holding `host` (what test/TestUtils.h createTensor does)
static Tensor makeTensor(GPUDevice& device, size_t batch, std::vector<size_t> dims, const std::vector<float>& host) {
    Shape shape(batch, dims);
    size_t bytes = sizeof(float) * shape.size();
    void* ptr = device.malloc(bytes);
    auto ref = static_cast<size_t*>(device.mallocCPU(sizeof(size_t)));
    TensorStorage storage(ptr, ref, bytes, &device);
    device.copyFromCPUToGPU(host.data(), ptr, bytes);
    return Tensor(storage, 0, shape, ElementType::from<float>());
}

static std::vector<float> download(GPUDevice& device, const Tensor& t) {
    std::vector<float> host(t.size());
    device.synchronize();
    device.copyFromGPUToCPU(t.raw(), host.data(), t.byteCount());
    return host;
}

// ---- test/MatrixMultiplyTest.h GPU1_float / GPU2_float shapes at the Math:: level
static void matmulMath(size_t xb, size_t xr, size_t xc, size_t yb, size_t yc) {
    GPUDevice device;
    size_t zb = std::max(xb, yb);
    auto hx = ints(xb * xr * xc), hy = ints(yb * xc * yc), hdz = ints(zb * xr * yc), hdx0 = ints(xb * xr * xc), hdy0 = ints(yb * xc * yc);
    Tensor x = makeTensor(device, xb, {xr, xc}, hx), y = makeTensor(device, yb, {xc, yc}, hy);
    Tensor z = makeTensor(device, zb, {xr, yc}, std::vector<float>(zb * xr * yc, -1.f));
    Tensor dz = makeTensor(device, zb, {xr, yc}, hdz), dx = makeTensor(device, xb, {xr, xc}, hdx0), dy = makeTensor(device, yb, {xc, yc}, hdy0);
    Math::MatrixMultiply(x, y, z);
    Math::MatrixMultiplyGradX(x, dx, y, z, dz);
    Math::MatrixMultiplyGradY(x, y, dy, z, dz);
    std::vector<float> rz(zb * xr * yc), rdx = hdx0, rdy = hdy0;
    d8o_matmul_forward_f32(hx.data(), xb, xr, xc, hy.data(), yb, yc, rz.data());
    d8o_matmul_grad_x_f32(rdx.data(), xb, xr, xc, hy.data(), yb, yc, hdz.data());
    d8o_matmul_grad_y_f32(hx.data(), xb, xr, xc, rdy.data(), yb, yc, hdz.data());
    EXPECT(same(download(device, z), rz));
    EXPECT(same(download(device, dx), rdx));   // += on top of the initial gradient
    EXPECT(same(download(device, dy), rdy));
}

// ---- graph level: parameter, feed, x * w, relu, backward from a host gradient, fetch (README usage of the reference)
static void mlpGraph() {
    EagerExecutor executor(DeviceType::GPU);
    const size_t rows = 96, din = 40, dhid = 72;
    auto hx = ints(rows * din, 5), hw1 = ints(din * dhid, 5), hw2 = ints(dhid * din, 5), hdy = ints(rows * din, 5);
    for (auto& v : hw1) v -= 2.f;  // make the ReLU cut something
    Variable& x = parameter(&executor, {rows, din});
    Variable& w1 = parameter(&executor, {din, dhid});
    Variable& w2 = parameter(&executor, {dhid, din});
    x.feed(hx.data());
    w1.feed(hw1.data());
    w2.feed(hw2.data());
    Variable& h = x * w1;
    Variable& a = relu(h);
    Variable& yv = matrixMultiply(a, w2);
    std::vector<float> gy(rows * din);
    yv.fetch(gy.data());
    // oracle
    std::vector<float> rh(rows * dhid), ra(rows * dhid), ry(rows * din);
    d8o_matmul_forward_f32(hx.data(), 1, rows, din, hw1.data(), 1, dhid, rh.data());
    for (size_t i = 0; i < rh.size(); ++i) ra[i] = rh[i] > 0 ? rh[i] : 0;
    d8o_matmul_forward_f32(ra.data(), 1, rows, dhid, hw2.data(), 1, din, ry.data());
    EXPECT(same(gy, ry));
    executor.backward(&yv, hdy.data(), false);
    std::vector<float> rda(rows * dhid, 0.f), rdw2(dhid * din, 0.f), rdh(rows * dhid, 0.f), rdx(rows * din, 0.f), rdw1(din * dhid, 0.f);
    d8o_matmul_grad_x_f32(rda.data(), 1, rows, dhid, hw2.data(), 1, din, hdy.data());
    d8o_matmul_grad_y_f32(ra.data(), 1, rows, dhid, rdw2.data(), 1, din, hdy.data());
    for (size_t i = 0; i < rdh.size(); ++i) rdh[i] = rh[i] > 0 ? rda[i] : 0;
    d8o_matmul_grad_x_f32(rdx.data(), 1, rows, din, hw1.data(), 1, dhid, rdh.data());
    d8o_matmul_grad_y_f32(hx.data(), 1, rows, din, rdw1.data(), 1, dhid, rdh.data());
    std::vector<float> gdx(rows * din), gdw1(din * dhid), gdw2(dhid * din);
    x.fetchGradient(gdx.data());
    w1.fetchGradient(gdw1.data());
    w2.fetchGradient(gdw2.data());
    EXPECT(same(gdx, rdx));
    EXPECT(same(gdw1, rdw1));
    EXPECT(same(gdw2, rdw2));
    EXPECT(executor.trainableParameters().size() == 3);
    executor.clearInterimNodes();
}

template <typename E>
static bool throws(const std::function<void()>& f);

// ---- the same MLP step with the executor's fusion and first-touch gradients on and off: every fetched tensor identical, and
// the fused step launches exactly its six contractions
struct MlpRun {
    std::vector<float> h, a, y, dx, dw1, dw2;
    unsigned long long forwardLaunches, backwardLaunches;
};
static MlpRun runMlp(bool fusion, bool firstTouch, const std::vector<float>& hx, const std::vector<float>& hw1, const std::vector<float>& hw2,
                     const std::vector<float>& hdy, size_t rows, size_t din, size_t dhid) {
    EagerExecutor executor(DeviceType::GPU);
    executor.setFusion(fusion);
    executor.setFirstTouch(firstTouch);
    Variable& x = parameter(&executor, {rows, din});
    Variable& w1 = parameter(&executor, {din, dhid});
    Variable& w2 = parameter(&executor, {dhid, din});
    x.feed(hx.data());
    w1.feed(hw1.data());
    w2.feed(hw2.data());
    MlpRun r;
    unsigned long long l0 = d8k_launch_count();
    Variable& h = x * w1;
    Variable& a = relu(h);
    Variable& yv = matrixMultiply(a, w2);
    executor.flush();
    r.forwardLaunches = d8k_launch_count() - l0;
    l0 = d8k_launch_count();
    executor.backward(&yv, hdy.data(), false);
    r.backwardLaunches = d8k_launch_count() - l0;
    r.h.resize(rows * dhid); r.a.resize(rows * dhid); r.y.resize(rows * din);
    r.dx.resize(rows * din); r.dw1.resize(din * dhid); r.dw2.resize(dhid * din);
    h.fetch(r.h.data());
    a.fetch(r.a.data());
    yv.fetch(r.y.data());
    x.fetchGradient(r.dx.data());
    w1.fetchGradient(r.dw1.data());
    w2.fetchGradient(r.dw2.data());
    executor.clearInterimNodes();
    return r;
}
static void fusedExecutorEqualsNodeByNode() {
    const size_t rows = 200, din = 72, dhid = 136;
    std::vector<float> hx(rows * din), hw1(din * dhid), hw2(dhid * din), hdy(rows * din);
    for (auto& v : hx) v = (std::rand() % 2001 - 1000) / 1000.f;     // real-valued data: the roundings must agree too
    for (auto& v : hw1) v = (std::rand() % 2001 - 1000) / 4000.f;
    for (auto& v : hw2) v = (std::rand() % 2001 - 1000) / 4000.f;
    for (auto& v : hdy) v = (std::rand() % 2001 - 1000) / 1000.f;
    MlpRun plain = runMlp(false, false, hx, hw1, hw2, hdy, rows, din, dhid);
    MlpRun fused = runMlp(true, true, hx, hw1, hw2, hdy, rows, din, dhid);
    EXPECT(same(plain.h, fused.h));
    EXPECT(same(plain.a, fused.a));
    EXPECT(same(plain.y, fused.y));
    EXPECT(same(plain.dx, fused.dx));
    EXPECT(same(plain.dw1, fused.dw1));
    EXPECT(same(plain.dw2, fused.dw2));
    EXPECT(plain.forwardLaunches == 3);                 // product, ReLu, product
    EXPECT(fused.forwardLaunches == 2);                 // product with ReLu inside, product
    EXPECT(fused.backwardLaunches == 4);                // dA (+ ReLu gradient), dW2, dX, dW1: no zero fill, no ReLuGrad launch
    EXPECT(plain.backwardLaunches == 5);                // + ReLuGrad (the zero fills are memsets, not kernels)
    MlpRun touchOnly = runMlp(false, true, hx, hw1, hw2, hdy, rows, din, dhid);
    EXPECT(same(plain.dx, touchOnly.dx) && same(plain.dw1, touchOnly.dw1) && same(plain.dw2, touchOnly.dw2));
}

// ---- Linear node after a product (one launch), its gradient, and AdamTrainer on the weights: equal to the oracle
static void linearNodeAndAdam() {
    EagerExecutor executor(DeviceType::GPU);
    const size_t rows = 40, din = 24, dout = 56;
    auto hx = ints(rows * din, 5), hw = ints(din * dout, 5), hdz = ints(rows * dout, 5);
    Variable& x = parameter(&executor, {rows, din}, false);
    Variable& w = parameter(&executor, {din, dout});
    x.feed(hx.data());
    w.feed(hw.data());
    unsigned long long l0 = d8k_launch_count();
    Variable& p = x * w;
    Variable& l = linear(p, 0.5f, -3.f);
    EXPECT(d8k_launch_count() - l0 == 1);               // the product ran with Linear in its epilogue
    std::vector<float> gp(rows * dout), gl(rows * dout), rp(rows * dout), rl(rows * dout);
    p.fetch(gp.data());
    l.fetch(gl.data());
    d8o_matmul_forward_f32(hx.data(), 1, rows, din, hw.data(), 1, dout, rp.data());
    d8o_linear_f32(rp.data(), 0.5f, -3.f, rl.data(), rl.size());
    EXPECT(same(gp, rp));
    EXPECT(same(gl, rl));
    executor.backward(&l, hdz.data(), false);
    std::vector<float> rdp(rows * dout, 0.f), rdw(din * dout, 0.f), gdw(din * dout);
    d8o_linear_grad_f32(rdp.data(), 0.5f, hdz.data(), rdp.size());
    d8o_matmul_grad_y_f32(hx.data(), 1, rows, din, rdw.data(), 1, dout, rdp.data());
    w.fetchGradient(gdw.data());
    EXPECT(same(gdw, rdw));
    // two AdamTrainer steps on w with the same gradient
    ConstantLearningRateIterator lr(0.0078125f);
    AdamTrainer trainer(&lr, 0.875f, 0.9990234375f, 1.f / 1048576.f, 0.00048828125f);
    std::vector<float> rw = hw, rg = rdw, rm(hw.size(), 0.f), rv(hw.size(), 0.f), gw(hw.size());
    for (int step = 0; step < 2; ++step) {
        trainer.train(&executor);
        d8o_adam_update_f32(rw.data(), rg.data(), rm.data(), rv.data(), 0.875f, 0.9990234375f, 1.f / 1048576.f, 0.00048828125f,
                            d8k_adam_ratio(0.0078125f, 0.875f, 0.9990234375f, step), rw.size());
        w.fetch(gw.data());
        EXPECT(same(gw, rw));
    }
    EXPECT(trainer.m.size() == 1 && trainer.v.size() == 1);
    executor.clearInterimNodes();
}

// ---- inputs through a CopyStream, upstream gradient from a device tensor: the same numbers as feed + backward(host gradient)
static void copyStreamStepEqualsSynchronousStep() {
    EagerExecutor executor(DeviceType::GPU);
    auto dev = static_cast<GPUDevice*>(executor.getDevice());
    const size_t rows = 96, din = 64, dout = 80;
    auto hx = ints(rows * din, 5), hw = ints(din * dout, 5), hdz = ints(rows * dout, 5);
    Variable& x = parameter(&executor, {rows, din});
    Variable& w = parameter(&executor, {din, dout});
    Variable& dzv = parameter(&executor, {rows, dout}, false);
    Variable& zkeep = parameter(&executor, {rows, dout}, false);
    w.feed(hw.data());
    // synchronous reference
    x.feed(hx.data());
    Variable& z0 = x * w;
    executor.backward(&z0, hdz.data(), false);
    std::vector<float> rz(rows * dout), rdx(rows * din), rdw(din * dout);
    z0.fetch(rz.data());
    x.fetchGradient(rdx.data());
    w.fetchGradient(rdw.data());
    executor.clearInterimNodes();
    // the same step with the copies on a second stream (page-locked host buffers)
    float *px, *pdz, *pz;
    cudaHostAlloc(&px, hx.size() * 4, cudaHostAllocDefault);
    cudaHostAlloc(&pdz, hdz.size() * 4, cudaHostAllocDefault);
    cudaHostAlloc(&pz, rz.size() * 4, cudaHostAllocDefault);
    std::copy(hx.begin(), hx.end(), px);
    std::copy(hdz.begin(), hdz.end(), pdz);
    x.zero();
    CopyStream copies(dev);
    copies.waitFor(copies.markExecutor());  // x.zero() above was the executor's
    copies.toDevice(px, x.value);
    copies.toDevice(pdz, dzv.value);
    copies.executorWaitsFor(copies.mark());
    Variable& z1 = x * w;
    executor.backward(&z1, dzv.value, false);
    copyOnExecutorStream(z1.value, zkeep.value);
    executor.clearInterimNodes();
    copies.waitFor(copies.markExecutor());
    copies.toHost(zkeep.value, pz);
    copies.synchronize();
    std::vector<float> gz(pz, pz + rz.size()), gdx(rows * din), gdw(din * dout);
    x.fetchGradient(gdx.data());
    w.fetchGradient(gdw.data());
    EXPECT(same(gz, rz));
    EXPECT(same(gdx, rdx));
    EXPECT(same(gdw, rdw));
    cudaFreeHost(px);
    cudaFreeHost(pdz);
    cudaFreeHost(pz);
}

// ---- x * w + b in one launch leaves the product unstored; asking for it, or using it again, computes it
static void fusedBiasKeepsTheProductAvailable() {
    EagerExecutor executor(DeviceType::GPU);
    const size_t rows = 33, din = 20, dout = 48;
    auto hx = ints(rows * din, 5), hw = ints(din * dout, 5), hb = ints(dout, 5);
    Variable& x = parameter(&executor, {rows, din}, false);
    Variable& w = parameter(&executor, {din, dout});
    Variable& b = parameter(&executor, {dout});
    x.feed(hx.data());
    w.feed(hw.data());
    b.feed(hb.data());
    unsigned long long l0 = d8k_launch_count();
    Variable& p = x * w;
    Variable& z = p + b;
    EXPECT(d8k_launch_count() - l0 == 1);
    EXPECT(p.valueStale);
    std::vector<float> rp(rows * dout), rz(rows * dout), gz(rows * dout), gp(rows * dout), gq(rows * dout);
    d8o_matmul_forward_f32(hx.data(), 1, rows, din, hw.data(), 1, dout, rp.data());
    d8o_add_bias_f32(rp.data(), hb.data(), rz.data(), rows, dout);
    z.fetch(gz.data());
    EXPECT(same(gz, rz));
    Variable& q = relu(p);          // a second consumer of the product: it is computed now
    EXPECT(!p.valueStale);
    p.fetch(gp.data());
    q.fetch(gq.data());
    EXPECT(same(gp, rp));
    for (size_t i = 0; i < gq.size(); ++i) EXPECT(gq[i] == (rp[i] > 0 ? rp[i] : 0));
    executor.clearInterimNodes();
}

// ---- z = x * w + b through the nodes, backward, then one SGDTrainer step: every tensor equal to the oracle's
static void linearWithBiasAndSgd() {
    EagerExecutor executor(DeviceType::GPU);
    const size_t batch = 3, rows = 40, din = 24, dout = 56;
    auto hx = ints(batch * rows * din, 5), hw = ints(din * dout, 5), hb = ints(dout, 5), hdz = ints(batch * rows * dout, 5);
    Variable& x = parameter(&executor, batch, {rows, din}, false);
    Variable& w = parameter(&executor, {din, dout});
    Variable& b = parameter(&executor, {dout});
    x.feed(hx.data());
    w.feed(hw.data());
    b.feed(hb.data());
    Variable& z = x * w + b;
    std::vector<float> gz(batch * rows * dout), rz(gz.size()), rmm(gz.size());
    z.fetch(gz.data());
    d8o_matmul_forward_f32(hx.data(), batch, rows, din, hw.data(), 1, dout, rmm.data());
    d8o_add_bias_f32(rmm.data(), hb.data(), rz.data(), batch * rows, dout);
    EXPECT(same(gz, rz));
    executor.backward(&z, hdz.data(), false);
    std::vector<float> rdw(din * dout, 0.f), rdb(dout, 0.f), gdw(din * dout), gdb(dout);
    d8o_matmul_grad_y_f32(hx.data(), batch, rows, din, rdw.data(), 1, dout, hdz.data());
    d8o_add_bias_grad_f32(rdb.data(), hdz.data(), batch * rows, dout);
    w.fetchGradient(gdw.data());
    b.fetchGradient(gdb.data());
    EXPECT(same(gdw, rdw));
    EXPECT(same(gdb, rdb));
    EXPECT(executor.trainableParameters().size() == 2);
    // SGDTrainer::update: value = gradient * (-lr) + value * (1 - lr * decay)
    ConstantLearningRateIterator lr(0.125f);
    SGDTrainer trainer(&lr, 0.5f);
    trainer.train(&executor);
    float alpha = -1 * 0.125f, beta = (1.0 - 0.125f * 0.5f);
    std::vector<float> rw(hw.size()), rb(hb.size()), gw(hw.size()), gb(hb.size());
    d8o_axpby_f32(rdw.data(), alpha, hw.data(), beta, rw.data(), rw.size());
    d8o_axpby_f32(rdb.data(), alpha, hb.data(), beta, rb.data(), rb.size());
    w.fetch(gw.data());
    b.fetch(gb.data());
    EXPECT(same(gw, rw));
    EXPECT(same(gb, rb));
    // equal shapes add too
    Variable& p = parameter(&executor, {7, 9});
    Variable& q = parameter(&executor, {7, 9});
    auto hp = ints(63, 9), hq = ints(63, 9);
    p.feed(hp.data());
    q.feed(hq.data());
    Variable& r = p + q;
    std::vector<float> gr(63);
    r.fetch(gr.data());
    for (size_t i = 0; i < 63; ++i) EXPECT(gr[i] == hp[i] + hq[i]);
    Variable& bad = parameter(&executor, {9, 7});
    EXPECT(throws<std::invalid_argument>([&] { p + bad; }));
    executor.clearInterimNodes();
}

// ---- test/Conv2dTest.h forwardGPU_float / backwardGPU_float through the node
static void convNode(size_t b, size_t ih, size_t iw, size_t ic, size_t oc, size_t fh, size_t fw, bool covered, int s, int d) {
    EagerExecutor executor(DeviceType::GPU);
    auto hx = ints(b * ih * iw * ic, 20), hw = ints(oc * fh * fw * ic, 20);
    Variable& x = parameter(&executor, b, {ih, iw, ic});
    Variable& w = parameter(&executor, {oc, fh, fw, ic});
    x.feed(hx.data());
    w.feed(hw.data());
    Variable& z = conv2d(x, w, covered, s, s, d, d);
    Shape zs = z.shape();
    int oh = (int)zs.dim(0), ow = (int)zs.dim(1);
    std::vector<float> gz(zs.size()), rz(zs.size());
    z.fetch(gz.data());
    d8o_conv2d_forward_f32(hx.data(), (int)b, (int)ih, (int)iw, (int)ic, hw.data(), (int)oc, (int)fh, (int)fw, rz.data(), oh, ow, s, s, d, d);
    EXPECT(same(gz, rz));
    auto hdz = ints(zs.size(), 20);
    executor.backward(&z, hdz.data(), false);
    std::vector<float> rdx(hx.size(), 0.f), rdw(hw.size(), 0.f), gdx(hx.size()), gdw(hw.size());
    d8o_conv2d_grad_x_f32(rdx.data(), (int)b, (int)ih, (int)iw, (int)ic, hw.data(), (int)oc, (int)fh, (int)fw, hdz.data(), oh, ow, s, s, d, d);
    d8o_conv2d_grad_y_f32(hx.data(), (int)b, (int)ih, (int)iw, (int)ic, rdw.data(), (int)oc, (int)fh, (int)fw, hdz.data(), oh, ow, s, s, d, d);
    x.fetchGradient(gdx.data());
    w.fetchGradient(gdw.data());
    EXPECT(same(gdx, rdx));
    EXPECT(same(gdw, rdw));
}

// ---- test/DeConv2dTest.h forwarGPU_float / backwarGPU_float through the node
static void deconvNode(size_t b, size_t ih, size_t iw, size_t ic, size_t oc, size_t fh, size_t fw, bool covered, int s) {
    EagerExecutor executor(DeviceType::GPU);
    auto hx = ints(b * ih * iw * ic, 20), hw = ints(oc * fh * fw * ic, 20);
    Variable& x = parameter(&executor, b, {ih, iw, ic});
    Variable& w = parameter(&executor, {oc, fh, fw, ic});
    x.feed(hx.data());
    w.feed(hw.data());
    Variable& z = deConv2d(x, w, covered, s, s);
    Shape zs = z.shape();
    int oh = (int)zs.dim(0), ow = (int)zs.dim(1);
    std::vector<float> gz(zs.size()), rz(zs.size());
    z.fetch(gz.data());
    d8o_deconv2d_forward_f32(hx.data(), (int)b, (int)ih, (int)iw, (int)ic, hw.data(), (int)oc, (int)fh, (int)fw, rz.data(), oh, ow, s, s);
    EXPECT(same(gz, rz));
    auto hdz = ints(zs.size(), 20);
    executor.backward(&z, hdz.data(), false);
    std::vector<float> rdx(hx.size(), 0.f), rdw(hw.size(), 0.f), gdx(hx.size()), gdw(hw.size());
    d8o_deconv2d_grad_x_f32(rdx.data(), (int)b, (int)ih, (int)iw, (int)ic, hw.data(), (int)oc, (int)fh, (int)fw, hdz.data(), oh, ow, s, s);
    d8o_deconv2d_grad_y_f32(hx.data(), (int)b, (int)ih, (int)iw, (int)ic, rdw.data(), (int)oc, (int)fh, (int)fw, hdz.data(), oh, ow, s, s);
    x.fetchGradient(gdx.data());
    w.fetchGradient(gdw.data());
    EXPECT(same(gdx, rdx));
    EXPECT(same(gdw, rdw));
}

// ---- the buddy pool contract (deep8/src/model/GPUMemoryPool.cu:132-279)
static void memoryPool() {
    GPUMemoryPool pool(0, static_cast<size_t>(1) << 24);  // 16 MiB blocks keep the test small
    EXPECT(pool.malloc(0) == nullptr);
    char* a = static_cast<char*>(pool.malloc(100));     // rounds to 128
    char* b = static_cast<char*>(pool.malloc(128));
    char* c = static_cast<char*>(pool.malloc(129));     // rounds to 256
    EXPECT(a && b && c && pool.blockCount() == 1);
    EXPECT(pool.bytesInUse() == 128 + 128 + 256);
    EXPECT((reinterpret_cast<uintptr_t>(c) & 255) == 0);   // a chunk is aligned to its own size
    EXPECT(b == a + 128);                                  // buddies
    pool.free(a);
    pool.free(b);
    char* d = static_cast<char*>(pool.malloc(256));     // the two freed buddies merged
    EXPECT(d == a);
    pool.free(c);
    pool.free(d);
    EXPECT(pool.bytesInUse() == 0);
    char* whole = static_cast<char*>(pool.malloc(static_cast<size_t>(1) << 24));   // everything merged back: one whole block fits
    EXPECT(whole && pool.blockCount() == 1);
    char* more = static_cast<char*>(pool.malloc(1024));  // needs a second block
    EXPECT(more && pool.blockCount() == 2);
    pool.free(whole);
    pool.free(more);
    bool threw = false;
    try {
        pool.malloc((static_cast<size_t>(1) << 24) + 1);  // larger than a block: "malloc too much memory"
    } catch (const std::invalid_argument&) {
        threw = true;
    }
    EXPECT(threw);
}

template <typename E>
static bool throws(const std::function<void()>& f) {
    try {
        f();
    } catch (const E&) {
        return true;
    } catch (...) {
        return false;
    }
    return false;
}

// ---- error behaviour: std::invalid_argument for argument checks, std::runtime_error for the rest
static void errors() {
    EXPECT(throws<std::runtime_error>([] { EagerExecutor cpu(DeviceType::CPU); }));
    EagerExecutor executor(DeviceType::GPU);
    Variable& x = parameter(&executor, {8, 16});
    Variable& bad = parameter(&executor, {15, 4});
    EXPECT(throws<std::invalid_argument>([&] { x * bad; }));                        // "the col of input1 must same to the row of input2"
    Variable& xb = parameter(&executor, 2, {8, 16});
    Variable& yb = parameter(&executor, 3, {16, 4});
    EXPECT(throws<std::invalid_argument>([&] { xb * yb; }));                        // "the batch of input is error"
    Variable& y = parameter(&executor, {16, 4});
    Variable& z = x * y;
    EXPECT(throws<std::invalid_argument>([&] { backward(z); }));                    // "the last Variable gradient must be scalar"
    Variable& dx = parameter(&executor, {8, 16}, true, DType::Float64);
    Variable& dy = parameter(&executor, {16, 4}, true, DType::Float64);
    EXPECT(throws<std::runtime_error>([&] { dx * dy; }));                           // "type double is not support"
    Variable& img = parameter(&executor, 1, {5, 5, 3});
    Variable& flt = parameter(&executor, {4, 7, 7, 3});
    EXPECT(throws<std::invalid_argument>([&] { conv2d(img, flt, false); }));        // filter larger than the image, not covered
    // scalar loss path of the reference: a 1x1 product can be differentiated without a supplied gradient
    Variable& p = parameter(&executor, {1, 4});
    Variable& q = parameter(&executor, {4, 1});
    float hp[4] = {1, 2, 3, 4}, hq[4] = {5, 6, 7, 8}, gp[4];
    p.feed(hp);
    q.feed(hq);
    Variable& s = p * q;
    backward(s, false);
    p.fetchGradient(gp);
    EXPECT(gp[0] == 5 && gp[1] == 6 && gp[2] == 7 && gp[3] == 8);
}

int main() {
    std::srand(1234);
    struct Case {
        const char* name;
        std::function<void()> run;
    };
    std::vector<Case> cases = {
        {"matmul Math:: x[10,400,200] * y[1,200,300] (test/MatrixMultiplyTest.h GPU1_float)", [] { matmulMath(10, 400, 200, 1, 300); }},
        {"matmul Math:: x[1,300,100] * y[10,100,1] (GPU2_float)", [] { matmulMath(1, 300, 100, 10, 1); }},
        {"matmul Math:: x[3,17,5] * y[3,5,9] (per-batch branch)", [] { matmulMath(3, 17, 5, 3, 9); }},
        {"graph: parameter, feed, x*w1, relu, *w2, backward(host gradient), fetch", mlpGraph},
        {"graph: x*w + b, backward, SGDTrainer step (Add, AddGradY, AXPBY)", linearWithBiasAndSgd},
        {"executor: fused launches + first-touch gradients equal the node-by-node walk bit for bit; launch counts", fusedExecutorEqualsNodeByNode},
        {"graph: linear(x*w) in one launch, LinearGrad, AdamTrainer steps", linearNodeAndAdam},
        {"graph: x*w + b in one launch, the unstored product computed on demand", fusedBiasKeepsTheProductAvailable},
        {"CopyStream: inputs and outputs on a second stream, backward from a device gradient, equal to feed / fetch", copyStreamStepEqualsSynchronousStep},
        {"Conv2d node 2x32x32x64, 4x4x64->32, covered, stride 2, dilation 2 (test/Conv2dTest.h)", [] { convNode(2, 32, 32, 64, 32, 4, 4, true, 2, 2); }},
        {"Conv2d node 2x32x32x64, 5x5, covered, stride 1", [] { convNode(2, 32, 32, 64, 32, 5, 5, true, 1, 1); }},
        {"Conv2d node not covered, stride 2, dilation 2", [] { convNode(2, 32, 32, 64, 32, 4, 4, false, 2, 2); }},
        {"DeConv2d node 2x32x32x64, 4x4, not covered, stride 3 (test/DeConv2dTest.h)", [] { deconvNode(2, 32, 32, 64, 32, 4, 4, false, 3); }},
        {"DeConv2d node covered, stride 3", [] { deconvNode(2, 32, 32, 64, 32, 4, 4, true, 3); }},
        {"GPUMemoryPool buddy contract", memoryPool},
        {"error behaviour", errors},
    };
    for (auto& c : cases) {
        int before = g_failed;
        try {
            c.run();
        } catch (const std::exception& e) {
            std::printf("  EXCEPTION: %s\n", e.what());
            ++g_failed;
        }
        std::printf("[%s] %s\n", g_failed == before ? "  OK  " : "FAILED", c.name);
        std::fflush(stdout);
    }
    std::printf("%d failed\n", g_failed);
    return g_failed ? 1 : 0;
}
