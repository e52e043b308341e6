// TEST INFRASTRUCTURE, not product code.
//
// C wrapper around the UNMODIFIED reference CPU implementation of the dense-contraction path
// (Deep8::Math::MatrixMultiply*/Conv2d*/DeConv2d*, deep8/src/math/{MatrixMultiply,Conv2d,DeConv2d}.cpp).
// The reference sources are compiled where they lie by oracle/Makefile and linked with this file into
// oracle/_ref/libd8ref.so.  Only tests, the smoke check and the benchmark's CPU-baseline leg may load it.
//
// Every entry point takes plain host pointers and dims.  dtype: 0 = float, 1 = double.
// Tensors are views over the caller's buffers: the storage refcount is pinned so that the reference's
// TensorStorage never hands a foreign pointer to its memory pool (deep8/src/model/TensorStorage.cpp:27-35).
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "model/Device.h"
#include "model/ElementType.h"
#include "model/Shape.h"
#include "model/Tensor.h"
#include "model/TensorStorage.h"
#include "math/MatrixMultiply.h"
#include "math/Conv2d.h"
#include "math/DeConv2d.h"
#include "math/AXPBY.h"
#include "math/Add.h"
#include "math/ReLu.h"
#include "math/Linear.h"
#include "math/AdamUpdate.h"

#define D8REF_API extern "C" __attribute__((visibility("default")))

namespace {

Deep8::CPUDevice* g_device = nullptr;
thread_local std::string g_error;

Deep8::CPUDevice* device() {
    if (!g_device) g_device = new Deep8::CPUDevice();
    return g_device;
}

Deep8::ElementType etype(int dtype) {
    return dtype == 0 ? Deep8::ElementType::from<float>() : Deep8::ElementType::from<double>();
}

struct View {
    size_t ref;
    Deep8::Tensor tensor;

    View(int dtype, const void* ptr, size_t batch, std::vector<size_t> dims) : ref(0) {
        Deep8::Shape shape(batch, dims);
        auto type = etype(dtype);
        Deep8::TensorStorage storage(const_cast<void*>(ptr), &ref, type.byteWidth * shape.size(), device());
        ref += (size_t(1) << 40);  // never reaches zero: the buffer belongs to the caller
        tensor = Deep8::Tensor(storage, 0, shape, type);
    }
};

std::vector<size_t> mat_dims(int ndims, size_t row, size_t col) {
    if (ndims == 1) return {row};
    return {row, col};
}

template <typename F>
int guarded(F f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    } catch (...) {
        g_error = "unknown exception";
        return 1;
    }
}

}  // namespace

D8REF_API const char* d8ref_last_error() { return g_error.c_str(); }

// threads of the reference's Eigen pool: sysconf(_SC_NPROCESSORS_CONF), deep8/src/model/Device.cpp:67-85.
// MatrixMultiply never uses the pool (dense Eigen::Map product, single thread).
D8REF_API int d8ref_threads() { return static_cast<int>(sysconf(_SC_NPROCESSORS_CONF)); }

// which: 0 = forward (z written), 1 = grad x (dx +=), 2 = grad y (dy +=).
// x: (xb, {xr, xc}) or (xb, {xr}) when xnd == 1; likewise y.  z: (max(xb, yb), {xr} if yc == 1 && ynd... see
// deep8/src/nodes/MatrixMultiply.cpp:10-28: z is 1-D when y.col() == 1, else 2-D.
D8REF_API int d8ref_matmul(int which, int dtype,
                           const void* x, void* dx, size_t xb, int xnd, size_t xr, size_t xc,
                           const void* y, void* dy, size_t yb, int ynd, size_t yr, size_t yc,
                           void* z, const void* dz) {
    return guarded([&] {
        size_t zb = xb > yb ? xb : yb;
        std::vector<size_t> zdims = (yc == 1) ? std::vector<size_t>{xr} : std::vector<size_t>{xr, yc};
        View vx(dtype, x, xb, mat_dims(xnd, xr, xc));
        View vy(dtype, y, yb, mat_dims(ynd, yr, yc));
        View vz(dtype, z, zb, zdims);
        if (which == 0) {
            Deep8::Math::MatrixMultiply(vx.tensor, vy.tensor, vz.tensor);
        } else if (which == 1) {
            View vdx(dtype, dx, xb, mat_dims(xnd, xr, xc));
            View vdz(dtype, dz, zb, zdims);
            Deep8::Math::MatrixMultiplyGradX(vx.tensor, vdx.tensor, vy.tensor, vz.tensor, vdz.tensor);
        } else {
            View vdy(dtype, dy, yb, mat_dims(ynd, yr, yc));
            View vdz(dtype, dz, zb, zdims);
            Deep8::Math::MatrixMultiplyGradY(vx.tensor, vy.tensor, vdy.tensor, vz.tensor, vdz.tensor);
        }
    });
}

// x: (b, {ih, iw, ic}); y: (1, {oc, fh, fw, ic}); z: (b, {oh, ow, oc}).
D8REF_API int d8ref_conv2d(int which, int dtype,
                           const void* x, void* dx, size_t b, size_t ih, size_t iw, size_t ic,
                           const void* y, void* dy, size_t oc, size_t fh, size_t fw,
                           void* z, const void* dz, size_t oh, size_t ow,
                           int covered, int strideY, int strideX, int dilationY, int dilationX) {
    return guarded([&] {
        View vx(dtype, x, b, {ih, iw, ic});
        View vy(dtype, y, 1, {oc, fh, fw, ic});
        View vz(dtype, z, b, {oh, ow, oc});
        if (which == 0) {
            Deep8::Math::Conv2d(vx.tensor, vy.tensor, vz.tensor, covered != 0, strideY, strideX, dilationY, dilationX, nullptr);
        } else if (which == 1) {
            View vdx(dtype, dx, b, {ih, iw, ic});
            View vdz(dtype, dz, b, {oh, ow, oc});
            Deep8::Math::Conv2dGradX(vx.tensor, vdx.tensor, vy.tensor, vz.tensor, vdz.tensor, covered != 0, strideY, strideX,
                                     dilationY, dilationX, nullptr);
        } else {
            View vdy(dtype, dy, 1, {oc, fh, fw, ic});
            View vdz(dtype, dz, b, {oh, ow, oc});
            Deep8::Math::Conv2dGradY(vx.tensor, vy.tensor, vdy.tensor, vz.tensor, vdz.tensor, covered != 0, strideY, strideX,
                                     dilationY, dilationX, nullptr);
        }
    });
}

D8REF_API int d8ref_deconv2d(int which, int dtype,
                             const void* x, void* dx, size_t b, size_t ih, size_t iw, size_t ic,
                             const void* y, void* dy, size_t oc, size_t fh, size_t fw,
                             void* z, const void* dz, size_t oh, size_t ow,
                             int covered, int strideY, int strideX) {
    return guarded([&] {
        View vx(dtype, x, b, {ih, iw, ic});
        View vy(dtype, y, 1, {oc, fh, fw, ic});
        View vz(dtype, z, b, {oh, ow, oc});
        if (which == 0) {
            Deep8::Math::DeConv2d(vx.tensor, vy.tensor, vz.tensor, covered != 0, strideY, strideX, nullptr);
        } else if (which == 1) {
            View vdx(dtype, dx, b, {ih, iw, ic});
            View vdz(dtype, dz, b, {oh, ow, oc});
            Deep8::Math::DeConv2dGradX(vx.tensor, vdx.tensor, vy.tensor, vz.tensor, vdz.tensor, covered != 0, strideY, strideX, nullptr);
        } else {
            View vdy(dtype, dy, 1, {oc, fh, fw, ic});
            View vdz(dtype, dz, b, {oh, ow, oc});
            Deep8::Math::DeConv2dGradY(vx.tensor, vy.tensor, vdy.tensor, vz.tensor, vdz.tensor, covered != 0, strideY, strideX, nullptr);
        }
    });
}

// Math::AXPBY (deep8/src/math/AXPBY.cpp:6-20): z = x * alpha + y * beta over n elements; z may alias x or y.
// This is the arithmetic of SGDTrainer::update (deep8/src/trainer/SGDTrainer.cpp:9-17).
D8REF_API int d8ref_axpby(int dtype, const void* x, float alpha, const void* y, float beta, void* z, size_t n) {
    return guarded([&] {
        View vx(dtype, x, 1, {n});
        View vy(dtype, y, 1, {n});
        View vz(dtype, z, 1, {n});
        Deep8::Math::AXPBY(vx.tensor, alpha, vy.tensor, beta, vz.tensor);
    });
}

// Math::Add / Math::AddGradY (deep8/src/math/Add.cpp:7-31, 71-110) for x (batch, {rows, cols}) and a bias y (1, {cols}).
// which: 0 = z = x + y; 2 = dy += sum of dz over batch and rows.
D8REF_API int d8ref_add_bias(int which, int dtype, const void* x, size_t batch, size_t rows, size_t cols, const void* y, void* dy, void* z,
                             const void* dz) {
    return guarded([&] {
        View vx(dtype, x, batch, {rows, cols});
        View vy(dtype, y, 1, {cols});
        View vz(dtype, z, batch, {rows, cols});
        if (which == 0) {
            Deep8::Math::Add(vx.tensor, vy.tensor, vz.tensor);
        } else {
            View vdy(dtype, dy, 1, {cols});
            View vdz(dtype, dz, batch, {rows, cols});
            Deep8::Math::AddGradY(vx.tensor, vy.tensor, vdy.tensor, vz.tensor, vdz.tensor);
        }
    });
}

// Math::ReLu / Math::ReLuGrad (deep8/src/math/ReLu.cpp:6-37).  which: 0 = y = max(x, 0); 1 = dx += (x > 0 ? dy : 0).
D8REF_API int d8ref_relu(int which, int dtype, const void* x, void* dx, void* y, const void* dy, size_t n) {
    return guarded([&] {
        View vx(dtype, x, 1, {n});
        View vy(dtype, y, 1, {n});
        if (which == 0) {
            Deep8::Math::ReLu(vx.tensor, vy.tensor);
        } else {
            View vdx(dtype, dx, 1, {n});
            View vdy(dtype, dy, 1, {n});
            Deep8::Math::ReLuGrad(vx.tensor, vdx.tensor, vy.tensor, vdy.tensor);
        }
    });
}

// Math::Linear / Math::LinearGrad (deep8/src/math/Linear.cpp:9-44).  which: 0 = y = x * a + b; 1 = dx += dy * a.
D8REF_API int d8ref_linear(int which, int dtype, const void* x, void* dx, float a, float b, void* y, const void* dy, size_t n) {
    return guarded([&] {
        View vx(dtype, x, 1, {n});
        View vy(dtype, y, 1, {n});
        if (which == 0) {
            Deep8::Math::Linear(vx.tensor, a, b, vy.tensor);
        } else {
            View vdx(dtype, dx, 1, {n});
            View vdy(dtype, dy, 1, {n});
            Deep8::Math::LinearGrad(vx.tensor, vdx.tensor, a, b, vy.tensor, vdy.tensor);
        }
    });
}

// Math::AdamUpdate (deep8/src/math/AdamUpdate.cpp:6-22): value, gradient, m and v are all updated in place.
D8REF_API int d8ref_adam_update(int dtype, void* value, void* gradient, void* m, void* v, float beta1, float beta2, float epsilon,
                                float learningRate, float weightDecay, long long steps, size_t n) {
    return guarded([&] {
        View vv(dtype, value, 1, {n});
        View vg(dtype, gradient, 1, {n});
        View vm(dtype, m, 1, {n});
        View vs(dtype, v, 1, {n});
        Deep8::Math::AdamUpdate(vv.tensor, vg.tensor, vm.tensor, vs.tensor, beta1, beta2, epsilon, learningRate, weightDecay, steps);
    });
}
