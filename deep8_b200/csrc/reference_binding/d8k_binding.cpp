// What a maintainer of the reference project adds to put libdeep8_b200.so behind Deep8's GPU functions: this one file
// replaces the `...GPU` definitions of deep8/src/math/MatrixMultiply.cu, Conv2d.cu and DeConv2d.cu (drop those three from the
// build, compile this file with -DHAVE_CUDA [-DHAVE_HALF], link -ldeep8_b200).  It is written against the reference's OWN
// headers, unmodified: tests/test_binding.py compiles it (syntax check, no GPU) with the reference's include directories, and
// the static_asserts below make that compilation fail when a signature of the reference
// (deep8/include/math/MatrixMultiply.h:17,26,35, Conv2d.h:24,35,46, DeConv2d.h:18,28,39) and a stub disagree.
//
// The d8k context stands where GPUDevice keeps its cuBLAS handle (deep8/include/model/GPUDevice.h:19-20).  With the
// header left as it is, the contexts live in a table beside the devices; a maintainer who edits GPUDevice.h keeps a
// `d8k_ctx* kernels` member instead and creates it where cublasCreate is called (deep8/src/model/GPUDevice.cu:10-65).
#include <mutex>
#include <stdexcept>
#include <type_traits>
#include <unordered_map>

#include "basic/GPUBasic.h"
#include "model/GPUDevice.h"
#include "math/MatrixMultiply.h"
#include "math/Conv2d.h"
#include "math/DeConv2d.h"

#include "d8k.h"

#ifndef HAVE_CUDA
#error "compile with -DHAVE_CUDA: the functions defined here are declared under it"
#endif

namespace Deep8 {
namespace Math {

namespace {

void d8kCheck(int rc) {
    if (rc == D8K_ERR_ARGUMENT) throw std::invalid_argument(d8k_last_error());  // the type DEEP8_ARGUMENT_CHECK throws
    if (rc != D8K_OK) throw std::runtime_error(d8k_last_error());               // the type DEEP8_RUNTIME_ERROR throws
}

int d8kType(const Tensor& t) {
    switch (t.elementType.id) {
    case DType::Float32:
        return D8K_F32;
#ifdef HAVE_HALF
    case DType::Float16:
        return D8K_F16;
#endif
    default:
        DEEP8_RUNTIME_ERROR("type " << t.elementType.name << " is not support");  // deep8/src/math/MatrixMultiply.cu:172-174
    }
}

d8k_ctx* kernelsOf(const Tensor& t) {
    static std::mutex lock;
    static std::unordered_map<int, d8k_ctx*> table;  // one context per GPU, for the life of the process
    auto device = static_cast<GPUDevice*>(t.device());
    std::lock_guard<std::mutex> guard(lock);
    auto it = table.find(device->deviceId);
    if (it != table.end()) return it->second;
    d8k_ctx* ctx = nullptr;
    d8kCheck(d8k_ctx_create(device->deviceId, 0, &ctx));
    table[device->deviceId] = ctx;
    return ctx;
}

struct Geometry {
    int batch, ih, iw, ic, oc, fh, fw, oh, ow;
};
Geometry geometry(const Tensor& x, const Tensor& y, const Tensor& z) {
    return Geometry{(int)x.batch(), (int)x.dim(0), (int)x.dim(1), (int)x.dim(2), (int)y.dim(0), (int)y.dim(1), (int)y.dim(2), (int)z.dim(0),
                    (int)z.dim(1)};
}

}  // namespace

// ---- deep8/src/math/MatrixMultiply.cu:139-176, 320-363, 508-551
void MatrixMultiplyGPU(const Tensor& x, const Tensor& y, Tensor& z) {
    d8kCheck(d8k_matmul_forward(kernelsOf(x), d8kType(x), x.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), y.raw(), (int)y.batch(),
                                (int)y.col(), z.raw()));
}
void MatrixMultiplyGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz) {
    d8kCheck(d8k_matmul_grad_x(kernelsOf(x), d8kType(x), dx.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), y.raw(), (int)y.batch(),
                               (int)y.col(), dz.raw()));
}
void MatrixMultiplyGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz) {
    d8kCheck(d8k_matmul_grad_y(kernelsOf(x), d8kType(x), x.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), dy.raw(), (int)y.batch(),
                               (int)y.col(), dz.raw()));
}

// ---- The GPU branch of the six ...InterimSize functions (deep8/src/math/Conv2d.cpp:42, 135, 232; DeConv2d.cpp:39, 118, 198):
// the maintainer returns these instead of the column-buffer size.  Same parameter lists as the reference's functions.
size_t d8kConv2dInterimSize(const Tensor& x, const Tensor& y, Tensor& z, bool, int, int, int, int) {
    Geometry g = geometry(x, y, z);
    return d8k_conv2d_interim_size(kernelsOf(x), 0, d8kType(x), g.batch, g.ih, g.iw, g.ic, g.oc, g.fh, g.fw, g.oh, g.ow);
}
size_t d8kConv2dGradXInterimSize(const Tensor& x, Tensor&, const Tensor& y, const Tensor& z, const Tensor&, bool, int, int, int, int) {
    Geometry g = geometry(x, y, z);
    return d8k_conv2d_interim_size(kernelsOf(x), 1, d8kType(x), g.batch, g.ih, g.iw, g.ic, g.oc, g.fh, g.fw, g.oh, g.ow);
}
size_t d8kConv2dGradYInterimSize(const Tensor& x, const Tensor& y, Tensor&, const Tensor& z, const Tensor&, bool, int, int, int, int) {
    Geometry g = geometry(x, y, z);
    return d8k_conv2d_interim_size(kernelsOf(x), 2, d8kType(x), g.batch, g.ih, g.iw, g.ic, g.oc, g.fh, g.fw, g.oh, g.ow);
}
size_t d8kDeConv2dInterimSize(const Tensor& x, const Tensor& y, Tensor& z, bool, int, int) {
    Geometry g = geometry(x, y, z);
    return d8k_deconv2d_interim_size(kernelsOf(x), 0, d8kType(x), g.batch, g.ih, g.iw, g.ic, g.oc, g.fh, g.fw, g.oh, g.ow);
}
size_t d8kDeConv2dGradXInterimSize(const Tensor& x, Tensor&, const Tensor& y, const Tensor& z, const Tensor&, bool, int, int) {
    Geometry g = geometry(x, y, z);
    return d8k_deconv2d_interim_size(kernelsOf(x), 1, d8kType(x), g.batch, g.ih, g.iw, g.ic, g.oc, g.fh, g.fw, g.oh, g.ow);
}
size_t d8kDeConv2dGradYInterimSize(const Tensor& x, const Tensor& y, Tensor&, const Tensor& z, const Tensor&, bool, int, int) {
    Geometry g = geometry(x, y, z);
    return d8k_deconv2d_interim_size(kernelsOf(x), 2, d8kType(x), g.batch, g.ih, g.iw, g.ic, g.oc, g.fh, g.fw, g.oh, g.ow);
}

// ---- deep8/src/math/Conv2d.cu:308-411, 607-721, 917-1031.  `covered` is already folded into z's shape by the node
// (deep8/src/nodes/Conv2d.cpp:47-63); the kernels derive the padding from the shapes as Conv2dGPU does.
void Conv2dGPU(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int strideY, int strideX, int dilationY, int dilationX, void* xcol) {
    Geometry g = geometry(x, y, z);
    d8kCheck(d8k_conv2d_forward(kernelsOf(x), d8kType(x), x.raw(), g.batch, g.ih, g.iw, g.ic, y.raw(), g.oc, g.fh, g.fw, z.raw(), g.oh, g.ow,
                                strideY, strideX, dilationY, dilationX, xcol,
                                xcol ? d8kConv2dInterimSize(x, y, z, covered, strideY, strideX, dilationY, dilationX) : 0));
}
void Conv2dGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX,
                    int dilationY, int dilationX, void* dxcol) {
    Geometry g = geometry(x, y, z);
    d8kCheck(d8k_conv2d_grad_x(kernelsOf(x), d8kType(x), dx.raw(), g.batch, g.ih, g.iw, g.ic, y.raw(), g.oc, g.fh, g.fw, dz.raw(), g.oh, g.ow,
                               strideY, strideX, dilationY, dilationX, dxcol,
                               dxcol ? d8kConv2dGradXInterimSize(x, dx, y, z, dz, covered, strideY, strideX, dilationY, dilationX) : 0));
}
void Conv2dGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX,
                    int dilationY, int dilationX, void* xcol) {
    Geometry g = geometry(x, y, z);
    d8kCheck(d8k_conv2d_grad_y(kernelsOf(x), d8kType(x), x.raw(), g.batch, g.ih, g.iw, g.ic, dy.raw(), g.oc, g.fh, g.fw, dz.raw(), g.oh, g.ow,
                               strideY, strideX, dilationY, dilationX, xcol,
                               xcol ? d8kConv2dGradYInterimSize(x, y, dy, z, dz, covered, strideY, strideX, dilationY, dilationX) : 0));
}

// ---- deep8/src/math/DeConv2d.cu:251-308, 557-622, 826-891
void DeConv2dGPU(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int strideY, int strideX, void* interimPtr) {
    Geometry g = geometry(x, y, z);
    d8kCheck(d8k_deconv2d_forward(kernelsOf(x), d8kType(x), x.raw(), g.batch, g.ih, g.iw, g.ic, y.raw(), g.oc, g.fh, g.fw, z.raw(), g.oh, g.ow,
                                  strideY, strideX, interimPtr, interimPtr ? d8kDeConv2dInterimSize(x, y, z, covered, strideY, strideX) : 0));
}
void DeConv2dGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX,
                      void* interimPtr) {
    Geometry g = geometry(x, y, z);
    d8kCheck(d8k_deconv2d_grad_x(kernelsOf(x), d8kType(x), dx.raw(), g.batch, g.ih, g.iw, g.ic, y.raw(), g.oc, g.fh, g.fw, dz.raw(), g.oh, g.ow,
                                 strideY, strideX, interimPtr,
                                 interimPtr ? d8kDeConv2dGradXInterimSize(x, dx, y, z, dz, covered, strideY, strideX) : 0));
}
void DeConv2dGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX,
                      void* interimPtr) {
    Geometry g = geometry(x, y, z);
    d8kCheck(d8k_deconv2d_grad_y(kernelsOf(x), d8kType(x), x.raw(), g.batch, g.ih, g.iw, g.ic, dy.raw(), g.oc, g.fh, g.fw, dz.raw(), g.oh, g.ow,
                                 strideY, strideX, interimPtr,
                                 interimPtr ? d8kDeConv2dGradYInterimSize(x, y, dy, z, dz, covered, strideY, strideX) : 0));
}

// ---- The definitions above must BE the functions the reference's headers declare.  Taking the address of an overloaded name
// is ill-formed, so a stub whose parameter list drifted from the header (which would silently add an overload) stops the
// compilation here; so does a stub of the right name with another type.
#define D8K_SAME_SIGNATURE(stub, reference) \
    static_assert(std::is_same<decltype(&stub), decltype(&reference)>::value, #stub " and " #reference " take different arguments")
static_assert(std::is_same<decltype(&MatrixMultiplyGPU), void (*)(const Tensor&, const Tensor&, Tensor&)>::value, "MatrixMultiplyGPU");
static_assert(std::is_same<decltype(&MatrixMultiplyGradXGPU), void (*)(const Tensor&, Tensor&, const Tensor&, const Tensor&, const Tensor&)>::value,
              "MatrixMultiplyGradXGPU");
static_assert(std::is_same<decltype(&MatrixMultiplyGradYGPU), void (*)(const Tensor&, const Tensor&, Tensor&, const Tensor&, const Tensor&)>::value,
              "MatrixMultiplyGradYGPU");
static_assert(std::is_same<decltype(&Conv2dGPU), void (*)(const Tensor&, const Tensor&, Tensor&, bool, int, int, int, int, void*)>::value, "Conv2dGPU");
static_assert(std::is_same<decltype(&Conv2dGradXGPU),
                           void (*)(const Tensor&, Tensor&, const Tensor&, const Tensor&, const Tensor&, bool, int, int, int, int, void*)>::value,
              "Conv2dGradXGPU");
static_assert(std::is_same<decltype(&Conv2dGradYGPU),
                           void (*)(const Tensor&, const Tensor&, Tensor&, const Tensor&, const Tensor&, bool, int, int, int, int, void*)>::value,
              "Conv2dGradYGPU");
static_assert(std::is_same<decltype(&DeConv2dGPU), void (*)(const Tensor&, const Tensor&, Tensor&, bool, int, int, void*)>::value, "DeConv2dGPU");
static_assert(std::is_same<decltype(&DeConv2dGradXGPU),
                           void (*)(const Tensor&, Tensor&, const Tensor&, const Tensor&, const Tensor&, bool, int, int, void*)>::value,
              "DeConv2dGradXGPU");
static_assert(std::is_same<decltype(&DeConv2dGradYGPU),
                           void (*)(const Tensor&, const Tensor&, Tensor&, const Tensor&, const Tensor&, bool, int, int, void*)>::value,
              "DeConv2dGradYGPU");
D8K_SAME_SIGNATURE(d8kConv2dInterimSize, Conv2dInterimSize);
D8K_SAME_SIGNATURE(d8kConv2dGradXInterimSize, Conv2dGradXInterimSize);
D8K_SAME_SIGNATURE(d8kConv2dGradYInterimSize, Conv2dGradYInterimSize);
D8K_SAME_SIGNATURE(d8kDeConv2dInterimSize, DeConv2dInterimSize);
D8K_SAME_SIGNATURE(d8kDeConv2dGradXInterimSize, DeConv2dGradXInterimSize);
D8K_SAME_SIGNATURE(d8kDeConv2dGradYInterimSize, DeConv2dGradYInterimSize);

}  // namespace Math
}  // namespace Deep8
