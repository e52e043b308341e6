// Implementation of include/deep8/Deep8.h: Deep8's operator / executor / device interface for the path, over the C ABI.
#include "../../../include/deep8/Deep8.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <queue>

namespace Deep8 {

namespace {

#define D8_CUDA_CHECK(call)                                                        \
    {                                                                              \
        cudaError_t d8_e__ = (call);                                               \
        if (d8_e__ != cudaSuccess) DEEP8_RUNTIME_ERROR("CUDA error: " << cudaGetErrorString(d8_e__)); \
    }

// D8K_ERR_ARGUMENT is the reference's std::invalid_argument, anything else its std::runtime_error
void d8kCheck(int rc) {
    if (rc == D8K_OK) return;
    if (rc == D8K_ERR_ARGUMENT) throw std::invalid_argument(d8k_last_error());
    throw std::runtime_error(d8k_last_error());
}

int d8kType(const Tensor& t) {
    switch (t.elementType.id) {
    case DType::Float32: return D8K_F32;
    case DType::Float16: return D8K_F16;
    default: DEEP8_RUNTIME_ERROR("type " << t.elementType.name << " is not support");
    }
}

GPUDevice* gpuOf(const Tensor& t) {
    DEEP8_ARGUMENT_CHECK(t.device() != nullptr && DeviceType::GPU == t.deviceType(), "the tensor must live on a GPU device");
    return static_cast<GPUDevice*>(t.device());
}

}  // namespace

// ================================================================================================ ElementType
ElementType ElementType::from(DType type) {
    switch (type) {
    case DType::Bool: return ElementType(type, 1, "bool");
    case DType::Uint8: return ElementType(type, 1, "uint8_t");
    case DType::Int8: return ElementType(type, 1, "int8_t");
    case DType::Uint16: return ElementType(type, 2, "uint16_t");
    case DType::Int16: return ElementType(type, 2, "int16_t");
    case DType::Uint32: return ElementType(type, 4, "uint32_t");
    case DType::Int32: return ElementType(type, 4, "int32_t");
    case DType::Uint64: return ElementType(type, 8, "uint64_t");
    case DType::Int64: return ElementType(type, 8, "int64_t");
    case DType::Float16: return ElementType(type, 2, "float16");
    case DType::Float32: return ElementType(type, 4, "float");
    case DType::Float64: return ElementType(type, 8, "double");
    default: return unknown();
    }
}

// ================================================================================================ Shape
Shape::Shape() : batch(0), nDims(0) {
    std::memset(dims, 0, sizeof(dims));
    std::memset(strides, 0, sizeof(strides));
}

Shape::Shape(size_t b, const Shape& other) : Shape(other) { batch = b; }

Shape::Shape(std::vector<size_t> list) : Shape(1, std::move(list)) {}

Shape::Shape(size_t b, std::vector<size_t> list) : batch(b), nDims(list.size()) {
    DEEP8_ARGUMENT_CHECK(list.size() <= MAX_TENSOR_DIMS, "the dim of a Tensor must not bigger than " << MAX_TENSOR_DIMS);
    DEEP8_ARGUMENT_CHECK(b > 0, "the batch must > 0");
    std::memset(dims, 0, sizeof(dims));
    for (size_t i = 0; i < list.size(); ++i) {
        DEEP8_ARGUMENT_CHECK(list[i] > 0, "the dim must > 0");
        dims[i] = list[i];
    }
    updateStrides();
}

void Shape::updateStrides() {
    std::memset(strides, 0, sizeof(strides));
    size_t s = 1;
    for (size_t i = nDims; i-- > 0;) {
        strides[i] = s;
        s *= dims[i];
    }
}

bool Shape::operator==(const Shape& o) const {
    if (batch != o.batch || nDims != o.nDims) return false;
    for (size_t i = 0; i < nDims; ++i)
        if (dims[i] != o.dims[i]) return false;
    return true;
}

bool Shape::equalExceptBatch(const Shape& o) const {
    if (nDims != o.nDims) return false;
    for (size_t i = 0; i < nDims; ++i)
        if (dims[i] != o.dims[i]) return false;
    return true;
}

size_t Shape::batchSize() const {
    size_t s = 1;
    for (size_t i = 0; i < nDims; ++i) s *= dims[i];
    return s;
}

size_t Shape::size() const { return batch * batchSize(); }

size_t Shape::dim(size_t d) const {
    DEEP8_ARGUMENT_CHECK(d < nDims, "the dim is out of the range");
    return dims[d];
}

size_t Shape::stride(size_t d) const {
    DEEP8_ARGUMENT_CHECK(d < nDims, "the dim is out of the range");
    return strides[d];
}

size_t Shape::row() const {
    DEEP8_ARGUMENT_CHECK(nDims >= 1, "the dimensions is error");
    return dims[0];
}

size_t Shape::col() const {
    DEEP8_ARGUMENT_CHECK(nDims >= 1, "the dimensions is error");
    return 1 == nDims ? 1 : dims[1];
}

void Shape::reShape(Shape& other) {
    DEEP8_ARGUMENT_CHECK(size() == other.size(), "the reShape operator needs this 2 Shape have the same size");
    *this = other;
}

std::string Shape::toStr() const {
    std::ostringstream oss;
    oss << "(" << batch;
    for (size_t i = 0; i < nDims; ++i) oss << ", " << dims[i];
    oss << ")";
    return oss.str();
}

// ================================================================================================ GPUMemoryPool
static constexpr size_t kMinChunk = 128;  // DEFAULT_MEMORY_MIN_SIZE of the reference (deep8/include/model/MemoryPool.h:13-23)

int GPUMemoryPool::levelFor(size_t size) {
    int level = 0;
    size_t s = kMinChunk;
    while (s < size) {
        s <<= 1;
        ++level;
    }
    return level;
}

GPUMemoryPool::GPUMemoryPool(int id, size_t blockSize) : deviceId(id), gpuBlockSize(blockSize) {
    DEEP8_ARGUMENT_CHECK(blockSize >= kMinChunk && (blockSize & (blockSize - 1)) == 0, "the block size must be a power of two >= 128");
    maxLevel = levelFor(blockSize);
    freeByLevel.resize(maxLevel + 1);
}

GPUMemoryPool::~GPUMemoryPool() {
    cudaSetDevice(deviceId);
    for (char* b : blocks) cudaFree(b);
}

void GPUMemoryPool::addBlock() {
    D8_CUDA_CHECK(cudaSetDevice(deviceId));
    char* p = nullptr;
    D8_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&p), gpuBlockSize));
    blocks.push_back(p);
    freeByLevel[maxLevel][{blocks.size() - 1, 0}] = true;
}

void* GPUMemoryPool::malloc(size_t size) {
    if (0 == size) return nullptr;
    DEEP8_ARGUMENT_CHECK(size <= gpuBlockSize, "malloc too much memory");
    const int want = levelFor(size);
    int level = want;
    while (level <= maxLevel && freeByLevel[level].empty()) ++level;
    if (level > maxLevel) {
        addBlock();
        level = maxLevel;
    }
    auto it = freeByLevel[level].begin();
    Chunk c{it->first.first, it->first.second, level};
    freeByLevel[level].erase(it);
    while (c.level > want) {  // split: keep the lower half, free the upper half
        --c.level;
        freeByLevel[c.level][{c.block, c.offset + (kMinChunk << c.level)}] = true;
    }
    void* p = blocks[c.block] + c.offset;
    live[p] = c;
    inUse += kMinChunk << c.level;
    return p;
}

void GPUMemoryPool::free(void* ptr) {
    if (nullptr == ptr) return;
    auto it = live.find(ptr);
    DEEP8_ARGUMENT_CHECK(it != live.end(), "free a pointer that this pool did not allocate");
    Chunk c = it->second;
    live.erase(it);
    inUse -= kMinChunk << c.level;
    while (c.level < maxLevel) {  // merge with the buddy while it is free
        size_t sz = kMinChunk << c.level;
        size_t buddy = c.offset ^ sz;
        auto b = freeByLevel[c.level].find({c.block, buddy});
        if (b == freeByLevel[c.level].end()) break;
        freeByLevel[c.level].erase(b);
        c.offset = std::min(c.offset, buddy);
        ++c.level;
    }
    freeByLevel[c.level][{c.block, c.offset}] = true;
}

void GPUMemoryPool::zero(void* ptr, size_t size) {
    D8_CUDA_CHECK(cudaSetDevice(deviceId));
    D8_CUDA_CHECK(cudaMemset(ptr, 0, size));
}
void GPUMemoryPool::copy(const void* from, void* to, size_t size) { copyFromGPUToGPU(from, to, size); }
void GPUMemoryPool::copyFromCPUToGPU(const void* from, void* to, size_t size) {
    D8_CUDA_CHECK(cudaSetDevice(deviceId));
    D8_CUDA_CHECK(cudaMemcpy(to, from, size, cudaMemcpyHostToDevice));
}
void GPUMemoryPool::copyFromGPUToCPU(const void* from, void* to, size_t size) {
    D8_CUDA_CHECK(cudaSetDevice(deviceId));
    D8_CUDA_CHECK(cudaMemcpy(to, from, size, cudaMemcpyDeviceToHost));
}
void GPUMemoryPool::copyFromGPUToGPU(const void* from, void* to, size_t size) {
    D8_CUDA_CHECK(cudaSetDevice(deviceId));
    D8_CUDA_CHECK(cudaMemcpy(to, from, size, cudaMemcpyDeviceToDevice));
}
void* GPUMemoryPool::mallocCPU(size_t size) { return std::malloc(size); }
void GPUMemoryPool::freeCPU(void* ptr) { std::free(ptr); }

std::string GPUMemoryPool::toString() const {
    std::ostringstream oss;
    oss << "GPUMemoryPool(device " << deviceId << ", " << blocks.size() << " block(s) of " << gpuBlockSize << " bytes, " << inUse
        << " bytes in use, " << live.size() << " live chunk(s))";
    return oss.str();
}
void GPUMemoryPool::printInfo() const { std::cout << toString() << std::endl; }

// ================================================================================================ GPUDevice
GPUDevice::GPUDevice() : GPUDevice(0) {}

GPUDevice::GPUDevice(int id, size_t poolBlockSize) : Device(DeviceType::GPU), memoryPool(nullptr), deviceId(id), kernels(nullptr) {
    D8_CUDA_CHECK(cudaSetDevice(deviceId));
    d8kCheck(d8k_ctx_create(deviceId, 0, &kernels));
    memoryPool = new GPUMemoryPool(deviceId, poolBlockSize);
}

GPUDevice::~GPUDevice() {
    cudaSetDevice(deviceId);
    cudaDeviceSynchronize();
    delete memoryPool;
    d8k_ctx_destroy(kernels);
}

void* GPUDevice::malloc(size_t size) { return memoryPool->malloc(size); }
void GPUDevice::free(void* ptr) { memoryPool->free(ptr); }
void* GPUDevice::mallocCPU(size_t size) { return memoryPool->mallocCPU(size); }
void GPUDevice::freeCPU(void* ptr) { memoryPool->freeCPU(ptr); }
void GPUDevice::zero(void* ptr, size_t size) { memoryPool->zero(ptr, size); }
void GPUDevice::copy(const void* from, void* to, size_t size) { memoryPool->copy(from, to, size); }
void GPUDevice::copyFromCPUToGPU(const void* from, void* to, size_t size) { memoryPool->copyFromCPUToGPU(from, to, size); }
void GPUDevice::copyFromGPUToCPU(const void* from, void* to, size_t size) { memoryPool->copyFromGPUToCPU(from, to, size); }
void GPUDevice::copyFromGPUToGPU(const void* from, void* to, size_t size) { memoryPool->copyFromGPUToGPU(from, to, size); }
void GPUDevice::synchronize() {
    int status = 0;
    d8kCheck(d8k_ctx_status(kernels, &status));
}

// ================================================================================================ TensorStorage / Tensor
TensorStorage::TensorStorage() : ptr(nullptr), refPtr(nullptr), size(0), device(nullptr) {}

TensorStorage::TensorStorage(void* p, size_t* refP, size_t s, Device* d) : ptr(p), refPtr(refP), size(s), device(d) {
    DEEP8_ARGUMENT_CHECK(nullptr != p && nullptr != refP && s > 0 && nullptr != d, "the memory is error");
    *refPtr = 1;
}

TensorStorage::TensorStorage(const TensorStorage& o) : ptr(o.ptr), refPtr(o.refPtr), size(o.size), device(o.device) {
    if (refPtr) ++(*refPtr);
}

TensorStorage::~TensorStorage() { release(); }

TensorStorage& TensorStorage::operator=(const TensorStorage& o) {
    if (o.refPtr) ++(*o.refPtr);
    release();
    ptr = o.ptr;
    refPtr = o.refPtr;
    size = o.size;
    device = o.device;
    return *this;
}

void TensorStorage::release() {
    if (refPtr && 0 == --(*refPtr)) {
        device->free(ptr);
        device->freeCPU(refPtr);
    }
    ptr = nullptr;
    refPtr = nullptr;
    size = 0;
    device = nullptr;
}

Tensor::Tensor() : storage(), offset(0), shape(), elementType(ElementType::unknown()) {}
Tensor::Tensor(Shape& s) : storage(), offset(0), shape(s), elementType(ElementType::unknown()) {}
Tensor::Tensor(TensorStorage& ts, size_t off, Shape& s, ElementType et) : storage(ts), offset(off), shape(s), elementType(et) {}
Tensor::Tensor(TensorStorage& ts, size_t off, std::vector<size_t>& list, ElementType et) : Tensor(ts, off, 1, list, et) {}
Tensor::Tensor(TensorStorage& ts, size_t off, size_t batch, std::vector<size_t>& list, ElementType et)
    : storage(ts), offset(off), shape(batch, list), elementType(et) {}

DeviceType Tensor::deviceType() const {
    DEEP8_ARGUMENT_CHECK(storage.device != nullptr, "the tensor has no storage");
    return storage.device->type;
}
Device* Tensor::device() const { return storage.device; }
void* Tensor::raw() const { return static_cast<char*>(storage.ptr) + offset; }
bool Tensor::isScalar() const { return 1 == shape.size(); }
size_t Tensor::byteCount() const { return elementType.byteWidth * shape.size(); }
void Tensor::zero() { Math::Constant(*this, 0); }

// ================================================================================================ Math
namespace Math {

namespace {
thread_local bool g_overwriteGradient = false;
int accumulateFlag() { return g_overwriteGradient ? 0 : 1; }
}  // namespace
OverwriteGradient::OverwriteGradient(bool on) : previous(g_overwriteGradient) { g_overwriteGradient = on; }
OverwriteGradient::~OverwriteGradient() { g_overwriteGradient = previous; }
bool OverwriteGradient::active() { return g_overwriteGradient; }

namespace {
void checkMatMul(const Tensor& x, const Tensor& y, const Tensor& z) {
    DEEP8_ARGUMENT_CHECK(x.deviceType() == y.deviceType() && x.deviceType() == z.deviceType(), "the device type must be same");
    DEEP8_ARGUMENT_CHECK(x.elementType == y.elementType && x.elementType == z.elementType, "the data type must be same");
    DEEP8_ARGUMENT_CHECK(1 == x.shape.batch || x.shape.batch == z.shape.batch, "the shape is error");
    DEEP8_ARGUMENT_CHECK(1 == y.shape.batch || y.shape.batch == z.shape.batch, "the shape is error");
    DEEP8_ARGUMENT_CHECK((1 == x.shape.nDims || 2 == x.shape.nDims) && (1 == y.shape.nDims || 2 == y.shape.nDims) &&
                             (1 == z.shape.nDims || 2 == z.shape.nDims),
                         "the shape is error");
    DEEP8_ARGUMENT_CHECK(x.shape.row() == z.shape.row() && y.shape.col() == z.shape.col() && x.shape.col() == y.shape.row(),
                         "the shape is error");
}
}  // namespace

void MatrixMultiply(const Tensor& x, const Tensor& y, Tensor& z) {
    checkMatMul(x, y, z);
    MatrixMultiplyGPU(x, y, z);
}
void MatrixMultiplyGPU(const Tensor& x, const Tensor& y, Tensor& z) {
    d8kCheck(d8k_matmul_forward(gpuOf(x)->kernels, d8kType(x), x.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), y.raw(), (int)y.batch(),
                                (int)y.col(), z.raw()));
}
void MatrixMultiplyGradX(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz) {
    checkMatMul(x, y, z);
    DEEP8_ARGUMENT_CHECK(x.elementType == dx.elementType && x.elementType == dz.elementType, "the data type must be same");
    DEEP8_ARGUMENT_CHECK(x.shape == dx.shape && z.shape == dz.shape, "the shape is error");
    MatrixMultiplyGradXGPU(x, dx, y, z, dz);
}
void MatrixMultiplyGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor&, const Tensor& dz) {
    d8kCheck(d8k_matmul_grad_x_into(gpuOf(x)->kernels, d8kType(x), dx.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), y.raw(),
                                    (int)y.batch(), (int)y.col(), dz.raw(), accumulateFlag()));
}
void MatrixMultiplyGradY(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz) {
    checkMatMul(x, y, z);
    DEEP8_ARGUMENT_CHECK(x.elementType == dy.elementType && x.elementType == dz.elementType, "the data type must be same");
    DEEP8_ARGUMENT_CHECK(y.shape == dy.shape && z.shape == dz.shape, "the shape is error");
    MatrixMultiplyGradYGPU(x, y, dy, z, dz);
}
void MatrixMultiplyGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor&, const Tensor& dz) {
    d8kCheck(d8k_matmul_grad_y_into(gpuOf(x)->kernels, d8kType(x), x.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), dy.raw(),
                                    (int)y.batch(), (int)y.col(), dz.raw(), accumulateFlag()));
}

namespace {
struct ConvGeom {
    int batch, ih, iw, ic, oc, fh, fw, oh, ow;
};

// the checks of Math::Conv2d (deep8/src/math/Conv2d.cpp:46-96): dtypes, ranks, and z's shape against the shape rule
ConvGeom convGeom(const Tensor& x, const Tensor& y, const Tensor& z, bool covered, int strideY, int strideX, int dilationY, int dilationX) {
    DEEP8_ARGUMENT_CHECK(x.elementType == y.elementType && x.elementType == z.elementType, "the data type must be same");
    DEEP8_ARGUMENT_CHECK(strideY >= 1 && strideX >= 1 && dilationY >= 1 && dilationX >= 1, "the stride or dilation is error");
    DEEP8_ARGUMENT_CHECK(3 == x.nDims() && 4 == y.nDims() && 3 == z.nDims(), "the shape is error");
    ConvGeom g{(int)x.batch(), (int)x.dim(0), (int)x.dim(1), (int)x.dim(2), (int)y.dim(0), (int)y.dim(1), (int)y.dim(2), 0, 0};
    DEEP8_ARGUMENT_CHECK(1 == y.batch() && (int)y.dim(3) == g.ic, "the shape is error");
    g.oh = d8k_conv2d_out_dim(g.ih, g.fh, strideY, dilationY, covered ? 1 : 0);
    g.ow = d8k_conv2d_out_dim(g.iw, g.fw, strideX, dilationX, covered ? 1 : 0);
    DEEP8_ARGUMENT_CHECK(g.batch == (int)z.batch() && g.oh == (int)z.dim(0) && g.ow == (int)z.dim(1) && g.oc == (int)z.dim(2),
                         "the shape is error");
    return g;
}

// Math::DeConv2d (deep8/src/math/DeConv2d.cpp:43-82)
ConvGeom deconvGeom(const Tensor& x, const Tensor& y, const Tensor& z, bool covered, int strideY, int strideX) {
    DEEP8_ARGUMENT_CHECK(x.elementType == y.elementType && x.elementType == z.elementType, "the data type must be same");
    DEEP8_ARGUMENT_CHECK(strideY >= 1 && strideX >= 1, "the stride must >= 1");
    DEEP8_ARGUMENT_CHECK(3 == x.nDims() && 4 == y.nDims() && 3 == z.nDims(), "the shape is error");
    ConvGeom g{(int)x.batch(), (int)x.dim(0), (int)x.dim(1), (int)x.dim(2), (int)y.dim(0), (int)y.dim(1), (int)y.dim(2), 0, 0};
    DEEP8_ARGUMENT_CHECK(1 == y.batch() && (int)y.dim(3) == g.ic, "the shape is error");
    g.oh = d8k_deconv2d_out_dim(g.ih, g.fh, strideY, covered ? 1 : 0);
    g.ow = d8k_deconv2d_out_dim(g.iw, g.fw, strideX, covered ? 1 : 0);
    DEEP8_ARGUMENT_CHECK(g.batch == (int)z.batch() && g.oh == (int)z.dim(0) && g.ow == (int)z.dim(1) && g.oc == (int)z.dim(2),
                         "the z shape is error");
    return g;
}

size_t interim(const Tensor& x, const ConvGeom& g, int which, bool deconv) {
    GPUDevice* dev = gpuOf(x);
    return deconv ? d8k_deconv2d_interim_size(dev->kernels, which, d8kType(x), g.batch, g.ih, g.iw, g.ic, g.oc, g.fh, g.fw, g.oh, g.ow)
                  : d8k_conv2d_interim_size(dev->kernels, which, d8kType(x), g.batch, g.ih, g.iw, g.ic, g.oc, g.fh, g.fw, g.oh, g.ow);
}
}  // namespace

size_t Conv2dInterimSize(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int sY, int sX, int dY, int dX) {
    return interim(x, convGeom(x, y, z, covered, sY, sX, dY, dX), 0, false);
}
size_t Conv2dGradXInterimSize(const Tensor& x, Tensor&, const Tensor& y, const Tensor& z, const Tensor&, bool covered, int sY, int sX, int dY,
                              int dX) {
    return interim(x, convGeom(x, y, z, covered, sY, sX, dY, dX), 1, false);
}
size_t Conv2dGradYInterimSize(const Tensor& x, const Tensor& y, Tensor&, const Tensor& z, const Tensor&, bool covered, int sY, int sX, int dY,
                              int dX) {
    return interim(x, convGeom(x, y, z, covered, sY, sX, dY, dX), 2, false);
}

void Conv2d(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int sY, int sX, int dY, int dX, void* interimPtr) {
    convGeom(x, y, z, covered, sY, sX, dY, dX);
    Conv2dGPU(x, y, z, covered, sY, sX, dY, dX, interimPtr);
}
void Conv2dGPU(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int sY, int sX, int dY, int dX, void* xcol) {
    ConvGeom g = convGeom(x, y, z, covered, sY, sX, dY, dX);
    d8kCheck(d8k_conv2d_forward(gpuOf(x)->kernels, d8kType(x), x.raw(), g.batch, g.ih, g.iw, g.ic, y.raw(), g.oc, g.fh, g.fw, z.raw(), g.oh,
                                g.ow, sY, sX, dY, dX, xcol, xcol ? interim(x, g, 0, false) : 0));
}
void Conv2dGradX(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int sY, int sX, int dY, int dX,
                 void* interimPtr) {
    convGeom(x, y, z, covered, sY, sX, dY, dX);
    DEEP8_ARGUMENT_CHECK(x.shape == dx.shape && z.shape == dz.shape && x.elementType == dx.elementType && x.elementType == dz.elementType,
                         "the shape is error");
    Conv2dGradXGPU(x, dx, y, z, dz, covered, sY, sX, dY, dX, interimPtr);
}
void Conv2dGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int sY, int sX, int dY,
                    int dX, void* dxcol) {
    ConvGeom g = convGeom(x, y, z, covered, sY, sX, dY, dX);
    d8kCheck(d8k_conv2d_grad_x_into(gpuOf(x)->kernels, d8kType(x), dx.raw(), g.batch, g.ih, g.iw, g.ic, y.raw(), g.oc, g.fh, g.fw, dz.raw(),
                                    g.oh, g.ow, sY, sX, dY, dX, dxcol, dxcol ? interim(x, g, 1, false) : 0, accumulateFlag()));
}
void Conv2dGradY(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int sY, int sX, int dY, int dX,
                 void* interimPtr) {
    convGeom(x, y, z, covered, sY, sX, dY, dX);
    DEEP8_ARGUMENT_CHECK(y.shape == dy.shape && z.shape == dz.shape && x.elementType == dy.elementType && x.elementType == dz.elementType,
                         "the shape is error");
    Conv2dGradYGPU(x, y, dy, z, dz, covered, sY, sX, dY, dX, interimPtr);
}
void Conv2dGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int sY, int sX, int dY,
                    int dX, void* xcol) {
    ConvGeom g = convGeom(x, y, z, covered, sY, sX, dY, dX);
    d8kCheck(d8k_conv2d_grad_y_into(gpuOf(x)->kernels, d8kType(x), x.raw(), g.batch, g.ih, g.iw, g.ic, dy.raw(), g.oc, g.fh, g.fw, dz.raw(),
                                    g.oh, g.ow, sY, sX, dY, dX, xcol, xcol ? interim(x, g, 2, false) : 0, accumulateFlag()));
}

size_t DeConv2dInterimSize(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int sY, int sX) {
    return interim(x, deconvGeom(x, y, z, covered, sY, sX), 0, true);
}
size_t DeConv2dGradXInterimSize(const Tensor& x, Tensor&, const Tensor& y, const Tensor& z, const Tensor&, bool covered, int sY, int sX) {
    return interim(x, deconvGeom(x, y, z, covered, sY, sX), 1, true);
}
size_t DeConv2dGradYInterimSize(const Tensor& x, const Tensor& y, Tensor&, const Tensor& z, const Tensor&, bool covered, int sY, int sX) {
    return interim(x, deconvGeom(x, y, z, covered, sY, sX), 2, true);
}
void DeConv2d(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int sY, int sX, void* interimPtr) {
    deconvGeom(x, y, z, covered, sY, sX);
    DeConv2dGPU(x, y, z, covered, sY, sX, interimPtr);
}
void DeConv2dGPU(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int sY, int sX, void* interimPtr) {
    ConvGeom g = deconvGeom(x, y, z, covered, sY, sX);
    d8kCheck(d8k_deconv2d_forward(gpuOf(x)->kernels, d8kType(x), x.raw(), g.batch, g.ih, g.iw, g.ic, y.raw(), g.oc, g.fh, g.fw, z.raw(), g.oh,
                                  g.ow, sY, sX, interimPtr, interimPtr ? interim(x, g, 0, true) : 0));
}
void DeConv2dGradX(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int sY, int sX,
                   void* interimPtr) {
    deconvGeom(x, y, z, covered, sY, sX);
    DEEP8_ARGUMENT_CHECK(x.shape == dx.shape && z.shape == dz.shape && x.elementType == dx.elementType && x.elementType == dz.elementType,
                         "the shape is error");
    DeConv2dGradXGPU(x, dx, y, z, dz, covered, sY, sX, interimPtr);
}
void DeConv2dGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int sY, int sX,
                      void* interimPtr) {
    ConvGeom g = deconvGeom(x, y, z, covered, sY, sX);
    d8kCheck(d8k_deconv2d_grad_x_into(gpuOf(x)->kernels, d8kType(x), dx.raw(), g.batch, g.ih, g.iw, g.ic, y.raw(), g.oc, g.fh, g.fw, dz.raw(),
                                      g.oh, g.ow, sY, sX, interimPtr, interimPtr ? interim(x, g, 1, true) : 0, accumulateFlag()));
}
void DeConv2dGradY(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int sY, int sX,
                   void* interimPtr) {
    deconvGeom(x, y, z, covered, sY, sX);
    DEEP8_ARGUMENT_CHECK(y.shape == dy.shape && z.shape == dz.shape && x.elementType == dy.elementType && x.elementType == dz.elementType,
                         "the shape is error");
    DeConv2dGradYGPU(x, y, dy, z, dz, covered, sY, sX, interimPtr);
}
void DeConv2dGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int sY, int sX,
                      void* interimPtr) {
    ConvGeom g = deconvGeom(x, y, z, covered, sY, sX);
    d8kCheck(d8k_deconv2d_grad_y_into(gpuOf(x)->kernels, d8kType(x), x.raw(), g.batch, g.ih, g.iw, g.ic, dy.raw(), g.oc, g.fh, g.fw, dz.raw(),
                                      g.oh, g.ow, sY, sX, interimPtr, interimPtr ? interim(x, g, 2, true) : 0, accumulateFlag()));
}

void ReLu(const Tensor& x, Tensor& y) {
    DEEP8_ARGUMENT_CHECK(x.elementType == y.elementType && x.shape == y.shape, "the shape or type is error");
    d8kCheck(d8k_relu_forward(gpuOf(x)->kernels, d8kType(x), x.raw(), y.raw(), x.size()));
}
void ReLuGrad(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& dy) {
    DEEP8_ARGUMENT_CHECK(x.elementType == dx.elementType && x.elementType == dy.elementType && x.shape == dx.shape && y.shape == dy.shape,
                         "the shape or type is error");
    d8kCheck(d8k_relu_backward(gpuOf(x)->kernels, d8kType(x), x.raw(), dx.raw(), dy.raw(), dx.size()));
}
namespace {
// the two shapes this path adds: 0 = equal shapes, 1 = y is a bias (1, {cols}) over x's last dimension
int addKind(const Tensor& x, const Tensor& y) {
    if (x.shape == y.shape) return 0;
    if (1 == y.batch() && 1 == y.nDims() && x.nDims() >= 1 && x.dim(x.nDims() - 1) == y.dim(0)) return 1;
    DEEP8_RUNTIME_ERROR("only equal shapes or a bias over the last dimension can be added on this path");
}
}  // namespace

void Add(const Tensor& x, const Tensor& y, Tensor& z) {
    DEEP8_ARGUMENT_CHECK(x.elementType == y.elementType && x.elementType == z.elementType, "the param data type must be same");
    DEEP8_ARGUMENT_CHECK(x.shape == z.shape, "the shape is error");
    if (0 == addKind(x, y)) {
        const void* src[2] = {x.raw(), y.raw()};
        d8kCheck(d8k_sum_shards(gpuOf(x)->kernels, d8kType(x), z.raw(), src, 2, x.size()));
    } else {
        d8kCheck(d8k_add_bias(gpuOf(x)->kernels, d8kType(x), x.raw(), y.raw(), z.raw(), x.size() / y.size(), (int)y.size()));
    }
}
void AddGradX(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz) {
    DEEP8_ARGUMENT_CHECK(x.shape == dx.shape && z.shape == dz.shape && x.shape == z.shape, "the shape is error");
    DEEP8_ARGUMENT_CHECK(x.elementType == dx.elementType && x.elementType == dz.elementType, "the param data type must be same");
    addKind(x, y);
    const void* src[2] = {dz.raw(), dx.raw()};  // dx += dz, or dx = dz for a first contribution
    d8kCheck(d8k_sum_shards(gpuOf(x)->kernels, d8kType(x), dx.raw(), src, OverwriteGradient::active() ? 1 : 2, dx.size()));
}
void AddGradY(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz) {
    DEEP8_ARGUMENT_CHECK(y.shape == dy.shape && z.shape == dz.shape && x.shape == z.shape, "the shape is error");
    DEEP8_ARGUMENT_CHECK(x.elementType == dy.elementType && x.elementType == dz.elementType, "the param data type must be same");
    if (0 == addKind(x, y)) {
        const void* src[2] = {dz.raw(), dy.raw()};
        d8kCheck(d8k_sum_shards(gpuOf(x)->kernels, d8kType(x), dy.raw(), src, OverwriteGradient::active() ? 1 : 2, dy.size()));
    } else {
        if (OverwriteGradient::active()) dy.zero();  // the column sums add into dy: a small vector, zeroed here for a first contribution
        d8kCheck(d8k_add_bias_grad(gpuOf(x)->kernels, d8kType(x), dy.raw(), dz.raw(), dz.size() / dy.size(), (int)dy.size()));
    }
}
// deep8/src/math/Linear.cpp:9-44
void Linear(const Tensor& x, const float a, const float b, Tensor& y) {
    DEEP8_ARGUMENT_CHECK(x.deviceType() == y.deviceType(), "the param device type must be same");
    DEEP8_ARGUMENT_CHECK(x.elementType == y.elementType, "the param data type must be same");
    DEEP8_ARGUMENT_CHECK(x.shape == y.shape, "the param shape must be same");
    d8kCheck(d8k_linear_forward(gpuOf(x)->kernels, d8kType(x), x.raw(), a, b, y.raw(), x.size()));
}
void LinearGrad(const Tensor& x, Tensor& dx, const float a, const float, const Tensor& y, const Tensor& dy) {
    DEEP8_ARGUMENT_CHECK(x.elementType == dx.elementType && x.elementType == y.elementType && x.elementType == dy.elementType,
                         "the param data type must be same");
    DEEP8_ARGUMENT_CHECK(x.shape == dx.shape && x.shape == y.shape && x.shape == dy.shape, "the param shape must be same");
    d8kCheck(d8k_linear_grad(gpuOf(x)->kernels, d8kType(x), dx.raw(), a, dy.raw(), dx.size()));
}
// deep8/src/math/AdamUpdate.cpp:6-22
void AdamUpdate(Tensor& value, Tensor& gradient, Tensor& m, Tensor& v, float beta1, float beta2, float epsilon, float learningRate,
                float weightDecay, int64_t steps) {
    DEEP8_ARGUMENT_CHECK(value.elementType == gradient.elementType && value.elementType == m.elementType && value.elementType == v.elementType,
                         "the param data type must be same");
    DEEP8_ARGUMENT_CHECK(value.shape.size() == gradient.shape.size() && value.shape.size() == m.shape.size() &&
                             value.shape.size() == v.shape.size(),
                         "the param shape size must be same");
    d8kCheck(d8k_adam_update(gpuOf(value)->kernels, d8kType(value), value.raw(), gradient.raw(), m.raw(), v.raw(), beta1, beta2, epsilon,
                             learningRate, weightDecay, steps, value.size()));
}

void MatrixMultiplyReLu(const Tensor& x, const Tensor& y, Tensor& z, Tensor& a) {
    checkMatMul(x, y, z);
    DEEP8_ARGUMENT_CHECK(z.shape == a.shape && z.elementType == a.elementType, "the shape or type is error");
    d8kCheck(d8k_matmul_forward_relu(gpuOf(x)->kernels, d8kType(x), x.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), y.raw(), (int)y.batch(),
                                     (int)y.col(), z.raw(), a.raw()));
}
void MatrixMultiplyLinear(const Tensor& x, const Tensor& y, Tensor& z, float a, float b, Tensor& l) {
    checkMatMul(x, y, z);
    DEEP8_ARGUMENT_CHECK(z.shape == l.shape && z.elementType == l.elementType, "the shape or type is error");
    d8kCheck(d8k_matmul_forward_linear(gpuOf(x)->kernels, d8kType(x), x.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), y.raw(),
                                       (int)y.batch(), (int)y.col(), z.raw(), a, b, l.raw()));
}
void MatrixMultiplyAddBias(const Tensor& x, const Tensor& y, const Tensor& bias, Tensor& z) {
    checkMatMul(x, y, z);
    DEEP8_ARGUMENT_CHECK(bias.elementType == z.elementType && 1 == bias.batch() && 1 == bias.nDims() && bias.dim(0) == y.col() && y.col() > 1,
                         "the bias must be one row of y.col() elements");
    d8kCheck(d8k_matmul_forward_bias(gpuOf(x)->kernels, d8kType(x), x.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), y.raw(), (int)y.batch(),
                                     (int)y.col(), bias.raw(), z.raw()));
}
void MatrixMultiplyGradXReLuGrad(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, const Tensor& h, Tensor& dh,
                                 bool accumulateDx, bool accumulateDh) {
    checkMatMul(x, y, z);
    DEEP8_ARGUMENT_CHECK(x.shape == dx.shape && z.shape == dz.shape && h.shape.size() == x.shape.size() && dh.shape.size() == x.shape.size(),
                         "the shape is error");
    DEEP8_ARGUMENT_CHECK(x.elementType == dx.elementType && x.elementType == dz.elementType && x.elementType == h.elementType &&
                             x.elementType == dh.elementType,
                         "the data type must be same");
    d8kCheck(d8k_matmul_grad_x_relu(gpuOf(x)->kernels, d8kType(x), dx.raw(), (int)x.batch(), (int)x.row(), (int)x.col(), y.raw(), (int)y.batch(),
                                    (int)y.col(), dz.raw(), accumulateDx ? 1 : 0, h.raw(), dh.raw(), accumulateDh ? 1 : 0));
}

void AXPBY(const Tensor& x, float alpha, const Tensor& y, float beta, Tensor& z) {
    DEEP8_ARGUMENT_CHECK(x.elementType == y.elementType && x.elementType == z.elementType, "the param data type must be same");
    DEEP8_ARGUMENT_CHECK(x.shape.size() == y.shape.size() && x.shape.size() == z.shape.size(), "the param shape size must be same");
    DEEP8_ARGUMENT_CHECK(y.raw() == z.raw(), "on this path AXPBY updates y in place (z must be y), as the trainers call it");
    d8kCheck(d8k_axpby(gpuOf(x)->kernels, d8kType(x), x.raw(), alpha, z.raw(), beta, x.size()));
}
void Constant(Tensor& x, float scalar) {
    DEEP8_ARGUMENT_CHECK(0.f == scalar, "only the constant 0 is supported on this path");
    d8kCheck(d8k_zero(gpuOf(x)->kernels, x.raw(), x.byteCount()));
}

}  // namespace Math

// ================================================================================================ nodes
Node* OutputEntry::first() const {
    DEEP8_ARGUMENT_CHECK(!entries.empty(), "the output is empty");
    return entries.begin()->first;
}

Node::Node() : type(NodeType::Unknow), id(-1), executor(nullptr) {}
Node::Node(Node* input) : Node() {
    inputs.push_back(input);
    input->outputs.add(this, 0);
}
Node::Node(std::vector<Node*>& in) : Node() {
    inputs = in;
    for (size_t i = 0; i < inputs.size(); ++i) inputs[i]->outputs.add(this, i);
}
Node::Node(int64_t i, std::string n, Executor* exe) : type(NodeType::Unknow), id(i), name(std::move(n)), executor(exe) {}
Node::Node(int64_t i, std::string n, Executor* exe, Node* input) : Node(i, std::move(n), exe) {
    inputs.push_back(input);
    input->outputs.add(this, 0);
}
Node::~Node() = default;
void Node::forward() {}
void Node::backward() {}
std::string Node::toString() { return name; }

Variable::Variable(int64_t i, std::string n, Executor* exe, Tensor& v) : Node(i, std::move(n), exe), value(v), updateGradient(false) {
    type = NodeType::Variable;
}
Variable::Variable(int64_t i, std::string n, Executor* exe, Tensor& v, Tensor& g)
    : Node(i, std::move(n), exe), value(v), gradient(g), updateGradient(true) {
    type = NodeType::Variable;
}
Variable::Variable(int64_t i, std::string n, Executor* exe, Node* input, Tensor& v)
    : Node(i, std::move(n), exe, input), value(v), updateGradient(false) {
    type = NodeType::Variable;
}
Variable::Variable(int64_t i, std::string n, Executor* exe, Node* input, Tensor& v, Tensor& g)
    : Node(i, std::move(n), exe, input), value(v), gradient(g), updateGradient(true) {
    type = NodeType::Variable;
}

void Variable::zeroGradient() {
    if (updateGradient) gradient.zero();
}
void Variable::removeGradient() {
    updateGradient = false;
    gradient = Tensor();
}
Variable& Variable::feed(const void* cpuPtr) {
    DEEP8_ARGUMENT_CHECK(nullptr != cpuPtr, "the pointer can not be null");
    if (executor) executor->flush();  // a held product was defined with the values of the moment it was added
    valueStale = false;
    value.device()->copyFromCPUToGPU(cpuPtr, value.raw(), value.byteCount());
    return *this;
}
Variable& Variable::fetch(void* cpuPtr) {
    DEEP8_ARGUMENT_CHECK(nullptr != cpuPtr, "the pointer can not be null");
    if (executor) {
        executor->flush();
        executor->materialise(this);
    }
    static_cast<GPUDevice*>(value.device())->synchronize();
    value.device()->copyFromGPUToCPU(value.raw(), cpuPtr, value.byteCount());
    return *this;
}
Variable& Variable::feedGradient(const void* cpuPtr) {
    DEEP8_ARGUMENT_CHECK(updateGradient && nullptr != cpuPtr, "the Variable has no gradient");
    gradient.device()->copyFromCPUToGPU(cpuPtr, gradient.raw(), gradient.byteCount());
    gradientTouched = true;
    return *this;
}
Variable& Variable::fetchGradient(void* cpuPtr) {
    DEEP8_ARGUMENT_CHECK(updateGradient && nullptr != cpuPtr, "the Variable has no gradient");
    static_cast<GPUDevice*>(gradient.device())->synchronize();
    gradient.device()->copyFromGPUToCPU(gradient.raw(), cpuPtr, gradient.byteCount());
    return *this;
}
Variable& Variable::zero() {
    if (executor) executor->flush();
    valueStale = false;
    value.zero();
    return *this;
}

Function::Function(std::vector<Node*>& in) : Node(in) { type = NodeType::Function; }

Shape Function::checkShape(std::vector<Shape>&) { DEEP8_RUNTIME_ERROR("can not call this checkShape by Function class"); }

ElementType Function::checkElementType(std::vector<ElementType>& inputTypes) {
    DEEP8_ARGUMENT_CHECK(!inputTypes.empty(), "the input can not be empty");
    for (auto& t : inputTypes) DEEP8_ARGUMENT_CHECK(t == inputTypes[0], "the input element type must be same");
    return inputTypes[0];
}

void Function::forward(const std::vector<const Tensor*>&, Tensor*) { DEEP8_RUNTIME_ERROR("can not call this forward by Function class"); }
void Function::backward(const std::vector<const Tensor*>&, const Tensor*, const Tensor*, size_t, Tensor*) {
    DEEP8_RUNTIME_ERROR("can not call this backward by Function class");
}

void Function::forward() {
    for (auto item : inputs) DEEP8_ARGUMENT_CHECK(NodeType::Variable == item->type, "the inputs must be a Variable type");
    DEEP8_ARGUMENT_CHECK(1 == outputs.size(), "the output size must be 1");
    DEEP8_ARGUMENT_CHECK(NodeType::Variable == outputs.first()->type, "the output must be a Variable type");
    auto out = static_cast<Variable*>(outputs.first());
    std::vector<const Tensor*> values;
    for (auto item : inputs) {
        auto in = static_cast<Variable*>(item);
        DEEP8_ARGUMENT_CHECK(out->deviceType() == in->deviceType(), "the device of input must be same with output");
        values.push_back(&in->value);
    }
    forward(values, &out->value);
}

void Function::backward() {
    for (auto item : inputs) DEEP8_ARGUMENT_CHECK(NodeType::Variable == item->type, "the inputs must be a Variable type");
    DEEP8_ARGUMENT_CHECK(1 == outputs.size(), "the output size must be 1");
    DEEP8_ARGUMENT_CHECK(NodeType::Variable == outputs.first()->type, "the output must be Variable type");
    auto out = static_cast<Variable*>(outputs.first());
    if (out->updateGradient && !out->gradientTouched) {  // nothing has contributed to it: the zeros the reference's zero fill leaves
        out->zeroGradient();
        out->gradientTouched = true;
    }
    std::vector<const Tensor*> values;
    for (auto item : inputs) values.push_back(&static_cast<Variable*>(item)->value);
    for (size_t i = 0; i < inputs.size(); ++i) {
        auto in = static_cast<Variable*>(inputs[i]);
        if (!in->updateGradient) continue;
        bool first = !in->gradientTouched;
        if (first && !canOverwriteGradient(i)) {  // this node can only add: give it zeros to add to
            in->zeroGradient();
            first = false;
        }
        {
            Math::OverwriteGradient guard(first);
            backward(values, &out->value, &out->gradient, i, &in->gradient);
        }
        in->gradientTouched = true;
    }
}

// ---- MatrixMultiply (deep8/src/nodes/MatrixMultiply.cpp)
MatrixMultiply::MatrixMultiply(std::vector<Node*>& in) : Function(in) { functionType = FunctionType::MatrixMultiply; }

Shape MatrixMultiply::checkShape(std::vector<Shape>& s) {
    DEEP8_ARGUMENT_CHECK(2 == s.size(), "the input count must be 2");
    const Shape &x = s[0], &y = s[1];
    DEEP8_ARGUMENT_CHECK(x.batch == y.batch || 1 == x.batch || 1 == y.batch, "the batch of input is error");
    DEEP8_ARGUMENT_CHECK((1 == x.nDims || 2 == x.nDims) && (1 == y.nDims || 2 == y.nDims), "the inputs dimensions is error");
    DEEP8_ARGUMENT_CHECK(x.col() == y.row(), "the col of input1 must same to the row of input2");
    size_t batch = std::max(x.batch, y.batch);
    if (1 == y.col()) return Shape(batch, {x.row()});
    return Shape(batch, {x.row(), y.col()});
}
void MatrixMultiply::forward(const std::vector<const Tensor*>& in, Tensor* out) { Math::MatrixMultiply(*in[0], *in[1], *out); }
void MatrixMultiply::backward(const std::vector<const Tensor*>& in, const Tensor* out, const Tensor* dOut, size_t index, Tensor* dIn) {
    if (0 == index) Math::MatrixMultiplyGradX(*in[0], *dIn, *in[1], *out, *dOut);
    else if (1 == index) Math::MatrixMultiplyGradY(*in[0], *in[1], *dIn, *out, *dOut);
    else DEEP8_RUNTIME_ERROR("the index is error");
}

// ---- Conv2d (deep8/src/nodes/Conv2d.cpp)
Conv2d::Conv2d(std::vector<Node*>& in, bool c, int sY, int sX, int dY, int dX)
    : Function(in), covered(c), strideY(sY), strideX(sX), dilationY(dY), dilationX(dX) {
    functionType = FunctionType::Conv2d;
    DEEP8_ARGUMENT_CHECK(strideY >= 1 && strideX >= 1 && dilationY >= 1 && dilationX >= 1, "the stride and dilation must >= 1");
}

Shape Conv2d::checkShape(std::vector<Shape>& s) {
    DEEP8_ARGUMENT_CHECK(2 == s.size(), "the input count must be 2");
    const Shape &x = s[0], &f = s[1];
    DEEP8_ARGUMENT_CHECK(3 == x.nDims, "Conv2d needs inputs nDims is 3");
    DEEP8_ARGUMENT_CHECK(4 == f.nDims && 1 == f.batch, "Conv2d needs filter nDims is 4, the batch must be 1");
    DEEP8_ARGUMENT_CHECK(x.dim(2) == f.dim(3), "the inputs dimension is error");
    if (!covered)
        DEEP8_ARGUMENT_CHECK(f.dim(1) <= x.dim(0) && f.dim(2) <= x.dim(1), "the not covered mode Padding type needs filter smaller than input");
    int oh = d8k_conv2d_out_dim((int)x.dim(0), (int)f.dim(1), strideY, dilationY, covered ? 1 : 0);
    int ow = d8k_conv2d_out_dim((int)x.dim(1), (int)f.dim(2), strideX, dilationX, covered ? 1 : 0);
    DEEP8_ARGUMENT_CHECK(oh > 0 && ow > 0, "the output height or width must > 0");
    return Shape(x.batch, {(size_t)oh, (size_t)ow, f.dim(0)});
}

namespace {
// the node-level wrapper of the reference: ask the interim size, take it from the pool, call, give it back
template <typename SizeFn, typename CallFn>
void withInterim(const Tensor& x, SizeFn size, CallFn call) {
    Device* device = x.device();
    size_t bytes = size();
    void* ptr = device->malloc(bytes);  // malloc(0) is nullptr
    try {
        call(ptr);
    } catch (...) {
        device->free(ptr);
        throw;
    }
    device->free(ptr);  // safe: one stream, host-side bookkeeping (as in deep8/src/nodes/Conv2d.cpp:77-82)
}
}  // namespace

void Conv2d::forward(const std::vector<const Tensor*>& in, Tensor* out) {
    withInterim(*in[0], [&] { return Math::Conv2dInterimSize(*in[0], *in[1], *out, covered, strideY, strideX, dilationY, dilationX); },
                [&](void* p) { Math::Conv2d(*in[0], *in[1], *out, covered, strideY, strideX, dilationY, dilationX, p); });
}
void Conv2d::backward(const std::vector<const Tensor*>& in, const Tensor* out, const Tensor* dOut, size_t index, Tensor* dIn) {
    if (0 == index) {
        withInterim(*in[0], [&] { return Math::Conv2dGradXInterimSize(*in[0], *dIn, *in[1], *out, *dOut, covered, strideY, strideX, dilationY, dilationX); },
                    [&](void* p) { Math::Conv2dGradX(*in[0], *dIn, *in[1], *out, *dOut, covered, strideY, strideX, dilationY, dilationX, p); });
    } else if (1 == index) {
        withInterim(*in[0], [&] { return Math::Conv2dGradYInterimSize(*in[0], *in[1], *dIn, *out, *dOut, covered, strideY, strideX, dilationY, dilationX); },
                    [&](void* p) { Math::Conv2dGradY(*in[0], *in[1], *dIn, *out, *dOut, covered, strideY, strideX, dilationY, dilationX, p); });
    } else {
        DEEP8_RUNTIME_ERROR("the index is error");
    }
}

// ---- DeConv2d (deep8/src/nodes/DeConv2d.cpp)
DeConv2d::DeConv2d(std::vector<Node*>& in, bool c, int sY, int sX) : Function(in), forwardCovered(c), forwardStrideY(sY), forwardStrideX(sX) {
    functionType = FunctionType::DeConv2d;
    DEEP8_ARGUMENT_CHECK(forwardStrideY >= 1 && forwardStrideX >= 1, "the stride must >= 1");
}

Shape DeConv2d::checkShape(std::vector<Shape>& s) {
    DEEP8_ARGUMENT_CHECK(2 == s.size(), "the input count must be 2");
    const Shape &x = s[0], &f = s[1];
    DEEP8_ARGUMENT_CHECK(3 == x.nDims, "Conv2d needs inputs nDims is 3");
    DEEP8_ARGUMENT_CHECK(4 == f.nDims && 1 == f.batch, "Conv2d needs filter nDims is 4, the batch must be 1");
    DEEP8_ARGUMENT_CHECK(x.dim(2) == f.dim(3), "the inputs dimension is error");
    int oh = d8k_deconv2d_out_dim((int)x.dim(0), (int)f.dim(1), forwardStrideY, forwardCovered ? 1 : 0);
    int ow = d8k_deconv2d_out_dim((int)x.dim(1), (int)f.dim(2), forwardStrideX, forwardCovered ? 1 : 0);
    DEEP8_ARGUMENT_CHECK(oh > 0 && ow > 0, "the output height/width must > 0");
    return Shape(x.batch, {(size_t)oh, (size_t)ow, f.dim(0)});
}
void DeConv2d::forward(const std::vector<const Tensor*>& in, Tensor* out) {
    withInterim(*in[0], [&] { return Math::DeConv2dInterimSize(*in[0], *in[1], *out, forwardCovered, forwardStrideY, forwardStrideX); },
                [&](void* p) { Math::DeConv2d(*in[0], *in[1], *out, forwardCovered, forwardStrideY, forwardStrideX, p); });
}
void DeConv2d::backward(const std::vector<const Tensor*>& in, const Tensor* out, const Tensor* dOut, size_t index, Tensor* dIn) {
    if (0 == index) {
        withInterim(*in[0], [&] { return Math::DeConv2dGradXInterimSize(*in[0], *dIn, *in[1], *out, *dOut, forwardCovered, forwardStrideY, forwardStrideX); },
                    [&](void* p) { Math::DeConv2dGradX(*in[0], *dIn, *in[1], *out, *dOut, forwardCovered, forwardStrideY, forwardStrideX, p); });
    } else if (1 == index) {
        withInterim(*in[0], [&] { return Math::DeConv2dGradYInterimSize(*in[0], *in[1], *dIn, *out, *dOut, forwardCovered, forwardStrideY, forwardStrideX); },
                    [&](void* p) { Math::DeConv2dGradY(*in[0], *in[1], *dIn, *out, *dOut, forwardCovered, forwardStrideY, forwardStrideX, p); });
    } else {
        DEEP8_RUNTIME_ERROR("the index is error");
    }
}

// ---- Add (deep8/src/nodes/Add.cpp): output shape = x's; y equal to it or a bias over the last dimension
Add::Add(std::vector<Node*>& in) : Function(in) { functionType = FunctionType::Add; }
Shape Add::checkShape(std::vector<Shape>& s) {
    DEEP8_ARGUMENT_CHECK(2 == s.size(), "the input count must be 2");
    const Shape &x = s[0], &y = s[1];
    bool bias = 1 == y.batch && 1 == y.nDims && x.nDims >= 1 && x.dim(x.nDims - 1) == y.dim(0);
    DEEP8_ARGUMENT_CHECK(x == y || bias, "the Shape can not Broadcast");
    return x;
}
void Add::forward(const std::vector<const Tensor*>& in, Tensor* out) { Math::Add(*in[0], *in[1], *out); }
void Add::backward(const std::vector<const Tensor*>& in, const Tensor* out, const Tensor* dOut, size_t index, Tensor* dIn) {
    if (0 == index) Math::AddGradX(*in[0], *dIn, *in[1], *out, *dOut);
    else if (1 == index) Math::AddGradY(*in[0], *in[1], *dIn, *out, *dOut);
    else DEEP8_RUNTIME_ERROR("the index is error");
}

// ---- ReLu (deep8/src/nodes/ReLu.cpp)
ReLu::ReLu(std::vector<Node*>& in) : Function(in) { functionType = FunctionType::ReLu; }
Shape ReLu::checkShape(std::vector<Shape>& s) {
    DEEP8_ARGUMENT_CHECK(1 == s.size(), "the input count must be 1");
    return s[0];
}
void ReLu::forward(const std::vector<const Tensor*>& in, Tensor* out) { Math::ReLu(*in[0], *out); }
void ReLu::backward(const std::vector<const Tensor*>& in, const Tensor* out, const Tensor* dOut, size_t index, Tensor* dIn) {
    DEEP8_ARGUMENT_CHECK(0 == index, "the index is error");
    Math::ReLuGrad(*in[0], *dIn, *out, *dOut);
}

// ---- Linear (deep8/src/nodes/Linear.cpp)
Linear::Linear(std::vector<Node*>& in, float aa, float bb) : Function(in), a(aa), b(bb) {
    functionType = FunctionType::Linear;
    DEEP8_ARGUMENT_CHECK(1 == this->inputs.size(), "the Linear Function needs 1 input");
}
Shape Linear::checkShape(std::vector<Shape>& s) {
    DEEP8_ARGUMENT_CHECK(1 == s.size(), "the input count must be 1");
    return s[0];
}
ElementType Linear::checkElementType(std::vector<ElementType>& t) {
    DEEP8_ARGUMENT_CHECK(1 == t.size(), "the input count must be 1");
    return Function::checkElementType(t);
}
void Linear::forward(const std::vector<const Tensor*>& in, Tensor* out) { Math::Linear(*in[0], a, b, *out); }
void Linear::backward(const std::vector<const Tensor*>& in, const Tensor* out, const Tensor* dOut, size_t index, Tensor* dIn) {
    DEEP8_ARGUMENT_CHECK(0 == index, "the index is error");
    Math::LinearGrad(*in[0], *dIn, a, b, *out, *dOut);
}

// ================================================================================================ executors
Executor::Executor(DeviceType deviceType, int deviceId) : uniqueId(0), device(nullptr) {
    if (DeviceType::GPU != deviceType) DEEP8_RUNTIME_ERROR("this build has no CPU device: the path runs on sm_100a kernels only");
    device = new GPUDevice(deviceId);
}

Executor::~Executor() {
    for (auto& item : allNodes) delete item.second;
    allNodes.clear();
    retainVariables.clear();
    interimNodes.clear();
    delete device;
}

std::string Executor::generateUniqueName(const char* prefix) { return std::string(prefix) + "_" + std::to_string(uniqueId); }

Tensor Executor::createTensor(Shape& shape, ElementType type) {
    size_t bytes = type.byteWidth * shape.size();
    void* ptr = device->malloc(bytes);
    auto ref = static_cast<size_t*>(device->mallocCPU(sizeof(size_t)));
    TensorStorage storage(ptr, ref, bytes, device);
    return Tensor(storage, 0, shape, type);
}

Variable* Executor::addVariable(Shape& shape, ElementType type, bool updateGradient, bool retain) {
    auto id = generateUniqueId();
    auto name = generateUniqueName("Variable");
    Variable* v;
    Tensor value = createTensor(shape, type);
    if (updateGradient) {
        Tensor gradient = createTensor(shape, type);
        v = new Variable(id, name, this, value, gradient);
    } else {
        v = new Variable(id, name, this, value);
    }
    allNodes[name] = v;
    if (retain) retainVariables[name] = v;
    else interimNodes[name] = v;
    return v;
}
Variable* Executor::addVariable(std::vector<size_t> list, ElementType type, bool updateGradient, bool retain) {
    Shape shape(1, std::move(list));
    return addVariable(shape, type, updateGradient, retain);
}
Variable* Executor::addVariable(size_t batch, std::vector<size_t> list, ElementType type, bool updateGradient, bool retain) {
    Shape shape(batch, std::move(list));
    return addVariable(shape, type, updateGradient, retain);
}
Variable* Executor::addVariable(size_t batch, std::vector<size_t> list, DType type, bool updateGradient, bool retain) {
    return addVariable(batch, std::move(list), ElementType::from(type), updateGradient, retain);
}

Variable* Executor::createVariableByFunction(Function* func) {
    auto id = generateUniqueId();
    auto name = generateUniqueName("Variable");
    bool updateGradient = false;
    std::vector<Shape> shapes;
    std::vector<ElementType> types;
    for (auto item : func->inputs) {
        DEEP8_ARGUMENT_CHECK(NodeType::Variable == item->type, "the input must be a Variable");
        auto in = static_cast<Variable*>(item);
        shapes.push_back(in->shape());
        types.push_back(in->elementType());
        updateGradient = updateGradient || in->updateGradient;
    }
    Shape shape = func->checkShape(shapes);
    ElementType type = func->checkElementType(types);
    Tensor value = createTensor(shape, type);
    if (updateGradient) {
        Tensor gradient = createTensor(shape, type);
        return new Variable(id, name, this, func, value, gradient);
    }
    return new Variable(id, name, this, func, value);
}

void Executor::clearInterimNodes() {
    flush();  // a held product belongs to the nodes about to be deleted
    for (auto& item : allNodes) {
        item.second->inputs.clear();
        item.second->outputs.clear();
    }
    for (auto& item : interimNodes) {
        allNodes.erase(item.first);
        retainVariables.erase(item.first);
        delete item.second;
    }
    interimNodes.clear();
}

void Executor::removeGradient() {
    for (auto& item : allNodes)
        if (NodeType::Variable == item.second->type) static_cast<Variable*>(item.second)->removeGradient();
}

std::vector<Variable*> Executor::trainableParameters() {
    std::vector<Variable*> out;
    for (auto& item : retainVariables)
        if (item.second->updateGradient) out.push_back(item.second);
    return out;
}

EagerExecutor::EagerExecutor(DeviceType deviceType, int deviceId) : Executor(deviceType, deviceId) {}

void EagerExecutor::setFusion(bool on) {
    flush();
    fuse = on;
}
void EagerExecutor::setFirstTouch(bool on) { touch = on; }

void EagerExecutor::flush() {
    if (nullptr == pending) return;
    Function* f = pending;
    pending = nullptr;
    f->forward();
}

void EagerExecutor::materialise(Variable* v) {
    if (nullptr == v || !v->valueStale) return;
    DEEP8_ARGUMENT_CHECK(1 == v->inputs.size() && NodeType::Function == v->inputs[0]->type, "a stale value needs the function that produces it");
    v->valueStale = false;
    static_cast<Function*>(v->inputs[0])->forward();
}

namespace {
bool isBias(const Variable* b, const Variable* of) {
    return 1 == b->value.batch() && 1 == b->value.nDims() && of->value.nDims() == 2 && b->value.dim(0) == of->value.col();
}
}  // namespace

Variable* EagerExecutor::addFunction(Function* function) {
    function->id = generateUniqueId();
    function->name = generateUniqueName("Function");
    function->executor = this;
    Variable* variable = createVariableByFunction(function);
    allNodes[function->name] = function;
    allNodes[variable->name] = variable;
    interimNodes[function->name] = function;
    interimNodes[variable->name] = variable;
    // eager: the output is computed as the graph is built - except that a MatrixMultiply waits for the next node, so that a
    // ReLu, a Linear or a bias Add of its product can run inside its launch
    if (nullptr != pending) {
        Function* prod = pending;
        auto z = static_cast<Variable*>(prod->outputs.first());
        auto x = static_cast<Variable*>(prod->inputs[0]);
        auto y = static_cast<Variable*>(prod->inputs[1]);
        const bool consumesProduct = !function->inputs.empty() && function->inputs[0] == z;
        if (consumesProduct && FunctionType::ReLu == function->functionType) {
            pending = nullptr;
            Math::MatrixMultiplyReLu(x->value, y->value, z->value, variable->value);
            return variable;
        }
        if (consumesProduct && FunctionType::Linear == function->functionType) {
            pending = nullptr;
            auto lin = static_cast<Linear*>(function);
            Math::MatrixMultiplyLinear(x->value, y->value, z->value, lin->a, lin->b, variable->value);
            return variable;
        }
        if (consumesProduct && FunctionType::Add == function->functionType && 2 == function->inputs.size() && function->inputs[1] != z &&
            isBias(static_cast<Variable*>(function->inputs[1]), z)) {
            pending = nullptr;
            Math::MatrixMultiplyAddBias(x->value, y->value, static_cast<Variable*>(function->inputs[1])->value, variable->value);
            z->valueStale = true;  // the product itself was never stored: computed if anybody asks for it
            return variable;
        }
        flush();
    }
    for (auto in : function->inputs) materialise(static_cast<Variable*>(in));
    if (fuse && FunctionType::MatrixMultiply == function->functionType) {
        (void)d8kType(variable->value);  // an unsupported element type is reported now, when the node is added, not when it runs
        pending = function;
        return variable;
    }
    function->forward();
    return variable;
}

void EagerExecutor::forward(Node*) { DEEP8_RUNTIME_ERROR("the EagerExecutor can not call the forward"); }

namespace {
// visit `last` and everything it depends on breadth first, in the reference's queue order (EagerExecutor.cpp:46-84)
template <typename F>
void bfs(Node* last, F visit) {
    std::queue<Node*> que;
    std::unordered_set<Node*> seen;
    que.push(last);
    seen.insert(last);
    while (!que.empty()) {
        Node* node = que.front();
        que.pop();
        visit(node);
        for (auto in : node->inputs)
            if (seen.insert(in).second) que.push(in);
    }
}
}  // namespace

void EagerExecutor::backward(Node* last, bool clearInterim) {
    DEEP8_ARGUMENT_CHECK(nullptr != last && last->type == NodeType::Variable, "the last node must be a Variable");
    auto v = static_cast<Variable*>(last);
    DEEP8_ARGUMENT_CHECK(v->isScalar(), "the last Variable gradient must be scalar");
    DEEP8_ARGUMENT_CHECK(v->updateGradient, "the last Variable has no gradient");
    const float one32 = 1.0f;
    const uint16_t one16 = 0x3C00;
    backward(v, v->elementType().id == DType::Float16 ? static_cast<const void*>(&one16) : static_cast<const void*>(&one32), clearInterim);
}

// One node of the backward walk.  A MatrixMultiply z = a * w whose first operand is a = ReLu(h), consumed by nothing else, runs
// its gradient of a together with ReLu's gradient (one launch); the ReLu node is then done.
void EagerExecutor::backwardNode(Node* n, std::unordered_set<Node*>& done) {
    if (done.count(n)) return;
    if (fuse && NodeType::Function == n->type && FunctionType::MatrixMultiply == static_cast<Function*>(n)->functionType && 2 == n->inputs.size() &&
        1 == n->outputs.size()) {
        auto f = static_cast<Function*>(n);
        auto z = static_cast<Variable*>(f->outputs.first());
        auto a = static_cast<Variable*>(f->inputs[0]);
        auto w = static_cast<Variable*>(f->inputs[1]);
        Function* r = (1 == a->inputs.size() && NodeType::Function == a->inputs[0]->type) ? static_cast<Function*>(a->inputs[0]) : nullptr;
        if (a->updateGradient && a != w && 1 == a->outputs.size() && nullptr != r && FunctionType::ReLu == r->functionType && !done.count(r) &&
            1 == r->inputs.size()) {
            auto h = static_cast<Variable*>(r->inputs[0]);
            if (h->updateGradient && h != a && h != w && h != z) {
                if (z->updateGradient && !z->gradientTouched) {
                    z->zeroGradient();
                    z->gradientTouched = true;
                }
                Math::MatrixMultiplyGradXReLuGrad(a->value, a->gradient, w->value, z->value, z->gradient, h->value, h->gradient, a->gradientTouched,
                                                  h->gradientTouched);
                a->gradientTouched = h->gradientTouched = true;
                done.insert(r);
                if (w->updateGradient) {
                    Math::OverwriteGradient guard(!w->gradientTouched);
                    Math::MatrixMultiplyGradY(a->value, w->value, w->gradient, z->value, z->gradient);
                    w->gradientTouched = true;
                }
                return;
            }
        }
    }
    n->backward();
}

void EagerExecutor::backward(Variable* last, const void* hostGradient, bool clearInterim) {
    backwardFrom(last, hostGradient, nullptr, clearInterim);
}
void EagerExecutor::backward(Variable* last, const Tensor& deviceGradient, bool clearInterim) {
    backwardFrom(last, nullptr, &deviceGradient, clearInterim);
}
void EagerExecutor::backwardFrom(Variable* last, const void* hostGradient, const Tensor* deviceGradient, bool clearInterim) {
    DEEP8_ARGUMENT_CHECK(nullptr != last && last->updateGradient && (nullptr != hostGradient || nullptr != deviceGradient),
                         "the last Variable needs a gradient");
    flush();
    bfs(last, [this](Node* n) {
        if (NodeType::Variable != n->type) return;
        auto v = static_cast<Variable*>(n);
        if (touch) v->gradientTouched = false;  // the first contribution will overwrite
        else v->zeroGradient();                 // the reference's walk: zero everything, then add
    });
    if (hostGradient) {
        last->feedGradient(hostGradient);
    } else {
        copyOnExecutorStream(*deviceGradient, last->gradient);
        last->gradientTouched = true;
    }
    std::unordered_set<Node*> done;
    bfs(last, [this, &done](Node* n) { backwardNode(n, done); });
    if (touch)
        bfs(last, [](Node* n) {  // a gradient nothing contributed to reads as zeros, as after the reference's zero fill
            if (NodeType::Variable != n->type) return;
            auto v = static_cast<Variable*>(n);
            if (v->updateGradient && !v->gradientTouched) v->zeroGradient();
            v->gradientTouched = true;
        });
    if (clearInterim) clearInterimNodes();
}

// ================================================================================================ overlapped copies
CopyStream::CopyStream(GPUDevice* d) : device(d), stream(nullptr), next(0) {
    DEEP8_ARGUMENT_CHECK(nullptr != d, "the device can not be null");
    D8_CUDA_CHECK(cudaSetDevice(d->deviceId));
    cudaStream_t st;
    D8_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    stream = st;
    for (auto& e : events) {
        cudaEvent_t ev;
        D8_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        e = ev;
    }
}
CopyStream::~CopyStream() {
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    for (auto e : events) cudaEventDestroy(static_cast<cudaEvent_t>(e));
    cudaStreamDestroy(static_cast<cudaStream_t>(stream));
}
void* CopyStream::fresh() {
    void* e = events[next];
    next = (next + 1) % 16;
    return e;
}
void CopyStream::toDevice(const void* pinned, Tensor& to) {
    DEEP8_ARGUMENT_CHECK(nullptr != pinned && to.device() == device, "the pointer is null or the tensor is on another device");
    D8_CUDA_CHECK(cudaMemcpyAsync(to.raw(), pinned, to.byteCount(), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
}
void CopyStream::toHost(const Tensor& from, void* pinned) {
    DEEP8_ARGUMENT_CHECK(nullptr != pinned && from.device() == device, "the pointer is null or the tensor is on another device");
    D8_CUDA_CHECK(cudaMemcpyAsync(pinned, from.raw(), from.byteCount(), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
}
void* CopyStream::mark() {
    void* e = fresh();
    D8_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(e), static_cast<cudaStream_t>(stream)));
    return e;
}
void* CopyStream::markExecutor() {  // the executor enqueues on the legacy default stream (GPUDevice's kernel context)
    void* e = fresh();
    D8_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(e), cudaStreamLegacy));
    return e;
}
void CopyStream::waitFor(void* m) { D8_CUDA_CHECK(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(m), 0)); }
void CopyStream::executorWaitsFor(void* m) { D8_CUDA_CHECK(cudaStreamWaitEvent(cudaStreamLegacy, static_cast<cudaEvent_t>(m), 0)); }
void CopyStream::synchronize() { D8_CUDA_CHECK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream))); }

void copyOnExecutorStream(const Tensor& from, Tensor& to) {
    DEEP8_ARGUMENT_CHECK(from.byteCount() == to.byteCount() && from.device() == to.device(), "the tensors differ in size or device");
    D8_CUDA_CHECK(cudaMemcpyAsync(to.raw(), from.raw(), to.byteCount(), cudaMemcpyDeviceToDevice, cudaStreamLegacy));
}

// ================================================================================================ Net.h sugar
void backward(Variable& v, bool clearInterim) { v.executor->backward(&v, clearInterim); }

Variable& parameter(Executor* executor, std::vector<size_t> list, bool updateGradient, DType type) {
    return *executor->addVariable(1, std::move(list), type, updateGradient, true);
}
Variable& parameter(Executor* executor, size_t batch, std::vector<size_t> list, bool updateGradient, DType type) {
    return *executor->addVariable(batch, std::move(list), type, updateGradient, true);
}
Variable& parameter(Executor* executor, Shape& shape, bool updateGradient, DType type) {
    return *executor->addVariable(shape, ElementType::from(type), updateGradient, true);
}

Variable& Variable::matrixMultiply(Variable& y) {
    std::vector<Node*> in = {this, &y};
    return *executor->addFunction(new MatrixMultiply(in));
}
Variable& Variable::conv2d(Variable& filter, bool covered, int sY, int sX, int dY, int dX) {
    std::vector<Node*> in = {this, &filter};
    return *executor->addFunction(new Conv2d(in, covered, sY, sX, dY, dX));
}
Variable& Variable::deConv2d(Variable& filter, bool covered, int sY, int sX) {
    std::vector<Node*> in = {this, &filter};
    return *executor->addFunction(new DeConv2d(in, covered, sY, sX));
}
Variable& Variable::relu() {
    std::vector<Node*> in = {this};
    return *executor->addFunction(new ReLu(in));
}

Variable& Variable::linear(float a, float b) {
    std::vector<Node*> in = {this};
    return *executor->addFunction(new Linear(in, a, b));
}
Variable& linear(Variable& x, float a, float b) { return x.linear(a, b); }

Variable& Variable::add(Variable& y) {
    std::vector<Node*> in = {this, &y};
    return *executor->addFunction(new Add(in));
}
Variable& operator+(Variable& x, Variable& y) { return x.add(y); }
Variable& add(Variable& x, Variable& y) { return x.add(y); }

// ================================================================================================ trainer
// deep8/src/trainer/{LearningRateIterator,ConstantLearningRateIterator,Trainer,SGDTrainer}.cpp
float LearningRateIterator::next(int64_t) { DEEP8_RUNTIME_ERROR("can not call this function in LearningRateIterator"); }
ConstantLearningRateIterator::ConstantLearningRateIterator(float lr) : learningRate(lr) {}
float ConstantLearningRateIterator::next(int64_t) { return learningRate; }

Trainer::Trainer(LearningRateIterator* lr, float decay) : steps(0), learningRate(lr), weightDecay(decay) {}
void Trainer::update(Executor*, Variable*, float, float, int64_t) { DEEP8_RUNTIME_ERROR("can not call this function in trainer"); }
void Trainer::train(Executor* executor, std::vector<Variable*> parameters) {
    if (parameters.empty()) return;
    executor->flush();  // a held product must read the weights as they are now
    float lr = learningRate->next(steps);
    for (auto parameter : parameters) {
        if (!parameter->updateGradient) continue;
        this->update(executor, parameter, lr, this->weightDecay, steps);
    }
    steps++;
}
void Trainer::train(Executor* executor) { train(executor, executor->trainableParameters()); }

SGDTrainer::SGDTrainer(LearningRateIterator* lr, float decay) : Trainer(lr, decay) {}
void SGDTrainer::update(Executor*, Variable* parameter, float learningRate, float weightDecay, int64_t) {
    float alpha = -1 * learningRate;
    float beta = (1.0 - learningRate * weightDecay);  // the reference's mix: float product, double difference (SGDTrainer.cpp:13-14)
    Math::AXPBY(parameter->gradient, alpha, parameter->value, beta, parameter->value);
}

// deep8/src/trainer/AdamTrainer.cpp
AdamTrainer::AdamTrainer(LearningRateIterator* lr, float b1, float b2, float e, float decay) : Trainer(lr, decay), beta1(b1), beta2(b2), epsilon(e) {}
void AdamTrainer::update(Executor* executor, Variable* parameter, float learningRate, float weightDecay, int64_t steps) {
    auto value = parameter->value;
    auto gradient = parameter->gradient;
    if (m.find(parameter) == m.end()) {
        auto mt = executor->addVariable(value.shape, value.elementType, false);
        mt->value.zero();
        m[parameter] = mt;
    }
    if (v.find(parameter) == v.end()) {
        auto vt = executor->addVariable(value.shape, value.elementType, false);
        vt->value.zero();
        v[parameter] = vt;
    }
    auto mt = m[parameter]->value;
    auto vt = v[parameter]->value;
    Math::AdamUpdate(value, gradient, mt, vt, beta1, beta2, this->epsilon, learningRate, weightDecay, steps);
}

Variable& operator*(Variable& x, Variable& y) { return x.matrixMultiply(y); }
Variable& matrixMultiply(Variable& x, Variable& y) { return x.matrixMultiply(y); }
Variable& conv2d(Variable& x, Variable& filter, bool covered, int sY, int sX, int dY, int dX) { return x.conv2d(filter, covered, sY, sX, dY, dX); }
Variable& deConv2d(Variable& x, Variable& filter, bool covered, int sY, int sX) { return x.deConv2d(filter, covered, sY, sX); }
Variable& relu(Variable& x) { return x.relu(); }

}  // namespace Deep8
