// C++ host side of the path: Deep8's operator / executor / device interface for MatrixMultiply, Conv2d, DeConv2d
// (and their neighbour ReLu), implemented over the C ABI of include/d8k.h.  Same class names, members, argument meaning
// and error behaviour as the reference (paths below are relative to the reference project):
//
//   Shape, ElementType/DType        deep8/include/model/Shape.h, ElementType.h
//   Device, GPUDevice, GPUMemoryPool deep8/include/model/Device.h, GPUDevice.h, GPUMemoryPool.h
//   TensorStorage, Tensor           deep8/include/model/TensorStorage.h, Tensor.h
//   Node, Variable, Function        deep8/include/nodes/Node.h, Variable.h, Function.h
//   MatrixMultiply, Conv2d, DeConv2d, ReLu, Add, Linear   deep8/include/nodes/*.h
//   Executor, EagerExecutor         deep8/include/model/Executor.h, EagerExecutor.h
//   Math::*                          deep8/include/math/{MatrixMultiply,Conv2d,DeConv2d,ReLu}.h
//   parameter(), operator*, conv2d(), deConv2d(), relu(), backward()   deep8/include/model/Net.h
//
// There is no CPU device here: every tensor lives on a GPU and every operator runs the sm_100a kernels.
#ifndef DEEP8_B200_DEEP8_H
#define DEEP8_B200_DEEP8_H

#include <cstddef>
#include <cstdint>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../d8k.h"

// Error convention of deep8/include/basic/Exception.h: "<file>:<line>: <text>."
#define DEEP8_RUNTIME_ERROR(message)                        \
    {                                                       \
        std::ostringstream d8_oss__;                        \
        d8_oss__ << __FILE__ << ":" << __LINE__ << ": " << message << "."; \
        throw std::runtime_error(d8_oss__.str());           \
    }

#define DEEP8_ARGUMENT_CHECK(condition, message)            \
    if (!(condition)) {                                     \
        std::ostringstream d8_oss__;                        \
        d8_oss__ << __FILE__ << ":" << __LINE__ << ": " << message << "."; \
        throw std::invalid_argument(d8_oss__.str());        \
    }

#define DEEP8_ASSERT(condition, message) DEEP8_ARGUMENT_CHECK(condition, message)

#define MAX_TENSOR_DIMS 4
#define DEEP8_API __attribute__((visibility("default")))

namespace Deep8 {

// ------------------------------------------------------------------------------------------------ element types
enum class DType {
    UnKnown = 0, Bool = 1, Uint8 = 2, Int8 = 3, Uint16 = 4, Int16 = 5, Uint32 = 6, Int32 = 7, Uint64 = 8, Int64 = 9,
    Float16 = 10, Float32 = 11, Float64 = 12,
};

struct half_t {  // storage-only stand-in for the reference's `half` on the host side
    uint16_t bits;
};

class DEEP8_API ElementType {
    ElementType(DType d, size_t bw, std::string n) : id(d), byteWidth(bw), name(std::move(n)) {}

public:
    DType id;
    size_t byteWidth;
    std::string name;

    bool operator==(const ElementType& o) const { return id == o.id; }
    bool operator!=(const ElementType& o) const { return id != o.id; }

    static ElementType unknown() { return ElementType(DType::UnKnown, 0, "unknown"); }
    static ElementType from(DType type);
    template <typename T>
    static ElementType from();
    template <typename T>
    bool is() const { return id == from<T>().id; }
};
template <> inline ElementType ElementType::from<float>() { return from(DType::Float32); }
template <> inline ElementType ElementType::from<double>() { return from(DType::Float64); }
template <> inline ElementType ElementType::from<half_t>() { return from(DType::Float16); }
template <> inline ElementType ElementType::from<int32_t>() { return from(DType::Int32); }
template <> inline ElementType ElementType::from<int64_t>() { return from(DType::Int64); }
template <> inline ElementType ElementType::from<uint8_t>() { return from(DType::Uint8); }

// ------------------------------------------------------------------------------------------------ Shape
class DEEP8_API Shape {
public:
    size_t batch;
    size_t nDims;
    size_t dims[MAX_TENSOR_DIMS];
    size_t strides[MAX_TENSOR_DIMS];

    Shape();
    Shape(const Shape&) = default;
    Shape(size_t batch, const Shape& other);
    explicit Shape(std::vector<size_t> list);
    explicit Shape(size_t batch, std::vector<size_t> list);
    Shape& operator=(const Shape&) = default;

    bool operator==(const Shape&) const;
    bool operator!=(const Shape& o) const { return !(*this == o); }
    size_t operator[](size_t d) const { return dim(d); }

    void reShape(Shape& other);
    bool equalExceptBatch(const Shape& other) const;
    size_t size() const;       // batch * dims[0] * dims[1] ...
    size_t batchSize() const;  // size() / batch
    size_t dim(size_t d) const;
    size_t stride(size_t d) const;
    size_t row() const;
    size_t col() const;
    std::string toStr() const;

private:
    void updateStrides();
};

// ------------------------------------------------------------------------------------------------ devices
enum class DeviceType { CPU = 0, GPU = 1 };

class DEEP8_API Device {
public:
    DeviceType type;
    explicit Device(DeviceType t) : type(t) {}
    virtual ~Device() = default;

    virtual void* malloc(size_t size) = 0;
    virtual void free(void* ptr) = 0;
    virtual void zero(void* ptr, size_t size) = 0;
    virtual void copy(const void* from, void* to, size_t size) = 0;
    virtual void copyFromCPUToGPU(const void* from, void* to, size_t size) = 0;
    virtual void copyFromGPUToCPU(const void* from, void* to, size_t size) = 0;
    virtual void copyFromGPUToGPU(const void* from, void* to, size_t size) = 0;
    virtual void* mallocCPU(size_t size) = 0;
    virtual void freeCPU(void* ptr) = 0;
};

// Buddy allocator over cudaMalloc'd blocks (deep8/include/model/GPUMemoryPool.h, MemoryPool.h:13-23): requests are rounded
// up to a power of two of at least 128 bytes, served from the smallest free chunk that fits (split in halves), and a
// freed chunk merges with its free buddy.  A request larger than one block throws; malloc(0) returns nullptr.  All
// bookkeeping is on the host.  The block size defaults to the reference's 512 MiB and can be raised for 180 GB parts.
class DEEP8_API GPUMemoryPool {
public:
    int deviceId;
    size_t gpuBlockSize;

    explicit GPUMemoryPool(int id = 0, size_t blockSize = (static_cast<size_t>(1) << 29));
    ~GPUMemoryPool();
    GPUMemoryPool(const GPUMemoryPool&) = delete;
    GPUMemoryPool& operator=(const GPUMemoryPool&) = delete;

    void* malloc(size_t size);
    void free(void* ptr);
    void zero(void* ptr, size_t size);
    void copy(const void* from, void* to, size_t size);  // device to device
    void copyFromCPUToGPU(const void* from, void* to, size_t size);
    void copyFromGPUToCPU(const void* from, void* to, size_t size);
    void copyFromGPUToGPU(const void* from, void* to, size_t size);
    void* mallocCPU(size_t size);
    void freeCPU(void* ptr);

    size_t blockCount() const { return blocks.size(); }
    size_t bytesInUse() const { return inUse; }
    std::string toString() const;
    void printInfo() const;

private:
    struct Chunk {
        size_t block;   // which cudaMalloc'd block
        size_t offset;  // byte offset inside the block, a multiple of its size
        int level;      // size = 128 << level
    };
    int maxLevel;
    std::vector<char*> blocks;
    std::vector<std::map<std::pair<size_t, size_t>, bool>> freeByLevel;  // (block, offset) of free chunks per level
    std::unordered_map<void*, Chunk> live;
    size_t inUse = 0;
    void addBlock();
    static int levelFor(size_t size);
};

class DEEP8_API GPUDevice : public Device {
public:
    GPUMemoryPool* memoryPool;
    int deviceId;
    d8k_ctx* kernels;  // stands where the reference keeps its cuBLAS handle

    GPUDevice();
    explicit GPUDevice(int id, size_t poolBlockSize = (static_cast<size_t>(1) << 29));
    ~GPUDevice() override;

    void* malloc(size_t size) override;
    void free(void* ptr) override;
    void* mallocCPU(size_t size) override;
    void freeCPU(void* ptr) override;
    void zero(void* ptr, size_t size) override;
    void copy(const void* from, void* to, size_t size) override;
    void copyFromCPUToGPU(const void* from, void* to, size_t size) override;
    void copyFromGPUToCPU(const void* from, void* to, size_t size) override;
    void copyFromGPUToGPU(const void* from, void* to, size_t size) override;
    void synchronize();
};

// ------------------------------------------------------------------------------------------------ tensors
// Reference-counted handle on a pool allocation; the last copy returns the memory to the device (TensorStorage.cpp).
class DEEP8_API TensorStorage {
public:
    void* ptr;
    size_t* refPtr;
    size_t size;
    Device* device;

    TensorStorage();
    TensorStorage(void* p, size_t* refP, size_t s, Device* d);
    TensorStorage(const TensorStorage& other);
    ~TensorStorage();
    TensorStorage& operator=(const TensorStorage& other);

private:
    void release();
};

class DEEP8_API Tensor {
public:
    TensorStorage storage;
    size_t offset;  // bytes into the storage
    Shape shape;
    ElementType elementType;

    Tensor();
    explicit Tensor(Shape& s);
    Tensor(TensorStorage& ts, size_t off, Shape& s, ElementType et);
    Tensor(TensorStorage& ts, size_t off, std::vector<size_t>& list, ElementType et);
    Tensor(TensorStorage& ts, size_t off, size_t batch, std::vector<size_t>& list, ElementType et);

    DeviceType deviceType() const;
    Device* device() const;
    size_t* refPtr() const { return storage.refPtr; }
    size_t refCount() const { return storage.refPtr ? *storage.refPtr : 0; }
    void* raw() const;
    bool isScalar() const;
    void zero();
    size_t byteCount() const;
    size_t batch() const { return shape.batch; }
    size_t nDims() const { return shape.nDims; }
    size_t size() const { return shape.size(); }
    size_t batchSize() const { return shape.batchSize(); }
    size_t row() const { return shape.row(); }
    size_t col() const { return shape.col(); }
    size_t dim(size_t d) const { return shape.dim(d); }
    size_t stride(size_t d) const { return shape.stride(d); }

    template <typename T>
    T* data() const {
        DEEP8_ARGUMENT_CHECK(elementType.is<T>(), "Tensor type is error, type is: " << elementType.name);
        return static_cast<T*>(raw());
    }
    template <typename T>
    bool is() const { return elementType.is<T>(); }
};

// ------------------------------------------------------------------------------------------------ math (GPU only)
namespace Math {
DEEP8_API void MatrixMultiply(const Tensor& x, const Tensor& y, Tensor& z);
DEEP8_API void MatrixMultiplyGPU(const Tensor& x, const Tensor& y, Tensor& z);
DEEP8_API void MatrixMultiplyGradX(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz);
DEEP8_API void MatrixMultiplyGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz);
DEEP8_API void MatrixMultiplyGradY(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz);
DEEP8_API void MatrixMultiplyGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz);

DEEP8_API size_t Conv2dInterimSize(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int strideY, int strideX, int dilationY, int dilationX);
DEEP8_API void Conv2d(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int strideY, int strideX, int dilationY, int dilationX, void* interimPtr);
DEEP8_API void Conv2dGPU(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int strideY, int strideX, int dilationY, int dilationX, void* xcol);
DEEP8_API size_t Conv2dGradXInterimSize(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, int dilationY, int dilationX);
DEEP8_API void Conv2dGradX(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, int dilationY, int dilationX, void* interimPtr);
DEEP8_API void Conv2dGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, int dilationY, int dilationX, void* dxcol);
DEEP8_API size_t Conv2dGradYInterimSize(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, int dilationY, int dilationX);
DEEP8_API void Conv2dGradY(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, int dilationY, int dilationX, void* interimPtr);
DEEP8_API void Conv2dGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, int dilationY, int dilationX, void* xcol);

DEEP8_API size_t DeConv2dInterimSize(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int strideY, int strideX);
DEEP8_API void DeConv2d(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int strideY, int strideX, void* interimPtr);
DEEP8_API void DeConv2dGPU(const Tensor& x, const Tensor& y, Tensor& z, bool covered, int strideY, int strideX, void* interimPtr);
DEEP8_API size_t DeConv2dGradXInterimSize(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX);
DEEP8_API void DeConv2dGradX(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, void* interimPtr);
DEEP8_API void DeConv2dGradXGPU(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, void* interimPtr);
DEEP8_API size_t DeConv2dGradYInterimSize(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX);
DEEP8_API void DeConv2dGradY(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, void* interimPtr);
DEEP8_API void DeConv2dGradYGPU(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz, bool covered, int strideY, int strideX, void* interimPtr);

DEEP8_API void ReLu(const Tensor& x, Tensor& y);
DEEP8_API void ReLuGrad(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& dy);
// deep8/include/math/Linear.h: y = x * a + b;  dx += dy * a
DEEP8_API void Linear(const Tensor& x, const float a, const float b, Tensor& y);
DEEP8_API void LinearGrad(const Tensor& x, Tensor& dx, const float a, const float b, const Tensor& y, const Tensor& dy);
// deep8/include/math/AdamUpdate.h: value, gradient, m and v are all updated in place
DEEP8_API void AdamUpdate(Tensor& value, Tensor& gradient, Tensor& m, Tensor& v, float beta1, float beta2, float epsilon, float learningRate,
                          float weightDecay, int64_t steps);

// ---- additions (no counterpart in the reference's Math namespace)
// While a guard constructed with `on == true` is alive on this thread, the GradX / GradY functions of MatrixMultiply,
// Conv2d, DeConv2d and Add OVERWRITE their gradient argument instead of adding to it: the executor uses it for the first
// contribution to a gradient tensor, which then needs no zero fill (deep8/src/model/EagerExecutor.cpp:51-65 zero-fills
// every gradient before the backward walk).  Other gradient functions ignore it.
class DEEP8_API OverwriteGradient {
public:
    explicit OverwriteGradient(bool on);
    ~OverwriteGradient();
    OverwriteGradient(const OverwriteGradient&) = delete;
    OverwriteGradient& operator=(const OverwriteGradient&) = delete;
    static bool active();

private:
    bool previous;
};
// One-launch forms of a MatrixMultiply followed by an element-wise node; each stores exactly what the two separate calls store.
DEEP8_API void MatrixMultiplyReLu(const Tensor& x, const Tensor& y, Tensor& z, Tensor& a);                              // a = ReLu(z)
DEEP8_API void MatrixMultiplyLinear(const Tensor& x, const Tensor& y, Tensor& z, float a, float b, Tensor& l);          // l = Linear(z)
DEEP8_API void MatrixMultiplyAddBias(const Tensor& x, const Tensor& y, const Tensor& bias, Tensor& z);                  // z = x * y + bias
// MatrixMultiplyGradX for x = ReLu(h) followed by ReLuGrad: dx (+)= dz * y^T, then dh (+)= (h > 0 ? dx : 0)
DEEP8_API void MatrixMultiplyGradXReLuGrad(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz, const Tensor& h,
                                           Tensor& dh, bool accumulateDx, bool accumulateDh);
DEEP8_API void Constant(Tensor& x, float scalar);  // only 0 is supported: what zeroGradient needs

// Math::Add (deep8/src/math/Add.cpp:7-110) for the two cases of the path: equal shapes, and y a bias of shape (1, {cols})
// added to every row of x (any batch, last dimension cols); other broadcasts throw std::runtime_error.
DEEP8_API void Add(const Tensor& x, const Tensor& y, Tensor& z);
DEEP8_API void AddGradX(const Tensor& x, Tensor& dx, const Tensor& y, const Tensor& z, const Tensor& dz);
DEEP8_API void AddGradY(const Tensor& x, const Tensor& y, Tensor& dy, const Tensor& z, const Tensor& dz);
// Math::AXPBY (deep8/src/math/AXPBY.cpp:6-20) with z == y, which is how every trainer calls it: y = x * alpha + y * beta
DEEP8_API void AXPBY(const Tensor& x, float alpha, const Tensor& y, float beta, Tensor& z);
}  // namespace Math

// ------------------------------------------------------------------------------------------------ graph nodes
class Executor;
class Node;

class DEEP8_API OutputEntry {
public:
    std::unordered_map<Node*, size_t> entries;
    void add(Node* node, size_t i) { entries[node] = i; }
    void remove(Node* node) { entries.erase(node); }
    void clear() { entries.clear(); }
    size_t size() const { return entries.size(); }
    Node* first() const;
};

enum class NodeType { Unknow = 0, Variable, Function };

class DEEP8_API Node {
public:
    NodeType type;
    int64_t id;
    std::string name;
    Executor* executor;
    std::vector<Node*> inputs;
    OutputEntry outputs;

protected:
    Node();
    explicit Node(Node* input);
    explicit Node(std::vector<Node*>& inputs);
    Node(int64_t id, std::string name, Executor* exe);
    Node(int64_t id, std::string name, Executor* exe, Node* input);

public:
    virtual ~Node();
    virtual void forward();
    virtual void backward();
    virtual std::string toString();
};

class DEEP8_API Variable : public Node {
public:
    Tensor value;
    Tensor gradient;
    bool updateGradient;
    // Executor bookkeeping (additions).  gradientTouched: a contribution has been written to `gradient` in the running
    // backward pass, so the next one adds.  valueStale: `value` has not been computed because its producing MatrixMultiply
    // ran fused with the Add that consumes it; it is computed when somebody asks for it (fetch, a second consumer).
    bool gradientTouched = true;
    bool valueStale = false;

    Variable(int64_t id, std::string name, Executor* exe, Tensor& v);
    Variable(int64_t id, std::string name, Executor* exe, Tensor& v, Tensor& g);
    Variable(int64_t id, std::string name, Executor* exe, Node* input, Tensor& v);
    Variable(int64_t id, std::string name, Executor* exe, Node* input, Tensor& v, Tensor& g);

    Shape shape() const { return value.shape; }
    ElementType elementType() const { return value.elementType; }
    DeviceType deviceType() const { return value.deviceType(); }
    bool isScalar() const { return value.isScalar(); }
    void zeroGradient();
    void removeGradient();
    void forward() override {}
    void backward() override {}

    Variable& feed(const void* cpuPtr);  // host -> value (synchronous, as in the reference)
    Variable& fetch(void* cpuPtr);       // value -> host
    Variable& feedGradient(const void* cpuPtr);
    Variable& fetchGradient(void* cpuPtr);
    Variable& zero();

    Variable& matrixMultiply(Variable& y);
    Variable& conv2d(Variable& filter, bool covered = true, int strideY = 1, int strideX = 1, int dilationY = 1, int dilationX = 1);
    Variable& deConv2d(Variable& filter, bool covered = false, int strideY = 1, int strideX = 1);
    Variable& relu();
    Variable& add(Variable& y);
    Variable& linear(float a = 1, float b = 0);
};

enum class FunctionType { Unkown = 0, Add, Conv2d, DeConv2d, Linear, MatrixMultiply, ReLu };

class DEEP8_API Function : public Node {
protected:
    explicit Function(std::vector<Node*>& inputs);

public:
    FunctionType functionType = FunctionType::Unkown;  // addition: lets the executor recognise the chains it can run in one launch
    virtual bool isShared() { return false; }
    // addition: true when backward(..., index, ...) honours Math::OverwriteGradient for that input, i.e. can write the first
    // contribution to the gradient without a zero fill
    virtual bool canOverwriteGradient(size_t /*index*/) { return false; }
    virtual Shape checkShape(std::vector<Shape>& inputShapes);
    virtual ElementType checkElementType(std::vector<ElementType>& inputTypes);
    virtual void forward(const std::vector<const Tensor*>& inputs, Tensor* output);
    virtual void backward(const std::vector<const Tensor*>& inputs, const Tensor* output, const Tensor* outputGradient, size_t index,
                          Tensor* iGradient);
    void forward() override;
    void backward() override;
};

class DEEP8_API MatrixMultiply : public Function {
public:
    bool canOverwriteGradient(size_t) override { return true; }
    explicit MatrixMultiply(std::vector<Node*>& inputs);
    Shape checkShape(std::vector<Shape>& inputShapes) override;
    void forward(const std::vector<const Tensor*>& inputs, Tensor* output) override;
    void backward(const std::vector<const Tensor*>& inputs, const Tensor* output, const Tensor* outputGradient, size_t index,
                  Tensor* iGradient) override;
};

class DEEP8_API Conv2d : public Function {
public:
    bool canOverwriteGradient(size_t) override { return true; }
    bool covered;
    int strideY, strideX, dilationY, dilationX;
    explicit Conv2d(std::vector<Node*>& inputs, bool covered = false, int strideY = 1, int strideX = 1, int dilationY = 1, int dilationX = 1);
    Shape checkShape(std::vector<Shape>& inputShapes) override;
    void forward(const std::vector<const Tensor*>& inputs, Tensor* output) override;
    void backward(const std::vector<const Tensor*>& inputs, const Tensor* output, const Tensor* outputGradient, size_t index,
                  Tensor* iGradient) override;
};

class DEEP8_API DeConv2d : public Function {
public:
    bool canOverwriteGradient(size_t) override { return true; }
    bool forwardCovered;
    int forwardStrideY, forwardStrideX;
    explicit DeConv2d(std::vector<Node*>& inputs, bool covered = false, int strideY = 1, int strideX = 1);
    Shape checkShape(std::vector<Shape>& inputShapes) override;
    void forward(const std::vector<const Tensor*>& inputs, Tensor* output) override;
    void backward(const std::vector<const Tensor*>& inputs, const Tensor* output, const Tensor* outputGradient, size_t index,
                  Tensor* iGradient) override;
};

class DEEP8_API ReLu : public Function {
public:
    explicit ReLu(std::vector<Node*>& inputs);
    Shape checkShape(std::vector<Shape>& inputShapes) override;
    void forward(const std::vector<const Tensor*>& inputs, Tensor* output) override;
    void backward(const std::vector<const Tensor*>& inputs, const Tensor* output, const Tensor* outputGradient, size_t index,
                  Tensor* iGradient) override;
};

// deep8/include/nodes/Add.h, deep8/src/nodes/Add.cpp: z = x + y with the shapes Math::Add accepts here
class DEEP8_API Add : public Function {
public:
    bool canOverwriteGradient(size_t) override { return true; }
    explicit Add(std::vector<Node*>& inputs);
    Shape checkShape(std::vector<Shape>& inputShapes) override;
    void forward(const std::vector<const Tensor*>& inputs, Tensor* output) override;
    void backward(const std::vector<const Tensor*>& inputs, const Tensor* output, const Tensor* outputGradient, size_t index,
                  Tensor* iGradient) override;
};

// deep8/include/nodes/Linear.h: y = a * x + b
class DEEP8_API Linear : public Function {
public:
    float a;
    float b;
    explicit Linear(std::vector<Node*>& inputs, float a, float b);
    Shape checkShape(std::vector<Shape>& inputShapes) override;
    ElementType checkElementType(std::vector<ElementType>& inputTypes) override;
    void forward(const std::vector<const Tensor*>& inputs, Tensor* output) override;
    void backward(const std::vector<const Tensor*>& inputs, const Tensor* output, const Tensor* outputGradient, size_t index,
                  Tensor* iGradient) override;
};

// ------------------------------------------------------------------------------------------------ executors
class DEEP8_API Executor {
protected:
    int64_t uniqueId;
    Device* device;
    std::unordered_map<std::string, Node*> allNodes;
    std::unordered_map<std::string, Variable*> retainVariables;
    std::unordered_map<std::string, Node*> interimNodes;

    explicit Executor(DeviceType deviceType, int deviceId);
    int64_t generateUniqueId() { return uniqueId++; }
    std::string generateUniqueName(const char* prefix);
    Tensor createTensor(Shape& shape, ElementType type);
    Variable* createVariableByFunction(Function* func);

public:
    virtual ~Executor();
    Device* getDevice() const { return device; }

    Variable* addVariable(Shape& shape, ElementType type, bool updateGradient = true, bool retain = true);
    Variable* addVariable(std::vector<size_t> list, ElementType type, bool updateGradient = true, bool retain = true);
    Variable* addVariable(size_t batch, std::vector<size_t> list, ElementType type, bool updateGradient = true, bool retain = true);
    Variable* addVariable(size_t batch, std::vector<size_t> list, DType type, bool updateGradient = true, bool retain = true);

    void clearInterimNodes();
    void removeGradient();
    std::vector<Variable*> trainableParameters();

    virtual Variable* addFunction(Function* func) = 0;
    virtual void forward(Node* last) = 0;
    virtual void backward(Node* last, bool clearInterim = true) = 0;
    // additions: run whatever an eager executor has put off (see EagerExecutor), and make a stale value real
    virtual void flush() {}
    virtual void materialise(Variable*) {}
};

class DEEP8_API EagerExecutor : public Executor {
public:
    // deviceId is an addition: the reference pins device 0 (deep8/src/model/Executor.cu:6-8); one executor per GPU needs it.
    explicit EagerExecutor(DeviceType deviceType = DeviceType::GPU, int deviceId = 0);
    Variable* addFunction(Function* func) override;
    void forward(Node* last) override;
    // the reference's rule: `last` must be a scalar Variable; its gradient is set to one
    void backward(Node* last, bool clearInterim = true) override;
    // addition: start from `last` with an upstream gradient given on the host (the benchmark configurations supply one)
    void backward(Variable* last, const void* hostGradient, bool clearInterim = true);
    // addition: the same with the upstream gradient already on the device (copied into last's gradient on the executor's
    // stream, no host synchronisation) - what a step that overlaps its copies with the previous step's kernels uses
    void backward(Variable* last, const Tensor& deviceGradient, bool clearInterim = true);

    // ---- additions: fewer launches and less memory traffic for the same tensors, on by default
    // Fusion: a MatrixMultiply is not launched at once but held until the next node is added.  If that node is a ReLu or a
    // Linear of the product, or an Add of the product and a bias, both run as ONE launch (the element-wise node inside the
    // contraction's epilogue); anything else - another node, feed, fetch, backward - launches the held product first.  In the
    // backward walk the gradient of x of z = ReLu(h) * w runs with ReLu's gradient in its epilogue when ReLu's output feeds
    // only that product.  Every tensor a caller can observe holds the bits the node-by-node sequence produces.
    // First touch: the backward walk zero-fills no gradient; the first contribution to each gradient tensor overwrites it
    // (Function::canOverwriteGradient) and later ones add, as the reference's zero fill + "+=" would.
    void setFusion(bool on);
    void setFirstTouch(bool on);
    bool fusion() const { return fuse; }
    bool firstTouch() const { return touch; }
    void flush() override;
    void materialise(Variable* v) override;

private:
    bool fuse = true, touch = true;
    Function* pending = nullptr;  // a MatrixMultiply whose launch is held
    void backwardNode(Node* n, std::unordered_set<Node*>& done);
    void backwardFrom(Variable* last, const void* hostGradient, const Tensor* deviceGradient, bool clearInterim);
};

// ------------------------------------------------------------------------------------------------ overlapped copies (addition)
// Variable::feed and fetch are synchronous, as in the reference.  A CopyStream is a second CUDA stream (non-blocking) on the
// executor's GPU for copies between page-locked host memory and tensors that run beside the executor's kernels.  Marks
// (CUDA events, recycled after 16 further marks) order it against the executor's stream; nothing here blocks the host
// except synchronize().
class DEEP8_API CopyStream {
public:
    explicit CopyStream(GPUDevice* device);
    ~CopyStream();
    CopyStream(const CopyStream&) = delete;
    CopyStream& operator=(const CopyStream&) = delete;
    void toDevice(const void* pinned, Tensor& to);    // enqueue host -> device
    void toHost(const Tensor& from, void* pinned);    // enqueue device -> host
    void* mark();                        // everything enqueued on this stream so far
    void* markExecutor();                // everything the executor has enqueued so far
    void waitFor(void* mark);            // what is enqueued here from now on starts after `mark`
    void executorWaitsFor(void* mark);   // what the executor enqueues from now on starts after `mark`
    void synchronize();                  // host waits for this stream
private:
    GPUDevice* device;
    void* stream;
    void* events[16];
    int next;
    void* fresh();
};
// device -> device on the executor's stream, without host synchronisation (Tensor::copyFrom's asynchronous form)
DEEP8_API void copyOnExecutorStream(const Tensor& from, Tensor& to);

// ------------------------------------------------------------------------------------------------ Net.h sugar for the path
DEEP8_API void backward(Variable& v, bool clearInterim = true);
DEEP8_API Variable& parameter(Executor* executor, std::vector<size_t> list, bool updateGradient = true, DType type = DType::Float32);
DEEP8_API Variable& parameter(Executor* executor, size_t batch, std::vector<size_t> list, bool updateGradient = true, DType type = DType::Float32);
DEEP8_API Variable& parameter(Executor* executor, Shape& shape, bool updateGradient = true, DType type = DType::Float32);
DEEP8_API Variable& operator*(Variable& x, Variable& y);
DEEP8_API Variable& matrixMultiply(Variable& x, Variable& y);
DEEP8_API Variable& conv2d(Variable& x, Variable& filter, bool covered = true, int strideY = 1, int strideX = 1, int dilationY = 1, int dilationX = 1);
DEEP8_API Variable& deConv2d(Variable& x, Variable& filter, bool covered = false, int strideY = 1, int strideX = 1);
DEEP8_API Variable& relu(Variable& x);
DEEP8_API Variable& linear(Variable& x, float a = 1, float b = 0);
DEEP8_API Variable& operator+(Variable& x, Variable& y);
DEEP8_API Variable& add(Variable& x, Variable& y);

// ------------------------------------------------------------------------------------------------ trainers (SGD, Adam)
// deep8/include/trainer/{LearningRateIterator,ConstantLearningRateIterator,Trainer,SGDTrainer,AdamTrainer}.h
class DEEP8_API LearningRateIterator {
public:
    virtual ~LearningRateIterator() = default;
    virtual float next(int64_t steps);
};
class DEEP8_API ConstantLearningRateIterator : public LearningRateIterator {
public:
    float learningRate;
    explicit ConstantLearningRateIterator(float lr = 0.01);
    float next(int64_t steps) override;
};
class DEEP8_API Trainer {
protected:
    int64_t steps;
    LearningRateIterator* learningRate;
    float weightDecay;
    explicit Trainer(LearningRateIterator* lr, float decay = 0);

public:
    virtual ~Trainer() = default;
    virtual void update(Executor* executor, Variable* parameter, float learningRate, float weightDecay, int64_t steps);
    void train(Executor* executor, std::vector<Variable*> parameters);
    void train(Executor* executor);
};
class DEEP8_API SGDTrainer : public Trainer {
public:
    explicit SGDTrainer(LearningRateIterator* lr, float decay = 0);
    void update(Executor* executor, Variable* parameter, float learningRate, float weightDecay, int64_t steps) override;
};

// deep8/include/trainer/AdamTrainer.h
class DEEP8_API AdamTrainer : public Trainer {
public:
    float beta1;
    float beta2;
    float epsilon;
    std::unordered_map<Variable*, Variable*> m;
    std::unordered_map<Variable*, Variable*> v;
    explicit AdamTrainer(LearningRateIterator* lr, float beta1 = 0.9, float beta2 = 0.999, float epsilon = 1e-7, float decay = 0);
    void update(Executor* executor, Variable* parameter, float learningRate, float weightDecay, int64_t steps) override;
};

// ------------------------------------------------------------------------------------------------ several GPUs (additions)
// The reference runs on one device (deep8/src/model/Executor.cu:6-8).  With the batch sharded over the GPUs of a box - one
// process and one EagerExecutor(DeviceType::GPU, rank) per GPU - the gradients of the parameters every rank holds a copy of
// must be summed over the ranks after backward() and before Trainer::train (deep8/src/trainer/Trainer.cpp:12-32).

// How the processes find each other on the host: handles and barriers only, no tensor data.
class DEEP8_API Rendezvous {
public:
    virtual ~Rendezvous() = default;
    virtual int rank() const = 0;
    virtual int world() const = 0;
    // every rank contributes `bytes` bytes; `all` receives world * bytes, rank r's at offset r * bytes
    virtual void allGather(const void* mine, size_t bytes, void* all) = 0;
    virtual void barrier() = 0;
};

// Rendezvous through a directory every rank can see (a tmpfs path on one box): each allGather writes one small file per rank
// (written under a temporary name, then renamed) and polls for the others', giving up with std::runtime_error after the timeout.
class DEEP8_API FileRendezvous : public Rendezvous {
public:
    FileRendezvous(std::string directory, int rank, int world, double timeoutSeconds = 60.0);
    int rank() const override { return myRank; }
    int world() const override { return worldSize; }
    void allGather(const void* mine, size_t bytes, void* all) override;
    void barrier() override;

private:
    std::string dir;
    int myRank, worldSize;
    double timeout;
    long round = 0;
};

// Sum of the listed parameters' gradients over the ranks, through GPU memory the peers map (d8k_peer_*): every rank owns a
// contiguous shard of the concatenated gradients, pulls that shard of every peer's copy with the copy engines, adds the
// shards in rank order in fp32 (every rank gets the same bits), and pushes the result to the peers.  Everything is enqueued
// on the executor's stream; a peer that does not arrive within the timeout raises std::runtime_error at the next
// synchronisation instead of hanging the GPU.  All parameters must share one element type (fp32 or fp16).
class DEEP8_API PeerGradientSum {
public:
    PeerGradientSum(Executor* executor, Rendezvous* rendezvous, std::vector<Variable*> parameters, double timeoutMs = 2000.0);
    ~PeerGradientSum();
    PeerGradientSum(const PeerGradientSum&) = delete;
    PeerGradientSum& operator=(const PeerGradientSum&) = delete;
    void sum();          // call after backward(); returns with the work enqueued
    void synchronize();  // waits for it and throws if a wait between the ranks expired
    size_t elements() const { return total; }

private:
    Rendezvous* rv;
    GPUDevice* device;
    std::vector<Variable*> params;
    std::vector<size_t> offsets;  // element offset of each gradient in the concatenation
    size_t total = 0, esize = 0, shardElems = 0;
    int dtype = 0, world = 1, rank = 0;
    unsigned step = 0;
    double timeout;
    char* base = nullptr;           // partial | result | one staging slot per rank | flags
    std::vector<char*> peers;       // the same allocation in every rank, as mapped here
    size_t offPartial = 0, offResult = 0, offStage = 0, offFlags = 0, stageBytes = 0;
    void* flag(int owner, int kind, int writer) const;
};

}  // namespace Deep8

#endif  // DEEP8_B200_DEEP8_H
