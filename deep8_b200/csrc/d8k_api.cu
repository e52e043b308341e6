// extern "C" layer (include/d8k.h): context management and the mapping of MatrixMultiply / Conv2d / DeConv2d,
// forward and gradients, onto the one contraction kernel, plus the two element-wise neighbours (ReLU, zero fill).
#include <atomic>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/d8k.h"
#include "gemm_host.h"

struct d8k_ctx : public d8k::Ctx {};

namespace d8k {

static thread_local std::string g_error;
static std::atomic<unsigned long long> g_launches{0};

void set_error(const std::string& msg) { g_error = msg; }
int fail(int code, const std::string& msg) {
    g_error = msg;
    return code;
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
static thread_local std::string g_last_kernel;
void set_last_kernel(const std::string& text) { g_last_kernel = text; }

namespace {

#define D8K_CUDA(call)                                                                             \
    do {                                                                                           \
        cudaError_t e__ = (call);                                                                  \
        if (e__ != cudaSuccess) return fail(D8K_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__)); \
    } while (0)

int check_ctx(const d8k_ctx* ctx) {
    if (!ctx) return fail(D8K_ERR_ARGUMENT, "null context");
    return 0;
}

int check_dtype(int dtype) {
    if (dtype != D8K_F16 && dtype != D8K_F32) return fail(D8K_ERR_ARGUMENT, "type is not support: dtype must be D8K_F16 or D8K_F32");
    return 0;
}

int max0(int v) { return v > 0 ? v : 0; }

// deep8/src/math/Conv2d.cu:334-335
int conv_pad_before(int in, int out, int f, int stride, int dilation) {
    int real = f + (f - 1) * (dilation - 1);
    return -(max0((out - 1) * stride + real - in) / 2);
}
// deep8/src/math/DeConv2d.cu:99-100
int deconv_pad_before(int in, int out, int f, int stride) { return -(max0(out + f - (in - 1) * stride - 2) / 2); }

struct ConvDims {
    int batch, ih, iw, ic, oc, fh, fw, oh, ow;
};

int check_conv(const ConvDims& d, int sy, int sx, int dy, int dx) {
    if (d.batch < 1 || d.ih < 1 || d.iw < 1 || d.ic < 1 || d.oc < 1 || d.fh < 1 || d.fw < 1 || d.oh < 1 || d.ow < 1)
        return fail(D8K_ERR_ARGUMENT, "the shape is error");
    if (sy < 1 || sx < 1 || dy < 1 || dx < 1) return fail(D8K_ERR_ARGUMENT, "the stride or dilation is error");
    long long m_in = 1LL * d.batch * d.ih * d.iw, m_out = 1LL * d.batch * d.oh * d.ow;
    long long kc = 1LL * d.fh * d.fw * (d.ic > d.oc ? d.ic : d.oc);
    if (m_in >= (1LL << 31) || m_out >= (1LL << 31) || kc >= (1LL << 31)) return fail(D8K_ERR_ARGUMENT, "the shape is too large");
    return 0;
}

ConvRule rule(int RH, int RW, int SH, int SW, int C, int FH, int FW, int mul_y, int mul_x, int e_y, int e_x, int off_y, int off_x, int div_y,
              int div_x) {
    ConvRule r;
    r.RH = RH; r.RW = RW; r.SH = SH; r.SW = SW; r.C = C; r.FW = FW; r.FH = FH;
    r.mul_y = mul_y; r.mul_x = mul_x; r.e_y = e_y; r.e_x = e_x; r.off_y = off_y; r.off_x = off_x; r.div_y = div_y; r.div_x = div_x;
    finish_rule(r);
    return r;
}

HostOperand plain(const void* ptr, bool mn, long long ld) {
    HostOperand o;
    o.ptr = ptr;
    o.mn = mn;
    o.ld = ld;
    return o;
}

HostOperand virt(const void* ptr, bool mn, const ConvRule& cr) {
    HostOperand o;
    o.ptr = ptr;
    o.mn = mn;
    o.is_virtual = true;
    o.cr = cr;
    return o;
}

// filter [oc, T, ic] read as the matrix W'[(t, co)][ci]: row g = t * oc + co lives at co * (T * ic) + t * ic
HostOperand filter_by_tap(const void* ptr, int oc, int taps, int ic) {
    HostOperand o;
    o.ptr = ptr;
    o.mn = true;
    o.rmod = oc;
    o.ld = 1LL * taps * ic;
    o.ld2 = ic;
    return o;
}

// ---- rules with a divisor, one residue class at a time
// A rule whose source pixel is (py*mul + fy*e + off) / div only touches the image where the numerator is divisible.  For
// the rows py = r (mod div) that holds for the taps fy = f0 + step*j alone, and there the quotient is
// py'*mul + off' + j*e' with py = r + div*py': a divisor-free rule over a sub-grid of rows and a sub-grid of taps, which
// the im2col tensor maps can describe.  The div_y*div_x classes are independent contractions: they write disjoint output
// pixels (forward, x-gradient) or disjoint filter taps (filter gradient), and none of them multiplies by the zeros that
// the undivided rule would gather (3/4 of the taps at stride 2).
struct AxisClass {
    int rows, f0, step, nf, e2, off2;
};
int gcd_int(int a, int b) {
    while (b) {
        int t = a % b;
        a = b;
        b = t;
    }
    return a < 0 ? -a : a;
}
AxisClass axis_class(int R, int F, int mul, int e, int off, int div, int r) {
    AxisClass c = {};
    c.rows = r < R ? (R - r + div - 1) / div : 0;
    c.step = div / gcd_int(e, div);
    c.f0 = -1;
    for (int f = 0; f < c.step; ++f)
        if ((((r * mul + off + f * e) % div) + div) % div == 0) {
            c.f0 = f;
            break;
        }
    if (c.f0 < 0 || c.f0 >= F) return c;  // nf == 0: these rows see no tap
    c.nf = (F - c.f0 + c.step - 1) / c.step;
    c.e2 = e * c.step / div;
    c.off2 = (r * mul + off + c.f0 * e) / div;
    return c;
}

// Runs contraction `which` of a convolution-like operator as one launch per residue class of `R` (the rule that has the
// divisor).  *done stays false - and nothing is launched - unless every class can go through the TMA producer; the
// caller then runs the undivided rule on the loader warps.
int conv_by_residue_class(d8k_ctx* ctx, int which, const GemmProblem& whole, const ConvDims& d, const ConvRule& R, const void* x,
                          const void* y, const void* dz, bool* done) {
    *done = false;
    const int taps = d.fh * d.fw;
    std::vector<GemmProblem> parts;
    bool uncovered = false;  // some output rows (or, for the filter gradient, taps) are written by no class
    for (int ry = 0; ry < R.div_y; ++ry) {
        for (int rx = 0; rx < R.div_x; ++rx) {
            AxisClass cy = axis_class(R.RH, R.FH, R.mul_y, R.e_y, R.off_y, R.div_y, ry);
            AxisClass cx = axis_class(R.RW, R.FW, R.mul_x, R.e_x, R.off_x, R.div_x, rx);
            if (cy.rows == 0 || cx.rows == 0) {
                if (which == 2) uncovered = true;  // the taps of a class without rows get no contribution
                continue;
            }
            if (cy.nf == 0 || cx.nf == 0) {
                uncovered = true;
                continue;
            }
            ConvRule sub = rule(cy.rows, cx.rows, R.SH, R.SW, R.C, cy.nf, cx.nf, R.mul_y, R.mul_x, cy.e2, cx.e2, cy.off2, cx.off2, 1, 1);
            GemmProblem g = whole;
            HostOperand::TapSubset t;
            t.on = 1; t.f0y = cy.f0; t.f0x = cx.f0; t.ty = cy.step; t.tx = cx.step; t.nfy = cy.nf; t.nfx = cx.nf;
            t.FH = d.fh; t.FW = d.fw; t.ic = d.ic; t.oc = d.oc;
            const int pixels = d.batch * cy.rows * cx.rows;
            if (which == 0) {
                g.M = pixels; g.N = d.oc; g.K = cy.nf * cx.nf * d.ic;
                g.a = virt(x, false, sub);
                g.b = plain(y, false, 1LL * taps * d.ic);
                g.b.sub = t;
            } else if (which == 1) {
                g.M = pixels; g.N = d.ic; g.K = cy.nf * cx.nf * d.oc;
                g.a = virt(dz, false, sub);
                g.b = filter_by_tap(y, d.oc, taps, d.ic);
                g.b.sub = t;
            } else {
                // the class's pixels of dz: an im2col walk with one tap, stride div, starting at (ry, rx)
                ConvRule pick = rule(cy.rows, cx.rows, R.RH, R.RW, d.oc, 1, 1, R.div_y, R.div_x, 1, 1, ry, rx, 1, 1);
                g.M = d.oc; g.N = cy.nf * cx.nf * d.ic; g.K = pixels;
                g.a = virt(dz, true, pick);
                g.b = virt(x, true, sub);
                g.out.cols_on = 1;
                g.out.C = d.ic; g.out.NFX = cx.nf; g.out.FW = d.fw;
                g.out.f0y = cy.f0; g.out.f0x = cx.f0; g.out.ty = cy.step; g.out.tx = cx.step;
            }
            if (which != 2) {
                g.out.rows_on = 1;
                g.out.RH = cy.rows; g.out.RW = cx.rows; g.out.OH = R.RH; g.out.OW = R.RW;
                g.out.sy = R.div_y; g.out.sx = R.div_x; g.out.ry = ry; g.out.rx = rx;
            }
            if (!gemm_goes_through_tma(ctx, g)) return 0;
            parts.push_back(g);
        }
    }
    if (whole.beta == 0 && uncovered) {  // an overwriting call: what no class writes is zeros
        const size_t elems = which == 0   ? static_cast<size_t>(d.batch) * d.oh * d.ow * d.oc
                             : which == 1 ? static_cast<size_t>(d.batch) * d.ih * d.iw * d.ic
                                          : static_cast<size_t>(d.oc) * d.fh * d.fw * d.ic;
        if (cudaMemsetAsync(whole.C, 0, elems * (whole.dtype == D8K_F32 ? 4 : 2), ctx->stream) != cudaSuccess)
            return fail(D8K_ERR_CUDA, "cudaMemsetAsync failed");
    }
    *done = true;
    return run_gemm_group(ctx, parts);
}

// The three contractions of a convolution-like operator over virtual im2col matrices.
//   forward : z[Mout x oc]      = V(x)[Mout x T*ic] * y^T
//   grad x  : dx[Min x ic]     += V'(dz)[Min x T*oc] * W'
//   grad y  : dy[oc x T*ic]    += dz^T[oc x Mout] * V(x)[Mout x T*ic]
// `fwd` is the rule of V (rows = output pixels, source = x); `bwd` the rule of V' (rows = input pixels, source = dz).
int conv_like(d8k_ctx* ctx, int which, int dtype, const ConvDims& d, const ConvRule& fwd, const ConvRule& bwd, const void* x, void* dx,
              const void* y, void* dy, void* z, const void* dz, void* interim, size_t interim_bytes, bool plan_only, size_t* need,
              int accumulate = 1) {
    const int taps = d.fh * d.fw;
    GemmProblem g;
    g.dtype = dtype;
    g.ws = interim;
    g.ws_bytes = interim_bytes;
    if (which == 0) {
        g.M = d.batch * d.oh * d.ow; g.N = d.oc; g.K = taps * d.ic;
        g.a = virt(x, false, fwd);
        g.b = plain(y, false, g.K);
        g.C = z; g.ldc = d.oc; g.beta = 0;
    } else if (which == 1) {
        g.M = d.batch * d.ih * d.iw; g.N = d.ic; g.K = taps * d.oc;
        g.a = virt(dz, false, bwd);
        g.b = filter_by_tap(y, d.oc, taps, d.ic);
        g.C = dx; g.ldc = d.ic; g.beta = accumulate ? 1 : 0;
    } else {
        g.M = d.oc; g.N = taps * d.ic; g.K = d.batch * d.oh * d.ow;
        g.a = plain(dz, true, d.oc);
        g.b = virt(x, true, fwd);
        g.C = dy; g.ldc = g.N; g.beta = accumulate ? 1 : 0;
    }
    if (plan_only) {
        *need = gemm_scratch_need(ctx, g);
        return 0;
    }
    const ConvRule& divided = which == 1 ? bwd : fwd;
    if (!divided.unit_div) {
        bool done = false;
        int rc = conv_by_residue_class(ctx, which, g, d, divided, x, y, dz, &done);
        if (done || rc != 0) return rc;
    }
    return run_gemm(ctx, g);
}

void conv_rules(const ConvDims& d, int sy, int sx, int dly, int dlx, ConvRule* fwd, ConvRule* bwd) {
    int pt = conv_pad_before(d.ih, d.oh, d.fh, sy, dly), pl = conv_pad_before(d.iw, d.ow, d.fw, sx, dlx);
    // deep8/src/math/Conv2d.cu:44-45: inY = padTop + oy*strideY + fy*dilationY
    *fwd = rule(d.oh, d.ow, d.ih, d.iw, d.ic, d.fh, d.fw, sy, sx, dly, dlx, pt, pl, 1, 1);
    // deep8/src/math/Conv2d.cu:99-113: oy = (iy - padTop - fy*dilationY) / strideY when divisible and inside
    *bwd = rule(d.ih, d.iw, d.oh, d.ow, d.oc, d.fh, d.fw, 1, 1, -dly, -dlx, -pt, -pl, sy, sx);
}

void deconv_rules(const ConvDims& d, int sy, int sx, ConvRule* fwd, ConvRule* bwd) {
    int pt = deconv_pad_before(d.ih, d.oh, d.fh, sy), pl = deconv_pad_before(d.iw, d.ow, d.fw, sx);
    // deep8/src/math/DeConv2d.cu:41-48: iy = (oy + padTop + fy) / strideY when divisible and inside
    *fwd = rule(d.oh, d.ow, d.ih, d.iw, d.ic, d.fh, d.fw, 1, 1, 1, 1, pt, pl, sy, sx);
    // deep8/src/math/DeConv2d.cu:342-343: oy = iy*strideY - padTop - fy
    *bwd = rule(d.ih, d.iw, d.oh, d.ow, d.oc, d.fh, d.fw, sy, sx, -1, -1, -pt, -pl, 1, 1);
}

// ------------------------------------------------------------------------------------------------ element-wise
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// 16 bytes per thread per step; the tail and unaligned buffers go element by element.
template <typename T>
__global__ void relu_forward_kernel(const T* __restrict__ x, T* __restrict__ y, size_t n, bool vec) {
    constexpr int V = 16 / sizeof(T);
    size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    size_t stride = gridDim.x * static_cast<size_t>(blockDim.x);
    size_t nv = vec ? n / V : 0;
    for (size_t i = tid; i < nv; i += stride) {
        uint4 in = reinterpret_cast<const uint4*>(x)[i];
        T* e = reinterpret_cast<T*>(&in);
#pragma unroll
        for (int k = 0; k < V; ++k) e[k] = to_f(e[k]) > 0.f ? e[k] : from_f<T>(0.f);
        reinterpret_cast<uint4*>(y)[i] = in;
    }
    for (size_t i = nv * V + tid; i < n; i += stride) y[i] = to_f(x[i]) > 0.f ? x[i] : from_f<T>(0.f);
}

template <typename T>
__global__ void relu_backward_kernel(const T* __restrict__ x, T* __restrict__ dx, const T* __restrict__ dy, size_t n, bool vec) {
    constexpr int V = 16 / sizeof(T);
    size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    size_t stride = gridDim.x * static_cast<size_t>(blockDim.x);
    size_t nv = vec ? n / V : 0;
    for (size_t i = tid; i < nv; i += stride) {
        uint4 xin = reinterpret_cast<const uint4*>(x)[i];
        uint4 gin = reinterpret_cast<const uint4*>(dy)[i];
        uint4 acc = reinterpret_cast<const uint4*>(dx)[i];
        const T* xe = reinterpret_cast<const T*>(&xin);
        const T* ge = reinterpret_cast<const T*>(&gin);
        T* ae = reinterpret_cast<T*>(&acc);
#pragma unroll
        for (int k = 0; k < V; ++k)
            if (to_f(xe[k]) > 0.f) ae[k] = from_f<T>(to_f(ae[k]) + to_f(ge[k]));
        reinterpret_cast<uint4*>(dx)[i] = acc;
    }
    for (size_t i = nv * V + tid; i < n; i += stride)
        if (to_f(x[i]) > 0.f) dx[i] = from_f<T>(to_f(dx[i]) + to_f(dy[i]));
}

// z[r][c] = x[r][c] + bias[c]: Math::Add with the bias broadcast over batch and rows (deep8/src/math/Add.cu).
template <typename T>
__global__ void add_bias_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ z, size_t rows, int cols, bool vec) {
    constexpr int V = 16 / sizeof(T);
    const size_t n = rows * static_cast<size_t>(cols);
    size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    size_t stride = gridDim.x * static_cast<size_t>(blockDim.x);
    if (vec) {  // cols is a multiple of V: a 16-byte piece stays inside one row
        for (size_t i = tid; i < n / V; i += stride) {
            uint4 a = reinterpret_cast<const uint4*>(x)[i];
            uint4 b = __ldg(reinterpret_cast<const uint4*>(bias) + (i % (cols / V)));
            T* ae = reinterpret_cast<T*>(&a);
            const T* be = reinterpret_cast<const T*>(&b);
#pragma unroll
            for (int k = 0; k < V; ++k) ae[k] = from_f<T>(to_f(ae[k]) + to_f(be[k]));
            reinterpret_cast<uint4*>(z)[i] = a;
        }
    } else {
        for (size_t i = tid; i < n; i += stride) z[i] = from_f<T>(to_f(x[i]) + to_f(bias[i % cols]));
    }
}

// Column sums for Math::AddGradY of a bias, in two fixed-order steps: CTA (strip, slice) adds its slice of rows for one
// strip of columns into partial[slice][col] (rows in order, fp32), then the last step adds the slices in order and
// accumulates into dbias.  Every run adds in the same order.  W columns per thread: 16-byte loads (W = 16 / sizeof(T))
// when rows and pitch allow, else one column per thread.
// With `scale` the rows are weighted, partial[slice][c] = sum of dz[r][c] * scale[r]: the matrix-vector product dz^T * scale of
// MatrixMultiply's gradient of y when y is a single column (deep8/src/math/MatrixMultiply.cu:393-398 with n == 1).
template <typename T, int W>
__global__ void bias_grad_partial_kernel(const T* __restrict__ dz, float* __restrict__ partial, size_t rows, int cols, int rows_per_slice,
                                         const T* __restrict__ scale = nullptr) {
    const int lane = threadIdx.x & 31;
    const int col = (blockIdx.x * 32 + lane) * W;
    const int sub = threadIdx.x >> 5;  // 8 warps share the slice's rows; their sums meet in shared memory in warp order
    __shared__ float part[8][32 * W];
    const size_t r0 = static_cast<size_t>(blockIdx.y) * rows_per_slice;
    size_t r1 = r0 + rows_per_slice;
    if (r1 > rows) r1 = rows;
    float acc[W];
#pragma unroll
    for (int k = 0; k < W; ++k) acc[k] = 0.f;
    if (col < cols) {
#pragma unroll 4
        for (size_t r = r0 + sub; r < r1; r += 8) {
            const float s = scale ? to_f(scale[r]) : 1.f;
            if constexpr (W == 1) {
                acc[0] += to_f(dz[r * cols + col]) * s;
            } else {
                const uint4 v = __ldcs(reinterpret_cast<const uint4*>(dz + r * cols + col));
                const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
                for (int k = 0; k < W; ++k) acc[k] += to_f(e[k]) * s;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < W; ++k) part[sub][lane * W + k] = acc[k];
    __syncthreads();
    if (sub == 0 && col < cols) {
#pragma unroll
        for (int k = 0; k < W; ++k) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += part[w][lane * W + k];
            partial[static_cast<size_t>(blockIdx.y) * cols + col + k] = t;
        }
    }
}
template <typename T>
__global__ void bias_grad_final_kernel(T* __restrict__ dbias, const float* __restrict__ partial, int slices, int cols, int accumulate = 1) {
    int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= cols) return;
    float t = 0.f;
    for (int s = 0; s < slices; ++s) t += partial[static_cast<size_t>(s) * cols + col];
    dbias[col] = from_f<T>((accumulate ? to_f(dbias[col]) : 0.f) + t);
}

// ---- MatrixMultiply with a single-column y (the n == 1 case of the reference's first branch, deep8/src/math/MatrixMultiply.cu:31-36,
// 205-213, 393-398): a matrix-vector product.  One useful column would waste 63 / 64 of a tensor-core tile and the whole
// matrix is read exactly once, so these are HBM-bound SIMT kernels: 16-byte loads, fp32 accumulation in a fixed order.
// z[r] (+)= sum over c of A[r][c] * v[c]; one warp per row, four 16-byte loads in flight per lane.
template <typename T>
__global__ void __launch_bounds__(256) matvec_rows_kernel(const T* __restrict__ A, const T* __restrict__ v, T* __restrict__ z, size_t rows,
                                                          int cols, int accumulate, bool vec) {
    constexpr int V = 16 / sizeof(T);
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
    const size_t nwarps = (gridDim.x * static_cast<size_t>(blockDim.x)) >> 5;
    for (size_t r = warp; r < rows; r += nwarps) {
        const T* a = A + r * cols;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (vec) {
            const int nv = cols / V;
            const uint4* a4 = reinterpret_cast<const uint4*>(a);
            const uint4* v4 = reinterpret_cast<const uint4*>(v);
            for (int i0 = lane; i0 < nv; i0 += 128) {
                uint4 av[4], vv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + 32 * u;
                    av[u] = i < nv ? __ldcs(a4 + i) : make_uint4(0u, 0u, 0u, 0u);
                    vv[u] = i < nv ? __ldg(v4 + i) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const T* ae = reinterpret_cast<const T*>(&av[u]);
                    const T* ve = reinterpret_cast<const T*>(&vv[u]);
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[u] = fmaf(to_f(ae[k]), to_f(ve[k]), acc[u]);
                }
            }
        } else {
            for (int c = lane; c < cols; c += 32) acc[0] = fmaf(to_f(a[c]), to_f(v[c]), acc[0]);
        }
        float t = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) z[r] = from_f<T>((accumulate ? to_f(z[r]) : 0.f) + t);
    }
}

// The same product for long rows: one CTA per row, so that the 256 threads read 4 KB of the row at a time, one after the
// other (whole DRAM pages) - with a warp per row thousands of 64 KB rows are streamed at once and the matrix arrived at
// 3.9 TB/s of the 6.4 TB/s a copy reaches.  A vector of up to 32 KB is copied to shared memory once per CTA (SMEM_V) instead
// of being read through L2 for every row.  Eight 16-byte loads of the row are in flight per thread.  The eight warps' sums meet in shared
// memory in warp order.
template <typename T, bool SMEM_V>
__global__ void __launch_bounds__(256) matvec_long_rows_kernel(const T* __restrict__ A, const T* __restrict__ v, T* __restrict__ z, size_t rows,
                                                               int cols, int accumulate) {
    constexpr int V = 16 / sizeof(T);
    constexpr int U = 8;
    extern __shared__ uint4 v_smem[];
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nv = cols / V;  // the caller guarantees 16-byte aligned rows of whole 16-byte pieces
    const uint4* v4 = reinterpret_cast<const uint4*>(v);
    if (SMEM_V) {
        for (int i = threadIdx.x; i < nv; i += 256) v_smem[i] = __ldg(v4 + i);
        __syncthreads();
    }
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const uint4* a4 = reinterpret_cast<const uint4*>(A + r * cols);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i0 = threadIdx.x; i0 < nv; i0 += 256 * U) {
            uint4 av[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + 256 * u;
                av[u] = i < nv ? __ldcs(a4 + i) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + 256 * u;
                const uint4 vv = i < nv ? (SMEM_V ? v_smem[i] : __ldg(v4 + i)) : make_uint4(0u, 0u, 0u, 0u);
                const T* ae = reinterpret_cast<const T*>(&av[u]);
                const T* ve = reinterpret_cast<const T*>(&vv);
#pragma unroll
                for (int k = 0; k < V; ++k) acc[u & 3] = fmaf(to_f(ae[k]), to_f(ve[k]), acc[u & 3]);
            }
        }
        float t = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) part[warp] = t;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) s += part[k];
            z[r] = from_f<T>((accumulate ? to_f(z[r]) : 0.f) + s);
        }
        __syncthreads();
    }
}

template <typename T>
static cudaError_t launch_matvec_long_rows(const d8k_ctx* ctx, const T* A, const T* v, T* z, size_t rows, int cols, int accumulate) {
    // the vector in shared memory while six CTAs per SM still fit (32 KB); a longer one would cost more in resident CTAs
    // than it saves in L2 traffic (measured: 64 KB rows 4.8 TB/s with the vector in shared memory, 128 KB rows 5.5 without)
    const size_t vbytes = static_cast<size_t>(cols) * sizeof(T);
    const bool smem_v = vbytes <= 32 * 1024;
    auto kernel = smem_v ? matvec_long_rows_kernel<T, true> : matvec_long_rows_kernel<T, false>;
    const size_t dyn = smem_v ? vbytes : 0;
    if (smem_v) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024);
        if (e != cudaSuccess) return e;
    }
    // as many CTAs as are resident at once, each walking over its share of the rows
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, dyn) != cudaSuccess || per_sm < 1) per_sm = smem_v ? 3 : 4;
    size_t ctas = static_cast<size_t>(ctx->num_sms) * per_sm;
    if (ctas > rows) ctas = rows;
    kernel<<<static_cast<unsigned>(ctas), 256, dyn, ctx->stream>>>(A, v, z, rows, cols, accumulate);
    return cudaGetLastError();
}

// D[r][c] (+)= u[r] * v[c]: the gradient of x for a single-column y.  A thread keeps its 16 bytes of v and walks down the rows.
template <typename T>
__global__ void __launch_bounds__(256) outer_product_kernel(T* __restrict__ D, const T* __restrict__ u, const T* __restrict__ v, size_t rows,
                                                            int cols, int accumulate, bool vec) {
    constexpr int V = 16 / sizeof(T);
    const int chunk = blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        if (chunk >= cols / V) return;
        const uint4 v4 = __ldg(reinterpret_cast<const uint4*>(v) + chunk);
        const T* ve = reinterpret_cast<const T*>(&v4);
        for (size_t r = blockIdx.y; r < rows; r += gridDim.y) {
            const float s = to_f(u[r]);
            uint4* dst = reinterpret_cast<uint4*>(D + r * cols) + chunk;
            uint4 d4 = accumulate ? *dst : make_uint4(0u, 0u, 0u, 0u);
            T* de = reinterpret_cast<T*>(&d4);
#pragma unroll
            for (int k = 0; k < V; ++k) de[k] = from_f<T>((accumulate ? to_f(de[k]) : 0.f) + s * to_f(ve[k]));
            *dst = d4;
        }
    } else {
        if (chunk >= cols) return;
        const float t = to_f(v[chunk]);
        for (size_t r = blockIdx.y; r < rows; r += gridDim.y)
            D[r * cols + chunk] = from_f<T>((accumulate ? to_f(D[r * cols + chunk]) : 0.f) + to_f(u[r]) * t);
    }
}

bool aligned16(const void* a, const void* b, const void* c) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0;
}

int elementwise_grid(const d8k_ctx* ctx, size_t n, int per_thread) {
    size_t blocks = (n / per_thread + 255) / 256;
    size_t cap = static_cast<size_t>(ctx->num_sms) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

}  // namespace
}  // namespace d8k

using namespace d8k;

extern "C" {

const char* d8k_last_error(void) { return g_error.c_str(); }
unsigned long long d8k_launch_count(void) { return g_launches.load(); }
const char* d8k_last_kernel(void) { return g_last_kernel.c_str(); }

int d8k_ctx_create(int device, size_t scratch_bytes, d8k_ctx** out) {
    if (!out) return fail(D8K_ERR_ARGUMENT, "d8k_ctx_create: null output pointer");
    *out = nullptr;
    int count = 0;
    D8K_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return fail(D8K_ERR_ARGUMENT, "d8k_ctx_create: no such device");
    D8K_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    D8K_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(D8K_ERR_CUDA, "d8k_ctx_create: these kernels are built for sm_100a (B200) only");
    d8k_ctx* ctx = new d8k_ctx();
    ctx->device = device;
    ctx->num_sms = prop.multiProcessorCount;
    ctx->scratch_bytes = scratch_bytes ? scratch_bytes : (static_cast<size_t>(64) << 20);
    cudaError_t e = cudaMalloc(&ctx->scratch, ctx->scratch_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->counters, (kMaxCounters + 1) * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->counters, 0, (kMaxCounters + 1) * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->group_buf, sizeof(GroupEntry) * kMaxGroups);
    if (e != cudaSuccess) {
        cudaFree(ctx->scratch);
        cudaFree(ctx->counters);
        cudaFree(ctx->group_buf);
        delete ctx;
        return fail(D8K_ERR_CUDA, std::string("d8k_ctx_create: ") + cudaGetErrorString(e));
    }
    ctx->status = ctx->counters + kMaxCounters;
    *out = ctx;
    return 0;
}

int d8k_ctx_destroy(d8k_ctx* ctx) {
    if (!ctx) return 0;
    cudaSetDevice(ctx->device);
    cudaFree(ctx->scratch);
    cudaFree(ctx->counters);
    cudaFree(ctx->group_buf);
    delete ctx;
    return 0;
}

int d8k_ctx_set_stream(d8k_ctx* ctx, void* stream) {
    if (int rc = check_ctx(ctx)) return rc;
    ctx->stream = static_cast<cudaStream_t>(stream);
    return 0;
}

int d8k_ctx_num_sms(const d8k_ctx* ctx) { return ctx ? ctx->num_sms : 0; }

int d8k_ctx_status(d8k_ctx* ctx, int* status) {
    if (int rc = check_ctx(ctx)) return rc;
    D8K_CUDA(cudaStreamSynchronize(ctx->stream));
    int host = 0;
    D8K_CUDA(cudaMemcpy(&host, ctx->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (status) *status = host;
    if (host != 0) {
        cudaMemset(ctx->status, 0, sizeof(int));  // (half-counted tile tickets need no care: the next launch has another epoch)
        return fail(D8K_ERR_KERNEL, "a kernel gave up on a bounded wait, status " + std::to_string(host));
    }
    return 0;
}

static int gemm_call(d8k_ctx* ctx, int dtype, int transA, int transB, int M, int N, int K, const void* A, long long lda, int batchA,
                     long long strideA, const void* B, long long ldb, int batchB, long long strideB, void* C, long long ldc, long long strideC,
                     int batch, int beta, int reduce_batch, int epi = 0, void* E1 = nullptr, void* E2 = nullptr, int beta2 = 0,
                     void* const* row_blocks = nullptr, int num_blocks = 0, int block_rows = 0, float epi_a = 0.f, float epi_b = 0.f) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (batchA < 1 || batchB < 1 || batch < 0) return fail(D8K_ERR_ARGUMENT, "d8k_gemm: batch counts must be positive");
    GemmProblem g;
    g.dtype = dtype;
    g.M = M; g.N = N; g.K = K;
    g.a = plain(A, transA != 0, lda);
    g.a.batch_count = batchA;
    g.a.batch_stride = strideA;
    g.b = plain(B, transB == 0, ldb);
    g.b.batch_count = batchB;
    g.b.batch_stride = strideB;
    g.C = C; g.ldc = ldc; g.c_batch_stride = strideC;
    g.batch = reduce_batch ? 1 : batch;
    g.kbatch = reduce_batch ? (batch > 0 ? batch : 1) : 1;
    if (reduce_batch && batch == 0) g.K = 0;
    g.beta = beta;
    g.epi = epi; g.E1 = E1; g.E2 = E2; g.beta2 = beta2;
    g.epi_a = epi_a; g.epi_b = epi_b;
    if (row_blocks) {
        if (num_blocks < 1 || num_blocks > kMaxScatter) return fail(D8K_ERR_ARGUMENT, "1 to 16 row blocks");
        g.scatter_rows = block_rows;
        g.scatter_count = num_blocks;
        for (int k = 0; k < num_blocks; ++k) g.scatter_base[k] = row_blocks[k];
    }
    return run_gemm(ctx, g);
}

int d8k_gemm(d8k_ctx* ctx, int dtype, int transA, int transB, int M, int N, int K, const void* A, long long lda, int batchA,
             long long strideA, const void* B, long long ldb, int batchB, long long strideB, void* C, long long ldc, long long strideC,
             int batch, int beta, int reduce_batch) {
    return gemm_call(ctx, dtype, transA, transB, M, N, K, A, lda, batchA, strideA, B, ldb, batchB, strideB, C, ldc, strideC, batch, beta,
                     reduce_batch);
}

static int check_matmul(int xb, int xr, int xc, int yb, int yc) {
    if (xb < 1 || yb < 1 || xr < 1 || xc < 1 || yc < 1) return fail(D8K_ERR_ARGUMENT, "the shape is error");
    if (xb != yb && xb != 1 && yb != 1) return fail(D8K_ERR_ARGUMENT, "the shape is error");  // deep8/src/nodes/MatrixMultiply.cpp:15-17
    if (1LL * (xb > yb ? xb : yb) * xr >= (1LL << 31)) return fail(D8K_ERR_ARGUMENT, "the shape is too large");
    return 0;
}

static int column_sums(d8k_ctx* ctx, int dtype, void* out, const void* src, size_t rows, int cols, const void* scale, int accumulate);

// z[rows] (+)= A[rows x cols] * v[cols]
static int matvec_rows(d8k_ctx* ctx, int dtype, const void* A, const void* v, void* z, size_t rows, int cols, int accumulate) {
    if (!A || !v || !z) return fail(D8K_ERR_ARGUMENT, "gemm: null pointer");
    const int per = dtype == D8K_F32 ? 4 : 8;
    const bool vec = aligned16(A, v, nullptr) && cols % per == 0;
    // rows of 16 KB and more: a CTA per row (measured on 4 KB .. 128 KB rows: shorter ones run faster with a warp per row)
    if (vec && static_cast<size_t>(cols) * (dtype == D8K_F32 ? 4 : 2) >= 16384) {
        D8K_CUDA(dtype == D8K_F32 ? launch_matvec_long_rows(ctx, static_cast<const float*>(A), static_cast<const float*>(v), static_cast<float*>(z), rows, cols, accumulate)
                                  : launch_matvec_long_rows(ctx, static_cast<const __half*>(A), static_cast<const __half*>(v), static_cast<__half*>(z), rows, cols,
                                                            accumulate));
        D8K_CUDA(cudaGetLastError());
        count_launch();
        set_last_kernel(std::string(dtype == D8K_F32 ? "f32" : "f16") + " matvec rows (cta per row)");
        return 0;
    }
    // one warp per row, eight warps per CTA, every CTA resident at once; when there are more rows than warps each warp takes the
    // same number of rows (k), so that no warp is left with one more than the others (16384 rows over 9472 warps ran at 86 %)
    const size_t cap = static_cast<size_t>(ctx->num_sms) * 8;
    const size_t k = (rows + 8 * cap - 1) / (8 * cap);
    size_t blocks = (rows + 8 * k - 1) / (8 * k);
    if (blocks < 1) blocks = 1;
    if (dtype == D8K_F32)
        matvec_rows_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(static_cast<const float*>(A), static_cast<const float*>(v),
                                                                                        static_cast<float*>(z), rows, cols, accumulate, vec);
    else
        matvec_rows_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(static_cast<const __half*>(A), static_cast<const __half*>(v),
                                                                                         static_cast<__half*>(z), rows, cols, accumulate, vec);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    set_last_kernel(std::string(dtype == D8K_F32 ? "f32" : "f16") + " matvec rows");
    return 0;
}

// D[rows x cols] (+)= u[rows] (x) v[cols]
static int outer_product(d8k_ctx* ctx, int dtype, void* D, const void* u, const void* v, size_t rows, int cols, int accumulate) {
    if (!D || !u || !v) return fail(D8K_ERR_ARGUMENT, "gemm: null pointer");
    const int per = dtype == D8K_F32 ? 4 : 8;
    const bool vec = aligned16(D, v, nullptr) && cols % per == 0;
    const int chunks = vec ? cols / per : cols;
    const int bx = (chunks + 255) / 256;
    size_t by = (static_cast<size_t>(ctx->num_sms) * 8 + bx - 1) / bx;
    if (by > rows) by = rows;
    if (by > 65535) by = 65535;
    dim3 grid(bx, static_cast<unsigned>(by));
    if (dtype == D8K_F32)
        outer_product_kernel<float><<<grid, 256, 0, ctx->stream>>>(static_cast<float*>(D), static_cast<const float*>(u), static_cast<const float*>(v),
                                                                 rows, cols, accumulate, vec);
    else
        outer_product_kernel<__half><<<grid, 256, 0, ctx->stream>>>(static_cast<__half*>(D), static_cast<const __half*>(u),
                                                                  static_cast<const __half*>(v), rows, cols, accumulate, vec);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    set_last_kernel(std::string(dtype == D8K_F32 ? "f32" : "f16") + " outer product");
    return 0;
}

static int matmul_forward_impl(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc, void* z,
                               int epi, void* relu_out, float epi_a = 0.f, float epi_b = 0.f) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (int rc = check_matmul(xb, xr, xc, yb, yc)) return rc;
    if (yb == 1 && yc == 1 && epi == 0)  // one column: a matrix-vector product over the folded rows
        return matvec_rows(ctx, dtype, x, y, z, static_cast<size_t>(xb) * xr, xc, 0);
    if (yb == 1)  // deep8/src/math/MatrixMultiply.cu:31-36: the batch folds into M
        return gemm_call(ctx, dtype, 0, 0, xb * xr, yc, xc, x, xc, 1, 0, y, yc, 1, 0, z, yc, 0, 1, 0, 0, epi, relu_out, nullptr, 0, nullptr, 0, 0,
                         epi_a, epi_b);
    if (xb == 1 && yc == 1 && (epi == 0 || epi == 1 || epi == 4))
        // deep8/src/math/MatrixMultiply.cu:37-42: z [yb x xr] = Y [yb x xc] * X^T, the batch of vectors as the rows of one matrix
        return gemm_call(ctx, dtype, 0, 1, yb, xr, xc, y, xc, 1, 0, x, xc, 1, 0, z, xr, 0, 1, 0, 0, epi, relu_out, nullptr, 0, nullptr, 0, 0,
                         epi_a, epi_b);
    int zb = xb > yb ? xb : yb;
    return gemm_call(ctx, dtype, 0, 0, xr, yc, xc, x, xc, xb, 1LL * xr * xc, y, yc, yb, 1LL * xc * yc, z, yc, 1LL * xr * yc, zb, 0, 0, epi,
                     relu_out, nullptr, 0, nullptr, 0, 0, epi_a, epi_b);
}

static int matmul_grad_x_impl(d8k_ctx* ctx, int dtype, void* dx, int xb, int xr, int xc, const void* y, int yb, int yc, const void* dz,
                              int accumulate, int epi, const void* h, void* dh, int accumulate_dh) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (int rc = check_matmul(xb, xr, xc, yb, yc)) return rc;
    void* hh = const_cast<void*>(h);
    const int beta = accumulate ? 1 : 0, beta2 = accumulate_dh ? 1 : 0;
    if (yb == 1 && yc == 1 && epi == 0)  // one column: dx [rows x xc] (+)= dz [rows] (x) y [xc]
        return outer_product(ctx, dtype, dx, dz, y, static_cast<size_t>(xb) * xr, xc, beta);
    if (xb == 1 && yc == 1 && yb > 1 && epi == 0)
        // deep8/src/math/MatrixMultiply.cu:214-219: dx [xr x xc] (+)= dZ^T [xr x yb] * Y [yb x xc]
        return gemm_call(ctx, dtype, 1, 0, xr, xc, yb, dz, xr, 1, 0, y, xc, 1, 0, dx, xc, 0, 1, beta, 0);
    // dx[M x xc] (+)= dz[M x yc] * y^T ; y is [xc x yc], i.e. already "N x K" for this product
    if (yb == 1) return gemm_call(ctx, dtype, 0, 1, xb * xr, xc, yc, dz, yc, 1, 0, y, yc, 1, 0, dx, xc, 0, 1, beta, 0, epi, hh, dh, beta2);
    int zb = xb > yb ? xb : yb;
    if (xb == 1 && zb > 1)  // broadcast x: every batch entry adds into the one dx (deep8/src/math/MatrixMultiply.cu:220-231)
        return gemm_call(ctx, dtype, 0, 1, xr, xc, yc, dz, yc, zb, 1LL * xr * yc, y, yc, yb, 1LL * xc * yc, dx, xc, 0, zb, beta, 1, epi, hh, dh,
                         beta2);
    return gemm_call(ctx, dtype, 0, 1, xr, xc, yc, dz, yc, zb, 1LL * xr * yc, y, yc, yb, 1LL * xc * yc, dx, xc, 1LL * xr * xc, zb, beta, 0, epi,
                     hh, dh, beta2);
}

static int matmul_grad_y_impl(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, void* dy, int yb, int yc, const void* dz,
                              int accumulate) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (int rc = check_matmul(xb, xr, xc, yb, yc)) return rc;
    const int beta = accumulate ? 1 : 0;
    if (yb == 1 && yc == 1) {  // one column: dy [xc] (+)= x^T [xc x rows] * dz [rows], column sums of x weighted by dz
        if (!x || !dy || !dz) return fail(D8K_ERR_ARGUMENT, "gemm: null pointer");
        set_last_kernel(std::string(dtype == D8K_F32 ? "f32" : "f16") + " matvec columns");
        return column_sums(ctx, dtype, dy, x, static_cast<size_t>(xb) * xr, xc, dz, beta);
    }
    if (xb == 1 && yc == 1 && yb > 1)
        // deep8/src/math/MatrixMultiply.cu:402-407: dy [yb x xc] (+)= dZ [yb x xr] * X [xr x xc]
        return gemm_call(ctx, dtype, 0, 0, yb, xc, xr, dz, xr, 1, 0, x, xc, 1, 0, dy, xc, 0, 1, beta, 0);
    // dy[xc x yc] (+)= x^T * dz ; with yb == 1 the batch joins the contraction: K = xb * xr (deep8/src/math/MatrixMultiply.cu:393-398)
    if (yb == 1) return gemm_call(ctx, dtype, 1, 0, xc, yc, xb * xr, x, xc, 1, 0, dz, yc, 1, 0, dy, yc, 0, 1, beta, 0);
    return gemm_call(ctx, dtype, 1, 0, xc, yc, xr, x, xc, xb, 1LL * xr * xc, dz, yc, yb, 1LL * xr * yc, dy, yc, 1LL * xc * yc, yb, beta, 0);
}

int d8k_matmul_forward(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc, void* z) {
    return matmul_forward_impl(ctx, dtype, x, xb, xr, xc, y, yb, yc, z, 0, nullptr);
}
int d8k_matmul_grad_x(d8k_ctx* ctx, int dtype, void* dx, int xb, int xr, int xc, const void* y, int yb, int yc, const void* dz) {
    return matmul_grad_x_impl(ctx, dtype, dx, xb, xr, xc, y, yb, yc, dz, 1, 0, nullptr, nullptr, 0);
}
int d8k_matmul_grad_y(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, void* dy, int yb, int yc, const void* dz) {
    return matmul_grad_y_impl(ctx, dtype, x, xb, xr, xc, dy, yb, yc, dz, 1);
}
int d8k_matmul_grad_x_into(d8k_ctx* ctx, int dtype, void* dx, int xb, int xr, int xc, const void* y, int yb, int yc, const void* dz,
                           int accumulate) {
    return matmul_grad_x_impl(ctx, dtype, dx, xb, xr, xc, y, yb, yc, dz, accumulate, 0, nullptr, nullptr, 0);
}
int d8k_matmul_grad_y_into(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, void* dy, int yb, int yc, const void* dz,
                           int accumulate) {
    return matmul_grad_y_impl(ctx, dtype, x, xb, xr, xc, dy, yb, yc, dz, accumulate);
}
int d8k_matmul_grad_y_scatter(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, int yc, const void* dz, void* const* row_blocks,
                              int num_blocks, int block_rows) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (int rc = check_matmul(xb, xr, xc, 1, yc)) return rc;
    if (!row_blocks) return fail(D8K_ERR_ARGUMENT, "d8k_matmul_grad_y_scatter: null pointer");
    // the yb == 1 case of matmul_grad_y_impl with the output rows sent to their blocks
    return gemm_call(ctx, dtype, 1, 0, xc, yc, xb * xr, x, xc, 1, 0, dz, yc, 1, 0, nullptr, yc, 0, 1, 0, 0, 0, nullptr, nullptr, 0, row_blocks,
                     num_blocks, block_rows);
}
int d8k_matmul_forward_relu(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc, void* z, void* a) {
    if (!a) return fail(D8K_ERR_ARGUMENT, "d8k_matmul_forward_relu: null pointer");
    return matmul_forward_impl(ctx, dtype, x, xb, xr, xc, y, yb, yc, z, 1, a);
}
int d8k_matmul_grad_x_relu(d8k_ctx* ctx, int dtype, void* dx, int xb, int xr, int xc, const void* y, int yb, int yc, const void* dz,
                           int accumulate_dx, const void* h, void* dh, int accumulate_dh) {
    if (!h || !dh) return fail(D8K_ERR_ARGUMENT, "d8k_matmul_grad_x_relu: null pointer");
    return matmul_grad_x_impl(ctx, dtype, dx, xb, xr, xc, y, yb, yc, dz, accumulate_dx, 2, h, dh, accumulate_dh);
}

int d8k_matmul_forward_linear(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc, void* z, float a,
                              float b, void* l) {
    if (!l) return fail(D8K_ERR_ARGUMENT, "d8k_matmul_forward_linear: null pointer");
    return matmul_forward_impl(ctx, dtype, x, xb, xr, xc, y, yb, yc, z, 4, l, a, b);
}

int d8k_matmul_forward_bias(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc, const void* bias,
                            void* z) {
    if (!bias) return fail(D8K_ERR_ARGUMENT, "d8k_matmul_forward_bias: null pointer");
    return matmul_forward_impl(ctx, dtype, x, xb, xr, xc, y, yb, yc, z, 3, const_cast<void*>(bias));
}

int d8k_add_bias(d8k_ctx* ctx, int dtype, const void* x, const void* bias, void* z, size_t rows, int cols) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (rows == 0 || cols <= 0) return cols < 0 ? fail(D8K_ERR_ARGUMENT, "the shape is error") : 0;
    if (!x || !bias || !z) return fail(D8K_ERR_ARGUMENT, "add_bias: null pointer");
    const size_t n = rows * static_cast<size_t>(cols);
    const int per = dtype == D8K_F32 ? 4 : 8;
    bool vec = aligned16(x, bias, z) && cols % per == 0;
    if (dtype == D8K_F32)
        add_bias_kernel<float><<<elementwise_grid(ctx, n, 4), 256, 0, ctx->stream>>>(static_cast<const float*>(x), static_cast<const float*>(bias),
                                                                                     static_cast<float*>(z), rows, cols, vec);
    else
        add_bias_kernel<__half><<<elementwise_grid(ctx, n, 8), 256, 0, ctx->stream>>>(static_cast<const __half*>(x), static_cast<const __half*>(bias),
                                                                                      static_cast<__half*>(z), rows, cols, vec);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

// out[c] (+)= sum over r < rows of src[r][c] (* scale[r] when scale is given), two fixed-order steps through the context's scratch
static int column_sums(d8k_ctx* ctx, int dtype, void* out, const void* src, size_t rows, int cols, const void* scale, int accumulate) {
    // 16-byte loads when every row starts on a 16-byte boundary and holds whole pieces
    const int per = dtype == D8K_F32 ? 4 : 8;
    const bool wide = (reinterpret_cast<uintptr_t>(src) & 15) == 0 && cols % per == 0;
    const int strip_cols = 32 * (wide ? per : 1);
    // enough slices to occupy the GPU, bounded by the context's scratch memory (slices * cols floats)
    const int strips = (cols + strip_cols - 1) / strip_cols;
    int slices = (ctx->num_sms * 4 + strips - 1) / strips;
    const size_t max_slices = ctx->scratch_bytes / (static_cast<size_t>(cols) * sizeof(float));
    if (max_slices < 1) return fail(D8K_ERR_ARGUMENT, "the context's scratch memory is smaller than one row of floats");
    if (static_cast<size_t>(slices) > max_slices) slices = static_cast<int>(max_slices);
    if (static_cast<size_t>(slices) > (rows + 63) / 64) slices = static_cast<int>((rows + 63) / 64);
    if (slices < 1) slices = 1;
    const int rows_per_slice = static_cast<int>((rows + slices - 1) / slices);
    slices = static_cast<int>((rows + rows_per_slice - 1) / rows_per_slice);
    dim3 grid(strips, slices);
    if (dtype == D8K_F32) {
        const float* in = static_cast<const float*>(src);
        const float* sc = static_cast<const float*>(scale);
        if (wide) bias_grad_partial_kernel<float, 4><<<grid, 256, 0, ctx->stream>>>(in, ctx->scratch, rows, cols, rows_per_slice, sc);
        else bias_grad_partial_kernel<float, 1><<<grid, 256, 0, ctx->stream>>>(in, ctx->scratch, rows, cols, rows_per_slice, sc);
        bias_grad_final_kernel<float><<<(cols + 255) / 256, 256, 0, ctx->stream>>>(static_cast<float*>(out), ctx->scratch, slices, cols, accumulate);
    } else {
        const __half* in = static_cast<const __half*>(src);
        const __half* sc = static_cast<const __half*>(scale);
        if (wide) bias_grad_partial_kernel<__half, 8><<<grid, 256, 0, ctx->stream>>>(in, ctx->scratch, rows, cols, rows_per_slice, sc);
        else bias_grad_partial_kernel<__half, 1><<<grid, 256, 0, ctx->stream>>>(in, ctx->scratch, rows, cols, rows_per_slice, sc);
        bias_grad_final_kernel<__half><<<(cols + 255) / 256, 256, 0, ctx->stream>>>(static_cast<__half*>(out), ctx->scratch, slices, cols, accumulate);
    }
    D8K_CUDA(cudaGetLastError());
    count_launch();
    count_launch();
    return 0;
}

int d8k_add_bias_grad(d8k_ctx* ctx, int dtype, void* dbias, const void* dz, size_t rows, int cols) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (rows == 0 || cols <= 0) return cols < 0 ? fail(D8K_ERR_ARGUMENT, "the shape is error") : 0;
    if (!dbias || !dz) return fail(D8K_ERR_ARGUMENT, "add_bias_grad: null pointer");
    return column_sums(ctx, dtype, dbias, dz, rows, cols, nullptr, 1);
}

int d8k_conv2d_out_dim(int in, int filter, int stride, int dilation, int covered) {
    int real = filter + (filter - 1) * (dilation - 1);
    return covered ? (in - 1) / stride + 1 : (in - real) / stride + 1;
}
int d8k_deconv2d_out_dim(int in, int filter, int stride, int covered) { return covered ? (in - 1) * stride + 1 : (in - 1) * stride + filter; }

size_t d8k_conv2d_interim_size(const d8k_ctx* ctx, int which, int dtype, int batch, int ih, int iw, int ic, int oc, int fh, int fw, int oh,
                               int ow) {
    if (!ctx || which < 0 || which > 2) return 0;
    ConvDims d{batch, ih, iw, ic, oc, fh, fw, oh, ow};
    ConvRule f, b;
    conv_rules(d, 1, 1, 1, 1, &f, &b);
    size_t need = 0;
    conv_like(const_cast<d8k_ctx*>(ctx), which, dtype, d, f, b, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, true, &need);
    return need;
}
size_t d8k_deconv2d_interim_size(const d8k_ctx* ctx, int which, int dtype, int batch, int ih, int iw, int ic, int oc, int fh, int fw,
                                 int oh, int ow) {
    return d8k_conv2d_interim_size(ctx, which, dtype, batch, ih, iw, ic, oc, fh, fw, oh, ow);  // same contraction shapes
}

#define D8K_CONV_PROLOGUE(strideY, strideX, dilY, dilX)                    \
    if (int rc = check_ctx(ctx)) return rc;                                \
    if (int rc = check_dtype(dtype)) return rc;                            \
    ConvDims d{batch, ih, iw, ic, oc, fh, fw, oh, ow};                     \
    if (int rc = check_conv(d, strideY, strideX, dilY, dilX)) return rc;   \
    ConvRule fwd, bwd;

int d8k_conv2d_forward(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                       void* z, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim, size_t interim_bytes) {
    D8K_CONV_PROLOGUE(strideY, strideX, dilationY, dilationX)
    conv_rules(d, strideY, strideX, dilationY, dilationX, &fwd, &bwd);
    return conv_like(ctx, 0, dtype, d, fwd, bwd, x, nullptr, y, nullptr, z, nullptr, interim, interim_bytes, false, nullptr);
}
int d8k_conv2d_grad_x(d8k_ctx* ctx, int dtype, void* dx, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                      const void* dz, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim,
                      size_t interim_bytes) {
    D8K_CONV_PROLOGUE(strideY, strideX, dilationY, dilationX)
    conv_rules(d, strideY, strideX, dilationY, dilationX, &fwd, &bwd);
    return conv_like(ctx, 1, dtype, d, fwd, bwd, nullptr, dx, y, nullptr, nullptr, dz, interim, interim_bytes, false, nullptr);
}
int d8k_conv2d_grad_y(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, void* dy, int oc, int fh, int fw,
                      const void* dz, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim,
                      size_t interim_bytes) {
    D8K_CONV_PROLOGUE(strideY, strideX, dilationY, dilationX)
    conv_rules(d, strideY, strideX, dilationY, dilationX, &fwd, &bwd);
    return conv_like(ctx, 2, dtype, d, fwd, bwd, x, nullptr, nullptr, dy, nullptr, dz, interim, interim_bytes, false, nullptr);
}

int d8k_conv2d_grad_x_into(d8k_ctx* ctx, int dtype, void* dx, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                           const void* dz, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim,
                           size_t interim_bytes, int accumulate) {
    D8K_CONV_PROLOGUE(strideY, strideX, dilationY, dilationX)
    conv_rules(d, strideY, strideX, dilationY, dilationX, &fwd, &bwd);
    return conv_like(ctx, 1, dtype, d, fwd, bwd, nullptr, dx, y, nullptr, nullptr, dz, interim, interim_bytes, false, nullptr, accumulate);
}
int d8k_conv2d_grad_y_into(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, void* dy, int oc, int fh, int fw,
                           const void* dz, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim,
                           size_t interim_bytes, int accumulate) {
    D8K_CONV_PROLOGUE(strideY, strideX, dilationY, dilationX)
    conv_rules(d, strideY, strideX, dilationY, dilationX, &fwd, &bwd);
    return conv_like(ctx, 2, dtype, d, fwd, bwd, x, nullptr, nullptr, dy, nullptr, dz, interim, interim_bytes, false, nullptr, accumulate);
}
int d8k_deconv2d_grad_x_into(d8k_ctx* ctx, int dtype, void* dx, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                             const void* dz, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes, int accumulate) {
    D8K_CONV_PROLOGUE(strideY, strideX, 1, 1)
    deconv_rules(d, strideY, strideX, &fwd, &bwd);
    return conv_like(ctx, 1, dtype, d, fwd, bwd, nullptr, dx, y, nullptr, nullptr, dz, interim, interim_bytes, false, nullptr, accumulate);
}
int d8k_deconv2d_grad_y_into(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, void* dy, int oc, int fh, int fw,
                             const void* dz, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes, int accumulate) {
    D8K_CONV_PROLOGUE(strideY, strideX, 1, 1)
    deconv_rules(d, strideY, strideX, &fwd, &bwd);
    return conv_like(ctx, 2, dtype, d, fwd, bwd, x, nullptr, nullptr, dy, nullptr, dz, interim, interim_bytes, false, nullptr, accumulate);
}

int d8k_deconv2d_forward(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                         void* z, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes) {
    D8K_CONV_PROLOGUE(strideY, strideX, 1, 1)
    deconv_rules(d, strideY, strideX, &fwd, &bwd);
    return conv_like(ctx, 0, dtype, d, fwd, bwd, x, nullptr, y, nullptr, z, nullptr, interim, interim_bytes, false, nullptr);
}
int d8k_deconv2d_grad_x(d8k_ctx* ctx, int dtype, void* dx, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                        const void* dz, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes) {
    D8K_CONV_PROLOGUE(strideY, strideX, 1, 1)
    deconv_rules(d, strideY, strideX, &fwd, &bwd);
    return conv_like(ctx, 1, dtype, d, fwd, bwd, nullptr, dx, y, nullptr, nullptr, dz, interim, interim_bytes, false, nullptr);
}
int d8k_deconv2d_grad_y(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, void* dy, int oc, int fh, int fw,
                        const void* dz, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes) {
    D8K_CONV_PROLOGUE(strideY, strideX, 1, 1)
    deconv_rules(d, strideY, strideX, &fwd, &bwd);
    return conv_like(ctx, 2, dtype, d, fwd, bwd, x, nullptr, nullptr, dy, nullptr, dz, interim, interim_bytes, false, nullptr);
}

int d8k_relu_forward(d8k_ctx* ctx, int dtype, const void* x, void* y, size_t n) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (n == 0) return 0;
    if (!x || !y) return fail(D8K_ERR_ARGUMENT, "relu: null pointer");
    bool vec = aligned16(x, y, nullptr);
    if (dtype == D8K_F32)
        relu_forward_kernel<float><<<elementwise_grid(ctx, n, 4), 256, 0, ctx->stream>>>(static_cast<const float*>(x), static_cast<float*>(y), n, vec);
    else
        relu_forward_kernel<__half><<<elementwise_grid(ctx, n, 8), 256, 0, ctx->stream>>>(static_cast<const __half*>(x), static_cast<__half*>(y), n, vec);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

int d8k_relu_backward(d8k_ctx* ctx, int dtype, const void* x, void* dx, const void* dy, size_t n) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (n == 0) return 0;
    if (!x || !dx || !dy) return fail(D8K_ERR_ARGUMENT, "relu: null pointer");
    bool vec = aligned16(x, dx, dy);
    if (dtype == D8K_F32)
        relu_backward_kernel<float><<<elementwise_grid(ctx, n, 4), 256, 0, ctx->stream>>>(static_cast<const float*>(x), static_cast<float*>(dx),
                                                                                        static_cast<const float*>(dy), n, vec);
    else
        relu_backward_kernel<__half><<<elementwise_grid(ctx, n, 8), 256, 0, ctx->stream>>>(static_cast<const __half*>(x), static_cast<__half*>(dx),
                                                                                         static_cast<const __half*>(dy), n, vec);
    D8K_CUDA(cudaGetLastError());
    count_launch();
    return 0;
}

int d8k_zero(d8k_ctx* ctx, void* ptr, size_t bytes) {
    if (int rc = check_ctx(ctx)) return rc;
    if (bytes == 0) return 0;
    if (!ptr) return fail(D8K_ERR_ARGUMENT, "zero: null pointer");
    D8K_CUDA(cudaMemsetAsync(ptr, 0, bytes, ctx->stream));
    return 0;
}

}  // extern "C"
