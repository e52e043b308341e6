/* TEST INFRASTRUCTURE, not product code.
 *
 * Plain-C restatement of the reference's dense-contraction path: MatrixMultiply, Conv2d and DeConv2d,
 * forward and both gradients, as direct loops over the index rules of the reference.  Only tests, the
 * smoke check and the benchmark's CPU-baseline leg may load this library; the product never does.
 *
 * Pinned: tests/test_oracle.py checks every function here against the reference's own CPU code
 * (oracle/_ref/libd8ref.so, built from the unmodified reference sources) on the shapes of the
 * reference's unit tests with integer-valued data (exact equality, as those tests assert) and on the
 * committed golden vectors under tests/golden/ (generated from the reference by tests/golden/make_golden.py).
 *
 * Arithmetic: every output element is one sum, accumulated in double in a fixed order and rounded once to
 * the storage type, so the result is the correctly rounded value of the exact contraction (up to double
 * rounding); the reference's Eigen float path differs from it only by float accumulation error.
 *
 * Each function cites the reference lines it follows (paths within the reference project).
 */
#ifndef D8O_T /* ---------------------------------------------------------------- first pass: shared part */

#include <math.h>
#include <stddef.h>
#include <stdint.h>

#define D8O_API __attribute__((visibility("default")))

static int d8o_max(int a, int b) { return a > b ? a : b; }

/* Output extent of Conv2d along one axis: deep8/src/nodes/Conv2d.cpp:47-63.
 * realF = f + (f-1)(dilation-1); not covered: (in - realF)/stride + 1; covered: (in - 1)/stride + 1. */
D8O_API int d8o_conv2d_out_dim(int in, int f, int stride, int dilation, int covered) {
    int realF = f + (f - 1) * (dilation - 1);
    if (covered) return (in - 1) / stride + 1;
    return (in - realF) / stride + 1;
}

/* Output extent of DeConv2d along one axis: deep8/src/nodes/DeConv2d.cpp:36-52.
 * not covered: (in-1)*stride + f; covered: (in-1)*stride + 1. */
D8O_API int d8o_deconv2d_out_dim(int in, int f, int stride, int covered) {
    if (covered) return (in - 1) * stride + 1;
    return (in - 1) * stride + f;
}

/* First input row touched by output row 0, a value <= 0: deep8/src/math/Conv2d.cu:334-335
 * padTop = -(max(0, (out-1)*stride + realF - in) / 2). */
D8O_API int d8o_conv2d_pad_before(int in, int out, int f, int stride, int dilation) {
    int realF = f + (f - 1) * (dilation - 1);
    return -(d8o_max(0, (out - 1) * stride + realF - in) / 2);
}

/* deep8/src/math/DeConv2d.cu:99-100: padTop = -(max(0, out + f - (in-1)*stride - 2) / 2). */
D8O_API int d8o_deconv2d_pad_before(int in, int out, int f, int stride) {
    return -(d8o_max(0, out + f - (in - 1) * stride - 2) / 2);
}

#define D8O_T float
#define D8O_(name) name##_f32
#include "d8_oracle.c"
#undef D8O_T
#undef D8O_

#define D8O_T double
#define D8O_(name) name##_f64
#include "d8_oracle.c"
#undef D8O_T
#undef D8O_

#else /* ------------------------------------------------------------------------ typed part (included twice) */

/* MatrixMultiply.  x is xb matrices [xr x xc], y is yb matrices [xc x yc], z is max(xb,yb) matrices [xr x yc];
 * a batch of 1 is broadcast (index b % batch).  All three branches of the reference
 * (deep8/src/math/MatrixMultiply.cpp:93-116: y.batch==1 folded into M; x.batch==1 && y.col()==1 as Y*X^T;
 * the general per-batch loop) compute exactly z_b = x_(b%xb) * y_(b%yb); they differ in blocking only. */
D8O_API void D8O_(d8o_matmul_forward)(const D8O_T* x, size_t xb, size_t xr, size_t xc,
                                     const D8O_T* y, size_t yb, size_t yc, D8O_T* z) {
    size_t zb = xb > yb ? xb : yb;
#pragma omp parallel for collapse(2) schedule(static)
    for (size_t b = 0; b < zb; ++b) {
        for (size_t i = 0; i < xr; ++i) {
            const D8O_T* xm = x + (b % xb) * xr * xc;
            const D8O_T* ym = y + (b % yb) * xc * yc;
            D8O_T* zm = z + b * xr * yc;
            for (size_t j = 0; j < yc; ++j) {
                double acc = 0;
                for (size_t k = 0; k < xc; ++k) acc += (double)xm[i * xc + k] * (double)ym[k * yc + j];
                zm[i * yc + j] = (D8O_T)acc;
            }
        }
    }
}

/* dX_(b%xb) += dZ_b * Y_(b%yb)^T, deep8/src/math/MatrixMultiply.cpp:133-163.  When x is broadcast (xb == 1 < zb) the
 * contributions of every b are summed into the one dX (the `b % xshape.batch` at :160). */
D8O_API void D8O_(d8o_matmul_grad_x)(D8O_T* dx, size_t xb, size_t xr, size_t xc,
                                    const D8O_T* y, size_t yb, size_t yc, const D8O_T* dz) {
    size_t zb = xb > yb ? xb : yb;
#pragma omp parallel for collapse(2) schedule(static)
    for (size_t bx = 0; bx < xb; ++bx) {
        for (size_t i = 0; i < xr; ++i) {
            for (size_t k = 0; k < xc; ++k) {
                double acc = 0;
                for (size_t b = bx; b < zb; b += xb) {
                    const D8O_T* ym = y + (b % yb) * xc * yc;
                    const D8O_T* dzm = dz + b * xr * yc;
                    for (size_t j = 0; j < yc; ++j) acc += (double)dzm[i * yc + j] * (double)ym[k * yc + j];
                }
                D8O_T* d = dx + bx * xr * xc + i * xc + k;
                *d = (D8O_T)((double)*d + acc);
            }
        }
    }
}

/* dY_(b%yb) += X_(b%xb)^T * dZ_b, deep8/src/math/MatrixMultiply.cpp:180-210.  With y.batch == 1 the sum over the
 * batch is the reference's K = xb*xr of one product (:186-194). */
D8O_API void D8O_(d8o_matmul_grad_y)(const D8O_T* x, size_t xb, size_t xr, size_t xc,
                                    D8O_T* dy, size_t yb, size_t yc, const D8O_T* dz) {
    size_t zb = xb > yb ? xb : yb;
#pragma omp parallel for collapse(2) schedule(static)
    for (size_t by = 0; by < yb; ++by) {
        for (size_t k = 0; k < xc; ++k) {
            for (size_t j = 0; j < yc; ++j) {
                double acc = 0;
                for (size_t b = by; b < zb; b += yb) {
                    const D8O_T* xm = x + (b % xb) * xr * xc;
                    const D8O_T* dzm = dz + b * xr * yc;
                    for (size_t i = 0; i < xr; ++i) acc += (double)xm[i * xc + k] * (double)dzm[i * yc + j];
                }
                D8O_T* d = dy + by * xc * yc + k * yc + j;
                *d = (D8O_T)((double)*d + acc);
            }
        }
    }
}

/* Conv2d forward.  x [b, ih, iw, ic], filter y [oc, fh, fw, ic], z [b, oh, ow, oc].
 * Index rule of the reference's im2col (deep8/src/math/Conv2d.cu:44-45): inY = padTop + oy*strideY + fy*dilationY
 * with padTop <= 0 from Conv2dGPU (:334-335); taps outside the image read zero (:49-53); then the GEMM
 * z[M x oc] = col[M x (fh*fw*ic)] * y^T (:188-195). */
D8O_API void D8O_(d8o_conv2d_forward)(const D8O_T* x, int b, int ih, int iw, int ic,
                                     const D8O_T* y, int oc, int fh, int fw,
                                     D8O_T* z, int oh, int ow,
                                     int strideY, int strideX, int dilationY, int dilationX) {
    int padTop = d8o_conv2d_pad_before(ih, oh, fh, strideY, dilationY);
    int padLeft = d8o_conv2d_pad_before(iw, ow, fw, strideX, dilationX);
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < b; ++n) {
        for (int oy = 0; oy < oh; ++oy) {
            for (int ox = 0; ox < ow; ++ox) {
                for (int o = 0; o < oc; ++o) {
                    double acc = 0;
                    for (int fy = 0; fy < fh; ++fy) {
                        int iy = padTop + oy * strideY + fy * dilationY;
                        if (iy < 0 || iy >= ih) continue;
                        for (int fx = 0; fx < fw; ++fx) {
                            int ix = padLeft + ox * strideX + fx * dilationX;
                            if (ix < 0 || ix >= iw) continue;
                            const D8O_T* xp = x + (((size_t)n * ih + iy) * iw + ix) * ic;
                            const D8O_T* wp = y + (((size_t)o * fh + fy) * fw + fx) * ic;
                            for (int c = 0; c < ic; ++c) acc += (double)xp[c] * (double)wp[c];
                        }
                    }
                    z[(((size_t)n * oh + oy) * ow + ox) * oc + o] = (D8O_T)acc;
                }
            }
        }
    }
}

/* Conv2d gradient of x: dcol = dz * y (deep8/src/math/Conv2d.cu:466-475), then col2im accumulates into dx
 * (:99-113): outY = inY - padTop - fy*dilationY must be a multiple of strideY and, divided, lie in [0, oh). */
D8O_API void D8O_(d8o_conv2d_grad_x)(D8O_T* dx, int b, int ih, int iw, int ic,
                                    const D8O_T* y, int oc, int fh, int fw,
                                    const D8O_T* dz, int oh, int ow,
                                    int strideY, int strideX, int dilationY, int dilationX) {
    int padTop = d8o_conv2d_pad_before(ih, oh, fh, strideY, dilationY);
    int padLeft = d8o_conv2d_pad_before(iw, ow, fw, strideX, dilationX);
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < b; ++n) {
        for (int iy = 0; iy < ih; ++iy) {
            for (int ix = 0; ix < iw; ++ix) {
                for (int c = 0; c < ic; ++c) {
                    double acc = 0;
                    for (int fy = 0; fy < fh; ++fy) {
                        int ny = iy - padTop - fy * dilationY;
                        if (ny < 0 || ny % strideY != 0 || ny / strideY >= oh) continue;
                        for (int fx = 0; fx < fw; ++fx) {
                            int nx = ix - padLeft - fx * dilationX;
                            if (nx < 0 || nx % strideX != 0 || nx / strideX >= ow) continue;
                            const D8O_T* dzp = dz + (((size_t)n * oh + ny / strideY) * ow + nx / strideX) * oc;
                            for (int o = 0; o < oc; ++o)
                                acc += (double)dzp[o] * (double)y[(((size_t)o * fh + fy) * fw + fx) * ic + c];
                        }
                    }
                    D8O_T* d = dx + (((size_t)n * ih + iy) * iw + ix) * ic + c;
                    *d = (D8O_T)((double)*d + acc);
                }
            }
        }
    }
}

/* Conv2d gradient of the filter: dy[oc x Kc] += dz^T[oc x M] * col[M x Kc] (deep8/src/math/Conv2d.cu:771-801),
 * col built by the same im2col rule as forward. */
D8O_API void D8O_(d8o_conv2d_grad_y)(const D8O_T* x, int b, int ih, int iw, int ic,
                                    D8O_T* dy, int oc, int fh, int fw,
                                    const D8O_T* dz, int oh, int ow,
                                    int strideY, int strideX, int dilationY, int dilationX) {
    int padTop = d8o_conv2d_pad_before(ih, oh, fh, strideY, dilationY);
    int padLeft = d8o_conv2d_pad_before(iw, ow, fw, strideX, dilationX);
#pragma omp parallel for collapse(3) schedule(static)
    for (int o = 0; o < oc; ++o) {
        for (int fy = 0; fy < fh; ++fy) {
            for (int fx = 0; fx < fw; ++fx) {
                for (int c = 0; c < ic; ++c) {
                    double acc = 0;
                    for (int n = 0; n < b; ++n) {
                        for (int oy = 0; oy < oh; ++oy) {
                            int iy = padTop + oy * strideY + fy * dilationY;
                            if (iy < 0 || iy >= ih) continue;
                            for (int ox = 0; ox < ow; ++ox) {
                                int ix = padLeft + ox * strideX + fx * dilationX;
                                if (ix < 0 || ix >= iw) continue;
                                acc += (double)dz[(((size_t)n * oh + oy) * ow + ox) * oc + o] *
                                       (double)x[(((size_t)n * ih + iy) * iw + ix) * ic + c];
                            }
                        }
                    }
                    D8O_T* d = dy + (((size_t)o * fh + fy) * fw + fx) * ic + c;
                    *d = (D8O_T)((double)*d + acc);
                }
            }
        }
    }
}

/* DeConv2d forward.  x [b, ih, iw, ic], filter y [oc, fh, fw, ic], z [b, oh, ow, oc].
 * zmat = x * ymat^T with ymat = y viewed [(oc,fy,fx) x ic] (deep8/src/math/DeConv2d.cu:102-109); the gather
 * (:41-52) sums the taps with (oy + padTop + fy) a multiple of strideY whose quotient lies in [0, ih);
 * padTop <= 0 from :99-100.  The output is overwritten (:56). */
D8O_API void D8O_(d8o_deconv2d_forward)(const D8O_T* x, int b, int ih, int iw, int ic,
                                       const D8O_T* y, int oc, int fh, int fw,
                                       D8O_T* z, int oh, int ow, int strideY, int strideX) {
    int padTop = d8o_deconv2d_pad_before(ih, oh, fh, strideY);
    int padLeft = d8o_deconv2d_pad_before(iw, ow, fw, strideX);
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < b; ++n) {
        for (int oy = 0; oy < oh; ++oy) {
            for (int ox = 0; ox < ow; ++ox) {
                for (int o = 0; o < oc; ++o) {
                    double acc = 0;
                    for (int fy = 0; fy < fh; ++fy) {
                        int ny = oy + padTop + fy;
                        if (ny < 0 || ny % strideY != 0 || ny / strideY >= ih) continue;
                        for (int fx = 0; fx < fw; ++fx) {
                            int nx = ox + padLeft + fx;
                            if (nx < 0 || nx % strideX != 0 || nx / strideX >= iw) continue;
                            const D8O_T* xp = x + (((size_t)n * ih + ny / strideY) * iw + nx / strideX) * ic;
                            const D8O_T* wp = y + (((size_t)o * fh + fy) * fw + fx) * ic;
                            for (int c = 0; c < ic; ++c) acc += (double)xp[c] * (double)wp[c];
                        }
                    }
                    z[(((size_t)n * oh + oy) * ow + ox) * oc + o] = (D8O_T)acc;
                }
            }
        }
    }
}

/* DeConv2d gradient of x: dzmat gathered by oy = iy*strideY - padTop - fy, zero outside (deep8/src/math/DeConv2d.cu:342-349),
 * then dx[m x ic] += dzmat[m x (oc,fy,fx)] * ymat (:420-428). */
D8O_API void D8O_(d8o_deconv2d_grad_x)(D8O_T* dx, int b, int ih, int iw, int ic,
                                      const D8O_T* y, int oc, int fh, int fw,
                                      const D8O_T* dz, int oh, int ow, int strideY, int strideX) {
    int padTop = d8o_deconv2d_pad_before(ih, oh, fh, strideY);
    int padLeft = d8o_deconv2d_pad_before(iw, ow, fw, strideX);
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < b; ++n) {
        for (int iy = 0; iy < ih; ++iy) {
            for (int ix = 0; ix < iw; ++ix) {
                for (int c = 0; c < ic; ++c) {
                    double acc = 0;
                    for (int fy = 0; fy < fh; ++fy) {
                        int oy = iy * strideY - padTop - fy;
                        if (oy < 0 || oy >= oh) continue;
                        for (int fx = 0; fx < fw; ++fx) {
                            int ox = ix * strideX - padLeft - fx;
                            if (ox < 0 || ox >= ow) continue;
                            const D8O_T* dzp = dz + (((size_t)n * oh + oy) * ow + ox) * oc;
                            for (int o = 0; o < oc; ++o)
                                acc += (double)dzp[o] * (double)y[(((size_t)o * fh + fy) * fw + fx) * ic + c];
                        }
                    }
                    D8O_T* d = dx + (((size_t)n * ih + iy) * iw + ix) * ic + c;
                    *d = (D8O_T)((double)*d + acc);
                }
            }
        }
    }
}

/* DeConv2d gradient of the filter: dy[(oc,fy,fx) x ic] += dzmat^T * x (deep8/src/math/DeConv2d.cu:668-699), dzmat as above. */
D8O_API void D8O_(d8o_deconv2d_grad_y)(const D8O_T* x, int b, int ih, int iw, int ic,
                                      D8O_T* dy, int oc, int fh, int fw,
                                      const D8O_T* dz, int oh, int ow, int strideY, int strideX) {
    int padTop = d8o_deconv2d_pad_before(ih, oh, fh, strideY);
    int padLeft = d8o_deconv2d_pad_before(iw, ow, fw, strideX);
#pragma omp parallel for collapse(3) schedule(static)
    for (int o = 0; o < oc; ++o) {
        for (int fy = 0; fy < fh; ++fy) {
            for (int fx = 0; fx < fw; ++fx) {
                for (int c = 0; c < ic; ++c) {
                    double acc = 0;
                    for (int n = 0; n < b; ++n) {
                        for (int iy = 0; iy < ih; ++iy) {
                            int oy = iy * strideY - padTop - fy;
                            if (oy < 0 || oy >= oh) continue;
                            for (int ix = 0; ix < iw; ++ix) {
                                int ox = ix * strideX - padLeft - fx;
                                if (ox < 0 || ox >= ow) continue;
                                acc += (double)dz[(((size_t)n * oh + oy) * ow + ox) * oc + o] *
                                       (double)x[(((size_t)n * ih + iy) * iw + ix) * ic + c];
                            }
                        }
                    }
                    D8O_T* d = dy + (((size_t)o * fh + fy) * fw + fx) * ic + c;
                    *d = (D8O_T)((double)*d + acc);
                }
            }
        }
    }
}

/* Math::AXPBY (deep8/src/math/AXPBY.cpp:22-31): z = x * alpha + y * beta, each product and the sum rounded in T
 * (the reference's build has no fused multiply-add: no -m flags, deep8/CMakeLists.txt:86).  z may be x or y.
 * SGDTrainer::update (deep8/src/trainer/SGDTrainer.cpp:9-17) is this with x = gradient, y = z = value,
 * alpha = -learningRate, beta = 1 - learningRate * weightDecay. */
D8O_API void D8O_(d8o_axpby)(const D8O_T* x, D8O_T alpha, const D8O_T* y, D8O_T beta, D8O_T* z, size_t n) {
#pragma STDC FP_CONTRACT OFF
    for (size_t i = 0; i < n; ++i) {
        volatile D8O_T a = x[i] * alpha;
        volatile D8O_T b = y[i] * beta;
        z[i] = a + b;
    }
}

/* Math::Add for a bias: x (batch, {rows, cols}) + y (1, {cols}) broadcast over batch and rows
 * (deep8/src/math/Add.cpp:7-31, 112-146; shapes aligned from the tail, deep8/include/utils/ShapeUtils.h:40-55). */
D8O_API void D8O_(d8o_add_bias)(const D8O_T* x, const D8O_T* bias, D8O_T* z, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) z[r * cols + c] = x[r * cols + c] + bias[c];
}

/* Math::AddGradY for that bias: dbias[c] += sum over batch and rows of dz (deep8/src/math/Add.cpp:165-187, the
 * broadcast dimensions are summed). */
D8O_API void D8O_(d8o_add_bias_grad)(D8O_T* dbias, const D8O_T* dz, size_t rows, size_t cols) {
    for (size_t c = 0; c < cols; ++c) {
        double acc = 0;
        for (size_t r = 0; r < rows; ++r) acc += (double)dz[r * cols + c];
        dbias[c] = (D8O_T)((double)dbias[c] + acc);
    }
}

/* Math::ReLu (deep8/src/math/ReLu.cpp:39-47): y = max(x, 0). */
D8O_API void D8O_(d8o_relu)(const D8O_T* x, D8O_T* y, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = x[i] > (D8O_T)0 ? x[i] : (D8O_T)0;
}

/* Math::ReLuGrad (deep8/src/math/ReLu.cpp:64-80): dx += (x > 0 ? dy : 0). */
D8O_API void D8O_(d8o_relu_grad)(const D8O_T* x, D8O_T* dx, const D8O_T* dy, size_t n) {
    for (size_t i = 0; i < n; ++i) dx[i] = dx[i] + (x[i] > (D8O_T)0 ? dy[i] : (D8O_T)0);
}

/* Math::Linear (deep8/src/math/Linear.cpp:46-54): y = x * a + b, product and sum rounded separately in T. */
D8O_API void D8O_(d8o_linear)(const D8O_T* x, D8O_T a, D8O_T b, D8O_T* y, size_t n) {
#pragma STDC FP_CONTRACT OFF
    for (size_t i = 0; i < n; ++i) {
        volatile D8O_T t = x[i] * a;
        y[i] = t + b;
    }
}

/* Math::LinearGrad (deep8/src/math/Linear.cpp:72-80): dx += dy * a. */
D8O_API void D8O_(d8o_linear_grad)(D8O_T* dx, D8O_T a, const D8O_T* dy, size_t n) {
#pragma STDC FP_CONTRACT OFF
    for (size_t i = 0; i < n; ++i) {
        volatile D8O_T t = dy[i] * a;
        dx[i] = dx[i] + t;
    }
}

/* Math::AdamUpdate (deep8/src/math/AdamUpdate.cpp:24-41), statement by statement, every operation rounded in T:
 *   gradient += value * weightDecay
 *   m = m * beta1 + gradient * (1 - beta1)
 *   v = v * beta2 + gradient^2 * (1 - beta2)
 *   value -= m / (sqrt(v) + epsilon) * ratio
 * `ratio` = learningRate * sqrt(1 - beta2^steps) / (1 - beta1^steps) is computed by the caller. */
D8O_API void D8O_(d8o_adam_update)(D8O_T* value, D8O_T* gradient, D8O_T* m, D8O_T* v, D8O_T beta1, D8O_T beta2, D8O_T epsilon,
                                   D8O_T weight_decay, D8O_T ratio, size_t n) {
#pragma STDC FP_CONTRACT OFF
    volatile D8O_T c1 = (D8O_T)1 - beta1, c2 = (D8O_T)1 - beta2;
    for (size_t i = 0; i < n; ++i) {
        volatile D8O_T t = value[i] * weight_decay;
        volatile D8O_T g = gradient[i] + t;
        gradient[i] = g;
        volatile D8O_T m1 = m[i] * beta1, m2 = g * c1;
        volatile D8O_T mm = m1 + m2;
        m[i] = mm;
        volatile D8O_T gg = g * g;
        volatile D8O_T v1 = v[i] * beta2, v2 = gg * c2;
        volatile D8O_T vv = v1 + v2;
        v[i] = vv;
        volatile D8O_T root = sizeof(D8O_T) == 4 ? (D8O_T)sqrtf((float)vv) : (D8O_T)sqrt((double)vv);
        volatile D8O_T den = root + epsilon;
        volatile D8O_T q = mm / den;
        volatile D8O_T step = q * ratio;
        value[i] = value[i] - step;
    }
}

#endif
