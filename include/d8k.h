/* deep8_b200 C ABI: the B200 (sm_100a) kernels behind Deep8's dense-contraction operators.
 *
 * Every entry point below stands where one GPU function of the reference stands; the reference's `Tensor` arguments
 * are flattened to raw device pointers and dims (row-major, batch outermost; images [batch, height, width, channel],
 * filters [outChannel, filterHeight, filterWidth, inChannel]).  Paths in the citations are relative to the
 * reference project.
 *
 * Conventions (the reference's, deep8/include/math/{MatrixMultiply,Conv2d,DeConv2d}.h):
 *   - forward overwrites z; every gradient entry point ACCUMULATES (+=) into dx / dy;
 *   - dtype is D8K_F16 (fp16 storage, fp32 accumulation) or D8K_F32 (3xTF32 split precision, fp32 accumulation);
 *   - all pointers are device pointers on the context's device; work is enqueued on the context's stream and the
 *     call returns without waiting;
 *   - return value 0 on success; otherwise an error code, with the text available from d8k_last_error()
 *     (D8K_ERR_ARGUMENT maps to the reference's std::invalid_argument, the others to std::runtime_error).
 * A context is to be used by one host thread / one stream at a time (it owns the split-K scratch memory), like the
 * cuBLAS handle inside the reference's GPUDevice (deep8/include/model/GPUDevice.h:12-70).
 */
#ifndef D8K_H
#define D8K_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define D8K_F16 0
#define D8K_F32 1

#define D8K_OK 0
#define D8K_ERR_ARGUMENT 1 /* bad shape, null pointer, unsupported dtype */
#define D8K_ERR_CUDA 2     /* a CUDA runtime or driver call failed */
#define D8K_ERR_KERNEL 3   /* a kernel gave up on a bounded wait; see d8k_ctx_status */

#if defined(__GNUC__)
#define D8K_API __attribute__((visibility("default")))
#else
#define D8K_API
#endif

typedef struct d8k_ctx d8k_ctx;

/* Replaces the GPU half of GPUDevice's constructor (deep8/src/model/GPUDevice.cu:10-65): selects `device`, allocates
 * the split-K scratch memory (scratch_bytes, 0 = default 64 MiB) and the kernel status word. */
D8K_API int d8k_ctx_create(int device, size_t scratch_bytes, d8k_ctx** out);
D8K_API int d8k_ctx_destroy(d8k_ctx* ctx);
/* Stream the kernels are enqueued on (a cudaStream_t); the default is the legacy default stream, as in the reference. */
D8K_API int d8k_ctx_set_stream(d8k_ctx* ctx, void* stream);
/* Waits for the stream, then reports the device status word: 0, or (role << 8 | barrier) of the first wait that
 * expired inside a kernel.  Returns D8K_ERR_KERNEL when it is non-zero (and clears it). */
D8K_API int d8k_ctx_status(d8k_ctx* ctx, int* status);
D8K_API int d8k_ctx_num_sms(const d8k_ctx* ctx);
D8K_API const char* d8k_last_error(void);

/* Number of kernels this library has launched from the calling process since it was loaded. */
D8K_API unsigned long long d8k_launch_count(void);
/* Which contraction kernel the calling thread's last launch used, as text: dtype, "pair" / "tma" / "gather", how the TMA
 * producer fetched each operand, tile width, split count, grid.  For tests and profiles; not a stable format. */
D8K_API const char* d8k_last_kernel(void);

/* General contraction, row-major:  C[b] (+)= op(A[b % batchA]) * op(B[b % batchB]),  b < batch.
 *   transA == 0: A[b] is M x K with pitch lda;  transA != 0: A[b] is K x M with pitch lda (its transpose is used)
 *   transB == 0: B[b] is K x N with pitch ldb;  transB != 0: B[b] is N x K with pitch ldb
 *   beta is 0 (overwrite C) or 1 (accumulate into C)
 *   reduce_batch != 0: one output C[0] (+)= sum over b < batch of op(A[b]) * op(B[b])  (the batch joins the contraction)
 * This is the cublas{S,H}gemm call of the reference (deep8/src/math/MatrixMultiply.cu:31-56, 205-231, 393-419) with the
 * host loop over the batch folded into one launch. */
D8K_API int d8k_gemm(d8k_ctx* ctx, int dtype, int transA, int transB, int M, int N, int K,
             const void* A, long long lda, int batchA, long long strideA,
             const void* B, long long ldb, int batchB, long long strideB,
             void* C, long long ldc, long long strideC, int batch, int beta, int reduce_batch);

/* No counterpart in the reference.  The same contraction as d8k_gemm for one matrix pair (no batch), for callers that
 * may not allocate device memory and therefore cannot create a context: the split-K scratch is a static device array
 * inside the library, 16 MiB of partial tiles (+ 20 KiB of bookkeeping) held by every GPU that loads the library until
 * the process exits.  Runs on the current device, on `stream` (a cudaStream_t, NULL = legacy default stream).  A
 * contraction whose split-K partial tiles need more than the 16 MiB is rejected with D8K_ERR_ARGUMENT.  The first call
 * on a device looks up the array's device address: make it before any stream capture.  Calls share the array: two calls
 * whose kernels overlap on the GPU race; issue them on one stream or serialise them.  A bounded wait that expires inside
 * the kernel is not reported through this entry point. */
D8K_API int d8k_gemm_static(int dtype, int transA, int transB, int M, int N, int K, const void* A, long long lda,
                            const void* B, long long ldb, void* C, long long ldc, int beta, void* stream);

/* MatrixMultiplyGPU (deep8/src/math/MatrixMultiply.cu:139-176): z[b] = x[b % xb] * y[b % yb];
 * x is xb matrices xr x xc, y is yb matrices xc x yc, z is max(xb, yb) matrices xr x yc; xb, yb equal or 1.
 * The three branches of the reference (MatrixMultiply.cu:31-56) map to: yb == 1 - one contraction with the batch folded into
 * the rows (a matrix-vector kernel when yc == 1); xb == 1 and yc == 1 - one contraction Z [yb x xr] = Y [yb x xc] * X^T;
 * otherwise one batched launch.  The gradients follow the same three cases (MatrixMultiply.cu:205-231, 393-419). */
D8K_API int d8k_matmul_forward(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc, void* z);
/* MatrixMultiplyGradXGPU (MatrixMultiply.cu:320-363): dx[b % xb] += dz[b] * y[b % yb]^T (summed over b when xb == 1). */
D8K_API int d8k_matmul_grad_x(d8k_ctx* ctx, int dtype, void* dx, int xb, int xr, int xc, const void* y, int yb, int yc, const void* dz);
/* MatrixMultiplyGradYGPU (MatrixMultiply.cu:508-551): dy[b % yb] += x[b % xb]^T * dz[b] (summed over b when yb == 1). */
D8K_API int d8k_matmul_grad_y(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, void* dy, int yb, int yc, const void* dz);

/* The two gradient entry points with the accumulation made explicit: accumulate != 0 is the reference's += (beta = 1 in
 * its gemm calls, MatrixMultiply.cu:203, 391); accumulate == 0 overwrites, for an executor that knows this is the first
 * contribution to the gradient and skips Variable::zeroGradient (deep8/src/model/EagerExecutor.cpp:51-65). */
D8K_API int d8k_matmul_grad_x_into(d8k_ctx* ctx, int dtype, void* dx, int xb, int xr, int xc, const void* y, int yb, int yc, const void* dz,
                           int accumulate);
D8K_API int d8k_matmul_grad_y_into(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, void* dy, int yb, int yc, const void* dz,
                           int accumulate);
/* MatrixMultiplyGPU followed by ReLuGPU (deep8/src/math/ReLu.cu:17-56) in one launch: z = x * y and a = max(z, 0), both
 * written from the accumulator in the epilogue; the results are those of the two separate calls. */
D8K_API int d8k_matmul_forward_relu(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc, void* z, void* a);
/* MatrixMultiplyGradXGPU followed by ReLuGradGPU (deep8/src/math/ReLu.cu:58-110) in one launch, for x = relu(h):
 * dx (+)= dz * y^T, then dh (+)= (h > 0 ? dx : 0) with the dx just stored.  Valid when this product is dx's only remaining
 * contribution, which holds for a chain x = relu(h), z = x * y.  Same rounding as the separate calls. */
D8K_API int d8k_matmul_grad_x_relu(d8k_ctx* ctx, int dtype, void* dx, int xb, int xr, int xc, const void* y, int yb, int yc, const void* dz,
                           int accumulate_dx, const void* h, void* dh, int accumulate_dh);

/* The sum and the all-gather in one kernel: as d8k_sum_shards (weights == NULL) or d8k_sum_shards_sgd (weights != NULL),
 * and every finished 16 bytes - of the sum, or of the updated weights - are also stored to copies[0..ncopies), the same
 * shard in each peer's buffer (d8k_peer_open addresses), over NVLink from the threads that computed them.  No copy
 * engine call and no second pass over the shard; signal the peers after it (d8k_peer_signal on the same stream). */
D8K_API int d8k_sum_shards_gather(d8k_ctx* ctx, int dtype, void* out, const void* const* srcs, int nsrc, size_t count, void* weights,
                                  float alpha, float beta, void* const* copies, int ncopies);

/* MatrixMultiplyGPU followed by AddGPU with a bias (deep8/src/math/Add.cu; shapes broadcast from the tail,
 * deep8/include/utils/ShapeUtils.h:40-55) in one launch: z = x * y + bias, bias one row of yc elements added to every
 * row of every batch entry, from the accumulator in the epilogue.  Rounded as the two calls would: the product to dtype,
 * then the sum. */
D8K_API int d8k_matmul_forward_bias(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc,
                                    const void* bias, void* z);
/* AddGPU for that bias alone: z[r][c] = x[r][c] + bias[c], r < rows (batch * rows of the operand); z may be x. */
D8K_API int d8k_add_bias(d8k_ctx* ctx, int dtype, const void* x, const void* bias, void* z, size_t rows, int cols);
/* AddGradYGPU for that bias (deep8/src/math/Add.cu, the broadcast dimensions are summed): dbias[c] += sum over r < rows of
 * dz[r][c], added in a fixed order (same bits every run) with fp32 accumulation; uses the context's scratch memory. */
D8K_API int d8k_add_bias_grad(d8k_ctx* ctx, int dtype, void* dbias, const void* dz, size_t rows, int cols);

/* Conv2d shape helpers: output extent (deep8/src/nodes/Conv2d.cpp:47-63) and DeConv2d's (deep8/src/nodes/DeConv2d.cpp:36-52). */
D8K_API int d8k_conv2d_out_dim(int in, int filter, int stride, int dilation, int covered);
D8K_API int d8k_deconv2d_out_dim(int in, int filter, int stride, int covered);

/* Conv2dInterimSize / GradXInterimSize / GradYInterimSize and the DeConv2d ones (deep8/src/math/Conv2d.cpp:6-44, 98-137,
 * 195-234; DeConv2d.cpp:6-41, 84-120, 164-200).  The reference returns the byte size of its im2col column buffer; these
 * kernels build the tiles in shared memory, so the answer is 0 unless the contraction would run split-K and the caller
 * wants to supply the scratch itself (`interim`).  The size is computed for the undivided contraction (stride and dilation
 * are not arguments of the reference's functions either); a strided call runs one contraction per residue class and may
 * want less or more.  The operator entry points therefore treat `interim` as an offer: it is used when it holds what the
 * launch wants, and the context's own scratch serves when interim is NULL, empty or smaller than that.
 * which: 0 forward, 1 gradient of x, 2 gradient of the filter. */
D8K_API size_t d8k_conv2d_interim_size(const d8k_ctx* ctx, int which, int dtype, int batch, int ih, int iw, int ic, int oc, int fh, int fw,
                               int oh, int ow);
D8K_API size_t d8k_deconv2d_interim_size(const d8k_ctx* ctx, int which, int dtype, int batch, int ih, int iw, int ic, int oc, int fh, int fw,
                                 int oh, int ow);

/* Conv2dGPU (deep8/src/math/Conv2d.cu:308-411).  x [batch, ih, iw, ic], y [oc, fh, fw, ic], z [batch, oh, ow, oc].
 * Padding follows the reference: the first input row read is -(max(0, (oh-1)*strideY + realFh - ih) / 2). */
D8K_API int d8k_conv2d_forward(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                       void* z, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim, size_t interim_bytes);
/* Conv2dGradXGPU (Conv2d.cu:607-721): dx += col2im(dz * y). */
D8K_API int d8k_conv2d_grad_x(d8k_ctx* ctx, int dtype, void* dx, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                      const void* dz, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim,
                      size_t interim_bytes);
/* Conv2dGradYGPU (Conv2d.cu:917-1031): dy += dz^T * im2col(x). */
D8K_API int d8k_conv2d_grad_y(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, void* dy, int oc, int fh, int fw,
                      const void* dz, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim,
                      size_t interim_bytes);

/* The four convolution gradients with the accumulation made explicit, like d8k_matmul_grad_{x,y}_into: accumulate != 0 is the
 * reference's += (Conv2d.cu:799, DeConv2d.cu:426, 697); accumulate == 0 overwrites - the first contribution to a gradient
 * needs no zero fill (Variable::zeroGradient, deep8/src/model/EagerExecutor.cpp:51-65).  Elements no filter tap reaches
 * (stride beyond the filter) are written as zeros. */
D8K_API int d8k_conv2d_grad_x_into(d8k_ctx* ctx, int dtype, void* dx, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                                   const void* dz, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim,
                                   size_t interim_bytes, int accumulate);
D8K_API int d8k_conv2d_grad_y_into(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, void* dy, int oc, int fh, int fw,
                                   const void* dz, int oh, int ow, int strideY, int strideX, int dilationY, int dilationX, void* interim,
                                   size_t interim_bytes, int accumulate);
D8K_API int d8k_deconv2d_grad_x_into(d8k_ctx* ctx, int dtype, void* dx, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                                     const void* dz, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes,
                                     int accumulate);
D8K_API int d8k_deconv2d_grad_y_into(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, void* dy, int oc, int fh, int fw,
                                     const void* dz, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes,
                                     int accumulate);

/* DeConv2dGPU (deep8/src/math/DeConv2d.cu:251-308).  x [batch, ih, iw, ic], y [oc, fh, fw, ic], z [batch, oh, ow, oc]. */
D8K_API int d8k_deconv2d_forward(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                         void* z, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes);
/* DeConv2dGradXGPU (DeConv2d.cu:557-622). */
D8K_API int d8k_deconv2d_grad_x(d8k_ctx* ctx, int dtype, void* dx, int batch, int ih, int iw, int ic, const void* y, int oc, int fh, int fw,
                        const void* dz, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes);
/* DeConv2dGradYGPU (DeConv2d.cu:826-891). */
D8K_API int d8k_deconv2d_grad_y(d8k_ctx* ctx, int dtype, const void* x, int batch, int ih, int iw, int ic, void* dy, int oc, int fh, int fw,
                        const void* dz, int oh, int ow, int strideY, int strideX, void* interim, size_t interim_bytes);

/* ReLuGPU / ReLuGradGPU (deep8/src/math/ReLu.cu:17-110): y = max(x, 0);  dx += (x > 0 ? dy : 0). */
D8K_API int d8k_relu_forward(d8k_ctx* ctx, int dtype, const void* x, void* y, size_t n);
D8K_API int d8k_relu_backward(d8k_ctx* ctx, int dtype, const void* x, void* dx, const void* dy, size_t n);
/* Math::Constant with scalar 0 as used by Variable::zeroGradient (deep8/src/nodes/Variable.cpp:119-123). */
D8K_API int d8k_zero(d8k_ctx* ctx, void* ptr, size_t bytes);

/* ---- Exchange of replicated-operand gradients between the GPUs of one box (one process per GPU).
 * No counterpart in the reference, whose Executor pins device 0 (deep8/src/model/Executor.cu:6-8).  The gradient of an
 * operand every sample shares (a batch-1 MatrixMultiply operand, a Conv2d/DeConv2d filter) is a sum over the batch; with
 * the batch sharded over GPUs each GPU holds a partial sum and the full gradient is their sum.  These entry points are
 * the pieces of a reduce-scatter + all-gather that uses no SM for the transfers: buffers that peers map (CUDA IPC), copy
 * engine transfers, a fixed-order sum kernel, and stream-ordered flags between processes.  Everything is enqueued on the
 * context's stream; a context per stream lets the exchange run beside the contractions. */
#define D8K_IPC_HANDLE_BYTES 64
/* Device memory other processes of this box can map: zero-filled; `handle` receives the bytes to send to the peers. */
D8K_API int d8k_peer_alloc(d8k_ctx* ctx, size_t bytes, void** ptr, unsigned char handle[D8K_IPC_HANDLE_BYTES]);
D8K_API int d8k_peer_free(d8k_ctx* ctx, void* ptr);
/* Maps a peer's d8k_peer_alloc memory into this process; *ptr is valid on the context's device until d8k_peer_close. */
D8K_API int d8k_peer_open(d8k_ctx* ctx, const unsigned char handle[D8K_IPC_HANDLE_BYTES], void** ptr);
D8K_API int d8k_peer_close(d8k_ctx* ctx, void* ptr);
/* After all work enqueued so far: *flags[i] = value for i < n (n <= 16), visible to every GPU; flags are 4-byte words in
 * d8k_peer_alloc memory of this or a peer process. */
D8K_API int d8k_peer_signal(d8k_ctx* ctx, void* const* flags, int n, unsigned value);
/* Holds the stream until flags[i] >= value for every i < n (n <= 16; words in this GPU's own memory that peers signal),
 * for at most timeout_ms; after that the status word is set ((5 << 8) | index of the first flag still behind, see
 * d8k_ctx_status) and the stream continues, so a peer that never arrives costs a bounded delay, not a hung GPU. */
D8K_API int d8k_peer_wait(d8k_ctx* ctx, const void* const* flags, int n, unsigned value, double timeout_ms);
/* Stream-ordered copy between any two device pointers this process can address (own or peer memory): the copy engines
 * move the bytes. */
D8K_API int d8k_peer_copy(d8k_ctx* ctx, void* dst, const void* src, size_t bytes);
/* MatrixMultiplyGradYGPU for a replicated y (yb == 1; MatrixMultiply.cu:508-551 with the batch folded into the
 * contraction) whose result leaves the kernel already scattered for the sum over GPUs: dy = x^T * dz is not stored as
 * one matrix; rows [k * block_rows, (k + 1) * block_rows) of it are written (overwritten, not accumulated) to
 * row_blocks[k], a block_rows x yc matrix that may live in a peer's d8k_peer_alloc memory - the epilogue stores straight
 * over NVLink, so the reduce-scatter's transfer happens tile by tile while the contraction runs.  block_rows is a
 * multiple of 128; num_blocks <= 16 blocks cover the xc rows.  The stores are complete, for every GPU, when the kernel
 * is: signal the peers after it (d8k_peer_signal on the same stream). */
D8K_API int d8k_matmul_grad_y_scatter(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, int yc, const void* dz,
                                      void* const* row_blocks, int num_blocks, int block_rows);
/* out[i] = srcs[0][i] + srcs[1][i] + ... + srcs[nsrc-1][i], i < count, added in that order in fp32 and rounded once to
 * dtype: every GPU that sums the same partials in the same order gets the same bits.  nsrc <= 16; out may be srcs[k]. */
D8K_API int d8k_sum_shards(d8k_ctx* ctx, int dtype, void* out, const void* const* srcs, int nsrc, size_t count);
/* Math::AXPBY as the trainers use it (deep8/src/math/AXPBY.cu:9-37, SGDTrainer::update deep8/src/trainer/SGDTrainer.cpp:9-17):
 * y = x * alpha + y * beta over n elements, with alpha = -learningRate and beta = 1 - learningRate * weightDecay for SGD.
 * Products and sum are rounded separately in fp32 (the reference's CPU arithmetic, bit for bit, for D8K_F32); fp16
 * operands are widened, and the result rounded once. */
D8K_API int d8k_axpby(d8k_ctx* ctx, int dtype, const void* x, float alpha, void* y, float beta, size_t n);
/* d8k_sum_shards and the SGD step in one pass over the shard a GPU owns: g = srcs[0] + ... + srcs[nsrc-1] (stored to
 * grad_out unless it is NULL), then weights = g * alpha + weights * beta on the same elements, g taken as stored (rounded
 * to dtype) so that the weights equal those of d8k_sum_shards followed by d8k_axpby.  The gradient is read once and the
 * updated weights, not the gradient, are what the all-gather then has to carry. */
D8K_API int d8k_sum_shards_sgd(d8k_ctx* ctx, int dtype, void* grad_out, const void* const* srcs, int nsrc, size_t count, void* weights,
                               float alpha, float beta);

/* LinearGPU (deep8/src/math/Linear.cu:25-58): y = x * a + b over n elements; y may be x.  fp32: the product and the sum
 * are rounded separately, which is the reference's CPU arithmetic bit for bit (deep8/src/math/Linear.cpp:46-54); fp16: in
 * half arithmetic with a and b converted to half, as the reference's half kernel does (Linear.cu:46-52). */
D8K_API int d8k_linear_forward(d8k_ctx* ctx, int dtype, const void* x, float a, float b, void* y, size_t n);
/* LinearGradGPU (Linear.cu:74-110): dx += dy * a. */
D8K_API int d8k_linear_grad(d8k_ctx* ctx, int dtype, void* dx, float a, const void* dy, size_t n);
/* MatrixMultiplyGPU followed by LinearGPU in one launch: z = x * y and l = z * a + b, both written from the accumulator in
 * the epilogue; the results are those of the two separate calls (l is computed from z as stored). */
D8K_API int d8k_matmul_forward_linear(d8k_ctx* ctx, int dtype, const void* x, int xb, int xr, int xc, const void* y, int yb, int yc, void* z,
                                      float a, float b, void* l);

/* AdamUpdateGPU (deep8/src/math/AdamUpdate.cu:9-58, called by AdamTrainer::update, deep8/src/trainer/AdamTrainer.cpp:9-31):
 *   gradient += value * weight_decay;  m = m * beta1 + gradient * (1 - beta1);  v = v * beta2 + gradient^2 * (1 - beta2);
 *   value -= m / (sqrt(v) + epsilon) * ratio,  ratio = d8k_adam_ratio(learning_rate, beta1, beta2, steps).
 * All four arrays are updated in place.  fp32: every operation rounded separately, IEEE sqrt and division - the
 * reference's CPU statements (deep8/src/math/AdamUpdate.cpp:24-41) with an exact square root; fp16 arrays are widened,
 * updated in fp32 and rounded once each. */
D8K_API int d8k_adam_update(d8k_ctx* ctx, int dtype, void* value, void* gradient, void* m, void* v, float beta1, float beta2, float epsilon,
                            float learning_rate, float weight_decay, long long steps, size_t n);
/* learning_rate * sqrt(1 - beta2^steps) / (1 - beta1^steps) in float, steps <= 0 taken as 1 (AdamUpdate.cpp:11-14, 38). */
D8K_API float d8k_adam_ratio(float learning_rate, float beta1, float beta2, long long steps);
/* d8k_sum_shards and Adam in one pass over the shard a GPU owns (the counterpart of d8k_sum_shards_sgd): g = srcs[0] + ...
 * + srcs[nsrc-1] rounded to dtype, then d8k_adam_update's statements on (weights, g, m, v) for the same elements; g after
 * the decay term is stored to grad_out unless it is NULL, and the updated weights are also stored to copies[0..ncopies) -
 * the same shard in each peer's buffer.  m and v cover the owned shard only: each GPU keeps 1 / N of the optimiser's state. */
D8K_API int d8k_sum_shards_adam(d8k_ctx* ctx, int dtype, void* grad_out, const void* const* srcs, int nsrc, size_t count, void* weights, void* m,
                                void* v, float beta1, float beta2, float epsilon, float learning_rate, float weight_decay, long long steps,
                                void* const* copies, int ncopies);

#ifdef __cplusplus
}
#endif
#endif /* D8K_H */
