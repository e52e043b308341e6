// Host-side description of one contraction and the context that launches it.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstddef>
#include <string>
#include <vector>

#include "gemm_kernel.cuh"

namespace d8k {

struct Ctx {
    int device = 0;
    int num_sms = 148;
    cudaStream_t stream = nullptr;
    float* scratch = nullptr;  // split-K partial tiles
    size_t scratch_bytes = 0;
    int* counters = nullptr;   // kMaxCounters tile ticket words (GemmParams::counters)
    unsigned epoch_counter = 0;  // this context's split launches so far, modulo 2^24 (GemmParams::epoch)
    int* status = nullptr;     // device status word
    GroupEntry* group_buf = nullptr;  // device memory for kMaxGroups entries of a grouped launch (null: launches are never grouped)
};
constexpr int kMaxCounters = 4096;
constexpr int kMaxGroups = 16;

// One operand as the host sees it.  mn == false: K-major (the contraction index is contiguous); mn == true: MN-major.
struct HostOperand {
    const void* ptr = nullptr;
    bool mn = false;
    bool is_virtual = false;   // virtual im2col matrix (cr) over the image at ptr
    long long ld = 0;          // pitch in elements of the stored matrix
    int rmod = 0;              // > 0: stored row g lives at (g % rmod) * ld + (g / rmod) * ld2
    long long ld2 = 0;
    long long batch_stride = 0;
    int batch_count = 1;
    ConvRule cr = {};
    // halo != 0 (set by run_gemm, fp32 only): the virtual matrix is fetched as per-tile patches of halo_rows x halo_wp pixels
    int halo = 0, halo_wp = 0, halo_rows = 0;
    // A filter [oc, FH, FW, ic] restricted to the taps (f0y + ty*j, f0x + tx*i), j < nfy, i < nfx - one residue class of a
    // strided convolution.  With rmod == 0 the operand is K-major rows of filters, columns (j, i, c); with rmod > 0 it is
    // the filter read by tap, W'[((j, i), co)][ci].  TMA only.
    struct TapSubset {
        int on = 0, f0y = 0, f0x = 0, ty = 1, tx = 1, nfy = 0, nfx = 0, FH = 0, FW = 0, ic = 0, oc = 0;
    } sub;
};

struct GemmProblem {
    int dtype = 0;
    int M = 0, N = 0, K = 0;
    HostOperand a, b;
    void* C = nullptr;
    long long ldc = 0, c_batch_stride = 0;
    int batch = 1;    // independent outputs
    int kbatch = 1;   // batches summed into one output
    int beta = 0;
    int epi = 0, beta2 = 0;  // fused element-wise tail (GemmParams::epi)
    float epi_a = 0.f, epi_b = 0.f;
    void* E1 = nullptr;
    void* E2 = nullptr;
    int force_splits = 0;    // > 0: this many splits (bounded by the k-block count and the scratch) instead of the plan's own choice
    int ticket_base = 0;     // first of the context's tickets this launch uses (grouped launches give every contraction its own range)
    bool ws_strict = false;  // split within ws / ws_bytes, never in the context's own scratch (run_gemm_group carves that up itself)
    void* ws = nullptr;  // optional caller scratch for split-K
    size_t ws_bytes = 0;
    // scatter_rows > 0: C is not used; output rows [k * scatter_rows, (k + 1) * scatter_rows) go to scatter_base[k], a
    // matrix of scatter_rows rows with pitch ldc (GemmParams::scatter_rows)
    int scatter_rows = 0, scatter_count = 0;
    void* scatter_base[kMaxScatter] = {};
    OutMap out = {};  // strided placement of rows / columns in the output tensor (GemmParams::out); FastDivs filled by run_gemm
};

// error reporting shared by the API layer
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
void count_launch();
void set_last_kernel(const std::string& text);

typedef cudaError_t (*GemmLaunchFn)(int grid, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p);

// Everything run_gemm works out for one contraction short of launching it
struct PreparedGemm {
    GemmParams p;
    CUtensorMap ta, tb;
    GemmLaunchFn fn = nullptr;
    int grid = 0, tiles = 0, splits = 1, total_kb = 0;
    bool pair = false, dual = false, halo = false, twin = false, f32 = false, a_mn = false, b_mn = false;
    int bn = 0;
    std::string text;  // what d8k_last_kernel reports
};

// capture != nullptr: prepare only (no clearing of tickets, no launch) and hand the result back
int run_gemm(Ctx* ctx, const GemmProblem& g, PreparedGemm* capture = nullptr);
// The contractions of one operator (the residue classes of a strided convolution): ONE launch whose work items are all of
// theirs when the context has a group buffer and every part runs the same one-CTA-per-SM kernel, otherwise one launch each.
int run_gemm_group(Ctx* ctx, std::vector<GemmProblem>& parts);
// scratch bytes run_gemm would use for this problem with its default split choice (0 when it runs unsplit)
size_t gemm_scratch_need(const Ctx* ctx, const GemmProblem& g);
// true when run_gemm would fetch both operands with the TMA producer (no loader warps)
bool gemm_goes_through_tma(const Ctx* ctx, const GemmProblem& g);

// one table per translation unit of instantiations; index [a_mn][b_mn][bn slot]
GemmLaunchFn lookup_f16_tma(bool a_mn, bool b_mn, int bn);
GemmLaunchFn lookup_f16_twin(bool a_mn, bool b_mn, int bn);  // lookup_f16_tma's tiles with twin issuing threads
GemmLaunchFn lookup_f16_grouped(bool a_mn, bool b_mn, int bn);  // the same for grouped launches
GemmLaunchFn lookup_f16_gather(bool a_mn, bool b_mn, int bn);
GemmLaunchFn lookup_f32_gather(bool a_mn, bool b_mn, int bn);
GemmLaunchFn lookup_f32_tma(bool a_mn, bool b_mn, int bn, bool a_in_tmem);
GemmLaunchFn lookup_f32_dual(bool a_mn, bool b_mn, int mode);  // two CTAs per SM (GemmCfg::DUAL, mode 1 or 2); launch 2 x SMs CTAs
GemmLaunchFn lookup_f32_halo(bool b_mn);  // K-major virtual A through patches, 64 columns
// paired-CTA kernel: the first argument of the launch function is the number of CTA pairs
GemmLaunchFn lookup_f16_pair(bool a_mn, bool b_mn);

template <class Cfg>
cudaError_t launch_cfg(int grid, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(d8k_gemm_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    d8k_gemm_kernel<Cfg><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, p);
    return cudaGetLastError();
}

}  // namespace d8k
