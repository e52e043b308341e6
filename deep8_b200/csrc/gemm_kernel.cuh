// One warp-specialised, persistent tcgen05 GEMM kernel for every contraction of the path:
//
//     D[b][M x N] (+)= sum_k A[b](m, k) * B[b](n, k)
//
// Operands are staged in shared memory as 128-byte rows under the 128-byte swizzle and multiplied by
// tcgen05.mma (cta_group::1, UMMA 128 x BN x {16 | 8}) into fp32 accumulators in tensor memory; two accumulator
// buffers let the epilogue of one tile overlap the main loop of the next.  Three ways of filling a stage:
//
//   TMA            (fp16)  one thread issues cp.async.bulk.tensor loads: tiled boxes of stored matrices, im2col boxes of
//                          NHWC images (a *virtual im2col matrix* whose rows are pixels and whose columns are (filter tap,
//                          channel): the column buffer of the reference's Conv2d/DeConv2d, deep8/src/math/Conv2d.cu:10-61,
//                          DeConv2d.cu:311-351, is never written to memory), boxes over a filter's taps.
//   TMA + CONVERT  (fp32)  the same loads deliver raw fp32 tiles, which the tensor core reads as the tf32 "hi" image (it
//                          drops the low 13 mantissa bits); converter warps write the "lo" image beside them - and, with
//                          ATMEM, A's hi and lo images into tensor memory (3xTF32: D += A_hi [B_hi ; B_lo] + A_lo B_hi).
//                          HALO additionally fetches a stride-1 image operand as per-tile patches (GemmCfg::HALO).
//   GATHER         (both)  helper warps read global memory with plain 16-byte loads and write the swizzled rows
//                          themselves, for whatever TMA cannot describe (unaligned pitches, odd channel counts, rules
//                          with a divisor); fp32 is split into tf32 hi and lo on the way.
//
// Split-K: when the output has few tiles and K is long, `splits` CTAs share one tile.  Each writes its fp32 partial
// tile to scratch memory, takes a ticket (a compare-and-swap on the tile's epoch-stamped word), and the CTA that draws
// the last ticket sums the partials in split order (so the result does not depend on arrival order), applies beta and
// stores.  Nobody waits on another CTA.
//
// Two forms beyond one CTA per SM with one thread per role (GemmCfg's last parameter): DUAL - two CTAs per SM, each with
// half the stages, one accumulator buffer and one converter group, for fp32 launches with more tiles than SMs and no
// split; TWIN - one CTA per SM with two TMA-issuing threads (A's boxes, B's boxes) and two MMA-issuing threads that take
// k-blocks in turn under a token, for every other TMA launch.  Both keep the order in which the sums are formed.
//
// Every mbarrier wait is bounded: on expiry the CTA records a status code, all roles leave their loops, and the
// kernel returns through the normal teardown (TMEM freed).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <type_traits>

#include "ptx_sm100.cuh"

namespace d8k {

constexpr int kBM = 128;                          // UMMA M
constexpr long long kWaitLimitCycles = 4000000000LL;  // ~2 s at the maximum SM clock

// status word values written by a kernel that gave up on a wait: (role << 8) | which barrier
enum : int { kStatusOk = 0, kRoleProducer = 1, kRoleMma = 2, kRoleEpilogue = 3, kRoleLoader = 4 };

// Exact n / d for 0 <= n < 2^32 without a divide instruction: the high 64 bits of n * ceil(2^64 / d).  With
// M = (2^64 + e) / d, 0 <= e < d, n * M / 2^64 = n / d + n e / (d 2^64) and n e < 2^64, so the floor is n / d.
// The loader warps decode pixel and tap indices for every 16-byte chunk; real divisions made them the bottleneck.
struct FastDiv {
    unsigned long long magic;  // 0 stands for d == 1
    int d;
};
inline FastDiv make_fastdiv(int d) {
    FastDiv f;
    f.d = d;
    f.magic = d <= 1 ? 0ull : (~0ull / static_cast<unsigned long long>(d)) + 1ull;
    return f;
}
__device__ __forceinline__ int fdiv(int n, const FastDiv& f) {
    return f.magic ? static_cast<int>(__umul64hi(static_cast<unsigned long long>(static_cast<unsigned>(n)), f.magic)) : n;
}

// Pixel/tap rule of a virtual im2col matrix.  Row g = (n, py, px) over an RH x RW grid; column = tap * C + c with
// tap = fy * FW + fx.  The source pixel is ((py*mul_y + fy*e_y + off_y) / div_y, likewise x) in an SH x SW image with
// C channels; the element is zero unless the numerators are >= 0, divisible, and the quotients are inside the image.
struct ConvRule {
    int RH, RW, SH, SW, C, FW, FH;
    int mul_y, mul_x, e_y, e_x, off_y, off_x, div_y, div_x;
    FastDiv f_plane, f_rw, f_c, f_fw, f_divy, f_divx;  // RH*RW, RW, C, FW, div_y, div_x
    int unit_div;                                      // div_y == div_x == 1: no divisibility test
    int low_y, low_x;  // unit_div: source pixel = anchor + tap offset with anchor = (py*mul_y + low_y, ...), tap offset >= 0
};
// tap offset along one axis for filter index f of F: the rule's e may be negative (taps walk backwards)
__host__ __device__ __forceinline__ int tap_offset(int f, int F, int e) { return e >= 0 ? f * e : (F - 1 - f) * (-e); }
inline void finish_rule(ConvRule& r) {
    r.f_plane = make_fastdiv(r.RH * r.RW);
    r.f_rw = make_fastdiv(r.RW);
    r.f_c = make_fastdiv(r.C);
    r.f_fw = make_fastdiv(r.FW);
    r.f_divy = make_fastdiv(r.div_y);
    r.f_divx = make_fastdiv(r.div_x);
    r.unit_div = (r.div_y == 1 && r.div_x == 1) ? 1 : 0;
    r.low_y = r.off_y + (r.e_y < 0 ? (r.FH - 1) * r.e_y : 0);
    r.low_x = r.off_x + (r.e_x < 0 ? (r.FW - 1) * r.e_x : 0);
}

// Where the loader warps find one operand.  Logical view: `rows` x `cols` elements, 128-byte windows of a row are
// fetched at a time.  kind 0: matrix, row g at base + g * ld, or with rmod > 0 at base + (g % rmod) * ld + (g / rmod) * ld2
// (+ batch).  kind 1: virtual im2col matrix described by `cr` over the NHWC image at base.
struct GatherSrc {
    const void* base;
    int kind;
    int rows, cols;
    int rmod;
    FastDiv f_rmod;
    long long ld, ld2;
    long long batch_stride;
    int batch_count;
    int vec_ok;  // base, pitches, batch stride (and channel count) keep every chunk 16-byte aligned and inside one tap
    ConvRule cr;
};

constexpr int kMaxScatter = 16;
// producer modes per operand (GemmParams::a_tma, b_tma)
enum : int {
    kTmaTiled = 0,      // K-major rows or MN-major chunks of a stored matrix (3-D map, or 4-D when *_chunked)
    kTmaIm2col = 1,     // virtual im2col matrix, K-major: one im2col box of 128 (or BN) pixels x one 128-byte channel slice of one tap
    kTmaIm2colMN = 2,   // virtual im2col matrix, MN-major: per 128-byte chunk one im2col box of BK pixels
    kTmaFilterTap = 3,  // filter [oc, taps, ic] as W'[(tap, co)][ci], MN-major: 4-D map {ce ci, oc, taps, ic / ce}
    kTmaFilterSub = 4,     // filter [oc, FH, FW, ic] restricted to a grid of taps, K-major: 4-D map {ic, taps x, taps y, oc}
    kTmaFilterTapSub = 5,  // the same subset read as W'[(tap, co)][ci], MN-major: 5-D map {ce ci, oc, taps x, taps y, ic / ce}
    kTmaHalo = 6,          // virtual im2col matrix of a stride-1 rule through per-tile patches (GemmCfg::HALO): 4-D tiled map {c, x, y, image}
};

// Where the result goes when it is a strided part of a larger tensor (one residue class of a strided convolution).
struct OutMap {
    int rows_on;  // row m = pixel (n, py, px) of an RH x RW sub-grid; it is stored at pixel (n, ry + sy*py, rx + sx*px) of an OH x OW image
    int RH, RW, OH, OW, sy, sx, ry, rx;
    int valid_w;  // > 0: only px < valid_w exist; the other columns of the RW-wide raster are padding whose rows are not stored
    FastDiv f_plane, f_rw;  // RH * RW, RW
    int cols_on;  // column = (j, i, c) over a sub-grid of taps; it is stored at ((f0y + ty*j) * FW + f0x + tx*i) * C + c
    int C, NFX, FW, f0y, f0x, ty, tx;
    FastDiv f_c, f_nfx;     // C, NFX
};

struct GroupEntry;

struct GemmParams {
    // Grouped launch (group_count > 1): the work items of several contractions of one operator - the residue classes of a strided
    // convolution - share ONE launch.  `groups` is an array in device memory with each contraction's own parameters and
    // tensor maps; work item w belongs to the group g with groups[g].first_work <= w < groups[g + 1].first_work and is item
    // w - first_work of that contraction.  The launch's own copy of the fields below is group 0's, with total_work the sum.
    int group_count;
    const GroupEntry* groups;
    int M, N, K;
    int batch;         // output batches (independent problems)
    int kbatch;        // batches folded into the contraction (sum over b of A[b] * B[b]); 1 otherwise
    int num_kb;        // k-blocks per batch = ceil(K / BK)
    int splits, kb_per_split;
    int tiles_m, tiles_n, raster_group;
    // Paired kernel only.  raster_n == 0: tiles are visited in groups of raster_group rows of tiles, each group sweeping all
    // columns (the group's A strips are what successive waves share); raster_n == 1: groups of raster_group columns sweeping
    // all rows (B strips shared).  l2_a / l2_b: L2 eviction priority of each operand's loads - 0 normal, 1 evict first
    // (a strip that streams through once per group), 2 evict last (the strips successive waves come back to).
    int raster_n, l2_a, l2_b;
    int epi_backoff_ns;  // paired kernel: sleep between the epilogue warps' polls for a finished accumulator (0 = poll back to back)
    // Halo kernels (GemmCfg::HALO): the A operand is a virtual im2col matrix of a stride-1 rule, and the rows of a tile are 128
    // consecutive pixels of one image's PADDED raster (halo_wp = RW + tap span columns per row).  One TMA box per (tile, 32-channel
    // slice) brings the tile's source pixels - its rows plus the taps' reach, halo_wp columns wide - into shared memory once; tap
    // (fy, fx) of the tile is then the same patch shifted by ty * halo_wp + tx rows.  k-blocks run slice-major: kk = slice * taps + tap.
    int halo_wp, halo_taps, halo_slices, halo_bytes;
    int total_work;    // batch * tiles_m * tiles_n * splits
    int beta;          // 0: overwrite, 1: accumulate into C
    int epi, beta2;    // fused element-wise tail, see store_row_chunk: 1 ReLU, 2 ReLU gradient, 3 bias row added (E1 = bias[N]), 4 Linear
    float epi_a, epi_b;  // epi 4: E1 = C * epi_a + epi_b
    void* E1;          // epi 1: relu(C) is written here; epi 2: ReLu's input is read here
    void* E2;          // epi 2: ReLu's input gradient, overwritten (beta2 == 0) or accumulated (beta2 == 1)
    void* C;
    long long ldc, c_batch_stride;
    float* ws;         // split-K partial tiles: total_work * 128 * BN floats
    int* counters;     // one ticket word per output tile: (epoch << 8 | tickets drawn by this launch's CTAs)
    int epoch;         // 24-bit number of this split launch on its context; ticket words of any other epoch count as zero
    int* status;
    int a_batch_mod, b_batch_mod;  // TMA: batch coordinate = b % mod
    int a_chunked, b_chunked;      // single-CTA TMA kernel: the MN-major operand comes through a 4-D {64, k, chunk, batch} map, one box per stage
    int a_tma, b_tma;              // single-CTA TMA kernels: how the producer fetches the operand (kTma*); a.cr / b.cr describe images
    long long* prof;   // optional, normally null: per CTA 8 counters of cycles each role spent waiting (paired kernel only)
    // Row-block scatter of the output (scatter_rows > 0): rows [k * scatter_rows, (k + 1) * scatter_rows) are stored at
    // C + scatter_off[k] (elements) instead of at C - each block may live in another allocation, on this GPU or a peer
    // mapped into this process.  scatter_rows is a multiple of 128, so no epilogue warp straddles two blocks.
    int scatter_rows;
    long long scatter_off[kMaxScatter];
    OutMap out;
    GatherSrc a, b;
};

struct alignas(128) GroupEntry {
    CUtensorMap ta, tb;
    GemmParams p;
    int first_work;
};

// Parameters, tensor maps and local index of work item w (see GemmParams::group_count)
struct SelectedWork {
    const GemmParams* p;
    const CUtensorMap* ta;
    const CUtensorMap* tb;
    int w;
};
__device__ __forceinline__ SelectedWork select_work(const GemmParams& launch, const CUtensorMap& ta, const CUtensorMap& tb, int w) {
    SelectedWork s = {&launch, &ta, &tb, w};
    if (launch.group_count > 1) {
        int g = 0;
        while (g + 1 < launch.group_count && w >= launch.groups[g + 1].first_work) ++g;
        const GroupEntry& e = launch.groups[g];
        s.p = &e.p;
        s.ta = &e.ta;
        s.tb = &e.tb;
        s.w = w - e.first_work;
    }
    return s;
}

// false for a row of the padded raster that stands for no output pixel (OutMap::valid_w)
__device__ __forceinline__ bool out_row_exists(const GemmParams& p, int row) {
    if (row >= p.M) return false;
    if (!p.out.rows_on || p.out.valid_w <= 0) return true;
    const OutMap& o = p.out;
    int n = fdiv(row, o.f_plane);
    int rem = row - n * (o.RH * o.RW);
    int py = fdiv(rem, o.f_rw);
    return rem - py * o.RW < o.valid_w;
}
// element offset of output row `row` (without the batch term)
__device__ __forceinline__ long long out_row_offset(const GemmParams& p, int row) {
    if (!p.out.rows_on) return static_cast<long long>(row) * p.ldc;
    const OutMap& o = p.out;
    int n = fdiv(row, o.f_plane);
    int rem = row - n * (o.RH * o.RW);
    int py = fdiv(rem, o.f_rw);
    int px = rem - py * o.RW;
    return ((static_cast<long long>(n) * o.OH + o.ry + o.sy * py) * o.OW + o.rx + o.sx * px) * p.ldc;
}
// stored column of logical column `col` (a multiple of 32; C is a multiple of 32 when the map is on, so 32 columns stay together)
__device__ __forceinline__ int out_col(const GemmParams& p, int col) {
    if (!p.out.cols_on) return col;
    const OutMap& o = p.out;
    int tap = fdiv(col, o.f_c);
    int c = col - tap * o.C;
    int j = fdiv(tap, o.f_nfx);
    int i = tap - j * o.NFX;
    return ((o.f0y + o.ty * j) * o.FW + o.f0x + o.tx * i) * o.C + c;
}

__device__ __forceinline__ long long scatter_offset(const GemmParams& p, int row) {
    if (p.scatter_rows == 0) return 0;
    int k = row / p.scatter_rows;
    return p.scatter_off[k < kMaxScatter ? k : kMaxScatter - 1];
}

template <bool F32_, bool A_MN_, bool B_MN_, int BN_, int STAGES_, bool GATHER_, bool ATMEM_ = false, bool HALO_ = false, int DUAL_ = 0>
struct GemmCfg {
    static constexpr bool F32 = F32_, A_MN = A_MN_, B_MN = B_MN_, GATHER = GATHER_;
    static constexpr int BN = BN_, STAGES = STAGES_;
    static constexpr int ESIZE = F32 ? 4 : 2;
    static constexpr int CE = 128 / ESIZE;       // elements in one 128-byte row
    static constexpr int BK = CE;                // k extent of one stage
    static constexpr int VEC = 16 / ESIZE;       // elements in one 16-byte chunk
    static constexpr int UMMA_K = 32 / ESIZE;
    static constexpr int KSTEPS = BK / UMMA_K;   // 4
    static constexpr int PARTS = F32 ? 2 : 1;    // hi and lo images for 3xTF32
    // MN-major tf32 operands must use the 128-byte swizzle with 32-byte atoms (4-row groups)
    static constexpr bool A_B32 = F32 && A_MN, B_B32 = F32 && B_MN;
    static constexpr int A_BYTES = kBM * 128;
    static constexpr int B_BYTES = BN * 128;
    // ATMEM (fp32 behind TMA only): the converter warps put A's hi and lo images into tensor memory instead of shared
    // memory - one row per lane, BK columns each - and the MMAs take A from there.  The stage keeps raw A and B hi/lo;
    // shared memory then holds six stages instead of four and the three MMA passes read only B from it.
    static constexpr bool ATMEM = ATMEM_;
    // HALO (with ATMEM, K-major A): A does not travel through the stages at all.  PATCH_SLOTS patch buffers of PATCH_BYTES hold
    // the source pixels of a tile's 32-channel slices (GemmParams::halo_*); the converter warps read each tap's rows from
    // the patch and write hi/lo to tensor memory.  A pixel is fetched once per tile and slice instead of once per tap.
    static constexpr bool HALO = HALO_;
    static constexpr int PATCH_SLOTS = HALO ? 3 : 0;
    static constexpr int PATCH_BYTES = 44 * 1024;
    static constexpr int A_PARTS = HALO ? 0 : (ATMEM ? 1 : PARTS);
    static constexpr int STAGE_BYTES = A_PARTS * A_BYTES + PARTS * B_BYTES;
    // STACK (fp32, 64 columns): B's hi and lo images lie one after the other in a stage, so ONE MMA of 2 BN columns multiplies
    // A_hi by both - columns [0, BN) of the accumulator receive A_hi B_hi, columns [BN, 2 BN) receive A_hi B_lo - and a second
    // MMA adds A_lo B_hi into the first half; the epilogue adds the halves.  Two instructions per k-step instead of three, and
    // the wide one runs at the tensor core's full rate (measured: a 128 x 64 x 8 tf32 MMA takes 48 clocks, not 32; a
    // 128 x 128 x 8 one takes its nominal 64).
    static constexpr bool STACK = F32 && BN == 64;
    static constexpr int ACC_COLS = STACK ? 2 * BN : BN;         // accumulator columns per buffer
    // DUAL (fp32 with ATMEM): TWO CTAs share an SM, each with half of everything - one accumulator buffer instead of two, half
    // the stages, one converter group, half of tensor memory.  The k-block period of one CTA is set by the latencies of its
    // single-thread roles (barrier round trips, commits), during which the tensor pipe idles; a second CTA's MMAs fill
    // those gaps, and its main loop runs while the first CTA's epilogue drains the one accumulator buffer.
    // DUAL_ == 2 (ALO): only A's lo image goes to tensor memory; the raw tile in shared memory serves as the hi image, read
    // by the wide MMA through a descriptor.  Half the tensor-memory columns per stage, so each CTA holds three stages.
    static constexpr bool DUAL = DUAL_ == 1 || DUAL_ == 2;
    static constexpr bool ALO = DUAL_ == 2;
    // DUAL_ == 4 (TWIN): one CTA per SM with a second TMA-issuing thread (one issues A's boxes, the other B's) and a second
    // MMA-issuing thread (the two take k-blocks in turn, ordered by a token, so the sums are formed in the same order).  A
    // k-block costs the single MMA thread about as long in barrier traffic and tcgen05.commit as in its eight MMAs, and the
    // single producer as long again; with two threads each, one thread's bookkeeping runs behind the other's issue.
    static constexpr bool TWIN = DUAL_ == 4 || DUAL_ == 5;
    // DUAL_ == 5: TWIN whose work items may belong to several contractions (GemmParams::group_count); a kernel of its own,
    // because per-item parameters read through a pointer cost the ungrouped kernels a fifth of their speed
    static constexpr bool GROUPED = DUAL_ == 5;
    static constexpr int A_TMEM_STRIDE = ALO ? BK : 2 * BK;     // tensor-memory columns of A per stage
    static constexpr int ACC_BUFS = DUAL ? 1 : 2;
    static constexpr int CTAS_PER_SM = DUAL ? 2 : 1;
    static constexpr int A_TMEM_COL0 = ACC_BUFS * ACC_COLS;     // after the accumulator buffers
    static constexpr int A_TMEM_COLS = ATMEM ? A_TMEM_STRIDE * STAGES : 0;  // per stage BK columns of hi (unless ALO), BK of lo
    static constexpr int TMEM_NEED = ACC_BUFS * ACC_COLS + A_TMEM_COLS;
    static_assert(!DUAL || (ATMEM && !HALO_ && STACK && TMEM_NEED <= 256), "two CTAs per SM share 512 columns of tensor memory");
    static constexpr int TMEM_COLS = (TMEM_NEED <= 32) ? 32 : (TMEM_NEED <= 64) ? 64 : (TMEM_NEED <= 128) ? 128 : (TMEM_NEED <= 256) ? 256 : 512;
    static_assert(TMEM_NEED <= 512, "tensor memory");
    static_assert(!ATMEM || (F32 && !GATHER), "A in tensor memory belongs to the fp32 TMA kernels");
    static_assert(!HALO || (ATMEM && !A_MN_), "the halo kernels read a K-major A from patches and keep it in tensor memory");
    // fp32 only: the tensor core adds into its fp32 accumulator with truncation, so a long chain drifts (about
    // 2e-5 of the result after 1300 accumulations).  Every CHUNK_KB k-blocks the accumulator buffer is handed to the
    // epilogue warps, which add it to register accumulators with round-to-nearest, and a fresh chain starts in the
    // other buffer.  0 = one chain per work item (fp16, whose output rounding is far coarser).
    static constexpr int CHUNK_KB = F32 ? 8 : 0;
    static constexpr int EPI_WARPS = 4;
    // GATHER: LOADER_GROUPS groups of four loader warps take the k-blocks in turn, so one group's address arithmetic and
    // conversions overlap the other group's global-load latency (a lone group spent 4-8 us per k-block).
    static constexpr int PRODUCER_WARP = 4, MMA_WARP = 5, LOADER_WARP0 = 6, LOADER_WARPS = 4;
    // fp32 with 128 columns keeps 128 accumulators per epilogue thread in registers: no room for a second group there
    static constexpr int LOADER_GROUPS = ((F32 && BN_ > 64) || DUAL) ? 1 : 2;
    // fp32 without GATHER: TMA brings the operands as stored.  The tensor core reads a raw fp32 word as tf32 by dropping
    // its low 13 mantissa bits, so the copy TMA made IS the hi image; the same warps that would gather only have to
    // write the lo image, tf32(v - trunc(v)), beside it - shared memory to shared memory, no global-load latency.
    static constexpr bool CONVERT = F32 && !GATHER;
    static constexpr bool HELPERS = GATHER || CONVERT;  // warps beyond the MMA warp exist
    static constexpr int BASE_WARPS = HELPERS ? LOADER_WARP0 + LOADER_WARPS * LOADER_GROUPS : 6;
    static constexpr int PRODUCER_B_WARP = BASE_WARPS, MMA2_WARP = BASE_WARPS + 1;  // TWIN only
    static constexpr int THREADS = 32 * (BASE_WARPS + (TWIN ? 2 : 0));
    static_assert(!TWIN || (!GATHER && !HALO_), "the twin roles belong to the TMA kernels");
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + PATCH_SLOTS * PATCH_BYTES + BAR_BYTES + 1024;  // + slack to align the ring to 1024
    static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N");
    static_assert(BN % CE == 0, "an MN-major B tile is whole 128-byte chunks");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
    static_assert(DUAL ? SMEM_BYTES <= 112 * 1024 : SMEM_BYTES > 114 * 1024, "one CTA per SM unless DUAL: more would compete for tensor memory");
};

struct WorkItem {
    int tile, split, batch, m0, n0, kb_begin, kb_end;
};

__device__ __forceinline__ WorkItem decode_work(const GemmParams& p, int w, int BN) {
    WorkItem it;
    it.tile = w / p.splits;
    it.split = w - it.tile * p.splits;
    int tpb = p.tiles_m * p.tiles_n;
    it.batch = it.tile / tpb;
    int t = it.tile - it.batch * tpb;
    int group_size = p.raster_group * p.tiles_n;
    int gid = t / group_size;
    int first_m = gid * p.raster_group;
    int gm = min(p.tiles_m - first_m, p.raster_group);
    int in_group = t - gid * group_size;
    int nt = in_group / gm;
    int mt = first_m + (in_group - nt * gm);
    it.m0 = mt * kBM;
    it.n0 = nt * BN;
    it.kb_begin = it.split * p.kb_per_split;
    it.kb_end = min(p.kbatch * p.num_kb, it.kb_begin + p.kb_per_split);
    return it;
}

// Bounded wait on an mbarrier phase.  `backoff_ns` > 0 sleeps between polls: used by roles that are not on the
// critical path (the epilogue waiting for a finished tile), because a warp that spins on mbarrier.try_wait competes
// with TMA writes and tensor-core operand reads for shared-memory bandwidth.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                         unsigned backoff_ns = 0) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    int spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
        if (backoff_ns) __nanosleep(backoff_ns);
        if ((++spins & 63) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

// wait_bar that also adds the cycles spent waiting to *acc when the diagnostics buffer is on (GemmParams::prof)
__device__ __forceinline__ bool wait_bar_timed(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code, bool timed,
                                               long long* acc, unsigned backoff_ns = 0) {
    if (!timed) return wait_bar(bar, parity, abort_flag, status, code, backoff_ns);
    const long long t0 = clock64();
    const bool ok = wait_bar(bar, parity, abort_flag, status, code, backoff_ns);
    *acc += clock64() - t0;
    return ok;
}

// ------------------------------------------------------------------------------------------------ gather loaders
// Column part of a virtual-matrix address: which tap and channel, and the tap's contribution to the pixel numerators.
struct ColCtx {
    int c, ty, tx;
    bool inside;  // the VEC-wide chunk starting here stays inside one tap and inside the matrix
};
template <int VEC>
__device__ __forceinline__ ColCtx col_ctx(const GatherSrc& s, int col) {
    const ConvRule& r = s.cr;
    ColCtx k;
    int tap = fdiv(col, r.f_c);
    k.c = col - tap * r.C;
    int fy = fdiv(tap, r.f_fw);
    int fx = tap - fy * r.FW;
    k.ty = fy * r.e_y + r.off_y;
    k.tx = fx * r.e_x + r.off_x;
    k.inside = (k.c + VEC <= r.C) && (col + VEC <= s.cols);
    return k;
}

// Element offset of (pixel row g, column context) in the source image; false where the tap falls on padding.
__device__ __forceinline__ bool locate(const ConvRule& r, int g, const ColCtx& k, long long& off) {
    int n = fdiv(g, r.f_plane);
    int rem = g - n * (r.RH * r.RW);
    int py = fdiv(rem, r.f_rw);
    int px = rem - py * r.RW;
    int ny = py * r.mul_y + k.ty, nx = px * r.mul_x + k.tx;
    if ((ny | nx) < 0) return false;
    int sy = fdiv(ny, r.f_divy), sx = fdiv(nx, r.f_divx);
    if (sy * r.div_y != ny || sx * r.div_x != nx || sy >= r.SH || sx >= r.SW) return false;
    off = (static_cast<long long>(n) * (r.SH * r.SW) + sy * r.SW + sx) * r.C + k.c;
    return true;
}

template <typename T, int VEC>
__device__ __forceinline__ uint4 load16(const T* p) {  // 16 bytes at p, by elements when p is not 16-byte aligned
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) return __ldg(reinterpret_cast<const uint4*>(p));
    T tmp[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) tmp[i] = __ldg(p + i);
    return *reinterpret_cast<uint4*>(tmp);
}

// 16 bytes of row g starting at column `col` of an operand, zero outside the logical extent.  `k` is the column context
// of `col` for a virtual matrix (the caller computes it once for all rows that share the column); `boff` the batch offset.
template <typename T, int VEC>
__device__ __forceinline__ uint4 fetch16(const GatherSrc& s, int g, int col, long long boff, const ColCtx& k) {
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (g >= s.rows || col >= s.cols) return out;
    const T* base = reinterpret_cast<const T*>(s.base);
    if (s.kind == 0) {
        const T* p = base + boff + col;
        if (s.rmod > 0) {
            int q = fdiv(g, s.f_rmod);
            p += static_cast<long long>(g - q * s.rmod) * s.ld + static_cast<long long>(q) * s.ld2;
        } else {
            p += static_cast<long long>(g) * s.ld;
        }
        if (col + VEC <= s.cols) return load16<T, VEC>(p);
        T tmp[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) tmp[i] = (col + i < s.cols) ? __ldg(p + i) : T(0);
        return *reinterpret_cast<uint4*>(tmp);
    }
    long long off;
    if (k.inside) {
        if (!locate(s.cr, g, k, off)) return out;
        return load16<T, VEC>(base + off);
    }
    T tmp[VEC];  // the chunk straddles taps (channel count not a multiple of the chunk) or the matrix edge
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        tmp[i] = T(0);
        if (col + i < s.cols) {
            ColCtx ke = col_ctx<1>(s, col + i);
            if (locate(s.cr, g, ke, off)) tmp[i] = __ldg(base + off);
        }
    }
    return *reinterpret_cast<uint4*>(tmp);
}

// ---- the fast path of the loaders.  An address is (row part) + (column part); for a K-major operand a thread keeps its
// rows for a whole tile and moves along the columns k-block by k-block, for an MN-major operand the other way round, so
// the part that does not change is worked out once per tile (RowState / ColState below) and a chunk's address costs a
// few additions.  Decoding pixel and tap for every chunk took about 145 instructions per 16 bytes.
struct RowState {  // kind 0: lo | hi = element offset of the row, ok = the row exists
    int lo, hi, ok;  // kind 1: lo = index of pixel (n, 0, 0), hi = py * mul_y, ok = px * mul_x; a missing row has hi far below zero
};
struct ColState {  // kind 0: c = the column; kind 1: channel and the tap's part of the pixel numerators
    int c, ty, tx;
    int how;       // kChunkZero: outside the matrix; kChunkFast: one aligned 16-byte load; kChunkSlow: element by element
};
enum : int { kChunkZero = 0, kChunkFast = 1, kChunkSlow = 2 };

__device__ __forceinline__ RowState row_state(const GatherSrc& s, int g) {
    RowState r;
    if (s.kind == 0) {
        long long off;
        if (s.rmod > 0) {
            int q = fdiv(g, s.f_rmod);
            off = static_cast<long long>(g - q * s.rmod) * s.ld + static_cast<long long>(q) * s.ld2;
        } else {
            off = static_cast<long long>(g) * s.ld;
        }
        r.lo = static_cast<int>(static_cast<unsigned long long>(off) & 0xffffffffull);
        r.hi = static_cast<int>(off >> 32);
        r.ok = g < s.rows;
    } else {
        const ConvRule& cr = s.cr;
        int n = fdiv(g, cr.f_plane);
        int rem = g - n * (cr.RH * cr.RW);
        int py = fdiv(rem, cr.f_rw);
        int px = rem - py * cr.RW;
        r.lo = n * (cr.SH * cr.SW);
        r.hi = g < s.rows ? py * cr.mul_y : -(1 << 30);
        r.ok = px * cr.mul_x;
    }
    return r;
}

template <int VEC>
__device__ __forceinline__ ColState col_state(const GatherSrc& s, int col) {
    ColState k;
    if (s.kind == 0) {
        k.c = col;
        k.ty = k.tx = 0;
        k.how = col >= s.cols ? kChunkZero : (col + VEC <= s.cols && s.vec_ok) ? kChunkFast : kChunkSlow;
    } else {
        ColCtx x = col_ctx<VEC>(s, col);
        k.c = x.c;
        k.ty = x.ty;
        k.tx = x.tx;
        k.how = col >= s.cols ? kChunkZero : (x.inside && s.vec_ok) ? kChunkFast : kChunkSlow;
    }
    return k;
}

// Address of a kChunkFast chunk, or 0 where the row is missing or the tap falls on padding.  `base` already includes
// the batch offset.
template <typename T>
__device__ __forceinline__ uintptr_t chunk_addr(const GatherSrc& s, const T* base, const RowState& r, const ColState& k) {
    if (s.kind == 0) {
        long long off = (static_cast<long long>(r.hi) << 32 | static_cast<unsigned>(r.lo)) + k.c;
        return r.ok ? reinterpret_cast<uintptr_t>(base + off) : 0;
    }
    const ConvRule& cr = s.cr;
    int ny = r.hi + k.ty, nx = r.ok + k.tx;
    int sy = ny, sx = nx;
    bool ok;
    if (cr.unit_div) {
        ok = static_cast<unsigned>(ny) < static_cast<unsigned>(cr.SH) && static_cast<unsigned>(nx) < static_cast<unsigned>(cr.SW);
    } else {
        ok = (ny | nx) >= 0;
        sy = fdiv(ny, cr.f_divy);
        sx = fdiv(nx, cr.f_divx);
        ok = ok && sy * cr.div_y == ny && sx * cr.div_x == nx && sy < cr.SH && sx < cr.SW;
    }
    long long off = static_cast<long long>(r.lo + sy * cr.SW + sx) * cr.C + k.c;
    return ok ? reinterpret_cast<uintptr_t>(base + off) : 0;
}

// One predicated 16-byte load.  A load inside an if/else made the compiler merge the loaded value at the join, which
// serialised the loads of a k-block: about one global-memory latency per chunk.
__device__ __forceinline__ uint4 ldg_pred(uintptr_t addr) {  // zeros unless addr is a real address
    uint4 v;
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.u64 q, %4, 0;\n\t"
        "mov.b32 %0, 0;\n\t"
        "mov.b32 %1, 0;\n\t"
        "mov.b32 %2, 0;\n\t"
        "mov.b32 %3, 0;\n\t"
        "@q ld.global.nc.v4.b32 {%0, %1, %2, %3}, [%4];\n\t"
        "}"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(addr)
        : "memory");
    return v;
}

// Swizzled position of 16-byte chunk j of row r inside a tile of 128-byte rows (tile base 1024-byte aligned).
// BASE32 == false: address bits [4,7) are XORed with bits [7,10), the pattern TMA and tcgen05 call SWIZZLE_128B.
// BASE32 == true : address bits [5,7) are XORed with bits [7,9) (32-byte atoms), for MN-major tf32 operands.
template <bool BASE32>
__device__ __forceinline__ uint32_t swz(int r, int j) {
    if constexpr (BASE32) return static_cast<uint32_t>(r * 128 + ((((j >> 1) ^ (r & 3)) << 5) | ((j & 1) << 4)));
    else return static_cast<uint32_t>(r * 128 + ((j ^ (r & 7)) << 4));
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// What the tensor core misses when it reads the fp32 word v as tf32 (it drops the low 13 bits): v - trunc(v), exact
// in fp32, rounded to tf32 (nearest, ties away from zero) with integer arithmetic - the conversion instruction runs at
// a quarter of the rate of the logic and add pipes, and this loop is the converter warps' whole job.
__device__ __forceinline__ uint4 tf32_low_part(const uint4& v) {
    uint4 o;
    const uint32_t* in = &v.x;
    uint32_t* out = &o.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float d = __uint_as_float(in[i]) - __uint_as_float(in[i] & 0xffffe000u);
        out[i] = (__float_as_uint(d) + 0x1000u) & 0xffffe000u;
    }
    return o;
}

// Write one fetched chunk: fp16 as is; fp32 as a tf32 hi image and a tf32 lo image `lo_offset` bytes further.
template <bool F32>
__device__ __forceinline__ void store_chunk_smem(uint32_t addr, uint32_t lo_offset, uint4 v) {
    if constexpr (!F32) {
        st_shared_v4(addr, v);
    } else {
        float f[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
        uint4 hi, lo;
        uint32_t* h = &hi.x;
        uint32_t* l = &lo.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float fh = ptx::to_tf32(f[i]);
            h[i] = __float_as_uint(fh);
            l[i] = __float_as_uint(ptx::to_tf32(f[i] - fh));
        }
        st_shared_v4(addr, hi);
        st_shared_v4(addr + lo_offset, lo);
    }
}

// ------------------------------------------------------------------------------------------------ epilogue helpers
__device__ __forceinline__ float epi_to_float(float v) { return v; }
__device__ __forceinline__ float epi_to_float(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T epi_from_float(float v);
template <>
__device__ __forceinline__ float epi_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half epi_from_float<__half>(float v) { return __float2half_rn(v); }

// 16 bytes of OutT <-> floats, two halves per conversion instruction
template <typename OutT>
struct EpiVec;
template <>
struct EpiVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& w, float* f) {
        f[0] = __uint_as_float(w.x); f[1] = __uint_as_float(w.y); f[2] = __uint_as_float(w.z); f[3] = __uint_as_float(w.w);
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};
template <>
struct EpiVec<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& w, float* f) {
        const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        uint4 w;
        __half2* h = reinterpret_cast<__half2*>(&w);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        return w;
    }
};

// Math::Linear on one stored value (widened): fp32 rounds the product and the sum separately (deep8/src/math/Linear.cpp:46-54);
// fp16 works in half arithmetic with a and b converted to half, like the reference's half kernel (deep8/src/math/Linear.cu:46-52).
template <typename OutT>
__device__ __forceinline__ float epi_linear(float c, float a, float b);
template <>
__device__ __forceinline__ float epi_linear<float>(float c, float a, float b) { return __fadd_rn(__fmul_rn(c, a), b); }
template <>
__device__ __forceinline__ float epi_linear<__half>(float c, float a, float b) {
    return __half2float(__hadd(__hmul(__float2half(a), __float2half(c)), __float2half(b)));
}

// Element-wise tail of the epilogue for one row and 32 columns [col0, col0 + 32), clipped to N.  `off` is the element
// offset of C(row, 0); E1 and E2 have C's shape and pitch.  With c = OutT(acc + (beta ? C : 0)):
//   EPI 0: C = c
//   EPI 1: C = c; E1 = c > 0 ? c : 0                     MatrixMultiply followed by ReLu (deep8/src/math/ReLu.cu:11-15)
//   EPI 2: C = c; E2 = (beta2 ? E2 : 0) + (E1 > 0 ? c : 0)   gradient of x followed by ReLu's gradient with E1 = ReLu's
//                                                        input (deep8/src/math/ReLu.cu:58-63); sums are rounded to OutT
//   EPI 3: C = OutT(c + bias[col])                        MatrixMultiply followed by Add with a bias row E1
//   EPI 4: C = c; E1 = c * epi_a + epi_b                  MatrixMultiply followed by Linear (deep8/src/math/Linear.cu:11-58)
template <typename OutT, int EPI>
__device__ __forceinline__ void store_row_chunk_epi(const GemmParams& p, long long off, int col0, const float* acc) {
    using V = EpiVec<OutT>;
    constexpr int VEC = V::N;
    const int colm = out_col(p, col0);
    OutT* dst = reinterpret_cast<OutT*>(p.C) + off + colm;
    // EPI 3: E1 is a bias row of N elements, indexed by the logical column alone
    OutT* e1 = EPI == 3 ? reinterpret_cast<OutT*>(p.E1) + col0 : reinterpret_cast<OutT*>(p.E1) + off + colm;
    OutT* e2 = reinterpret_cast<OutT*>(p.E2) + off + colm;
    bool vec_ok = (col0 + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
    if (EPI >= 1) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(e1) & 15) == 0);
    if (EPI == 2) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(e2) & 15) == 0);
    if (vec_ok) {
#pragma unroll
        for (int v = 0; v < 32 / VEC; ++v) {
            float c[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) c[i] = acc[v * VEC + i];
            if (p.beta) {
                float old[VEC];
                V::unpack(reinterpret_cast<const uint4*>(dst)[v], old);
#pragma unroll
                for (int i = 0; i < VEC; ++i) c[i] += old[i];
            }
            uint4 cw = V::pack(c);
            if (EPI == 3) {  // z = round(round(x * y) + bias): the two roundings of MatrixMultiply followed by Add
                float b[VEC];
                V::unpack(cw, c);
                V::unpack(reinterpret_cast<const uint4*>(e1)[v], b);
#pragma unroll
                for (int i = 0; i < VEC; ++i) c[i] += b[i];
                cw = V::pack(c);
            }
            reinterpret_cast<uint4*>(dst)[v] = cw;
            if (EPI == 1 || EPI == 2 || EPI == 4) V::unpack(cw, c);  // the stored (rounded) values drive the fused tails
            if (EPI == 1) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) c[i] = c[i] > 0.f ? c[i] : 0.f;
                reinterpret_cast<uint4*>(e1)[v] = V::pack(c);
            } else if (EPI == 4) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) c[i] = epi_linear<OutT>(c[i], p.epi_a, p.epi_b);
                reinterpret_cast<uint4*>(e1)[v] = V::pack(c);
            } else if (EPI == 2) {
                float x[VEC], g[VEC];
                V::unpack(reinterpret_cast<const uint4*>(e1)[v], x);
                if (p.beta2) {
                    V::unpack(reinterpret_cast<const uint4*>(e2)[v], g);
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) g[i] = 0.f;
                }
#pragma unroll
                for (int i = 0; i < VEC; ++i)
                    if (x[i] > 0.f) g[i] += c[i];
                reinterpret_cast<uint4*>(e2)[v] = V::pack(g);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {  // fully unrolled: a dynamic index would push the accumulators to local memory
            if (col0 + i < p.N) {
                float v = acc[i];
                if (p.beta) v += epi_to_float(dst[i]);
                OutT c = epi_from_float<OutT>(v);
                if (EPI == 3) c = epi_from_float<OutT>(epi_to_float(c) + epi_to_float(e1[i]));
                dst[i] = c;
                if (EPI == 1) {
                    e1[i] = epi_to_float(c) > 0.f ? c : epi_from_float<OutT>(0.f);
                } else if (EPI == 4) {
                    e1[i] = epi_from_float<OutT>(epi_linear<OutT>(epi_to_float(c), p.epi_a, p.epi_b));
                } else if (EPI == 2) {
                    OutT g = p.beta2 ? e2[i] : epi_from_float<OutT>(0.f);
                    if (epi_to_float(e1[i]) > 0.f) g = epi_from_float<OutT>(epi_to_float(g) + epi_to_float(c));
                    e2[i] = g;
                }
            }
        }
    }
}

template <typename OutT>
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, long long off, int col0, const float* acc) {
    if (p.epi == 0) store_row_chunk_epi<OutT, 0>(p, off, col0, acc);
    else if (p.epi == 1) store_row_chunk_epi<OutT, 1>(p, off, col0, acc);
    else if (p.epi == 2) store_row_chunk_epi<OutT, 2>(p, off, col0, acc);
    else if (p.epi == 3) store_row_chunk_epi<OutT, 3>(p, off, col0, acc);
    else store_row_chunk_epi<OutT, 4>(p, off, col0, acc);
}

// ------------------------------------------------------------------------------------------------ the kernel
// Producer side of one operand for one stage (one elected lane).  ROWS: tile rows of the operand (kBM or BN); mn0: first
// row (M or N index) of the tile; k0: first contraction index of the k-block.  Every mode delivers ROWS * 128 bytes.
template <class Cfg, bool MN, int ROWS>
__device__ __forceinline__ void produce_operand(int mode, int chunked, const GatherSrc& src, const void* map, uint32_t dst, uint32_t bar,
                                                int k0, int mn0, int batch) {
    constexpr int BK = Cfg::BK, CE = Cfg::CE;
    if (mode == kTmaTiled) {
        if constexpr (!MN) {
            ptx::tma_load_3d(dst, map, bar, k0, mn0, batch);
        } else {
            if (chunked) {  // one box for all 128-byte chunks of the tile: the TMA unit is bound by box count
                ptx::tma_load_4d(dst, map, bar, 0, k0, mn0 / CE, batch);
            } else {
#pragma unroll
                for (int c = 0; c < ROWS / CE; ++c) ptx::tma_load_3d(dst + c * BK * 128, map, bar, mn0 + c * CE, k0, batch);
            }
        }
        return;
    }
    const ConvRule& r = src.cr;
    if (mode == kTmaFilterTap) {  // k = tap * oc + co: the k-block is BK filters co of one tap
        int t = fdiv(k0, src.f_rmod);
        ptx::tma_load_4d(dst, map, bar, 0, k0 - t * src.rmod, t, mn0 / CE);
        return;
    }
    if (mode == kTmaFilterSub) {  // k = (j * NFX + i) * C + c over the tap sub-grid; rows = filters
        int tap = fdiv(k0, r.f_c);
        int j = fdiv(tap, r.f_fw);
        ptx::tma_load_4d(dst, map, bar, k0 - tap * r.C, tap - j * r.FW, j, mn0);
        return;
    }
    if (mode == kTmaFilterTapSub) {  // k = (j * NFX + i) * oc + co
        int tap = fdiv(k0, src.f_rmod);
        int j = fdiv(tap, r.f_fw);
        ptx::tma_load_5d(dst, map, bar, 0, k0 - tap * src.rmod, tap - j * r.FW, j, mn0 / CE);
        return;
    }
    // the im2col modes start from one pixel index: the tile's first row (K-major) or the k-block's first row (MN-major)
    const int g = mode == kTmaIm2col ? mn0 : k0;
    const int n = fdiv(g, r.f_plane);
    const int rem = g - n * (r.RH * r.RW);
    const int py = fdiv(rem, r.f_rw);
    const int px = rem - py * r.RW;
    const int w = px * r.mul_x + r.low_x, h = py * r.mul_y + r.low_y;
    if (mode == kTmaIm2col) {  // columns k0 .. k0 + BK: channels c0.. of one tap
        int tap = fdiv(k0, r.f_c);
        int c0 = k0 - tap * r.C;
        int fy = fdiv(tap, r.f_fw);
        int fx = tap - fy * r.FW;
        ptx::tma_load_im2col_4d(dst, map, bar, c0, w, h, n, tap_offset(fx, r.FW, r.e_x), tap_offset(fy, r.FH, r.e_y));
    } else {  // kTmaIm2colMN: each 128-byte chunk of columns is a channel slice of one tap
#pragma unroll
        for (int c = 0; c < ROWS / CE; ++c) {
            int col = mn0 + c * CE;
            int tap = fdiv(col, r.f_c);
            int c0 = col - tap * r.C;
            int fy = fdiv(tap, r.f_fw);
            int fx = tap - fy * r.FW;
            if (col >= src.cols) {  // past the matrix: a channel coordinate outside the image makes the box all zeros
                c0 = r.C;
                fy = fx = 0;
            }
            ptx::tma_load_im2col_4d(dst + c * BK * 128, map, bar, c0, w, h, n, tap_offset(fx, r.FW, r.e_x), tap_offset(fy, r.FH, r.e_y));
        }
    }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::CTAS_PER_SM)
d8k_gemm_kernel(const __grid_constant__ CUtensorMap tmA_launch, const __grid_constant__ CUtensorMap tmB_launch, const GemmParams p_launch) {
    // the roles' work loops shadow these three with the ones of the work item's group (select_work)
    const GemmParams& p = p_launch;
    const CUtensorMap& tmA = tmA_launch;
    const CUtensorMap& tmB = tmB_launch;
    using OutT = typename std::conditional<Cfg::F32, float, __half>::type;
    using InT = OutT;
    constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES, BK = Cfg::BK, CE = Cfg::CE;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;  // ring of stages, 1024-byte aligned
    const uint32_t patch_base = smem_base + STAGES * Cfg::STAGE_BYTES;  // HALO: PATCH_SLOTS buffers, each 1024-byte aligned
    const uint32_t bar_base = patch_base + Cfg::PATCH_SLOTS * Cfg::PATCH_BYTES;
    // barrier block: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then the TMEM base address word
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
    auto raw_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 5 + s); };  // CONVERT: TMA's bytes have landed
    auto patch_full = [&](int i) { return bar_base + 8u * (3 * STAGES + 5 + i); };                     // HALO: the box has landed
    auto patch_empty = [&](int i) { return bar_base + 8u * (3 * STAGES + 5 + Cfg::PATCH_SLOTS + i); };  // HALO: every converter is done with it
    auto patch_addr = [&](int i) { return patch_base + static_cast<uint32_t>(i) * Cfg::PATCH_BYTES; };
    auto turn_bar = [&](int w) { return bar_base + 8u * (3 * STAGES + 5 + 2 * Cfg::PATCH_SLOTS + w); };  // TWIN: MMA thread w may issue
    static_assert(8 * (3 * Cfg::STAGES + 5 + 2 * Cfg::PATCH_SLOTS + 2) <= Cfg::BAR_BYTES, "barrier block");

    __shared__ volatile int s_abort;
    __shared__ int s_last;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), Cfg::HELPERS ? 32 * Cfg::LOADER_WARPS : (Cfg::TWIN ? 2 : 1));
            ptx::mbar_init(empty_bar(s), 1);
            ptx::mbar_init(raw_bar(s), Cfg::TWIN ? 2 : 1);
        }
        ptx::mbar_init(turn_bar(0), 1);
        ptx::mbar_init(turn_bar(1), 1);
        for (int i = 0; i < Cfg::PATCH_SLOTS; ++i) {
            ptx::mbar_init(patch_full(i), 1);
            ptx::mbar_init(patch_empty(i), 32 * Cfg::LOADER_WARPS * Cfg::LOADER_GROUPS);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(tfull_bar(a), 1);
            ptx::mbar_init(tempty_bar(a), 32 * Cfg::EPI_WARPS);
        }
        ptx::fence_mbar_init();
        if (Cfg::TWIN) ptx::mbar_arrive(turn_bar(0));  // the first k-block has no predecessor: thread 0's first turn is open
    }
    if (warp == Cfg::MMA_WARP) {
        ptx::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    if (!Cfg::GATHER && warp == Cfg::PRODUCER_WARP && lane == 0) {
        ptx::tma_prefetch_desc(&tmA);
        ptx::tma_prefetch_desc(&tmB);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    auto stage_a = [&](int s) { return smem_base + s * Cfg::STAGE_BYTES; };
    auto stage_b = [&](int s) { return smem_base + s * Cfg::STAGE_BYTES + Cfg::A_PARTS * Cfg::A_BYTES; };

    if (!Cfg::GATHER && (warp == Cfg::PRODUCER_WARP || (Cfg::TWIN && warp == Cfg::PRODUCER_B_WARP))) {
        // ============================================================================ TMA producer
        // TWIN: this code runs in two warps; the first issues A's boxes, the second B's, each announcing its own bytes
        const bool do_a = !Cfg::TWIN || warp == Cfg::PRODUCER_WARP, do_b = !Cfg::TWIN || warp != Cfg::PRODUCER_WARP;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        // HALO: patch q of this CTA belongs to its (q / slices)-th work item and that item's slice q % slices; it lands in slot
        // q % PATCH_SLOTS.  Patches are requested PATCH_SLOTS - 1 slices ahead of the k-blocks that read them.
        int q_issued = 0, item_seq = 0;
        const bool timed = p.prof != nullptr;
        long long w_empty = 0, w_patch = 0;
        const long long t_begin = timed ? clock64() : 0;
        auto issue_patches_before = [&](int q_end) {
            if constexpr (Cfg::HALO) {
                while (ok && q_issued < q_end) {
                    const int seq = q_issued / p.halo_slices, slice = q_issued - seq * p.halo_slices;
                    const long long w2 = static_cast<long long>(blockIdx.x) + static_cast<long long>(seq) * gridDim.x;
                    if (w2 >= p.total_work) {
                        q_issued = q_end;  // nothing left to fetch
                        break;
                    }
                    const WorkItem it2 = decode_work(p, static_cast<int>(w2), BN);
                    const int slot = q_issued % Cfg::PATCH_SLOTS;
                    ok = wait_bar_timed(patch_empty(slot), ((q_issued / Cfg::PATCH_SLOTS) & 1) ^ 1, &s_abort, p.status, (kRoleProducer << 8) | 4, timed,
                                        &w_patch);
                    if (!ok) break;
                    if (lane == 0) {
                        const ConvRule& r = p.a.cr;
                        ptx::mbar_arrive_expect_tx(patch_full(slot), static_cast<uint32_t>(p.halo_bytes));
                        // box {32 channels, halo_wp columns, rows, 1 image} whose corner is the tile's first source pixel; what
                        // lies outside the image arrives as zeros
                        ptx::tma_load_4d(patch_addr(slot), &tmA, patch_full(slot), slice * CE, r.low_x, it2.m0 / p.halo_wp + r.low_y,
                                         it2.batch % p.a_batch_mod);
                    }
                    __syncwarp();
                    ++q_issued;
                }
            }
        };
        for (int w_all = blockIdx.x; ok && w_all < p_launch.total_work; w_all += gridDim.x, ++item_seq) {
            SelectedWork sel = {&p_launch, &tmA_launch, &tmB_launch, w_all};
            if constexpr (Cfg::GROUPED) sel = select_work(p_launch, tmA_launch, tmB_launch, w_all);
            const GemmParams& p = Cfg::GROUPED ? *sel.p : p_launch;
            const CUtensorMap& tmA = Cfg::GROUPED ? *sel.ta : tmA_launch;
            const CUtensorMap& tmB = Cfg::GROUPED ? *sel.tb : tmB_launch;
            const int w = Cfg::GROUPED ? sel.w : w_all;
            (void)tmA; (void)tmB; (void)w;
            WorkItem it = decode_work(p, w, BN);
            // GROUPED: what the k-loop reads, copied out of the item's parameters once - read through the pointer every field
            // would be loaded again after each asm statement with a memory clobber
            GatherSrc src_copy;
            int kbatch_l = p.kbatch, num_kb_l = p.num_kb, tma_l = 0, chunked_l = 0, batch_mod_l = 1;
            if constexpr (Cfg::GROUPED) {
                src_copy = do_a ? p.a : p.b;
                tma_l = do_a ? p.a_tma : p.b_tma;
                chunked_l = do_a ? p.a_chunked : p.b_chunked;
                batch_mod_l = do_a ? p.a_batch_mod : p.b_batch_mod;
            }
            for (int kk = it.kb_begin; kk < it.kb_end; ++kk) {
                int k0_halo = 0;
                if constexpr (Cfg::HALO) {
                    const int slice = kk / p.halo_taps, tap = kk - slice * p.halo_taps;
                    if (tap == 0) issue_patches_before(item_seq * p.halo_slices + slice + Cfg::PATCH_SLOTS);
                    if (!ok) break;
                    k0_halo = tap * p.a.cr.C + slice * CE;
                }
                ok = wait_bar_timed(empty_bar(stage), phase ^ 1, &s_abort, p.status, (kRoleProducer << 8) | 1, timed, &w_empty);
                if (!ok) break;
                if (lane == 0) {
                    int b = it.batch, kb = kk;
                    if (kbatch_l > 1) {
                        b = kk / num_kb_l;
                        kb = kk - b * num_kb_l;
                    }
                    int k0 = Cfg::HALO ? k0_halo : kb * BK;
                    // CONVERT: the boxes fill the hi halves of the stage and complete on the raw barrier
                    const uint32_t bar = Cfg::CONVERT ? raw_bar(stage) : full_bar(stage);
                    if constexpr (Cfg::TWIN) ptx::mbar_arrive_expect_tx(bar, do_a ? Cfg::A_BYTES : Cfg::B_BYTES);
                    else ptx::mbar_arrive_expect_tx(bar, Cfg::HALO ? Cfg::B_BYTES : Cfg::CONVERT ? Cfg::A_BYTES + Cfg::B_BYTES : Cfg::STAGE_BYTES);
                    if constexpr (Cfg::GROUPED) {  // always TWIN: this thread issues one operand
                        if (do_a) produce_operand<Cfg, Cfg::A_MN, kBM>(tma_l, chunked_l, src_copy, &tmA, stage_a(stage), bar, k0, it.m0, b % batch_mod_l);
                        else produce_operand<Cfg, Cfg::B_MN, BN>(tma_l, chunked_l, src_copy, &tmB, stage_b(stage), bar, k0, it.n0, b % batch_mod_l);
                    } else {
                        if constexpr (!Cfg::HALO)
                            if (do_a) produce_operand<Cfg, Cfg::A_MN, kBM>(p.a_tma, p.a_chunked, p.a, &tmA, stage_a(stage), bar, k0, it.m0, b % p.a_batch_mod);
                        if (do_b) produce_operand<Cfg, Cfg::B_MN, BN>(p.b_tma, p.b_chunked, p.b, &tmB, stage_b(stage), bar, k0, it.n0, b % p.b_batch_mod);
                    }
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (timed && lane == 0 && warp == Cfg::PRODUCER_WARP) {
            p.prof[blockIdx.x * 16 + 0] = clock64() - t_begin;
            p.prof[blockIdx.x * 16 + 1] = w_empty;
            p.prof[blockIdx.x * 16 + 2] = w_patch;
        }
    } else if (warp == Cfg::MMA_WARP || (Cfg::TWIN && warp == Cfg::MMA2_WARP)) {
        // ============================================================================ MMA issuer
        // A from tensor memory is always one row per lane, whatever the stored layout was
        constexpr uint32_t idesc = ptx::make_idesc(Cfg::F32 ? 2u : 0u, Cfg::A_MN && !Cfg::ATMEM, Cfg::B_MN, kBM, BN);
        constexpr uint32_t idesc_wide =
            ptx::make_idesc(Cfg::F32 ? 2u : 0u, Cfg::A_MN && (!Cfg::ATMEM || Cfg::ALO), Cfg::B_MN, kBM, Cfg::STACK ? 2 * BN : BN);
        // descriptor step per UMMA_K: K-major advances 32 bytes inside the swizzled row; MN-major advances UMMA_K rows
        constexpr uint32_t a_step = Cfg::A_MN ? Cfg::UMMA_K * 128 : 32;
        constexpr uint32_t b_step = Cfg::B_MN ? Cfg::UMMA_K * 128 : 32;
        constexpr uint32_t a_lbo = Cfg::A_MN ? BK * 128 : 16;
        constexpr uint32_t b_lbo = Cfg::B_MN ? BK * 128 : 16;
        constexpr uint32_t a_sbo = Cfg::A_B32 ? 512 : 1024, b_sbo = Cfg::B_B32 ? 512 : 1024;
        constexpr uint32_t a_lay = Cfg::A_B32 ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
        constexpr uint32_t b_lay = Cfg::B_B32 ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
        // The tensor pipe holds only a couple of MMAs ahead of the one it runs (measured: issuing costs what executing
        // costs), so whatever this warp does between two k-blocks is time the pipe idles: a 128 x 64 x 8 tf32 MMA is 48 clocks
        // and the bookkeeping of a k-block used to cost over 600.  Everything that moves with the stage - barrier addresses,
        // descriptors, the tensor-memory column of A - is therefore a running value stepped once per k-block, not recomputed.
        constexpr uint64_t kStageStep = static_cast<uint64_t>(Cfg::STAGE_BYTES >> 4);  // a stage further on, in descriptor units
        const uint64_t da_first = ptx::smem_desc(stage_a(0), a_lbo, a_sbo, a_lay), db_first = ptx::smem_desc(stage_b(0), b_lbo, b_sbo, b_lay);
        const uint32_t ta_first = tmem_base + Cfg::A_TMEM_COL0;
        int stage = 0;
        uint32_t phase = 0;
        uint64_t da_run = da_first, db_run = db_first;
        uint32_t ta_run = ta_first, full_run = full_bar(0), empty_run = empty_bar(0);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool timed = p.prof != nullptr;
        long long w_full = 0, w_tmem = 0;
        const long long t_begin = timed ? clock64() : 0;
        // TWIN: both MMA warps walk every k-block to keep the running state; warp `me` issues the k-blocks t with t % 2 == me
        const int me = (Cfg::TWIN && warp != Cfg::MMA_WARP) ? 1 : 0;
        int t = 0;
        uint32_t my_turns = 0;
        for (int w_all = blockIdx.x; ok && w_all < p_launch.total_work; w_all += gridDim.x) {
            SelectedWork sel = {&p_launch, &tmA_launch, &tmB_launch, w_all};
            if constexpr (Cfg::GROUPED) sel = select_work(p_launch, tmA_launch, tmB_launch, w_all);
            const GemmParams& p = Cfg::GROUPED ? *sel.p : p_launch;
            const CUtensorMap& tmA = Cfg::GROUPED ? *sel.ta : tmA_launch;
            const CUtensorMap& tmB = Cfg::GROUPED ? *sel.tb : tmB_launch;
            const int w = Cfg::GROUPED ? sel.w : w_all;
            (void)tmA; (void)tmB; (void)w;
            WorkItem it = decode_work(p, w, BN);
            uint32_t d_tmem = 0;
            int in_chain = 0;
            for (int kk = it.kb_begin; kk < it.kb_end; ++kk, ++t) {
                const bool mine = !Cfg::TWIN || (t & 1) == me;
                if (in_chain == 0) d_tmem = tmem_base + acc * Cfg::ACC_COLS;
                if (mine && in_chain == 0) {  // a new accumulation chain needs a drained accumulator buffer
                    ok = wait_bar_timed(tempty_bar(acc), acc_phase ^ 1, &s_abort, p.status, (kRoleMma << 8) | 2, timed, &w_tmem);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                }
                if (mine) {
                    ok = wait_bar_timed(full_run, phase, &s_abort, p.status, (kRoleMma << 8) | 1, timed, &w_full);
                    if (!ok) break;
                    if constexpr (Cfg::TWIN) {  // the other thread has issued the k-block before this one
                        ok = wait_bar(turn_bar(me), my_turns & 1, &s_abort, p.status, (kRoleMma << 8) | 5);
                        if (!ok) break;
                        ++my_turns;
                    }
                    ptx::tc_fence_after_sync();
                }
                const bool chain_ends = (kk + 1 == it.kb_end) || (Cfg::CHUNK_KB > 0 && in_chain + 1 == Cfg::CHUNK_KB);
                if (mine && lane == 0) {
#pragma unroll
                    for (int s = 0; s < Cfg::KSTEPS; ++s) {
                        // a k-step moves the start address by a few 16-byte units, far below the 14-bit field's range: a plain add
                        const uint64_t da = da_run + ((s * a_step) >> 4), db = db_run + ((s * b_step) >> 4);
                        const uint32_t accumulate = (in_chain > 0 || s > 0) ? 1u : 0u;
                        if constexpr (Cfg::ATMEM) {
                            const uint32_t ta_hi = ta_run + s * Cfg::UMMA_K;
                            if constexpr (Cfg::ALO) {
                                ptx::mma_tf32(d_tmem, da, db, idesc_wide, accumulate);    // A_hi (shared memory) [B_hi ; B_lo]
                                ptx::mma_tf32_a_tmem(d_tmem, ta_hi, db, idesc, 1u);      // A_lo (tensor memory) B_hi
                            } else if constexpr (Cfg::STACK) {
                                ptx::mma_tf32_a_tmem(d_tmem, ta_hi, db, idesc_wide, accumulate);  // A_hi [B_hi ; B_lo]
                                ptx::mma_tf32_a_tmem(d_tmem, ta_hi + BK, db, idesc, 1u);          // A_lo B_hi
                            } else {
                                ptx::mma_tf32_a_tmem(d_tmem, ta_hi + BK, db, idesc, accumulate);  // small terms first
                                ptx::mma_tf32_a_tmem(d_tmem, ta_hi, db + (Cfg::B_BYTES >> 4), idesc, 1u);
                                ptx::mma_tf32_a_tmem(d_tmem, ta_hi, db, idesc, 1u);
                            }
                        } else if constexpr (Cfg::F32) {
                            const uint64_t da_lo = da + (Cfg::A_BYTES >> 4), db_lo = db + (Cfg::B_BYTES >> 4);
                            if constexpr (Cfg::STACK) {
                                ptx::mma_tf32(d_tmem, da, db, idesc_wide, accumulate);  // A_hi [B_hi ; B_lo]
                                ptx::mma_tf32(d_tmem, da_lo, db, idesc, 1u);           // A_lo B_hi
                            } else {
                                ptx::mma_tf32(d_tmem, da_lo, db, idesc, accumulate);  // small terms first
                                ptx::mma_tf32(d_tmem, da, db_lo, idesc, 1u);
                                ptx::mma_tf32(d_tmem, da, db, idesc, 1u);
                            }
                        } else {
                            ptx::mma_f16(d_tmem, da, db, idesc, accumulate);
                        }
                    }
                    if constexpr (Cfg::TWIN) {  // pass the token before this thread's own bookkeeping
                        ptx::tc_fence_before_sync();
                        ptx::mbar_arrive(turn_bar(me ^ 1));
                    }
                    ptx::tc_commit(empty_run);  // the stage may be refilled once these MMAs have read it
                    // the pipe completes MMAs in issue order: this commit also covers the other thread's earlier k-blocks of the chain
                    if (chain_ends) ptx::tc_commit(tfull_bar(acc));
                }
                __syncwarp();
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1;
                    da_run = da_first; db_run = db_first; ta_run = ta_first; full_run = full_bar(0); empty_run = empty_bar(0);
                } else {
                    da_run += kStageStep; db_run += kStageStep; ta_run += Cfg::A_TMEM_STRIDE; full_run += 8; empty_run += 8;
                }
                if (chain_ends) {
                    in_chain = 0;
                    if (++acc == Cfg::ACC_BUFS) { acc = 0; acc_phase ^= 1; }
                } else {
                    ++in_chain;
                }
            }
        }
        if (timed && lane == 0 && warp == Cfg::MMA_WARP) {
            p.prof[blockIdx.x * 16 + 3] = clock64() - t_begin;
            p.prof[blockIdx.x * 16 + 4] = w_full;
            p.prof[blockIdx.x * 16 + 5] = w_tmem;
        }
    } else if (warp < Cfg::EPI_WARPS) {
        // ============================================================================ epilogue (TMEM -> C)
        const int quarter = warp;  // warp w may read TMEM lanes [32 (w % 4), +32)
        const int row_in_tile = quarter * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool timed = p.prof != nullptr;
        long long w_tfull = 0;
        const long long t_begin = timed ? clock64() : 0;
        for (int w_all = blockIdx.x; ok && w_all < p_launch.total_work; w_all += gridDim.x) {
            SelectedWork sel = {&p_launch, &tmA_launch, &tmB_launch, w_all};
            if constexpr (Cfg::GROUPED) sel = select_work(p_launch, tmA_launch, tmB_launch, w_all);
            const GemmParams& p = Cfg::GROUPED ? *sel.p : p_launch;
            const CUtensorMap& tmA = Cfg::GROUPED ? *sel.ta : tmA_launch;
            const CUtensorMap& tmB = Cfg::GROUPED ? *sel.tb : tmB_launch;
            const int w = Cfg::GROUPED ? sel.w : w_all;
            (void)tmA; (void)tmB; (void)w;
            WorkItem it = decode_work(p, w, BN);
            const int row = it.m0 + row_in_tile;
            const bool row_ok = out_row_exists(p, row);
            const long long crow = static_cast<long long>(it.batch) * p.c_batch_stride + out_row_offset(p, row) + scatter_offset(p, row);
            float* part = p.ws + (static_cast<size_t>(w) * kBM + row_in_tile) * BN;
            if constexpr (Cfg::CHUNK_KB == 0) {
                ok = wait_bar_timed(tfull_bar(acc), acc_phase, &s_abort, p.status, (kRoleEpilogue << 8) | 3, timed, &w_tfull,
                                    static_cast<unsigned>(p.epi_backoff_ns));
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t taddr = tmem_base + acc * Cfg::ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    __syncwarp();
                    ptx::tmem_ld_32x32(taddr + c * 32, r);
                    ptx::tmem_ld_wait();
                    if (p.splits == 1) {
                        if (row_ok && it.n0 + c * 32 < p.N) {
                            float accv[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) accv[i] = __uint_as_float(r[i]);
                            store_row_chunk<OutT>(p, crow, it.n0 + c * 32, accv);
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            __stcg(reinterpret_cast<uint4*>(part + c * 32) + v, make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]));
                    }
                }
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(tempty_bar(acc));  // accumulator buffer free for the tile after next
                if (++acc == Cfg::ACC_BUFS) { acc = 0; acc_phase ^= 1; }
            } else {
                // one accumulation chain per CHUNK_KB k-blocks: add each finished chain into registers (round to nearest)
                float accv[BN];
#pragma unroll
                for (int i = 0; i < BN; ++i) accv[i] = 0.f;
                const int chains = (it.kb_end - it.kb_begin + Cfg::CHUNK_KB - 1) / Cfg::CHUNK_KB;
                for (int ch = 0; ch < chains; ++ch) {
                    ok = wait_bar_timed(tfull_bar(acc), acc_phase, &s_abort, p.status, (kRoleEpilogue << 8) | 3, timed, &w_tfull,
                                        static_cast<unsigned>(p.epi_backoff_ns));
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    const uint32_t taddr = tmem_base + acc * Cfg::ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
                    if constexpr (Cfg::DUAL) {  // 16 columns at a time: two CTAs per SM leave 96 registers per thread
#pragma unroll
                        for (int c = 0; c < Cfg::ACC_COLS / 16; ++c) {
                            uint32_t r[16];
                            __syncwarp();
                            ptx::tmem_ld_32x16(taddr + c * 16, r);
                            ptx::tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) accv[(c % (BN / 16)) * 16 + i] += __uint_as_float(r[i]);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < Cfg::ACC_COLS / 32; ++c) {  // STACK: the second half of the columns holds the A_hi B_lo terms
                            uint32_t r[32];
                            __syncwarp();
                            ptx::tmem_ld_32x32(taddr + c * 32, r);
                            ptx::tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) accv[(c % (BN / 32)) * 32 + i] += __uint_as_float(r[i]);
                        }
                    }
                    ptx::tc_fence_before_sync();
                    ptx::mbar_arrive(tempty_bar(acc));
                    if (++acc == Cfg::ACC_BUFS) { acc = 0; acc_phase ^= 1; }
                }
                if (!ok) break;
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) {
                    if (p.splits == 1) {
                        if (row_ok && it.n0 + c * 32 < p.N) store_row_chunk<OutT>(p, crow, it.n0 + c * 32, &accv[c * 32]);
                    } else {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            __stcg(reinterpret_cast<float4*>(part + c * 32) + v,
                                   make_float4(accv[c * 32 + 4 * v], accv[c * 32 + 4 * v + 1], accv[c * 32 + 4 * v + 2], accv[c * 32 + 4 * v + 3]));
                    }
                }
            }

            if (p.splits > 1) {
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 0) {
                    // A ticket word is (launch epoch << 8 | tickets drawn).  A word left by another launch - finished, or one that
                    // gave up on a wait half-way - carries another epoch and counts as zero, so tickets are never cleared.
                    unsigned* word = reinterpret_cast<unsigned*>(p.counters + it.tile);
                    const unsigned fresh = static_cast<unsigned>(p_launch.epoch) << 8;
                    unsigned cur = *reinterpret_cast<volatile unsigned*>(word);
                    unsigned drawn;
                    for (;;) {
                        const unsigned want = ((cur & 0xffffff00u) == fresh ? cur : fresh) + 1u;
                        const unsigned old = atomicCAS(word, cur, want);
                        if (old == cur) {
                            drawn = want & 0xffu;
                            break;
                        }
                        cur = old;
                    }
                    s_last = (static_cast<int>(drawn) == p.splits);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (s_last) {
                    __threadfence();
                    if (row_ok) {
                        const float* first = p.ws + (static_cast<size_t>(it.tile) * p.splits * kBM + row_in_tile) * BN;
#pragma unroll 1
                        for (int c = 0; c < BN / 32; ++c) {
                            if (it.n0 + c * 32 >= p.N) break;
                            float accv[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) accv[i] = 0.f;
                            for (int s = 0; s < p.splits; ++s) {
                                const float4* src = reinterpret_cast<const float4*>(first + static_cast<size_t>(s) * kBM * BN + c * 32);
#pragma unroll
                                for (int v = 0; v < 8; ++v) {
                                    float4 t = __ldcg(src + v);
                                    accv[4 * v] += t.x; accv[4 * v + 1] += t.y; accv[4 * v + 2] += t.z; accv[4 * v + 3] += t.w;
                                }
                            }
                            store_row_chunk<OutT>(p, crow, it.n0 + c * 32, accv);
                        }
                    }
                }
            }
        }
        // scattered rows may sit in a peer GPU's memory: order this thread's stores before whatever the host enqueues next
        if (p.scatter_rows) __threadfence_system();
        if (timed && threadIdx.x == 0) {
            p.prof[blockIdx.x * 16 + 6] = clock64() - t_begin;
            p.prof[blockIdx.x * 16 + 7] = w_tfull;
        }
    } else if (Cfg::CONVERT && warp >= Cfg::LOADER_WARP0) {
        // ============================================================================ converters (fp32 behind TMA)
        // The stage's hi halves hold the operands as TMA wrote them, already in the swizzled layout; the lo image has
        // the same layout A_BYTES (B_BYTES) further on, so this is a linear pass over 16-byte chunks.
        const int group = (warp - Cfg::LOADER_WARP0) / Cfg::LOADER_WARPS;
        const int tid = threadIdx.x - 32 * (Cfg::LOADER_WARP0 + Cfg::LOADER_WARPS * group);  // 0..127 inside the group
        constexpr int A_CHUNKS = Cfg::A_BYTES / 16 / 128, B_CHUNKS = Cfg::B_BYTES / 16 / 128;
        int t = 0;
        bool ok = true;
        int item_seq = 0;
        const bool timed = p.prof != nullptr;
        long long w_raw = 0, w_pfull = 0;
        const long long t_begin = timed ? clock64() : 0;
        for (int w_all = blockIdx.x; ok && w_all < p_launch.total_work; w_all += gridDim.x, ++item_seq) {
            SelectedWork sel = {&p_launch, &tmA_launch, &tmB_launch, w_all};
            if constexpr (Cfg::GROUPED) sel = select_work(p_launch, tmA_launch, tmB_launch, w_all);
            const GemmParams& p = Cfg::GROUPED ? *sel.p : p_launch;
            const CUtensorMap& tmA = Cfg::GROUPED ? *sel.ta : tmA_launch;
            const CUtensorMap& tmB = Cfg::GROUPED ? *sel.tb : tmB_launch;
            const int w = Cfg::GROUPED ? sel.w : w_all;
            (void)tmA; (void)tmB; (void)w;
            WorkItem it = decode_work(p, w, BN);
            const int tile_col0 = Cfg::HALO ? it.m0 % p.halo_wp : 0;  // HALO: raster position of the tile's first pixel inside its first patch row
            for (int kk = it.kb_begin; kk < it.kb_end; ++kk, ++t) {
                // HALO: which patch this k-block reads, and where its tap starts inside it
                int pslot = 0, prow0 = 0;
                bool last_tap = false;
                if constexpr (Cfg::HALO) {
                    const int slice = kk / p.halo_taps, tap = kk - slice * p.halo_taps;
                    const int pq = item_seq * p.halo_slices + slice;
                    pslot = pq % Cfg::PATCH_SLOTS;
                    last_tap = tap + 1 == p.halo_taps;
                    if (t % Cfg::LOADER_GROUPS != group) {
                        // not this group's k-block; its earlier reads of the patch are over, so the slot is done with on the last tap
                        if (last_tap) ptx::mbar_arrive(patch_empty(pslot));
                        continue;
                    }
                    ok = wait_bar_timed(patch_full(pslot), (pq / Cfg::PATCH_SLOTS) & 1, &s_abort, p.status, (kRoleLoader << 8) | 4, timed, &w_pfull);
                    if (!ok) break;
                    const ConvRule& r = p.a.cr;
                    const int fy = fdiv(tap, r.f_fw), fx = tap - fy * r.FW;
                    prow0 = tile_col0 + tap_offset(fy, r.FH, r.e_y) * p.halo_wp + tap_offset(fx, r.FW, r.e_x);
                } else {
                    if (t % Cfg::LOADER_GROUPS != group) continue;
                }
                const int stage = t % STAGES;
                const uint32_t phase = (t / STAGES) & 1;
                ok = wait_bar_timed(raw_bar(stage), phase, &s_abort, p.status, (kRoleLoader << 8) | 2, timed, &w_raw);  // every reader observes the phase itself
                if (!ok) break;
                if constexpr (Cfg::ATMEM) {
                    // A: this thread owns tile row 32 (warp % 4) + lane, the tensor-memory lane its warp may write
                    const int q = warp & 3;
                    uint32_t hi[32];
                    if constexpr (!Cfg::A_MN) {
                        // HALO: the row sits in the patch at its pixel's raster position shifted by the tap; else in the stage
                        const int row = Cfg::HALO ? prow0 + q * 32 + lane : q * 32 + lane;
                        const uint32_t base = (Cfg::HALO ? patch_addr(pslot) : stage_a(stage)) + 128u * row;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {  // the row's eight 16-byte chunks, un-swizzled on the way
                            uint4 v = ptx::ld_shared_v4(base + ((c ^ (row & 7)) << 4));
                            hi[4 * c] = v.x; hi[4 * c + 1] = v.y; hi[4 * c + 2] = v.z; hi[4 * c + 3] = v.w;
                        }
                        if constexpr (Cfg::HALO) {
                            if (last_tap) ptx::mbar_arrive(patch_empty(pslot));  // the values are in registers: the slot may be refilled
                        }
                    } else {
                        // MN-major: chunk q holds BK k-rows of 32 m's; this thread's m is `lane`, one word per k-row
                        const uint32_t base = stage_a(stage) + q * (BK * 128) + ((lane & 3) << 2);
                        const int c16 = lane >> 2;
#pragma unroll
                        for (int k = 0; k < 32; ++k) hi[k] = ptx::ld_shared_b32(base + swz<true>(k, c16));
                    }
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::A_TMEM_COL0 + stage * Cfg::A_TMEM_STRIDE;
                    // the store takes its operands when it issues: the registers are reused for lo
                    if constexpr (!Cfg::ALO) ptx::tmem_st_32x32(taddr, hi);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float d = __uint_as_float(hi[i]) - __uint_as_float(hi[i] & 0xffffe000u);
                        hi[i] = (__float_as_uint(d) + 0x1000u) & 0xffffe000u;
                    }
                    ptx::tmem_st_32x32(taddr + (Cfg::ALO ? 0 : BK), hi);
                    uint4 vb[B_CHUNKS];
                    const uint32_t b0 = stage_b(stage) + 16u * tid;
#pragma unroll
                    for (int i = 0; i < B_CHUNKS; ++i) vb[i] = ptx::ld_shared_v4(b0 + 2048u * i);
#pragma unroll
                    for (int i = 0; i < B_CHUNKS; ++i) st_shared_v4(b0 + 2048u * i + Cfg::B_BYTES, tf32_low_part(vb[i]));
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before_sync();
                } else {
                uint4 va[A_CHUNKS], vb[B_CHUNKS];
                const uint32_t a0 = stage_a(stage) + 16u * tid, b0 = stage_b(stage) + 16u * tid;
#pragma unroll
                for (int i = 0; i < A_CHUNKS; ++i) va[i] = ptx::ld_shared_v4(a0 + 2048u * i);
#pragma unroll
                for (int i = 0; i < B_CHUNKS; ++i) vb[i] = ptx::ld_shared_v4(b0 + 2048u * i);
#pragma unroll
                for (int i = 0; i < A_CHUNKS; ++i) st_shared_v4(a0 + 2048u * i + Cfg::A_BYTES, tf32_low_part(va[i]));
#pragma unroll
                for (int i = 0; i < B_CHUNKS; ++i) st_shared_v4(b0 + 2048u * i + Cfg::B_BYTES, tf32_low_part(vb[i]));
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(full_bar(stage));
            }
        }
        if (timed && tid == 0) {
            p.prof[blockIdx.x * 16 + 8 + 3 * group] = clock64() - t_begin;
            p.prof[blockIdx.x * 16 + 9 + 3 * group] = w_raw;
            p.prof[blockIdx.x * 16 + 10 + 3 * group] = w_pfull;
        }
    } else if (Cfg::GATHER && warp >= Cfg::LOADER_WARP0) {
        // ============================================================================ gather loaders
        const int lw = (warp - Cfg::LOADER_WARP0) % Cfg::LOADER_WARPS;
        const int group = (warp - Cfg::LOADER_WARP0) / Cfg::LOADER_WARPS;
        const int sub = lane >> 3;  // row inside a group of four
        const int j = lane & 7;     // 16-byte chunk of the row
        constexpr int A_ITERS = kBM / 16, B_ITERS = BN / 16;
        // Chunk i of this thread sits in tile row r_i = 16 i + r0.  K-major: r_i is the operand row, the column is the
        // k-block's.  MN-major: r_i = (chunk of 128 bytes along M or N) * BK + (k row), so i % NPIX picks one of the
        // thread's NPIX k rows and i / NPIX the 128-byte chunk.
        constexpr int NPIX = BK / 16;
        constexpr int A_NROW = Cfg::A_MN ? NPIX : A_ITERS, A_NCOL = Cfg::A_MN ? A_ITERS / NPIX : 1;
        constexpr int B_NROW = Cfg::B_MN ? NPIX : B_ITERS, B_NCOL = Cfg::B_MN ? B_ITERS / NPIX : 1;
        static_assert(A_ITERS % NPIX == 0 && B_ITERS % NPIX == 0, "an MN-major tile is whole 128-byte chunks");
        const int r0 = lw * 4 + sub;
        // 16 i + r0 keeps its low three bits, so the swizzled position is that of row r0 plus 2048 i
        const uint32_t sw_a = swz<Cfg::A_B32>(r0, j), sw_b = swz<Cfg::B_B32>(r0, j);
        const InT* const base_a0 = reinterpret_cast<const InT*>(p.a.base);
        const InT* const base_b0 = reinterpret_cast<const InT*>(p.b.base);
        int t = 0;                  // running k-block count of this CTA: k-block t uses stage t % STAGES
        bool ok = true;
        for (int w_all = blockIdx.x; ok && w_all < p_launch.total_work; w_all += gridDim.x) {
            SelectedWork sel = {&p_launch, &tmA_launch, &tmB_launch, w_all};
            if constexpr (Cfg::GROUPED) sel = select_work(p_launch, tmA_launch, tmB_launch, w_all);
            const GemmParams& p = Cfg::GROUPED ? *sel.p : p_launch;
            const CUtensorMap& tmA = Cfg::GROUPED ? *sel.ta : tmA_launch;
            const CUtensorMap& tmB = Cfg::GROUPED ? *sel.tb : tmB_launch;
            const int w = Cfg::GROUPED ? sel.w : w_all;
            (void)tmA; (void)tmB; (void)w;
            WorkItem it = decode_work(p, w, BN);
            RowState ra[A_NROW], rb[B_NROW];
            ColState ca[A_NCOL], cb[B_NCOL];
            // the half of each address that stays put for the whole tile
            if constexpr (!Cfg::A_MN) {
#pragma unroll
                for (int i = 0; i < A_ITERS; ++i) ra[i] = row_state(p.a, it.m0 + 16 * i + r0);
            } else {
#pragma unroll
                for (int q = 0; q < A_NCOL; ++q) ca[q] = col_state<Cfg::VEC>(p.a, it.m0 + q * CE + j * Cfg::VEC);
            }
            if constexpr (!Cfg::B_MN) {
#pragma unroll
                for (int i = 0; i < B_ITERS; ++i) rb[i] = row_state(p.b, it.n0 + 16 * i + r0);
            } else {
#pragma unroll
                for (int q = 0; q < B_NCOL; ++q) cb[q] = col_state<Cfg::VEC>(p.b, it.n0 + q * CE + j * Cfg::VEC);
            }
            for (int kk = it.kb_begin; kk < it.kb_end; ++kk, ++t) {
                if (t % Cfg::LOADER_GROUPS != group) continue;
                const int stage = t % STAGES;
                const uint32_t phase = (t / STAGES) & 1;
                ok = wait_bar(empty_bar(stage), phase ^ 1, &s_abort, p.status, (kRoleLoader << 8) | 1);
                if (!ok) break;
                int b = it.batch, kb = kk;
                if (p.kbatch > 1) {
                    b = kk / p.num_kb;
                    kb = kk - b * p.num_kb;
                }
                const int k0 = kb * BK;
                const long long boff_a = p.a.batch_count > 1 ? static_cast<long long>(b % p.a.batch_count) * p.a.batch_stride : 0;
                const long long boff_b = p.b.batch_count > 1 ? static_cast<long long>(b % p.b.batch_count) * p.b.batch_stride : 0;
                // the half that moves with the k-block
                if constexpr (!Cfg::A_MN) {
                    ca[0] = col_state<Cfg::VEC>(p.a, k0 + j * Cfg::VEC);
                } else {
#pragma unroll
                    for (int h = 0; h < NPIX; ++h) ra[h] = row_state(p.a, k0 + 16 * h + r0);
                }
                if constexpr (!Cfg::B_MN) {
                    cb[0] = col_state<Cfg::VEC>(p.b, k0 + j * Cfg::VEC);
                } else {
#pragma unroll
                    for (int h = 0; h < NPIX; ++h) rb[h] = row_state(p.b, k0 + 16 * h + r0);
                }
                const InT* const base_a = base_a0 + (p.a.kind == 0 ? boff_a : 0);
                const InT* const base_b = base_b0 + (p.b.kind == 0 ? boff_b : 0);
                uint4 va[A_ITERS], vb[B_ITERS];
                unsigned slow = 0;  // bit i: chunk i of A, bit 16 + i: chunk i of B
#pragma unroll
                for (int i = 0; i < A_ITERS; ++i) {
                    const RowState& r = ra[Cfg::A_MN ? i % NPIX : i];
                    const ColState& k = ca[Cfg::A_MN ? i / NPIX : 0];
                    uintptr_t addr = chunk_addr<InT>(p.a, base_a, r, k);
                    if (k.how == kChunkSlow) slow |= 1u << i;
                    va[i] = ldg_pred(k.how == kChunkFast ? addr : 0);
                }
#pragma unroll
                for (int i = 0; i < B_ITERS; ++i) {
                    const RowState& r = rb[Cfg::B_MN ? i % NPIX : i];
                    const ColState& k = cb[Cfg::B_MN ? i / NPIX : 0];
                    uintptr_t addr = chunk_addr<InT>(p.b, base_b, r, k);
                    if (k.how == kChunkSlow) slow |= 1u << (16 + i);
                    vb[i] = ldg_pred(k.how == kChunkFast ? addr : 0);
                }
                if (slow) {  // ragged edges, unaligned rows, chunks that straddle filter taps: element by element
#pragma unroll
                    for (int i = 0; i < A_ITERS; ++i) {
                        if (!(slow >> i & 1u)) continue;
                        int r = 16 * i + r0;
                        int g = Cfg::A_MN ? k0 + (r % BK) : it.m0 + r;
                        int col = Cfg::A_MN ? it.m0 + (r / BK) * CE + j * Cfg::VEC : k0 + j * Cfg::VEC;
                        ColCtx kc = {};
                        if (p.a.kind == 1) kc = col_ctx<Cfg::VEC>(p.a, col);
                        va[i] = fetch16<InT, Cfg::VEC>(p.a, g, col, boff_a, kc);
                    }
#pragma unroll
                    for (int i = 0; i < B_ITERS; ++i) {
                        if (!(slow >> (16 + i) & 1u)) continue;
                        int r = 16 * i + r0;
                        int g = Cfg::B_MN ? k0 + (r % BK) : it.n0 + r;
                        int col = Cfg::B_MN ? it.n0 + (r / BK) * CE + j * Cfg::VEC : k0 + j * Cfg::VEC;
                        ColCtx kc = {};
                        if (p.b.kind == 1) kc = col_ctx<Cfg::VEC>(p.b, col);
                        vb[i] = fetch16<InT, Cfg::VEC>(p.b, g, col, boff_b, kc);
                    }
                }
#pragma unroll
                for (int i = 0; i < A_ITERS; ++i) store_chunk_smem<Cfg::F32>(stage_a(stage) + sw_a + 2048u * i, Cfg::A_BYTES, va[i]);
#pragma unroll
                for (int i = 0; i < B_ITERS; ++i) store_chunk_smem<Cfg::F32>(stage_b(stage) + sw_b + 2048u * i, Cfg::B_BYTES, vb[i]);
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(full_bar(stage));
            }
        }
    }

    // ================================================================================ teardown
    if (s_abort) {
        // give copies and MMAs still in flight time to land before shared and tensor memory are released
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == Cfg::MMA_WARP) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace d8k
