// Host side of the contraction kernel: picks the tile configuration and the split, encodes TMA tensor maps, launches.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>

#include "gemm_host.h"

namespace d8k {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*,
                                   const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeIm2colFn encode_im2col() {
    static EncodeIm2colFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeIm2colFn>(sym);
    });
    return fn;
}

int env_int(const char* name, int fallback) {
    const char* v = std::getenv(name);
    return v ? std::atoi(v) : fallback;
}

bool tma_ok(const HostOperand& o, int esize) {
    if (o.is_virtual || o.rmod > 0) return false;
    if (reinterpret_cast<uintptr_t>(o.ptr) & 15) return false;
    if ((o.ld * esize) % 16 != 0) return false;
    if (o.batch_count > 1 && (o.batch_stride * esize) % 16 != 0) return false;
    return true;
}

// 3-D map {inner, rows, batch} over a row-major fp16 matrix stack, 128-byte swizzle, zero fill outside.
bool make_map(CUtensorMap* map, const HostOperand& o, long long inner, long long rows, int box_rows, int esize = 2, bool atom32 = false) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(o.batch_count)};
    long long bstride = o.batch_count > 1 ? o.batch_stride : rows * o.ld;
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(o.ld * esize), static_cast<cuuint64_t>(bstride * esize)};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / esize), static_cast<cuuint32_t>(box_rows), 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(o.ptr), dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// 4-D map that delivers several 128-byte-wide pieces of an operand as ONE box (the TMA unit is bound by box count).
// With ce = 128 / esize elements per piece:
//   K-major  (mn == false): {ce k, rows, K / ce, batch},      box {ce, box_k rows, box_groups k-pieces, 1} - needs K % ce == 0
//   MN-major (mn == true) : {ce m/n, K, extent / ce, batch},  box {ce, box_k k rows, box_groups chunks, 1} - needs extent % ce == 0
// The second and third strides are not in increasing order (the 128-byte step comes after the row pitch); TMA only
// computes addresses from them.  atom32: the 128-byte swizzle with 32-byte atoms that MN-major tf32 operands need.
bool make_pair_map(CUtensorMap* map, const HostOperand& o, long long extent, long long K, int box_k = 128, int box_groups = 2,
                   int esize = 2, bool atom32 = false) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const long long ce = 128 / esize;
    long long rows = o.mn ? K : extent;           // stored rows
    long long groups = (o.mn ? extent : K) / ce;  // 128-byte groups along the stored row
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(ce), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(groups),
                          static_cast<cuuint64_t>(o.batch_count)};
    long long bstride = o.batch_count > 1 ? o.batch_stride : rows * o.ld;
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(o.ld * esize), 128u, static_cast<cuuint64_t>(bstride * esize)};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(ce), static_cast<cuuint32_t>(box_k), static_cast<cuuint32_t>(box_groups), 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(o.ptr), dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// How the TMA producer can fetch an operand (kTma*), or -1 when only the loader warps can.  extent: M or N.
int tma_mode(const HostOperand& o, int esize, long long extent, long long K) {
    const long long ce = 128 / esize;  // elements per 128-byte row; also the k-block
    if (reinterpret_cast<uintptr_t>(o.ptr) & 15) return -1;
    if (o.halo) return encode_tiled() != nullptr ? kTmaHalo : -1;
    if (o.sub.on) {  // a grid of taps of a filter [oc, FH, FW, ic]
        if (o.is_virtual || o.batch_count > 1 || o.sub.ic % ce != 0 || encode_tiled() == nullptr) return -1;
        if (o.rmod == 0) return o.mn ? -1 : kTmaFilterSub;
        return (o.mn && o.sub.oc % ce == 0) ? kTmaFilterTapSub : -1;
    }
    if (!o.is_virtual && o.rmod == 0) return tma_ok(o, esize) ? kTmaTiled : -1;
    if (!o.is_virtual) {  // filter [oc, taps, ic] read as W'[(tap, co)][ci]: ld = taps * ic, ld2 = ic, rmod = oc
        if (!o.mn || o.batch_count > 1 || o.ld2 % ce != 0 || o.rmod % ce != 0 || extent != o.ld2 || encode_tiled() == nullptr) return -1;
        return kTmaFilterTap;
    }
    const ConvRule& r = o.cr;
    if (!r.unit_div || r.C % ce != 0 || r.mul_y > 8 || r.mul_x > 8 || encode_im2col() == nullptr || o.batch_count > 1) return -1;
    const int up_y = r.low_y + (r.RH - 1) * r.mul_y - (r.SH - 1), up_x = r.low_x + (r.RW - 1) * r.mul_x - (r.SW - 1);
    auto corner_ok = [](int v) { return v >= -128 && v <= 127; };
    if (!corner_ok(r.low_y) || !corner_ok(r.low_x) || !corner_ok(up_y) || !corner_ok(up_x)) return -1;
    const int span_y = (r.FH - 1) * (r.e_y < 0 ? -r.e_y : r.e_y), span_x = (r.FW - 1) * (r.e_x < 0 ? -r.e_x : r.e_x);
    if (span_y > 255 || span_x > 255) return -1;
    (void)K;
    return o.mn ? kTmaIm2colMN : kTmaIm2col;
}

// im2col map over the NHWC image of a virtual operand: `pixels` anchor pixels per box, one 128-byte channel slice.
// rows: logical pixel rows of the virtual matrix (images * RH * RW).
bool make_im2col_map(CUtensorMap* map, const HostOperand& o, long long rows, int pixels, int esize, bool atom32) {
    EncodeIm2colFn enc = encode_im2col();
    if (!enc) return false;
    const ConvRule& r = o.cr;
    const long long images = rows / (static_cast<long long>(r.RH) * r.RW);
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(r.C), static_cast<cuuint64_t>(r.SW), static_cast<cuuint64_t>(r.SH),
                          static_cast<cuuint64_t>(images)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(r.C) * esize, static_cast<cuuint64_t>(r.SW) * r.C * esize,
                             static_cast<cuuint64_t>(r.SH) * r.SW * r.C * esize};
    // anchors run over [low, low + (R - 1) * mul] in each axis: the box's far corner, relative to the image's
    int lower[2] = {r.low_x, r.low_y};
    int upper[2] = {r.low_x + (r.RW - 1) * r.mul_x - (r.SW - 1), r.low_y + (r.RH - 1) * r.mul_y - (r.SH - 1)};
    cuuint32_t estr[4] = {1u, static_cast<cuuint32_t>(r.mul_x), static_cast<cuuint32_t>(r.mul_y), 1u};
    CUresult rc = enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(o.ptr), dims,
                      strides, lower, upper, static_cast<cuuint32_t>(128 / esize), static_cast<cuuint32_t>(pixels), estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

// 4-D map {ce ci, oc, taps, ic / ce} over a filter [oc, taps, ic]: one box = box_k filters of one tap x `chunks` 128-byte
// slices of input channels, laid out chunk by chunk as an MN-major operand wants.
bool make_filter_tap_map(CUtensorMap* map, const HostOperand& o, int box_k, int chunks, int esize, bool atom32) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const long long ce = 128 / esize, ic = o.ld2, taps = o.ld / o.ld2, oc = o.rmod;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(ce), static_cast<cuuint64_t>(oc), static_cast<cuuint64_t>(taps), static_cast<cuuint64_t>(ic / ce)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(o.ld) * esize, static_cast<cuuint64_t>(ic) * esize, 128u};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(ce), static_cast<cuuint32_t>(box_k), 1u, static_cast<cuuint32_t>(chunks)};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult rc = enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(o.ptr), dims,
                      strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

// Maps over a tap sub-grid of a filter [oc, FH, FW, ic] (HostOperand::TapSubset), all strides in bytes.
//   K-major : {ic, nfx, nfy, oc}, box {ce, 1, 1, rows_tile}: rows_tile filters x one 128-byte channel slice of one tap
//   by tap  : {ce ci, oc, nfx, nfy, ic / ce}, box {ce, ce filters, 1, 1, chunks}
bool make_filter_sub_map(CUtensorMap* map, const HostOperand& o, int rows_tile, int esize, bool by_tap, bool atom32) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const HostOperand::TapSubset& t = o.sub;
    const cuuint64_t es = esize, ce = 128 / esize, ic = t.ic, oc = t.oc;
    const char* base = static_cast<const char*>(o.ptr) + (static_cast<size_t>(t.f0y) * t.FW + t.f0x) * ic * es;
    const cuuint64_t step_x = static_cast<cuuint64_t>(t.tx) * ic * es, step_y = static_cast<cuuint64_t>(t.ty) * t.FW * ic * es,
                     step_f = static_cast<cuuint64_t>(t.FH) * t.FW * ic * es;
    CUresult rc;
    const CUtensorMapDataType dt = esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapSwizzle sw = atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    if (!by_tap) {
        cuuint64_t dims[4] = {ic, static_cast<cuuint64_t>(t.nfx), static_cast<cuuint64_t>(t.nfy), oc};
        cuuint64_t strides[3] = {step_x, step_y, step_f};
        cuuint32_t box[4] = {static_cast<cuuint32_t>(ce), 1u, 1u, static_cast<cuuint32_t>(rows_tile)};
        cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
        rc = enc(map, dt, 4, const_cast<char*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        cuuint64_t dims[5] = {ce, oc, static_cast<cuuint64_t>(t.nfx), static_cast<cuuint64_t>(t.nfy), ic / ce};
        cuuint64_t strides[4] = {step_f, step_x, step_y, 128u};
        cuuint32_t box[5] = {static_cast<cuuint32_t>(ce), static_cast<cuuint32_t>(ce), 1u, 1u, static_cast<cuuint32_t>(rows_tile / ce)};
        cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
        rc = enc(map, dt, 5, const_cast<char*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    return rc == CUDA_SUCCESS;
}

// Patch map of a halo operand: the NHWC image as {C, W, H, images}, box {32 channels, halo_wp columns, halo_rows rows, 1}.
bool make_halo_map(CUtensorMap* map, const HostOperand& o, long long images, int esize) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const ConvRule& r = o.cr;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(r.C), static_cast<cuuint64_t>(r.SW), static_cast<cuuint64_t>(r.SH), static_cast<cuuint64_t>(images)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(r.C) * esize, static_cast<cuuint64_t>(r.SW) * r.C * esize,
                             static_cast<cuuint64_t>(r.SH) * r.SW * r.C * esize};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / esize), static_cast<cuuint32_t>(o.halo_wp), static_cast<cuuint32_t>(o.halo_rows), 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult rc = enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(o.ptr), dims, strides,
                      box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

// The halo form of a convolution-like contraction whose A operand is a virtual im2col matrix with unit stride between
// neighbouring rows (Conv2d forward and gradient of x at stride 1, the residue classes of a strided DeConv2d, ...), or false
// when it does not apply.  The rows of one image become its PADDED raster - halo_wp = RW + (tap span in x) columns per output
// row, so that a tap is a constant row shift - and the images become the batch; rows that stand for padding columns are
// computed and not stored (OutMap::valid_w).  fp32 only: the converter warps rebuild each tap's A rows from the patch.
constexpr int kHaloPatchBytes = 44 * 1024;  // GemmCfg::PATCH_BYTES
bool to_halo(const GemmProblem& g, GemmProblem* out) {
    if (g.a.halo || g.dtype != 1 || !g.a.is_virtual || g.a.mn || g.batch != 1 || g.kbatch != 1 || g.scatter_rows != 0 || g.out.cols_on || g.a.sub.on) return false;
    if (!env_int("D8K_HALO", 0)) return false;
    const ConvRule& r = g.a.cr;
    if (!r.unit_div || r.mul_y != 1 || r.mul_x != 1 || r.C % 32 != 0) return false;
    const long long plane = static_cast<long long>(r.RH) * r.RW;
    if (plane <= 0 || g.M % plane != 0) return false;
    const long long images = g.M / plane;
    const int span_x = (r.FW - 1) * (r.e_x < 0 ? -r.e_x : r.e_x), span_y = (r.FH - 1) * (r.e_y < 0 ? -r.e_y : r.e_y);
    const int wp = r.RW + span_x;
    // patch rows a tile can read: its 128 raster positions starting anywhere in a row, shifted by the farthest tap
    const long long reach = static_cast<long long>(wp - 1) + 127 + static_cast<long long>(span_y) * wp + span_x + 1;
    const long long rows = (reach + wp - 1) / wp;
    if (wp > 256 || rows > 256 || 128LL * wp * rows > kHaloPatchBytes) return false;
    if (g.out.rows_on && (g.out.RH != r.RH || g.out.RW != r.RW)) return false;
    if (static_cast<long long>(r.RH) * wp >= (1LL << 31) || images >= (1LL << 31)) return false;
    if (g.K != static_cast<long long>(r.FH) * r.FW * r.C) return false;
    GemmProblem h = g;
    h.batch = static_cast<int>(images);
    h.M = r.RH * wp;
    h.a.halo = 1;
    h.a.halo_wp = wp;
    h.a.halo_rows = static_cast<int>(rows);
    h.a.batch_count = static_cast<int>(images);
    OutMap& o = h.out;
    if (!o.rows_on) {  // rows are the pixels of the output itself
        o.rows_on = 1;
        o.OH = r.RH; o.OW = r.RW; o.sy = 1; o.sx = 1; o.ry = 0; o.rx = 0;
    }
    o.RH = r.RH;
    o.RW = wp;
    o.valid_w = r.RW;
    h.c_batch_stride = static_cast<long long>(o.OH) * o.OW * g.ldc;
    *out = h;
    return true;
}

GatherSrc to_gather(const HostOperand& o, int rows, int cols, int esize) {
    GatherSrc s;
    std::memset(&s, 0, sizeof(s));
    s.base = o.ptr;
    s.kind = o.is_virtual ? 1 : 0;
    s.rows = rows;
    s.cols = cols;
    s.rmod = o.rmod;
    s.f_rmod = make_fastdiv(o.rmod > 0 ? o.rmod : 1);
    s.ld = o.ld;
    s.ld2 = o.ld2;
    s.batch_stride = o.batch_stride;
    s.batch_count = o.batch_count > 0 ? o.batch_count : 1;
    s.cr = o.cr;
    const long long vec = 16 / esize;
    s.vec_ok = (reinterpret_cast<uintptr_t>(o.ptr) & 15) == 0 && o.ld % vec == 0 && o.ld2 % vec == 0 && o.batch_stride % vec == 0 &&
               (!o.is_virtual || o.cr.C % vec == 0);
    if (o.sub.on) {  // the producer decodes k = (j * nfx + i) * C + c (or * oc + co) with these
        s.cr.C = o.sub.ic;
        s.cr.FW = o.sub.nfx;
        s.cr.f_c = make_fastdiv(o.sub.ic);
        s.cr.f_fw = make_fastdiv(o.sub.nfx);
        s.rmod = o.rmod > 0 ? o.sub.oc : 0;
        s.f_rmod = make_fastdiv(o.sub.oc > 0 ? o.sub.oc : 1);
    }
    return s;
}

struct Plan {
    bool f32, tma, pair;
    int a_tma, b_tma;  // kTma* of each operand when tma
    int bn, bk, tiles_m, tiles_n, tiles, num_kb, total_kb, splits, kb_per_split;
    size_t scratch;
};

// An overwriting fp16 product with a long contraction goes to the paired kernel from a third of a wave of 256 x 256 tiles
// on (measured: 2048^3 forward 33.6 -> 27.4 us, 2048 x 4096 x 2048 57.4 -> 38.9, 1024 x 8192 x 4096 104.9 -> 63.5; accumulating
// products and shorter contractions of that size are faster on the single-CTA kernel and keep the half-wave threshold)
bool pair_early(const Ctx* ctx, const GemmProblem& g) {
    if (g.dtype != 0 || g.beta != 0 || g.epi != 0 || g.K < 2048 || g.kbatch != 1 || !env_int("D8K_PAIR_EARLY", 1)) return false;
    const long long tiles256 = static_cast<long long>(g.batch) * ((g.M + 255) / 256) * ((g.N + 255) / 256);
    return tiles256 * 3 >= ctx->num_sms && tiles256 * 2 < ctx->num_sms;
}

Plan make_plan(const Ctx* ctx, const GemmProblem& g, size_t scratch_limit) {
    Plan pl;
    pl.f32 = g.dtype == 1;
    int esize = pl.f32 ? 4 : 2;
    pl.a_tma = tma_mode(g.a, esize, g.M, g.K);
    pl.b_tma = tma_mode(g.b, esize, g.N, g.K);
    pl.tma = pl.a_tma >= 0 && pl.b_tma >= 0 && encode_tiled() != nullptr && !env_int("D8K_FORCE_GATHER", 0);
    if ((pl.a_tma > kTmaTiled || pl.b_tma > kTmaTiled) && !env_int("D8K_IM2COL", 1)) pl.tma = false;
    // fp32 behind TMA: an MN-major stored matrix arrives as one box of whole 32-element chunks
    if (pl.f32 && ((pl.a_tma == kTmaTiled && g.a.mn && g.M % 32 != 0) || (pl.b_tma == kTmaTiled && g.b.mn && g.N % 32 != 0) ||
                   !env_int("D8K_F32_TMA", 1)))
        pl.tma = false;
    if (pl.f32) pl.bn = 64;  // the 64-column fp32 kernels run two groups of helper warps (see GemmCfg::LOADER_GROUPS)
    else if (pl.tma) {
        pl.bn = g.N > 128 ? 256 : 128;
        // 256 columns only when such tiles alone give every SM one: a small problem prefers twice as many narrower tiles
        const long long tiles256 = static_cast<long long>(g.batch) * ((g.M + kBM - 1) / kBM) * ((g.N + 255) / 256);
        if (pl.bn == 256 && tiles256 < ctx->num_sms) pl.bn = 128;
        // ... unless the paired kernel takes the problem at a lower tile count (see below): it needs 256-column tiles
        if (pair_early(ctx, g)) pl.bn = 256;
    }
    else pl.bn = g.N > 64 ? 128 : 64;
    int forced_bn = env_int("D8K_BN", 0);
    if (forced_bn == 64 && !pl.tma) pl.bn = 64;
    if (forced_bn == 128 && !(pl.f32 && pl.tma)) pl.bn = 128;
    if (forced_bn == 256 && pl.tma) pl.bn = 256;
    pl.bk = 128 / esize;
    pl.tiles_m = (g.M + kBM - 1) / kBM;
    pl.tiles_n = (g.N + pl.bn - 1) / pl.bn;
    pl.tiles = g.batch * pl.tiles_m * pl.tiles_n;
    pl.num_kb = (g.K + pl.bk - 1) / pl.bk;
    pl.total_kb = pl.num_kb * g.kbatch;
    // split the contraction when the output alone cannot occupy half of the SMs
    int splits = 1;
    if (pl.tiles * 2 <= ctx->num_sms && pl.total_kb >= 8 && pl.tiles <= kMaxCounters) {
        splits = ctx->num_sms / pl.tiles;
        // a split costs about a dozen k-blocks' time (partial tiles, tickets, the reduction): at least 24 k-blocks per split
        // (measured: a 256 x 512 x 128 fp32 product ran in 22.5 us with 4 splits of 4 k-blocks, in 17.4 us unsplit; the filter
        // gradient of 64 x [128 x 256] * [256 x 256] in 50 us with 16 splits of 16 k-blocks, in 46 us with 8 to 12)
        if (splits > pl.total_kb / 24) splits = pl.total_kb / 24;
    }
    int forced = env_int("D8K_SPLITS", 0);
    if (forced <= 0) forced = g.force_splits;
    if (forced > 0 && pl.tiles <= kMaxCounters) splits = forced < pl.total_kb ? forced : pl.total_kb;
    size_t per_split = static_cast<size_t>(pl.tiles) * kBM * pl.bn * sizeof(float);
    if (splits > 1 && per_split * splits > scratch_limit) splits = static_cast<int>(scratch_limit / per_split);
    if (splits < 1) splits = 1;
    if (splits > 255) splits = 255;  // a tile's ticket word counts its splits in eight bits
    pl.kb_per_split = (pl.total_kb + splits - 1) / splits;
    pl.splits = (pl.total_kb + pl.kb_per_split - 1) / pl.kb_per_split;
    pl.scratch = pl.splits > 1 ? per_split * pl.splits : 0;
    // CTA pairs on 256 x 256 tiles once the output alone fills the machine (74 pairs) and nothing is split
    int tiles256 = g.batch * ((g.M + 255) / 256) * ((g.N + 255) / 256);
    pl.pair = pl.tma && pl.a_tma == kTmaTiled && pl.b_tma == kTmaTiled && !g.out.rows_on && !g.out.cols_on && pl.bn == 256 && pl.splits == 1 && (tiles256 * 2 >= ctx->num_sms || pair_early(ctx, g) || env_int("D8K_PAIR", 1) == 2) && env_int("D8K_PAIR", 1) != 0 &&
              g.K % 64 == 0 && (!g.a.mn || g.M % 64 == 0) && (!g.b.mn || g.N % 64 == 0);
    if (pl.pair) {
        pl.tiles_m = (g.M + 255) / 256;
        pl.tiles_n = (g.N + 255) / 256;
        pl.tiles = tiles256;
    }
    return pl;
}

// Tile order of the paired kernel, chosen to keep DRAM traffic down when the operands exceed the L2.
// A wave is the `pairs` tiles in flight together; all of them walk along K in step, so within a wave every distinct operand
// strip (256 rows x K) is fetched from DRAM once.  With groups of g tiles along one axis sweeping the other axis a wave
// touches about g + pairs / g strips.  If in addition the g strips of a group are small enough to stay in L2 while the
// group's sweeps stream past (loads marked evict-last), later waves of the group find them there, and the traffic drops to
// (resident operand once) + (number of groups) x (streamed operand).  The model below picks axis, g and residency by the
// bytes each choice would read.
struct Raster {
    int group, along_n, l2_a, l2_b;
};
Raster pick_raster(long long M, long long N, long long K, int tiles_m, int tiles_n, int pairs) {
    const double strip = 256.0 * static_cast<double>(K) * 2.0;
    const double a_total = static_cast<double>(M) * K * 2.0, b_total = static_cast<double>(N) * K * 2.0;
    const double budget = static_cast<double>(env_int("D8K_L2_RESIDENT_MB", 40)) * 1048576.0;
    Raster best = {16, 0, 0, 0};
    double best_cost = -1.0;
    for (int along_n = 0; along_n < 2; ++along_n) {
        const int along = along_n ? tiles_n : tiles_m;
        const double res_total = along_n ? b_total : a_total, str_total = along_n ? a_total : b_total;
        for (int g = 1; g <= along && g <= 32; ++g) {
            const int groups = (along + g - 1) / g;
            // strips of the group resident in L2 across its waves
            if (g * strip <= budget && env_int("D8K_L2_HINTS", 0)) {
                const double cost = res_total + groups * str_total;
                if (best_cost < 0 || cost < best_cost * 0.999) {
                    best_cost = cost;
                    best = {g, along_n, along_n ? 1 : 2, along_n ? 2 : 1};
                }
            }
            // no residency: every wave fetches the strips it touches (the last group may be narrower)
            const int across = along_n ? tiles_m : tiles_n;
            double cost = 0.0;
            for (int first = 0; first < along; first += g) {
                const int gi = along - first < g ? along - first : g;
                cost += static_cast<double>(gi) * across / pairs * (gi + static_cast<double>(pairs) / gi) * strip;
            }
            if (best_cost < 0 || cost < best_cost * 0.999) {
                best_cost = cost;
                best = {g, along_n, 0, 0};
            }
        }
    }
    if (!env_int("D8K_L2_STREAM_FIRST", 1)) {  // the streamed operand at normal priority instead of evict-first
        if (best.l2_a == 1) best.l2_a = 0;
        if (best.l2_b == 1) best.l2_b = 0;
    }
    return best;
}

}  // namespace

size_t gemm_scratch_need(const Ctx* ctx, const GemmProblem& g) {
    if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.batch <= 0) return 0;
    return make_plan(ctx, g, ~static_cast<size_t>(0)).scratch;
}

bool gemm_goes_through_tma(const Ctx* ctx, const GemmProblem& g) {
    Plan pl = make_plan(ctx, g, ~static_cast<size_t>(0));
    return pl.tma;
}

// The epoch of the context's next split launch: 1 .. 2^24 - 1, then round again.  At the wrap every ticket word is cleared once,
// so that a word written 2^24 launches ago cannot pass for a current one.
static int next_epoch(Ctx* ctx) {
    ctx->epoch_counter = (ctx->epoch_counter + 1) & 0xffffffu;
    if (ctx->epoch_counter == 0) {
        cudaMemsetAsync(ctx->counters, 0, static_cast<size_t>(kMaxCounters) * sizeof(int), ctx->stream);
        ctx->epoch_counter = 1;
    }
    return static_cast<int>(ctx->epoch_counter);
}

int run_gemm(Ctx* ctx, const GemmProblem& g, PreparedGemm* capture) {
    if (g.M < 0 || g.N < 0 || g.K < 0 || g.batch < 0 || g.kbatch < 1) return fail(1, "gemm: negative extent");
    if (g.M == 0 || g.N == 0 || g.batch == 0) return 0;
    if ((!g.C && g.scatter_rows == 0) || (g.K > 0 && (!g.a.ptr || !g.b.ptr))) return fail(1, "gemm: null pointer");
    if (g.dtype != 0 && g.dtype != 1) return fail(1, "gemm: dtype must be D8K_F16 or D8K_F32");
    if (g.beta != 0 && g.beta != 1) return fail(1, "gemm: beta must be 0 or 1");
    if (g.epi < 0 || g.epi > 4 || (g.epi >= 1 && !g.E1) || (g.epi == 2 && !g.E2)) return fail(1, "gemm: bad fused epilogue arguments");
    if (g.epi == 3 && (g.beta != 0 || g.scatter_rows != 0 || g.out.cols_on)) return fail(1, "gemm: the bias tail belongs to an overwriting forward product");
    const int esize = g.dtype == 1 ? 4 : 2;
    if (g.scatter_rows != 0) {
        if (g.scatter_rows < 0 || g.scatter_rows % 128 != 0) return fail(1, "gemm: scattered row blocks must be multiples of 128 rows");
        if (g.scatter_count < 1 || g.scatter_count > kMaxScatter || static_cast<long long>(g.scatter_count) * g.scatter_rows < g.M)
            return fail(1, "gemm: 1 to 16 row blocks that cover every output row");
        if (g.beta != 0 || g.epi != 0 || g.batch != 1 || g.K == 0) return fail(1, "gemm: a scattered output is overwritten, unbatched, without a fused tail");
        for (int k = 0; k < g.scatter_count; ++k)
            if (!g.scatter_base[k] || (reinterpret_cast<uintptr_t>(g.scatter_base[k]) & 15)) return fail(1, "gemm: null or unaligned row block");
    }
    if (g.K == 0) {  // an empty contraction is a zero matrix
        if (g.beta == 0) {
            for (int b = 0; b < g.batch; ++b) {
                char* c = static_cast<char*>(g.C) + static_cast<size_t>(b) * g.c_batch_stride * esize;
                cudaError_t e = cudaMemset2DAsync(c, g.ldc * esize, 0, static_cast<size_t>(g.N) * esize, g.M, ctx->stream);
                if (e != cudaSuccess) return fail(2, std::string("gemm: cudaMemset2DAsync: ") + cudaGetErrorString(e));
            }
        }
        return 0;
    }

    // a stride-1 virtual operand in fp32: per-tile patches instead of one fetch per filter tap, when the plan stays unsplit
    GemmProblem halo_problem;
    if (!capture && to_halo(g, &halo_problem)) {
        const Plan hp = make_plan(ctx, halo_problem, 0);
        if (hp.tma && hp.splits == 1 && hp.bn == 64 && hp.tiles * 2 > ctx->num_sms) return run_gemm(ctx, halo_problem);
    }
    // The caller's scratch (a node's interim buffer) is used when it holds everything the split plan wants; a buffer that is
    // missing, empty or smaller than that would silently cost splits, so the context's own scratch serves instead.
    bool own_scratch = g.ws == nullptr || g.ws_bytes == 0;
    if (!own_scratch && !g.ws_strict && g.ws_bytes < ctx->scratch_bytes && make_plan(ctx, g, ctx->scratch_bytes).scratch > g.ws_bytes) own_scratch = true;
    float* scratch = own_scratch ? ctx->scratch : static_cast<float*>(g.ws);
    size_t scratch_limit = own_scratch ? ctx->scratch_bytes : g.ws_bytes;
    if (reinterpret_cast<uintptr_t>(scratch) & 15) return fail(1, "gemm: scratch memory must be 16-byte aligned");
    Plan pl = make_plan(ctx, g, scratch_limit);
    if ((g.a.sub.on || g.b.sub.on) && !pl.tma) return fail(1, "gemm: a tap subset of a filter is only read through TMA");
    if (g.a.halo && (!pl.tma || pl.splits != 1 || pl.bn != 64)) return fail(2, "gemm: the halo form needs the unsplit fp32 TMA kernel");

    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.batch = g.batch;
    p.kbatch = g.kbatch;
    p.num_kb = pl.num_kb;
    p.splits = pl.splits;
    p.kb_per_split = pl.kb_per_split;
    p.tiles_m = pl.tiles_m;
    p.tiles_n = pl.tiles_n;
    p.raster_group = 16;
    if (pl.pair && g.batch == 1) {
        const Raster r = pick_raster(g.M, g.N, static_cast<long long>(g.K) * g.kbatch, pl.tiles_m, pl.tiles_n, ctx->num_sms / 2);
        p.raster_group = r.group;
        p.raster_n = r.along_n;
        p.l2_a = r.l2_a;
        p.l2_b = r.l2_b;
    }
    p.epi_backoff_ns = env_int("D8K_EPI_BACKOFF", 0);
    if (env_int("D8K_RASTER", 0) > 0) p.raster_group = env_int("D8K_RASTER", 0);
    if (env_int("D8K_RASTER_N", -1) >= 0) p.raster_n = env_int("D8K_RASTER_N", 0) ? 1 : 0;
    if (env_int("D8K_L2_A", -1) >= 0) p.l2_a = env_int("D8K_L2_A", 0);
    if (env_int("D8K_L2_B", -1) >= 0) p.l2_b = env_int("D8K_L2_B", 0);
    if (p.raster_group < 1) p.raster_group = 1;
    p.total_work = pl.tiles * pl.splits;
    p.beta = g.beta;
    p.epi = g.epi;
    p.epi_a = g.epi_a;
    p.epi_b = g.epi_b;
    p.beta2 = g.beta2;
    p.E1 = g.E1;
    p.E2 = g.E2;
    p.C = g.C;
    if (g.scatter_rows > 0) {  // offsets are relative to block 0, which stands in for C
        p.C = g.scatter_base[0];
        p.scatter_rows = g.scatter_rows;
        for (int k = 0; k < kMaxScatter; ++k) {
            const int kk = k < g.scatter_count ? k : g.scatter_count - 1;
            const long long bytes = static_cast<const char*>(g.scatter_base[kk]) - static_cast<const char*>(g.scatter_base[0]);
            p.scatter_off[k] = bytes / esize - static_cast<long long>(kk) * g.scatter_rows * g.ldc;
        }
    }
    p.out = g.out;
    if (p.out.rows_on) {
        p.out.f_plane = make_fastdiv(p.out.RH * p.out.RW);
        p.out.f_rw = make_fastdiv(p.out.RW);
    }
    if (p.out.cols_on) {
        p.out.f_c = make_fastdiv(p.out.C);
        p.out.f_nfx = make_fastdiv(p.out.NFX);
    }
    p.ldc = g.ldc;
    p.c_batch_stride = g.c_batch_stride;
    p.ws = scratch;
    p.counters = ctx->counters + g.ticket_base;
    p.status = ctx->status;
    if (const char* pp = std::getenv("D8K_PROF_PTR"))  // diagnostics: device address of 8 cycle counters per CTA (paired kernel)
        p.prof = reinterpret_cast<long long*>(static_cast<uintptr_t>(std::strtoull(pp, nullptr, 0)));
    p.a_batch_mod = g.a.batch_count > 0 ? g.a.batch_count : 1;
    p.b_batch_mod = g.b.batch_count > 0 ? g.b.batch_count : 1;

    CUtensorMap ta, tb;
    std::memset(&ta, 0, sizeof(ta));
    std::memset(&tb, 0, sizeof(tb));
    GemmLaunchFn fn = nullptr;
    bool dual = false;  // two CTAs per SM (fp32, A in tensor memory)
    bool twin = false;  // one CTA per SM with twin TMA and MMA threads
    if (pl.pair) {
        if (!make_pair_map(&ta, g.a, g.M, g.K) || !make_pair_map(&tb, g.b, g.N, g.K)) return fail(2, "gemm: cuTensorMapEncodeTiled (4-D) failed");
        fn = lookup_f16_pair(g.a.mn, g.b.mn);
    } else if (pl.tma) {
        // one map per operand, by producer mode; fp32 MN-major operands use the 32-byte-atom swizzle; the raw fp32 tiles
        // are the hi images and converter warps add the lo images
        const int ce = 128 / esize;
        p.a_tma = pl.a_tma;
        p.b_tma = pl.b_tma;
        p.a = g.a.mn ? to_gather(g.a, g.K, g.M, esize) : to_gather(g.a, g.M, g.K, esize);
        p.b = g.b.mn ? to_gather(g.b, g.K, g.N, esize) : to_gather(g.b, g.N, g.K, esize);
        auto build = [&](CUtensorMap* map, const HostOperand& o, int mode, long long extent, int rows_tile, int* chunked) -> bool {
            const bool atom32 = pl.f32 && o.mn;
            if (mode == kTmaHalo) return make_halo_map(map, o, g.batch, esize);
            if (mode == kTmaIm2col) return make_im2col_map(map, o, extent, rows_tile, esize, atom32);
            if (mode == kTmaIm2colMN) return make_im2col_map(map, o, g.K, ce, esize, atom32);
            if (mode == kTmaFilterTap) return make_filter_tap_map(map, o, ce, rows_tile / ce, esize, atom32);
            if (mode == kTmaFilterSub) return make_filter_sub_map(map, o, rows_tile, esize, false, atom32);
            if (mode == kTmaFilterTapSub) return make_filter_sub_map(map, o, rows_tile, esize, true, atom32);
            if (!o.mn) return make_map(map, o, g.K, extent, rows_tile, esize);
            *chunked = (pl.f32 || extent % ce == 0) && env_int("D8K_CHUNKED", 1);
            if (pl.f32 && !*chunked) return false;
            return *chunked ? make_pair_map(map, o, extent, g.K, ce, rows_tile / ce, esize, atom32) : make_map(map, o, extent, g.K, ce, esize);
        };
        if (!build(&ta, g.a, pl.a_tma, g.M, kBM, &p.a_chunked) || !build(&tb, g.b, pl.b_tma, g.N, pl.bn, &p.b_chunked))
            return fail(2, "gemm: cuTensorMapEncode failed");
        fn = pl.f32 ? lookup_f32_tma(g.a.mn, g.b.mn, pl.bn, env_int("D8K_F32_ATMEM", 1) != 0) : lookup_f16_tma(g.a.mn, g.b.mn, pl.bn);
        // fp16 single-CTA kernels: twin TMA-issuing and MMA-issuing threads (GemmCfg::TWIN) - same bits, never slower and up
        // to 20 % faster on the measured shapes; D8K_F16_TWIN=0 keeps one thread each
        if (!pl.f32 && env_int("D8K_F16_TWIN", 1)) {
            fn = lookup_f16_twin(g.a.mn, g.b.mn, pl.bn);
            twin = true;
        }
        if (pl.f32 && pl.bn == 64 && !g.a.halo && env_int("D8K_F32_ATMEM", 1)) {
            // Two CTAs per SM (GemmCfg::DUAL) when there is more than one tile per SM and no split: the second CTA's MMAs fill
            // the tensor pipe while the first one's single-thread roles go round their barriers.  Mode 2 (three stages, A's hi
            // image read from shared memory) wins on long accumulation loops, mode 1 (A entirely in tensor memory) on short
            // ones.  With a split, or with fewer work items than SMs, a CTA is alone on its SM anyway: there the one-CTA kernel
            // with twin TMA and MMA threads runs (mode 4, GemmCfg::TWIN; never slower than the single-thread roles of mode 0
            // on twenty-seven measured shapes, up to 20 % faster).  D8K_F32_DUAL = 0 / 1 / 2 / 4 overrides.
            int mode = env_int("D8K_F32_DUAL", -1);
            if (mode < 0) mode = (pl.splits == 1 && p.total_work > ctx->num_sms) ? (pl.total_kb > 8 ? 2 : 1) : 4;
            if (mode == 1 || mode == 2) {
                fn = lookup_f32_dual(g.a.mn, g.b.mn, mode);
                dual = true;
            } else if (mode == 4) {
                fn = lookup_f32_dual(g.a.mn, g.b.mn, mode);
                twin = true;
            }
        }
        if (g.a.halo) {
            fn = lookup_f32_halo(g.b.mn);
            p.halo_wp = g.a.halo_wp;
            p.halo_taps = g.a.cr.FH * g.a.cr.FW;
            p.halo_slices = g.a.cr.C / ce;
            p.halo_bytes = 128 * g.a.halo_wp * g.a.halo_rows;
        }
    } else {
        p.a = g.a.mn ? to_gather(g.a, g.K, g.M, esize) : to_gather(g.a, g.M, g.K, esize);
        p.b = g.b.mn ? to_gather(g.b, g.K, g.N, esize) : to_gather(g.b, g.N, g.K, esize);
        fn = pl.f32 ? lookup_f32_gather(g.a.mn, g.b.mn, pl.bn) : lookup_f16_gather(g.a.mn, g.b.mn, pl.bn);
    }
    if (!fn) return fail(2, "gemm: no kernel for this configuration");
    int grid = p.total_work < ctx->num_sms ? p.total_work : ctx->num_sms;
    if (dual) grid = p.total_work < 2 * ctx->num_sms ? p.total_work : 2 * ctx->num_sms;
    if (pl.pair) grid = p.total_work < ctx->num_sms / 2 ? p.total_work : ctx->num_sms / 2;  // pairs
    std::string text;
    {
        static const char* const kModes[] = {"tiled", "im2col", "im2col-mn", "filter-tap", "filter-sub", "filter-tap-sub", "halo"};
        std::ostringstream os;
        os << (pl.f32 ? "f32 " : "f16 ") << (pl.pair ? "pair" : pl.tma ? "tma" : "gather");
        if (pl.tma && !pl.pair) os << " a=" << kModes[pl.a_tma] << " b=" << kModes[pl.b_tma];
        os << " bn=" << (pl.pair ? 256 : pl.bn) << " splits=" << pl.splits << " grid=" << grid;
        if (dual) os << " dual";
        if (twin) os << " twin";
        if (pl.pair) os << " raster=" << (p.raster_n ? "n" : "m") << p.raster_group << " l2=" << p.l2_a << p.l2_b;
        text = os.str();
    }
    if (capture) {
        capture->p = p;
        capture->ta = ta;
        capture->tb = tb;
        capture->fn = fn;
        capture->grid = grid;
        capture->tiles = pl.tiles;
        capture->splits = pl.splits;
        capture->total_kb = pl.total_kb;
        capture->pair = pl.pair;
        capture->dual = dual;
        capture->halo = g.a.halo != 0;
        capture->twin = twin;
        capture->f32 = pl.f32;
        capture->a_mn = g.a.mn;
        capture->b_mn = g.b.mn;
        capture->bn = pl.bn;
        capture->text = text;
        return 0;
    }
    if (pl.splits > 1) p.epoch = next_epoch(ctx);
    cudaError_t e = fn(grid, ctx->stream, ta, tb, p);
    if (e != cudaSuccess) return fail(2, std::string("gemm: launch failed: ") + cudaGetErrorString(e));
    count_launch();
    set_last_kernel(text);
    return 0;
}

int run_gemm_group(Ctx* ctx, std::vector<GemmProblem>& parts) {
    const int n = static_cast<int>(parts.size());
    if (n == 0) return 0;
    bool grouped = ctx->group_buf != nullptr && n >= 2 && n <= kMaxGroups && env_int("D8K_GROUP", 1);
    std::vector<PreparedGemm> prep(grouped ? n : 0);
    int tickets = 0;
    int group_splits = 0;
    if (grouped) {
        // Splits are chosen for the group as a whole: the parts' tiles together are what has to fill the SMs.  (Each part
        // planning for itself split four times too often: configuration 4's filter gradient took 114 us with 9 splits
        // per class and takes 56 with 2.)
        long long all_tiles = 0;
        int min_kb = 0;
        for (int i = 0; i < n && grouped; ++i) {
            PreparedGemm probe;
            if (parts[i].M <= 0 || parts[i].N <= 0 || parts[i].K <= 0 || parts[i].batch <= 0) grouped = false;
            else if (int rc = run_gemm(ctx, parts[i], &probe)) return rc;
            else {
                all_tiles += probe.tiles;
                if (min_kb == 0 || probe.total_kb < min_kb) min_kb = probe.total_kb;
            }
        }
        group_splits = (all_tiles > 0 && all_tiles * 2 <= ctx->num_sms) ? static_cast<int>(ctx->num_sms / all_tiles) : 1;
        if (group_splits > min_kb / 24) group_splits = min_kb / 24;  // at least 24 k-blocks per split, as in a single launch's plan
        if (group_splits < 1) group_splits = 1;
    }
    if (grouped) {
        // every contraction gets its own part of the context's scratch memory and its own range of tickets
        const size_t region = (ctx->scratch_bytes / n) & ~static_cast<size_t>(255);
        for (int i = 0; i < n && grouped; ++i) {
            GemmProblem g = parts[i];
            g.ws = reinterpret_cast<char*>(ctx->scratch) + static_cast<size_t>(i) * region;
            g.ws_bytes = region;
            g.ws_strict = true;
            g.ticket_base = tickets;
            g.force_splits = group_splits;
            if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.batch <= 0) grouped = false;  // degenerate parts keep run_gemm's own handling
            else if (int rc = run_gemm(ctx, g, &prep[i])) return rc;
            if (!grouped) break;
            tickets += prep[i].tiles;
            // one launch needs one kernel: the same instantiation for every part, one CTA per SM
            if (prep[i].pair || prep[i].dual || prep[i].halo || !prep[i].twin || prep[i].fn != prep[0].fn || tickets > kMaxCounters) grouped = false;
        }
    }
    if (!grouped) {
        for (GemmProblem& g : parts)
            if (int rc = run_gemm(ctx, g)) return rc;
        return 0;
    }
    std::vector<GroupEntry> entries(n);
    int total = 0;
    for (int i = 0; i < n; ++i) {
        std::memset(&entries[i], 0, sizeof(GroupEntry));
        entries[i].ta = prep[i].ta;
        entries[i].tb = prep[i].tb;
        entries[i].p = prep[i].p;
        entries[i].first_work = total;
        total += prep[i].p.total_work;
    }
    cudaError_t e = cudaMemcpyAsync(ctx->group_buf, entries.data(), sizeof(GroupEntry) * n, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) return fail(2, std::string("gemm: preparing a grouped launch: ") + cudaGetErrorString(e));
    GemmParams launch = prep[0].p;
    launch.epoch = next_epoch(ctx);
    launch.group_count = n;
    launch.groups = ctx->group_buf;
    launch.total_work = total;
    const int grid = total < ctx->num_sms ? total : ctx->num_sms;
    const GemmLaunchFn fn = prep[0].f32 ? lookup_f32_dual(prep[0].a_mn, prep[0].b_mn, 5) : lookup_f16_grouped(prep[0].a_mn, prep[0].b_mn, prep[0].bn);
    if (!fn) return fail(2, "gemm: no grouped kernel for this configuration");
    e = fn(grid, ctx->stream, prep[0].ta, prep[0].tb, launch);
    if (e != cudaSuccess) return fail(2, std::string("gemm: launch failed: ") + cudaGetErrorString(e));
    count_launch();
    set_last_kernel(prep[0].text + " grouped x" + std::to_string(n) + " grid=" + std::to_string(grid));
    return 0;
}

}  // namespace d8k
