// The paired-CTA variant of the TMA-fed fp16 contraction kernel: two CTAs of a cluster work on one 256 x 256 output
// tile with tcgen05.mma.cta_group::2.
//
// Why: a lone CTA on a 128 x 256 tile stages 48 KB of operands per k-block of 64 (94 bytes per SM clock at full
// tensor rate) and only four stages fit in shared memory; measured, the tensor pipe then waits on operand delivery
// 43 % of the time.  In a pair, CTA r stages rows [128 r, 128 r + 128) of the A tile and rows [128 r, 128 r + 128) of the
// B tile (N side) - 32 KB per k-block - and the pair's MMA reads both halves of B from both CTAs' shared memory, so each
// SM moves two thirds of the bytes.
//
// Protocol (all barriers live at the same shared-memory offsets in both CTAs; "leader" = cluster rank 0):
//   full[s]    leader only, count 1: the leader's producer arrives with expect_tx = both CTAs' bytes; both CTAs' TMA
//              loads (cp.async.bulk.tensor ... cta_group::2) complete their bytes on the leader's barrier.
//   empty[s]   both CTAs, count 1: tcgen05.commit.cta_group::2 from the leader's MMA thread, sent to both CTAs.
//   tfull[a]   both CTAs, count 1: same commit form once a tile's last MMA is issued; each CTA's epilogue warps then
//              read their own 128 accumulator rows from their own tensor memory.
//   tempty[a]  leader only, count 2 x 128: every epilogue thread of both CTAs arrives (the peer's remotely).
// Epilogue: accumulator rows leave tensor memory one thread per row; each warp transposes its 32 x 32 chunk through a
// private shared-memory slot so that global memory sees whole 64-byte row segments (and reads C, ReLu's input and its
// gradient the same way when beta or a fused tail needs them).
// One TMA instruction per operand per stage: measured on B200, a CTA's TMA unit retires about two tile loads per 260 ns
// whatever their size (16 KB or 32 KB), so a stage holds SUB = 2 k-blocks of 64 and each operand arrives as ONE 32 KB box
// of a 4-D tensor map {64 elements, rows, k-blocks (or 64-element chunks), batch}; with 16 KB boxes (one k-block per
// stage) the tensor pipe waited on operand delivery a third of the time.
// No load uses multicast.  Every wait is bounded as in the single-CTA kernel; the two cluster barriers (after set-up,
// before tensor memory is freed) are reached by every thread on every path.
#pragma once
#include "gemm_kernel.cuh"

namespace d8k {

template <bool A_MN_, bool B_MN_, int STAGES_, int SUB_ = 2>
struct Gemm2Cfg {
    static constexpr bool A_MN = A_MN_, B_MN = B_MN_;
    static constexpr int STAGES = STAGES_;
    static constexpr int SUB = SUB_;             // k-blocks of 64 per stage
    static constexpr int BM = 256, BN = 256;     // tile of the pair
    static constexpr int HALF_N = BN / 2;        // B rows staged by one CTA
    static constexpr int CE = 64, BK = 64 * SUB, UMMA_K = 16, KSTEPS = BK / UMMA_K;
    static constexpr int A_BYTES = 128 * 128 * SUB;    // this CTA's 128 rows of A, SUB k-blocks
    static constexpr int B_BYTES = HALF_N * 128 * SUB;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // per CTA
    static constexpr int TMEM_COLS = 512;        // two accumulator buffers of 256 columns
    static constexpr int EPI_WARPS = 4, PRODUCER_WARP = 4, MMA_WARP = 5;
    static constexpr int THREADS = 32 * 6;
    static constexpr int BAR_BYTES = 256;
    // epilogue staging: per epilogue warp three slots (C, E1, E2) of 32 rows x 64 bytes (32 fp16 columns)
    static constexpr int SLOT_BYTES = 32 * 64, STAGING_BYTES = EPI_WARPS * 3 * SLOT_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + STAGING_BYTES + 1024;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
    static_assert(SMEM_BYTES > 114 * 1024, "one CTA per SM");
};

namespace ptx {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load into this CTA's shared memory whose byte count completes on an mbarrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster_addr, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster_addr, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// the same load with an L2 eviction priority (createpolicy value)
__device__ __forceinline__ void tma_load_4d_pair_hint(uint32_t dst, const void* tmap, uint32_t bar_cluster_addr, int c0, int c1, int c2, int c3,
                                                      uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        ::"r"(dst), "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
        : "memory");
}
// L2 eviction priority for loads: 0 normal, 1 evict first, 2 evict last
__device__ __forceinline__ uint64_t l2_policy(int kind) {
    uint64_t pol;
    if (kind == 2) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    else if (kind == 1) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    else asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at this shared-memory offset in every CTA of `mask` once the pair's MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(mask)
                 : "memory");
}


}  // namespace ptx

// 16-byte chunk c16 (0..3) of row r (0..31) inside a staging slot of 64-byte rows: the chunk index is XORed with bits of
// the row so that both access patterns of the epilogue - one thread per row, and four threads per row over eight rows -
// touch every bank group once.
__device__ __forceinline__ uint32_t slot_off(int r, int c16) { return static_cast<uint32_t>(r * 64 + ((c16 ^ ((r >> 1) & 3)) << 4)); }

struct PairWork {
    int batch, m0, n0;
};

__device__ __forceinline__ PairWork decode_pair_work(const GemmParams& p, int w) {
    PairWork it;
    int tpb = p.tiles_m * p.tiles_n;
    it.batch = w / tpb;
    int t = w - it.batch * tpb;
    // groups of `raster_group` tiles along one axis sweep the whole other axis, fastest along the grouped axis
    const int along = p.raster_n ? p.tiles_n : p.tiles_m, across = p.raster_n ? p.tiles_m : p.tiles_n;
    int group_size = p.raster_group * across;
    int gid = t / group_size;
    int first = gid * p.raster_group;
    int g = min(along - first, p.raster_group);
    int in_group = t - gid * group_size;
    int sweep = in_group / g;
    int pos = first + (in_group - sweep * g);
    it.m0 = (p.raster_n ? sweep : pos) * 256;
    it.n0 = (p.raster_n ? pos : sweep) * 256;
    return it;
}

// p.tiles_m counts 256-row tiles here, p.total_work = batch * tiles_m * tiles_n, p.splits == 1; the grid is 2 x (pairs).
template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::THREADS, 1)
d8k_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
    constexpr int STAGES = Cfg::STAGES, BK = Cfg::BK;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
    static_assert(8 * (2 * Cfg::STAGES + 4) + 8 <= Cfg::BAR_BYTES, "barrier block");

    __shared__ volatile int s_abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(tfull_bar(a), 1);
            ptx::mbar_init(tempty_bar(a), 2 * 32 * Cfg::EPI_WARPS);
        }
        ptx::fence_mbar_init();
    }
    if (warp == Cfg::MMA_WARP) {
        ptx::tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    if (warp == Cfg::PRODUCER_WARP && lane == 0) {
        ptx::tma_prefetch_desc(&tmA);
        ptx::tma_prefetch_desc(&tmB);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive();  // the peer's barriers are initialised before anything is sent to them
    ptx::cluster_wait();
    ptx::tc_fence_after_sync();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    auto stage_a = [&](int s) { return smem_base + s * Cfg::STAGE_BYTES; };
    auto stage_b = [&](int s) { return smem_base + s * Cfg::STAGE_BYTES + Cfg::A_BYTES; };
    const int its_per_batch = (p.num_kb + Cfg::SUB - 1) / Cfg::SUB;  // stages per batch entry of the contraction
    const int total_it = p.kbatch * its_per_batch;

    if (warp == Cfg::PRODUCER_WARP) {
        // ============================================================================ TMA producer (both CTAs)
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        long long waited = 0;
        const long long t_begin = p.prof ? clock64() : 0;
        const bool hinted = (p.l2_a | p.l2_b) != 0;
        const uint64_t pol_a = ptx::l2_policy(p.l2_a), pol_b = ptx::l2_policy(p.l2_b);
        for (int w = pair; ok && w < p.total_work; w += num_pairs) {
            PairWork it = decode_pair_work(p, w);
            const int my_m0 = it.m0 + 128 * static_cast<int>(rank);
            const int my_n0 = it.n0 + Cfg::HALF_N * static_cast<int>(rank);
            for (int kk = 0; kk < total_it; ++kk) {
                const long long tw = p.prof ? clock64() : 0;
                ok = wait_bar(empty_bar(stage), phase ^ 1, &s_abort, p.status, (kRoleProducer << 8) | 1);
                if (!ok) break;
                if (p.prof) waited += clock64() - tw;
                if (lane == 0) {
                    int b = it.batch, ki = kk;
                    if (p.kbatch > 1) {
                        b = kk / its_per_batch;
                        ki = kk - b * its_per_batch;
                    }
                    const int kb0 = ki * Cfg::SUB;  // first k-block of 64 of this stage
                    const uint32_t bar = ptx::map_to_rank(full_bar(stage), 0);
                    if (leader) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * Cfg::STAGE_BYTES);
                    // K-major: {k in block, row, k-block, batch}; MN-major: {m/n in chunk, k, chunk of 64, batch}
                    const int a1 = Cfg::A_MN ? kb0 * 64 : my_m0, a2 = Cfg::A_MN ? my_m0 / 64 : kb0;
                    const int b1 = Cfg::B_MN ? kb0 * 64 : my_n0, b2 = Cfg::B_MN ? my_n0 / 64 : kb0;
                    if (hinted) {
                        ptx::tma_load_4d_pair_hint(stage_a(stage), &tmA, bar, 0, a1, a2, b % p.a_batch_mod, pol_a);
                        ptx::tma_load_4d_pair_hint(stage_b(stage), &tmB, bar, 0, b1, b2, b % p.b_batch_mod, pol_b);
                    } else {
                        ptx::tma_load_4d_pair(stage_a(stage), &tmA, bar, 0, a1, a2, b % p.a_batch_mod);
                        ptx::tma_load_4d_pair(stage_b(stage), &tmB, bar, 0, b1, b2, b % p.b_batch_mod);
                    }
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (p.prof && lane == 0) {
            p.prof[blockIdx.x * 8 + 0] = clock64() - t_begin;
            p.prof[blockIdx.x * 8 + 1] = waited;
        }
    } else if (warp == Cfg::MMA_WARP) {
        // ============================================================================ MMA issuer (leader CTA only)
        if (leader) {
            constexpr uint32_t idesc = ptx::make_idesc(0u, Cfg::A_MN, Cfg::B_MN, 256, 256);
            // K-major: k-block j of the stage is a 16 KB tile at j * 16 KB, a k-step is 32 bytes inside its swizzled rows.
            // MN-major: a 64-wide chunk holds BK k-rows of 128 bytes (chunk stride = LBO), a k-step is 16 rows.
            auto a_off = [](int s) -> uint32_t { return Cfg::A_MN ? s * Cfg::UMMA_K * 128 : (s >> 2) * (128 * 128) + (s & 3) * 32; };
            auto b_off = [](int s) -> uint32_t { return Cfg::B_MN ? s * Cfg::UMMA_K * 128 : (s >> 2) * (Cfg::HALF_N * 128) + (s & 3) * 32; };
            constexpr uint32_t a_lbo = Cfg::A_MN ? BK * 128 : 16;
            constexpr uint32_t b_lbo = Cfg::B_MN ? BK * 128 : 16;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            long long waited_full = 0, waited_tmem = 0;
            const long long t_begin = p.prof ? clock64() : 0;
            for (int w = pair; ok && w < p.total_work; w += num_pairs) {
                const long long tt = p.prof ? clock64() : 0;
                ok = wait_bar(tempty_bar(acc), acc_phase ^ 1, &s_abort, p.status, (kRoleMma << 8) | 2);
                if (!ok) break;
                if (p.prof) waited_tmem += clock64() - tt;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * 256;
                for (int kk = 0; kk < total_it; ++kk) {
                    const long long tw = p.prof ? clock64() : 0;
                    ok = wait_bar(full_bar(stage), phase, &s_abort, p.status, (kRoleMma << 8) | 1);
                    if (!ok) break;
                    if (p.prof) waited_full += clock64() - tw;
                    ptx::tc_fence_after_sync();
                    if (lane == 0) {
#pragma unroll
                        for (int s = 0; s < Cfg::KSTEPS; ++s) {
                            uint64_t da = ptx::smem_desc(stage_a(stage) + a_off(s), a_lbo, 1024, ptx::kLayoutSw128);
                            uint64_t db = ptx::smem_desc(stage_b(stage) + b_off(s), b_lbo, 1024, ptx::kLayoutSw128);
                            ptx::mma_f16_pair(d_tmem, da, db, idesc, (kk > 0 || s > 0) ? 1u : 0u);
                        }
                        ptx::tc_commit_pair(empty_bar(stage), 3);
                        if (kk + 1 == total_it) ptx::tc_commit_pair(tfull_bar(acc), 3);
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
            if (p.prof && lane == 0) {
                p.prof[blockIdx.x * 8 + 2] = clock64() - t_begin;
                p.prof[blockIdx.x * 8 + 3] = waited_full;
                p.prof[blockIdx.x * 8 + 4] = waited_tmem;
            }
        }
    } else if (warp < Cfg::EPI_WARPS) {
        // ============================================================================ epilogue (both CTAs, own rows)
        using OutT = __half;
        const int quarter = warp;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t tempty_leader0 = ptx::map_to_rank(tempty_bar(0), 0);
        const uint32_t tempty_leader1 = ptx::map_to_rank(tempty_bar(1), 0);
        const uint32_t staging = bar_base + Cfg::BAR_BYTES + warp * (3 * Cfg::SLOT_BYTES);
        // whole 16-byte pieces everywhere: bases, pitch and batch stride multiples of 8 elements
        const bool coalesced = ((reinterpret_cast<uintptr_t>(p.C) | (p.epi ? reinterpret_cast<uintptr_t>(p.E1) : 0) |
                                 (p.epi == 2 ? reinterpret_cast<uintptr_t>(p.E2) : 0)) & 15) == 0 &&
                               (p.ldc & 7) == 0 && (p.c_batch_stride & 7) == 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        long long waited = 0;
        const long long t_begin = p.prof ? clock64() : 0;
        for (int w = pair; ok && w < p.total_work; w += num_pairs) {
            PairWork it = decode_pair_work(p, w);
            const int row = it.m0 + 128 * static_cast<int>(rank) + row_in_tile;
            const long long crow = static_cast<long long>(it.batch) * p.c_batch_stride + static_cast<long long>(row) * p.ldc + scatter_offset(p, row);
            const int warp_row0 = it.m0 + 128 * static_cast<int>(rank) + quarter * 32;  // first row of this warp
            const long long warp_off = static_cast<long long>(it.batch) * p.c_batch_stride + static_cast<long long>(warp_row0) * p.ldc +
                                       scatter_offset(p, warp_row0);
            const int lr = lane >> 2, lc = lane & 3;  // coalesced pattern: row 8 i + lr, 16-byte chunk lc
            // ReLu's input for the fused gradient tail is read once, from DRAM: the loads of a 32-column chunk are issued
            // one chunk ahead (the first before the accumulator is even finished), so their latency overlaps the previous
            // chunk's work instead of adding to every chunk - with four epilogue warps per CTA that latency, serialised,
            // made the epilogue longer than a short-K tile's main loop.
            // The old values of an accumulating store (beta) travel the same way: without it a 256 x 256 tile's read-modify-write
            // took longer than a K = 1024 main loop (dY += X^T dZ with 8192 x 4096 outputs ran at 384 TFLOP/s).
            uint4 pre[4] = {}, pre_c[4] = {};
            const bool prefetch = coalesced && p.epi == 2, prefetch_c = coalesced && p.beta != 0;
            auto issue_e1 = [&](int c) {
                const int pc0 = it.n0 + c * 32;
                if (!prefetch || pc0 + 32 > p.N) return;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = 8 * i + lr;
                    if (warp_row0 + rr < p.M)
                        pre[i] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const OutT*>(p.E1) + warp_off + static_cast<long long>(rr) * p.ldc +
                                                                       pc0 + lc * 8));
                }
            };
            auto issue_c = [&](int c) {
                const int pc0 = it.n0 + c * 32;
                if (!prefetch_c || pc0 + 32 > p.N) return;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = 8 * i + lr;
                    if (warp_row0 + rr < p.M)
                        pre_c[i] = *reinterpret_cast<const uint4*>(reinterpret_cast<const OutT*>(p.C) + warp_off + static_cast<long long>(rr) * p.ldc + pc0 +
                                                                   lc * 8);
                }
            };
            issue_c(0);
            issue_e1(0);
            const long long tw = p.prof ? clock64() : 0;
            ok = wait_bar(tfull_bar(acc), acc_phase, &s_abort, p.status, (kRoleEpilogue << 8) | 3, static_cast<unsigned>(p.epi_backoff_ns));
            if (!ok) break;
            if (p.prof) waited += clock64() - tw;
            ptx::tc_fence_after_sync();
            const uint32_t taddr = tmem_base + acc * 256 + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < 256 / 32; ++c) {
                uint32_t r[32];
                __syncwarp();
                ptx::tmem_ld_32x32(taddr + c * 32, r);
                ptx::tmem_ld_wait();
                const int col0 = it.n0 + c * 32;
                if (col0 >= p.N) continue;
                if (coalesced && col0 + 32 <= p.N) {
                    // Rows leave as whole 64-byte segments: the values cross from "one thread per row" (the tensor
                    // memory layout) to "four threads per row" through this warp's private staging slots.
                    const uint32_t s0 = staging + 0 * Cfg::SLOT_BYTES, s1 = staging + 1 * Cfg::SLOT_BYTES, s2 = staging + 2 * Cfg::SLOT_BYTES;
                    if (p.beta || p.epi == 2) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rr = 8 * i + lr;
                            if (warp_row0 + rr < p.M) {
                                const long long e = warp_off + static_cast<long long>(rr) * p.ldc + col0 + lc * 8;
                                if (p.beta) st_shared_v4(s0 + slot_off(rr, lc), pre_c[i]);
                                if (p.epi == 2) {
                                    st_shared_v4(s1 + slot_off(rr, lc), pre[i]);
                                    if (p.beta2) st_shared_v4(s2 + slot_off(rr, lc), *reinterpret_cast<const uint4*>(reinterpret_cast<const OutT*>(p.E2) + e));
                                }
                            }
                        }
                        if (c + 1 < 256 / 32) {
                            issue_e1(c + 1);
                            issue_c(c + 1);
                        }
                        __syncwarp();
                    }
                    using V = EpiVec<OutT>;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {  // this thread's row, eight columns at a time
                        float cv[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) cv[i] = __uint_as_float(r[v * 8 + i]);
                        if (p.beta) {
                            float old[8];
                            V::unpack(ptx::ld_shared_v4(s0 + slot_off(lane, v)), old);
#pragma unroll
                            for (int i = 0; i < 8; ++i) cv[i] += old[i];
                        }
                        uint4 cw = V::pack(cv);
                        if (p.epi == 3) {  // + bias row, after the product's own rounding (MatrixMultiply then Add)
                            float b[8];
                            V::unpack(cw, cv);
                            V::unpack(__ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const OutT*>(p.E1) + col0) + v), b);
#pragma unroll
                            for (int i = 0; i < 8; ++i) cv[i] += b[i];
                            cw = V::pack(cv);
                        }
                        st_shared_v4(s0 + slot_off(lane, v), cw);
                        if (p.epi == 1 || p.epi == 2 || p.epi == 4) V::unpack(cw, cv);  // the stored (rounded) values drive the fused tails
                        if (p.epi == 1) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) cv[i] = cv[i] > 0.f ? cv[i] : 0.f;
                            st_shared_v4(s1 + slot_off(lane, v), V::pack(cv));
                        } else if (p.epi == 4) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) cv[i] = epi_linear<OutT>(cv[i], p.epi_a, p.epi_b);
                            st_shared_v4(s1 + slot_off(lane, v), V::pack(cv));
                        } else if (p.epi == 2) {
                            float x[8], g[8];
                            V::unpack(ptx::ld_shared_v4(s1 + slot_off(lane, v)), x);
                            if (p.beta2) {
                                V::unpack(ptx::ld_shared_v4(s2 + slot_off(lane, v)), g);
                            } else {
#pragma unroll
                                for (int i = 0; i < 8; ++i) g[i] = 0.f;
                            }
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if (x[i] > 0.f) g[i] += cv[i];
                            st_shared_v4(s2 + slot_off(lane, v), V::pack(g));
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int rr = 8 * i + lr;
                        if (warp_row0 + rr < p.M) {
                            const long long e = warp_off + static_cast<long long>(rr) * p.ldc + col0 + lc * 8;
                            *reinterpret_cast<uint4*>(reinterpret_cast<OutT*>(p.C) + e) = ptx::ld_shared_v4(s0 + slot_off(rr, lc));
                            if (p.epi == 1 || p.epi == 4) *reinterpret_cast<uint4*>(reinterpret_cast<OutT*>(p.E1) + e) = ptx::ld_shared_v4(s1 + slot_off(rr, lc));
                            if (p.epi == 2) *reinterpret_cast<uint4*>(reinterpret_cast<OutT*>(p.E2) + e) = ptx::ld_shared_v4(s2 + slot_off(rr, lc));
                        }
                    }
                } else if (row < p.M) {
                    float accv[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) accv[i] = __uint_as_float(r[i]);
                    store_row_chunk<OutT>(p, crow, col0, accv);
                }
            }
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive_cluster(acc == 0 ? tempty_leader0 : tempty_leader1);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        // scattered rows may sit in a peer GPU's memory: order this thread's stores before whatever the host enqueues next
        if (p.scatter_rows) __threadfence_system();
        if (p.prof && threadIdx.x == 0) {
            p.prof[blockIdx.x * 8 + 5] = clock64() - t_begin;
            p.prof[blockIdx.x * 8 + 6] = waited;
        }
    }

    // ================================================================================ teardown
    if (s_abort) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive();  // neither CTA frees tensor memory or exits while its peer may still use either CTA's memory
    ptx::cluster_wait();
    if (warp == Cfg::MMA_WARP) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    }
}

template <class Cfg>
cudaError_t launch_pair_cfg(int pairs, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(d8k_gemm_pair_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    d8k_gemm_pair_kernel<Cfg><<<2 * pairs, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, p);
    return cudaGetLastError();
}

}  // namespace d8k
