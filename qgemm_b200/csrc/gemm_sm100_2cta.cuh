// CTA-pair variant of the persistent tcgen05 GEMM: two CTAs of a 2-CTA cluster share one
// 256 x 256 output tile through tcgen05.mma.cta_group::2.
//
// Each CTA loads 128 rows of A and only its 128-row half of the B tile (32 KB per 128-byte K block
// instead of the 48 KB a lone 128 x 256 tile needs), so a third fewer bytes cross L2 -> SM and
// shared memory per flop, and six pipeline stages fit where the lone-CTA kernel has four. The
// even-ranked ("leader") CTA issues every MMA; the instruction reads both CTAs' shared memory and
// writes rows 0..127 of the tile into the leader's tensor memory and rows 128..255 into the peer's.
//
// Barriers (all mbarriers, every wait bounded as in gemm_sm100.cuh):
//   full[stage]   leader only; one arrive.expect_tx by the leader's producer for both CTAs' bytes;
//                 both producers' TMA loads credit it (cta_group::2 loads may signal the peer's barrier);
//   empty[stage]  one per CTA; the leader's tcgen05.commit arrives on both;
//   tmem_full[a]  one per CTA; the leader's tcgen05.commit arrives on both;
//   tmem_empty[a] leader only; the 4 epilogue warps of each CTA arrive on it (count 8).
// No TMA load is multicast.
#pragma once
#include "gemm_sm100.cuh"

namespace qgemm {

constexpr int kPairTileM = 256;
constexpr int kPairTileN = 256;

// BN = tile width: 256, or 128 (256 x 128 tiles: a CTA then loads 128 rows of A and 64 rows of B, 24 KB per K block for
// its 128 x 128 share of the output where a lone CTA on a 128 x 128 tile loads 32 KB; eight stages fit).
// ONE (256 x 128 tiles only) = one tile per cluster: the epilogue's staging buffers lie over the start of the ring,
// which is idle by then in both CTAs, and a ninth stage takes their place (see GemmSmem).
template <int BN, bool ONE = false>
struct PairSmemT {
    static_assert(!ONE || BN == 128, "one-tile layout: 256 x 128 tiles");
    static constexpr int kStages = BN == 256 ? 6 : (ONE ? 9 : 8);
    static constexpr int kAStage = 128 * 128;
    static constexpr int kBStage = (BN / 2) * 128;
    static constexpr int kTiles = kStages * (kAStage + kBStage);
    static constexpr int kOutOffset = ONE ? 0 : kTiles;  // epilogue staging (see epilogue_tma)
    static constexpr int kBarOffset = kTiles + (ONE ? 0 : kEpilogueStagingBytes);
    static constexpr int kMiscOffset = kBarOffset + (2 * kStages + 4) * 8;
    static constexpr int kTotal = kMiscOffset + 16;
    static constexpr int kDynamicBytes = kTotal + 1024;
};
using PairSmem = PairSmemT<kPairTileN>;
constexpr int kPairStages = PairSmem::kStages;

template <bool GATHER>
struct ExtraDstParam {
    using type = NoExtraDst;
};
template <>
struct ExtraDstParam<true> {
    using type = ExtraDst;
};

// p.m_tiles / p.n_tiles count 256 x BN pair tiles; the grid is 2 * (number of clusters). BN = 128 takes a K-major B
// only and has no last-wave split.
// GATHER: the epilogue also stores every tile to the p.n_extra_dst destinations of `extra` (see ExtraDst).

template <int KIND, int OUT, bool GATHER = false, int BN = kPairTileN, bool ONE = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_ws,
                         const __grid_constant__ typename ExtraDstParam<GATHER>::type extra, const GemmParams p) {
    using L = PairSmemT<BN, ONE>;
    static_assert(BN == 256 || BN == 128, "pair tile width");
    constexpr int STAGES = L::kStages;
    constexpr int ELT = (KIND == ptx::KIND_F16) ? 2 : 1;
    constexpr int BK = 128 / ELT;
    constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    const uint32_t smem_a = smem_base;
    const uint32_t smem_b = smem_base + STAGES * L::kAStage;
    const uint32_t bar_full = smem_base + L::kBarOffset;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_tfull = bar_empty + STAGES * 8;
    const uint32_t bar_tempty = bar_tfull + 2 * 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 4);

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;
    const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
    const int cluster_id = static_cast<int>(blockIdx.x) >> 1;
    const int n_clusters = static_cast<int>(gridDim.x) >> 1;
    const int total_work = p.total_work;
    // a wait that runs out raises the abort flag of both CTAs of the pair, so that they leave together
    const uint32_t peer_abort = ptx::mapa_shared(ptx::smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + s * 8, 1);
            ptx::mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(bar_tfull + a * 8, 1);
            ptx::mbar_init(bar_tempty + a * 8, 8);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        if (p.c_tma_ok) ptx::prefetch_tensormap(&tmap_c);
        if (p.tail_begin > 0 || p.sk_parts > 0) ptx::prefetch_tensormap(&tmap_ws);
        if constexpr (GATHER)
            for (int d = 0; d < p.n_extra_dst; ++d) ptx::prefetch_tensormap(&extra.map[d]);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    // Both CTAs' barriers must exist before either CTA signals the other's.
    ptx::cluster_arrive();
    ptx::cluster_wait();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (ptx::elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int w = cluster_id; ok && w < total_work; w += n_clusters) {
                const WorkItem item = decode_work(w, p);
                const TileCoord t = item.t;
                const int kb0 = item.kb0, kb1 = item.kb1;
                const int row_a = (t.m_blk * 2 + static_cast<int>(rank)) * 128;
                const int row_b = t.n_blk * BN + static_cast<int>(rank) * (BN / 2);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!wait_bounded(bar_empty + stage * 8, phase ^ 1u, abort_flag, p.status, ROLE_PRODUCER, kb, peer_abort)) {
                        ok = false;
                        break;
                    }
                    if (kb == p.test_skip_kb) {
                        // test hook: neither CTA fills this slot, so the leader's MMA issuer's wait on it runs out
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    if (rank == 0) ptx::mbar_arrive_expect_tx(bar_full + stage * 8, 2 * (L::kAStage + L::kBStage));
                    const uint32_t leader_full = ptx::mapa_shared(bar_full + stage * 8, 0);
                    ptx::tma_load_2d_pair(smem_a + stage * L::kAStage, &tmap_a, leader_full, kb * BK, row_a);
                    if (p.b_mn_major) {
                        constexpr int CHUNK = 128 / ELT;  // this CTA's BN / 2 columns of B: 128-byte chunks of N
#pragma unroll
                        for (int j = 0; j < (BN / 2) / CHUNK; ++j)
                            ptx::tma_load_2d_pair(smem_b + stage * L::kBStage + j * (BK * 128), &tmap_b, leader_full,
                                                  row_b + j * CHUNK, kb * BK);
                    } else {
                        ptx::tma_load_2d_pair(smem_b + stage * L::kBStage, &tmap_b, leader_full, kb * BK, row_b);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (rank == 0 && ptx::elect_one()) {
            uint32_t stage = 0, phase = 0;
            uint32_t it = 0;
            bool ok = true;
            for (int w = cluster_id; ok && w < total_work; w += n_clusters, ++it) {
                const WorkItem item = decode_work(w, p);
                const int kb0 = item.kb0, kb1 = item.kb1;
                if (kb0 >= kb1) {  // an empty item (GemmParams::sk_parts): no accumulator is taken for it
                    --it;
                    continue;
                }
                const uint32_t acc = it & 1u;
                const uint32_t acc_phase = (it >> 1) & 1u;
                if (!wait_bounded(bar_tempty + acc * 8, acc_phase ^ 1u, abort_flag, p.status, ROLE_MMA, -1, peer_abort)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!wait_bounded(bar_full + stage * 8, phase, abort_flag, p.status, ROLE_MMA, kb, peer_abort)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint64_t a_desc = ptx::make_kmajor_sw128_desc(smem_a + stage * L::kAStage);
                    const uint64_t b_desc =
                        p.b_mn_major ? ptx::make_mnmajor_sw128_desc(smem_b + stage * L::kBStage, BK * 128)
                                     : ptx::make_kmajor_sw128_desc(smem_b + stage * L::kBStage);
                    const uint32_t b_step = p.b_mn_major ? static_cast<uint32_t>((32 / ELT) * 128 / 16) : 2u;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        ptx::umma_ss_pair<KIND>(d_tmem, a_desc + 2u * k, b_desc + b_step * k, p.idesc,
                                                (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    ptx::tc_commit_pair(bar_empty + stage * 8, 3);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) ptx::tc_commit_pair(bar_tfull + acc * 8, 3);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs)
        const int quad = warp & 3;
        float alpha = 1.0f;
        if constexpr (OUT != OUT_RAW32) {
            if (p.scale_a != nullptr) alpha *= __ldg(p.scale_a);
            if (p.scale_b != nullptr) alpha *= __ldg(p.scale_b);
        }
        uint32_t it = 0;
        uint32_t out_buf = 0;
        for (int w = cluster_id; w < total_work; w += n_clusters, ++it) {
            const WorkItem item = decode_work(w, p);
            if (item.kb0 >= item.kb1) {  // an empty item: the MMA issuer passed over it as well
                --it;
                continue;
            }
            const TileCoord t = item.t;
            const uint32_t acc = it & 1u;
            const uint32_t acc_phase = (it >> 1) & 1u;
            if (!wait_bounded(bar_tfull + acc * 8, acc_phase, abort_flag, p.status, ROLE_EPILOGUE, w, peer_abort)) break;
            ptx::tc_fence_after();
            const long long row =
                (static_cast<long long>(t.m_blk) * 2 + static_cast<long long>(rank)) * 128 + quad * 32 + lane;
            uint8_t* c_base = reinterpret_cast<uint8_t*>(p.C) +
                              static_cast<long long>(t.split) * p.split_stride * OutBytes<OUT>::value;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
            const int row0 = (t.m_blk * 2 + static_cast<int>(rank)) * 128 + quad * 32;
            const CUtensorMap* extra_maps = nullptr;
            int n_extra = 0;
            if constexpr (GATHER) {  // launched only with valid tensor maps for C and every further destination
                extra_maps = &extra.map[0];
                n_extra = p.n_extra_dst;
            }
            if (item.slot >= 0) {
                // K slice of a last-wave tile: raw 32-bit partial sums into a whole scratch slot, nothing to clip
                epilogue_tma<KIND, OUT_RAW32, BN>(&tmap_ws, t_addr,
                                                  (item.slot * 2 + static_cast<int>(rank)) * 128 + quad * 32, 0x7fffffff,
                                                  0, BN, t.split, smem_base + L::kOutOffset + (warp - 2) * 8192, lane,
                                                  1.0f, out_buf);
            } else if (GATHER || p.c_tma_ok) {
                epilogue_tma<KIND, OUT, BN>(&tmap_c, t_addr, row0, p.M, t.n_blk * BN, p.N, t.split,
                                            smem_base + L::kOutOffset + (warp - 2) * 8192, lane, alpha, out_buf,
                                            extra_maps, n_extra);
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int n0 = t.n_blk * BN + c * 32;
                    if (n0 >= p.N) break;
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(t_addr + c * 32, v);
                    ptx::tmem_ld_wait();
                    if (row < p.M)
                        store_chunk<KIND, OUT>(c_base, p.ldc, row, n0, min(32, p.N - n0), p.c_vec_ok != 0, v, alpha);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(bar_tempty + acc * 8, 0));
        }
        if (lane == 0) {
            // stores to another GPU are waited for to completion, not just until shared memory was read
            if constexpr (GATHER) ptx::tma_store_wait_all<0>();
            else ptx::tma_store_wait_read<0>();
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    // Neither CTA may release its shared or tensor memory while the other can still touch it.
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(20000);
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

}  // namespace qgemm
