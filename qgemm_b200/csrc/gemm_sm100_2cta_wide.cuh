// "Wide" CTA-pair variant of the persistent tcgen05 GEMM: a 2-CTA cluster computes a 512 x 256 output tile.
//
// Each CTA owns 256 rows of the tile as two 128-row halves, one accumulator each, which together fill its tensor
// memory (2 x 256 columns). Per 128-byte K block a CTA loads 256 rows of A (32 KB) and its 128-row half of the B tile
// (16 KB), and the leader issues two rounds of tcgen05.mma.cta_group::2 (M = 256: 128 rows from each CTA), one per
// accumulator, against the same B. Compared with the 256 x 256 pair kernel (gemm_sm100_2cta.cuh) this moves a quarter
// fewer operand bytes from L2 to the SMs per flop -- (512 + 256) / (512 * 256) against (256 + 256) / (256 * 256) --
// which on a part that sits at its power cap buys clock. The price: both accumulators are busy until the last K
// block, so there is no second accumulator to compute into while the epilogue drains the first; the next tile's MMAs
// on accumulator j start as soon as accumulator j has been drained (tmem_empty[j]).
//
// Barriers (all waits bounded as in gemm_sm100.cuh): full[stage] leader only, credited by both CTAs' loads;
// empty[stage] and tmem_full one per CTA, signalled by the leader's tcgen05.commit to both; tmem_empty[0..1] leader
// only, 4 epilogue warps of each CTA arrive (count 8). No TMA load is multicast. splits == 1 only.
#pragma once
#include "gemm_sm100_2cta.cuh"

namespace qgemm {

constexpr int kWideStages = 4;
constexpr int kWideTileM = 512;
constexpr int kWideTileN = 256;

struct WideSmem {
    static constexpr int kAStage = 256 * 128;
    static constexpr int kBStage = 128 * 128;
    static constexpr int kTiles = kWideStages * (kAStage + kBStage);
    static constexpr int kOutOffset = kTiles;  // epilogue staging (see epilogue_tma)
    static constexpr int kBarOffset = kTiles + kEpilogueStagingBytes;  // full[S], empty[S], tfull, tempty[2]
    static constexpr int kMiscOffset = kBarOffset + (2 * kWideStages + 3) * 8;
    static constexpr int kTotal = kMiscOffset + 16;
    static constexpr int kDynamicBytes = kTotal + 1024;
};

// p.m_tiles / p.n_tiles count 512 x 256 tiles; the grid is 2 * (number of clusters).
template <int KIND, int OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_wide_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                              const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
    using L = WideSmem;
    constexpr int STAGES = kWideStages;
    constexpr int ELT = (KIND == ptx::KIND_F16) ? 2 : 1;
    constexpr int BK = 128 / ELT;
    constexpr int BN = kWideTileN;
    constexpr uint32_t TMEM_COLS = 512;

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
    const uint32_t bar_tempty = bar_tfull + 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 4);

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;
    const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
    const int cluster_id = static_cast<int>(blockIdx.x) >> 1;
    const int n_clusters = static_cast<int>(gridDim.x) >> 1;
    const int total_work = p.m_tiles * p.n_tiles;
    // a wait that runs out raises the abort flag of both CTAs of the pair, so that they leave together
    const uint32_t peer_abort = ptx::mapa_shared(ptx::smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + s * 8, 1);
            ptx::mbar_init(bar_empty + s * 8, 1);
        }
        ptx::mbar_init(bar_tfull, 1);
        for (int a = 0; a < 2; ++a) ptx::mbar_init(bar_tempty + a * 8, 8);
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        ptx::prefetch_tensormap(&tmap_c);
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
                const TileCoord t = decode_tile(w, p);
                const int row_a = (t.m_blk * 2 + static_cast<int>(rank)) * 256;
                const int row_b = t.n_blk * BN + static_cast<int>(rank) * 128;
                for (int kb = 0; kb < p.kb_total; ++kb) {
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
                    // 256 rows of A in one box: rows 0..127 land in the first 16 KB of the stage, 128..255 in the second
                    ptx::tma_load_2d_pair(smem_a + stage * L::kAStage, &tmap_a, leader_full, kb * BK, row_a);
                    if (p.b_mn_major) {
                        constexpr int CHUNK = 128 / ELT;  // this CTA's 128 columns of B: 128-byte chunks of N
#pragma unroll
                        for (int j = 0; j < 128 / CHUNK; ++j)
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
                for (int kb = 0; ok && kb < p.kb_total; ++kb) {
                    if (!wait_bounded(bar_full + stage * 8, phase, abort_flag, p.status, ROLE_MMA, kb, peer_abort)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint64_t b_desc =
                        p.b_mn_major ? ptx::make_mnmajor_sw128_desc(smem_b + stage * L::kBStage, BK * 128)
                                     : ptx::make_kmajor_sw128_desc(smem_b + stage * L::kBStage);
                    const uint32_t b_step = p.b_mn_major ? static_cast<uint32_t>((32 / ELT) * 128 / 16) : 2u;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        if (kb == 0) {
                            // accumulator j of the previous tile must have been drained by both CTAs' epilogues
                            if (!wait_bounded(bar_tempty + j * 8, (it & 1u) ^ 1u, abort_flag, p.status, ROLE_MMA, -1 - j, peer_abort)) {
                                ok = false;
                                break;
                            }
                            ptx::tc_fence_after();
                        }
                        const uint64_t a_desc = ptx::make_kmajor_sw128_desc(smem_a + stage * L::kAStage + j * (128 * 128));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            ptx::umma_ss_pair<KIND>(tmem_base + j * BN, a_desc + 2u * k, b_desc + b_step * k, p.idesc,
                                                    (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    if (!ok) break;
                    ptx::tc_commit_pair(bar_empty + stage * 8, 3);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) ptx::tc_commit_pair(bar_tfull, 3);
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
            const TileCoord t = decode_tile(w, p);
            if (!wait_bounded(bar_tfull, it & 1u, abort_flag, p.status, ROLE_EPILOGUE, w, peer_abort)) break;
            ptx::tc_fence_after();
#pragma unroll 1
            for (int j = 0; j < 2; ++j) {
                const int row0 = (t.m_blk * 2 + static_cast<int>(rank)) * 256 + j * 128 + quad * 32;
                const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + j * BN;
                epilogue_tma<KIND, OUT, BN>(&tmap_c, t_addr, row0, p.M, t.n_blk * BN, p.N, 0,
                                            smem_base + L::kOutOffset + (warp - 2) * 8192, lane, alpha, out_buf);
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(bar_tempty + j * 8, 0));
            }
        }
        if (lane == 0) ptx::tma_store_wait_read<0>();
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
