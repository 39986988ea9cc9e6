// Split-K inside one launch for CTA pairs: a cluster of 2 S CTAs (S = 2 or 4 pairs) shares one 256 x 128 output tile.
//
// Pair s (cluster ranks 2 s and 2 s + 1) multiplies K slice s of the tile with tcgen05.mma.cta_group::2, exactly as
// gemm_tcgen05_pair_kernel does for a whole tile: each CTA loads 128 rows of A and its 64-row half of the B tile,
// the even-ranked CTA of the pair issues the MMAs, rows 0..127 of the tile accumulate in its tensor memory and rows
// 128..255 in its partner's. Then, as in gemm_sm100_kcluster.cuh:
//   1. every CTA copies its raw 128 x 128 accumulator into its own shared memory (the ring, idle by then);
//   2. cluster barrier;
//   3. the S CTAs that hold the same row half (equal rank parity) deal its valid rows out among themselves; each adds
//      up its rows of the S partial tiles, read with ld.shared::cluster, in slice order starting from zero (the order
//      of splitk_reduce_kernel: bit-identical to the two-launch split, int8 exact), scales, casts and stores them;
//   4. cluster barrier.
// For mid-size problems (a few dozen 256 x 128 tiles, K of several thousand): a CTA of a pair moves 24 KB per K block
// from L2 for its 128 x 128 share of the output, where the 64-wide lone tiles that otherwise occupy the SMs for such a
// problem move 24 KB for 128 x 64, and the kernel is bound by what a CTA can pull; without K slices too few pairs
// exist to occupy the SMs, and with the two-launch split the partial sums make a round trip through global memory.
// (The same on 256 x 256 tiles, 128 KB of partial sums per CTA, was measured and is no faster than two launches.)
// K-major B only. One tile per cluster. Every mbarrier wait is bounded; a CTA whose wait runs out raises the abort
// flag of every CTA of the cluster, and the cluster barriers are executed unconditionally by every thread.
#pragma once
#include "gemm_sm100_2cta.cuh"
#include "gemm_sm100_kcluster.cuh"

namespace qgemm {

template <int KIND, int OUT, int S>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kcluster_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                  const GemmParams p) {
    constexpr int BN = 128;
    using L = PairSmemT<BN, true>;  // no staging buffers (results are stored from registers): nine stages
    static_assert(S == 2 || S == 4, "pairs per cluster");
    constexpr int STAGES = L::kStages;
    constexpr int ELT = (KIND == ptx::KIND_F16) ? 2 : 1;
    constexpr int BK = 128 / ELT;
    constexpr uint32_t TMEM_COLS = BN;
    constexpr int ROW_WORDS = BN + kKcPad;
    constexpr int TPR = BN / 4;  // threads per row in the reduction
    static_assert(kBM * ROW_WORDS * 4 <= L::kTiles, "the partial tile fits in the pipeline's ring");

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
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 4);

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const uint32_t half = rank & 1u;         // 0 = the pair's leader, rows 0..127 of the tile
    const uint32_t slice = rank >> 1;        // which pair of the cluster = which K slice
    const uint32_t leader = rank & ~1u;      // cluster rank of this pair's leader
    const uint16_t pair_mask = static_cast<uint16_t>(3u << leader);
    const int tile = static_cast<int>(blockIdx.x) / (2 * S);

    ptx::pdl_launch_dependents();  // the successor may start its set-up; it waits for this grid before touching memory
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + s * 8, 1);
            ptx::mbar_init(bar_empty + s * 8, 1);
        }
        ptx::mbar_init(bar_tfull, 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    const TileCoord t = decode_tile(tile, p);  // p.splits == 1: work item == tile
    const int kb0 = static_cast<int>(slice) * p.kb_per_split;
    const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
    ptx::tc_fence_before();
    __syncthreads();
    // Every CTA's barriers and abort flag must exist before any other CTA of the cluster signals them.
    ptx::cluster_arrive();
    ptx::cluster_wait();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    ptx::pdl_wait();

    auto raise_peers = [&]() {
        const uint32_t own = ptx::smem_u32(const_cast<int*>(abort_flag));
#pragma unroll
        for (uint32_t r = 0; r < static_cast<uint32_t>(2 * S); ++r)
            if (r != rank) ptx::st_shared_cluster_u32(ptx::mapa_shared(own, r), 1u);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (every CTA)
        if (ptx::elect_one()) {
            uint32_t stage = 0, phase = 0;
            const int row_a = (t.m_blk * 2 + static_cast<int>(half)) * 128;
            const int row_b = t.n_blk * BN + static_cast<int>(half) * (BN / 2);
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!wait_bounded(bar_empty + stage * 8, phase ^ 1u, abort_flag, p.status, ROLE_PRODUCER, kb)) {
                    raise_peers();
                    break;
                }
                if (kb != p.test_skip_kb) {  // test hook: a slot that neither CTA of the pair fills
                    if (half == 0) ptx::mbar_arrive_expect_tx(bar_full + stage * 8, 2 * (L::kAStage + L::kBStage));
                    const uint32_t leader_full = ptx::mapa_shared(bar_full + stage * 8, leader);
                    ptx::tma_load_2d_pair(smem_a + stage * L::kAStage, &tmap_a, leader_full, kb * BK, row_a);
                    ptx::tma_load_2d_pair(smem_b + stage * L::kBStage, &tmap_b, leader_full, kb * BK, row_b);
                }
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (the pair's leader only)
        if (half == 0 && ptx::elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!wait_bounded(bar_full + stage * 8, phase, abort_flag, p.status, ROLE_MMA, kb)) {
                    raise_peers();
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint64_t a_desc = ptx::make_kmajor_sw128_desc(smem_a + stage * L::kAStage);
                const uint64_t b_desc = ptx::make_kmajor_sw128_desc(smem_b + stage * L::kBStage);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    ptx::umma_ss_pair<KIND>(tmem_base, a_desc + 2u * k, b_desc + 2u * k, p.idesc,
                                            (kb > kb0 || k > 0) ? 1u : 0u);
                ptx::tc_commit_pair(bar_empty + stage * 8, pair_mask);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (ok) ptx::tc_commit_pair(bar_tfull, pair_mask);
        }
    } else {
        // ------------------------------------------------------------ epilogue warps: accumulator -> own shared memory
        const int quad = warp & 3;
        if (wait_bounded(bar_tfull, 0u, abort_flag, p.status, ROLE_EPILOGUE, tile)) {
            ptx::tc_fence_after();
            const uint32_t row_addr = smem_base + static_cast<uint32_t>((quad * 32 + lane) * ROW_WORDS * 4);
            if ((t.m_blk * 2 + static_cast<int>(half)) * 128 + quad * 32 < p.M) {  // warp-uniform: rows that exist
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    if (t.n_blk * BN + c * 32 >= p.N) break;  // columns that exist
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c * 32, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        ptx::st_shared_v4(row_addr + static_cast<uint32_t>((c * 32 + 4 * j) * 4), v[4 * j], v[4 * j + 1],
                                          v[4 * j + 2], v[4 * j + 3]);
                }
            }
            ptx::tc_fence_before();
        } else {
            raise_peers();
        }
    }

    // ---------------------------------------------------------------- every CTA's partial tile is in place
    __syncthreads();
    ptx::cluster_arrive();
    ptx::cluster_wait();

    // ---------------------------------------------------------------- this CTA's rows of the sum
    // The valid rows of this CTA's row half are dealt out over the S CTAs of equal parity; 32 threads share a row,
    // four columns each: a warp reads 512 contiguous bytes of a peer's shared memory and stores a contiguous run of C.
    if (warp >= 2 && *abort_flag == 0) {
        const int e = static_cast<int>(threadIdx.x) - 64;  // 0..127
        const int sub = e & (TPR - 1);
        const int half_row0 = (t.m_blk * 2 + static_cast<int>(half)) * 128;
        const int rows_valid = max(0, min(kBM, p.M - half_row0));
        const int rows_per_cta = (rows_valid + S - 1) / S;
        const int r0 = static_cast<int>(slice) * rows_per_cta;
        const int r1 = min(rows_valid, r0 + rows_per_cta);
        const int n0 = t.n_blk * BN + sub * 4;
        const int n_valid = min(4, p.N - n0);
        float alpha = 1.0f;
        if constexpr (OUT != OUT_RAW32) {
            if (p.scale_a != nullptr) alpha *= __ldg(p.scale_a);
            if (p.scale_b != nullptr) alpha *= __ldg(p.scale_b);
        }
        constexpr int OB = OutBytes<OUT>::value;
        if (n_valid > 0) {
#pragma unroll 2
            for (int r = r0 + e / TPR; r < r1; r += 128 / TPR) {
                const uint32_t own = smem_base + static_cast<uint32_t>((r * ROW_WORDS + sub * 4) * 4);
                uint32_t w[S][4];
#pragma unroll
                for (uint32_t k = 0; k < static_cast<uint32_t>(S); ++k)
                    ptx::ld_shared_cluster_v4(ptx::mapa_shared(own, 2u * k + half), w[k][0], w[k][1], w[k][2], w[k][3]);
                uint32_t acc[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if constexpr (KIND == ptx::KIND_I8) {
                        int a = 0;
#pragma unroll
                        for (int k = 0; k < S; ++k) a += static_cast<int>(w[k][j]);
                        acc[j] = static_cast<uint32_t>(a);
                    } else {
                        float a = 0.0f;
#pragma unroll
                        for (int k = 0; k < S; ++k) a += __uint_as_float(w[k][j]);
                        acc[j] = __float_as_uint(a);
                    }
                }
                const long long row = static_cast<long long>(half_row0) + r;
                uint8_t* dst = reinterpret_cast<uint8_t*>(p.C) + (row * p.ldc + n0) * OB;
                const bool vec = p.c_vec_ok != 0 && n_valid == 4;
                if constexpr (OUT == OUT_RAW32) {
                    if (vec) {
                        *reinterpret_cast<uint4*>(dst) = make_uint4(acc[0], acc[1], acc[2], acc[3]);
                    } else {
                        for (int j = 0; j < n_valid; ++j) reinterpret_cast<uint32_t*>(dst)[j] = acc[j];
                    }
                } else {
                    float f[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        f[j] = ((KIND == ptx::KIND_I8) ? static_cast<float>(static_cast<int>(acc[j])) : __uint_as_float(acc[j])) *
                               alpha;
                    if constexpr (OUT == OUT_F32) {
                        if (vec) {
                            *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
                        } else {
                            for (int j = 0; j < n_valid; ++j) reinterpret_cast<float*>(dst)[j] = f[j];
                        }
                    } else {
                        uint32_t pk[2];
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            if constexpr (OUT == OUT_BF16) {
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                                pk[j] = *reinterpret_cast<uint32_t*>(&h2);
                            } else {
                                __half2 h2 = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                                pk[j] = *reinterpret_cast<uint32_t*>(&h2);
                            }
                        }
                        if (vec) {
                            *reinterpret_cast<uint2*>(dst) = make_uint2(pk[0], pk[1]);
                        } else {
                            for (int j = 0; j < n_valid; ++j)
                                reinterpret_cast<uint16_t*>(dst)[j] =
                                    static_cast<uint16_t>((j & 1) ? (pk[j >> 1] >> 16) : (pk[j >> 1] & 0xffffu));
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    // No CTA may release its shared or tensor memory while another can still touch it.
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
