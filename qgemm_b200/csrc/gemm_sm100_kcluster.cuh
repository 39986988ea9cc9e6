// Split-K inside one launch: the S CTAs of a thread-block cluster each multiply one K slice of the same 128 x BN
// output tile, and the partial sums are added up through distributed shared memory.
//
// The two-launch split-K (partial sums to global scratch, then splitk_reduce_kernel) costs a second launch on problems
// whose whole body is a few microseconds -- small M and N, long K, where there are too few output tiles to occupy the
// SMs. Here the partial sums never leave the cluster:
//   1. every CTA runs the usual pipeline (TMA producer warp, MMA issuer warp) over its K slice into a tensor-memory
//      accumulator;
//   2. its four epilogue warps copy the raw 32-bit accumulator into the CTA's own shared memory (the pipeline's ring,
//      idle by then);
//   3. cluster barrier;
//   4. the tile's valid rows are dealt out over the S CTAs; each adds up its rows of all S partial tiles, read with
//      ld.shared::cluster, in slice order starting from zero (the order of splitk_reduce_kernel: results are
//      bit-identical to the two-launch path, int8 stays exact), scales, casts and stores them;
//   5. cluster barrier, so that no CTA's shared memory goes away while a peer may still read it.
// The reference has no split-K (README.md:28 lists it as a to-do; src/gemm/sm89_gemm_kernel_v5.cu:319 carries an
// unused `split_k = 2`).
//
// One tile per cluster (grid = tiles x S, at most one wave). Every mbarrier wait is bounded as in gemm_sm100.cuh; the
// two cluster barriers are executed by every thread of every CTA whatever happened before them, so a CTA that gave up
// a wait still meets its peers there, and it raises their abort flags on the way.
#pragma once
#include "gemm_sm100.cuh"

namespace qgemm {

constexpr int kKcPad = 4;  // words of padding per row of the partial tile in shared memory (bank spread for 16-byte rows)

template <int KIND, int BN, int STAGES, int OUT, int AM, int S>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kcluster_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                             const GemmParams p) {
    using L = GemmSmem<BN, STAGES, AM, true>;  // no staging buffers: results are stored from registers
    static_assert(S == 2 || S == 4 || S == 8, "cluster size (8 is the largest portable one)");
    static_assert(BN == 64 || BN == 128, "BN / 4 threads x four columns cover a row of the tile");
    static_assert(kBM * (BN + kKcPad) * 4 <= L::kTiles, "the partial tile fits in the pipeline's ring");
    static_assert(STAGES * L::kAStage + (kBM - AM) * 128 <= L::kTiles, "the MMA's 128-row read of A stays inside the tile area");
    constexpr int ELT = (KIND == ptx::KIND_F16) ? 2 : 1;
    constexpr int BK = 128 / ELT;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr int ROW_WORDS = BN + kKcPad;

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
    const int tile = static_cast<int>(blockIdx.x) / S;  // one tile per cluster

    ptx::pdl_launch_dependents();  // the successor may start its set-up; it waits for this grid before touching memory
    if (warp == 0) {  // the barriers are set up by the lanes of one warp side by side
        static_assert(STAGES <= 32, "one lane per ring slot");
        if (lane < STAGES) {
            ptx::mbar_init(bar_full + lane * 8, 1);
            ptx::mbar_init(bar_empty + lane * 8, 1);
        }
        if (lane == 0) {
            ptx::mbar_init(bar_tfull, 1);
            *abort_flag = 0;
            ptx::prefetch_tensormap(&tmap_a);
            ptx::prefetch_tensormap(&tmap_b);
        }
        ptx::fence_barrier_init();
    }
    const TileCoord t = decode_tile(tile, p);  // p.splits == 1: work item == tile
    const int kb0 = static_cast<int>(rank) * p.kb_per_split;
    const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
    const int group = p.kgroup > 1 ? p.kgroup : 1;  // K blocks per TMA instruction (GemmParams::kgroup)
    const int skip_kb = p.test_skip_kb;
    // The loads of `group` K blocks starting at kb into ring slots stage .. stage + group - 1.
    auto load_group = [&](int kb, uint32_t stage) {
        const uint32_t full = bar_full + stage * 8;
        if (!(skip_kb >= kb && skip_kb < kb + group)) {  // test hook: a slot that is never filled
            ptx::mbar_arrive_expect_tx(full, group * (L::kAStage + L::kBStage));
            if (group == 1) {
                ptx::tma_load_2d(smem_a + stage * L::kAStage, &tmap_a, full, kb * BK, t.m_blk * kBM);
                ptx::tma_load_2d(smem_b + stage * L::kBStage, &tmap_b, full, kb * BK, t.n_blk * BN);
            } else {
                ptx::tma_load_3d(smem_a + stage * L::kAStage, &tmap_a, full, 0, t.m_blk * kBM, kb);
                ptx::tma_load_3d(smem_b + stage * L::kBStage, &tmap_b, full, 0, t.n_blk * BN, kb);
            }
        }
    };
    // As in gemm_tcgen05_kernel: the producer lane sends the first two groups of loads on their way as soon as the
    // predecessor in the stream is done, before the CTA-wide barrier (tensor-memory allocation and the barrier then
    // overlap the first bytes' flight); its loop state is carried into the main loop.
    uint32_t prod_stage = 0, prod_phase = 0, prod_filled = 0;
    int prod_kb = kb0;
    if (warp == 0) {
        __syncwarp();  // the other lanes' barrier set-up
        if (ptx::elect_one()) {
            ptx::pdl_wait();
            while (prod_kb < kb1 && prod_filled < static_cast<uint32_t>(min(STAGES, p.early_groups * group))) {
                load_group(prod_kb, prod_stage);
                prod_kb += group;
                prod_filled += group;
                prod_stage += group;
                if (prod_stage >= static_cast<uint32_t>(STAGES)) {
                    prod_stage = 0;
                    prod_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    ptx::pdl_wait();

    // A wait that runs out raises the abort flag of every CTA of the cluster, so that all of them stop waiting and
    // go on to the cluster barriers.
    auto raise_peers = [&]() {
        const uint32_t own = ptx::smem_u32(const_cast<int*>(abort_flag));
#pragma unroll
        for (uint32_t r = 0; r < static_cast<uint32_t>(S); ++r)
            if (r != rank) ptx::st_shared_cluster_u32(ptx::mapa_shared(own, r), 1u);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            uint32_t stage = prod_stage, phase = prod_phase, filled = prod_filled;
            for (int kb = prod_kb; kb < kb1; kb += group) {
                // the first STAGES slots are free without asking
                if (filled >= static_cast<uint32_t>(STAGES) &&
                    !wait_bounded(bar_empty + stage * 8, phase ^ 1u, abort_flag, p.status, ROLE_PRODUCER, kb)) {
                    raise_peers();
                    break;
                }
                if (filled < static_cast<uint32_t>(STAGES)) filled += group;
                load_group(kb, stage);
                stage += group;
                if (stage >= STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            const int G = p.kgroup > 1 ? p.kgroup : 1;
            for (int kb = kb0; kb < kb1; kb += G) {
                if (!wait_bounded(bar_full + stage * 8, phase, abort_flag, p.status, ROLE_MMA, kb)) {
                    raise_peers();
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const int blocks = min(G, kb1 - kb);
                for (int j = 0; j < blocks; ++j) {
                    const uint64_t a_desc = ptx::make_kmajor_sw128_desc(smem_a + (stage + j) * L::kAStage);
                    const uint64_t b_desc = ptx::make_kmajor_sw128_desc(smem_b + (stage + j) * L::kBStage);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        ptx::umma_ss<KIND>(tmem_base, a_desc + 2u * k, b_desc + 2u * k, p.idesc,
                                           (kb + j > kb0 || k > 0) ? 1u : 0u);
                }
                ptx::tc_commit(bar_empty + stage * 8);
                stage += G;
                if (stage >= STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (ok) ptx::tc_commit(bar_tfull);
        }
    } else {
        // ------------------------------------------------------------ epilogue warps, step 2: accumulator -> own shared memory
        const int quad = warp & 3;
        if (wait_bounded(bar_tfull, 0u, abort_flag, p.status, ROLE_EPILOGUE, tile)) {
            ptx::tc_fence_after();
            // the ring is idle: every load has landed and every MMA that read it has completed
            const uint32_t row_addr = smem_base + static_cast<uint32_t>((quad * 32 + lane) * ROW_WORDS * 4);
            if (t.m_blk * kBM + quad * 32 < p.M) {  // warp-uniform: rows that exist
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
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

    // ---------------------------------------------------------------- step 3: every CTA's partial tile is in place
    __syncthreads();
    ptx::cluster_arrive();
    ptx::cluster_wait();

    // ---------------------------------------------------------------- step 4: this CTA's rows of the sum
    // The tile's valid rows are dealt out over the S CTAs. BN / 4 threads share a row, four columns each, so that a
    // warp's read of a peer's shared memory is one or two contiguous runs of 256 bytes or more, and its store to C too.
    if (warp >= 2 && *abort_flag == 0) {
        const int e = static_cast<int>(threadIdx.x) - 64;  // 0..127
        constexpr int TPR = BN / 4;  // threads per row
        const int sub = e & (TPR - 1);
        const int rows_valid = min(kBM, p.M - t.m_blk * kBM);
        const int rows_per_cta = (rows_valid + S - 1) / S;
        const int r0 = static_cast<int>(rank) * rows_per_cta;
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
                    ptx::ld_shared_cluster_v4(ptx::mapa_shared(own, k), w[k][0], w[k][1], w[k][2], w[k][3]);
                uint32_t acc[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // slice order starting from zero: the order of the two-launch reduction
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
                const long long row = static_cast<long long>(t.m_blk) * kBM + r;
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
                                __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                                pk[j] = *reinterpret_cast<uint32_t*>(&h);
                            } else {
                                __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                                pk[j] = *reinterpret_cast<uint32_t*>(&h);
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

    // ---------------------------------------------------------------- step 5 and teardown
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (*abort_flag != 0) {
        // let TMA copies and MMAs that were already issued finish before the memory they touch is released
        for (int i = 0; i < 64; ++i) __nanosleep(20000);
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace qgemm
