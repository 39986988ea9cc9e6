// FP8 e4m3 GEMM with block scales -- the one mixed kernel the reference actually implements
// (FP8_GEMM_kernel, src/mix_gemm/hip_mix_gemm_kernel.cpp:249-378, AMD rocWMMA only):
//
//   C[m,n] = sum_kb ( sum_{k in block kb} A[m,k] * B[k,n] ) * a_scale[kb*M + m] * b_scale[kb*ceil(N/128) + n/128]
//
// with 128-wide K blocks, one A scale per row and block, one B scale per 128 x 128 block, fp32
// accumulation and one rounding to the output type (:193-244, :363-367, layouts :425-439).
//
// sm_100a shape of it: a 128-element FP8 K block is exactly one 128-byte TMA / UMMA K block. The MMA
// warp issues each K block (4 x tcgen05.mma.kind::f8f6f4, 128 x 128 x 32) into one of four *partial*
// tensor-memory accumulators with the accumulate flag off, so a partial holds the unscaled product of
// one block only. The epilogue warps drain each partial with tcgen05.ld and fold it into fp32
// registers with one fused multiply-add per element, scale = a_scale * b_scale, while the tensor
// cores already work on the next blocks in the other partials -- the rescale in CUDA cores that the
// reference does per K tile in registers. After the last block the registers are rounded and leave
// through the same swizzled-staging + TMA-store path as the plain GEMM.
//
// Barriers: full[stage] (TMA bytes landed), done[blk % 12] (one tcgen05.commit per K block: the block has been
// multiplied, which both frees its stage and publishes its partial), pempty[partial] (all eight rescale warps
// have the partial in registers). Loads run the whole ring ahead (the producer waits for a free stage only); the MMA
// issuers wait for a free partial -- with the wait in the producer a TMA round trip sat inside the partial's cycle
// (measured 7 % slower at 4096 x 7168 x 7168).
// Two warps issue the MMAs, one the even K blocks and one the odd ones (blocks go into different partials, so their
// MMAs are independent): measured 12-16 % faster on shapes below about 4096^3, no change above.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_launch.cuh"
#include "qgemm_internal.h"

namespace qgemm {

namespace {

constexpr int kBsBN = 128;
constexpr int kBsStages = 6;
constexpr int kBsPartials = 4;                           // partial accumulators in flight (4 x 128 = all 512 columns)
constexpr int kBsDone = 12;                              // "K block multiplied" barriers: lcm(stages, partials)
constexpr int kBsEpilogueWarps = 8;                      // two warps per tensor-memory lane quadrant
constexpr int kBsIssuerB = 2 + kBsEpilogueWarps;         // second MMA-issuing warp (odd K blocks), after the rescale warps
constexpr int kBsThreads = 32 * (3 + kBsEpilogueWarps);  // producer, MMA issuer (even blocks), 8 rescale warps, issuer (odd)
constexpr int kBsColsPerWarp = kBsBN / 2;                // each of the two warps of a quadrant takes 64 columns

struct BsSmem {
    static constexpr int kAStage = 128 * 128;
    static constexpr int kBStage = kBsBN * 128;
    static constexpr int kTiles = kBsStages * (kAStage + kBStage);
    static constexpr int kOutOffset = kTiles;
    static constexpr int kBarOffset = kTiles + kBsEpilogueWarps * 4096;  // full[S], done[12], pempty[P]
    static constexpr int kMiscOffset = kBarOffset + (kBsStages + kBsDone + kBsPartials) * 8;
    static constexpr int kTotal = kMiscOffset + 16;
    static constexpr int kDynamicBytes = kTotal + 1024;
};

// Work item -> tile: groups of 8 tile rows walked column by column, so that the tiles resident at one
// time share A and B panels in L2 (the same grouping as decode_tile in gemm_sm100.cuh).
__device__ __forceinline__ void bs_decode(int w, const BlockScaleParams& p, int& m_blk, int& n_blk) {
    const int G = p.group_m;
    const int group_sz = G * p.n_tiles;
    const int g = w / group_sz;
    const int first_m = g * G;
    const int gm = min(p.m_tiles - first_m, G);
    const int r = w - g * group_sz;
    n_blk = r / gm;
    m_blk = first_m + (r - n_blk * gm);
}

template <int OUT>
__global__ void __launch_bounds__(kBsThreads, 1)
fp8_blockscale_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const BlockScaleParams p) {
    using L = BsSmem;
    constexpr int STAGES = kBsStages;
    constexpr int BN = kBsBN;
    constexpr int BK = 128;  // FP8 elements per 128-byte K block == the scale block
    constexpr uint32_t TMEM_COLS = kBsPartials * BN;
    constexpr uint32_t PMASK = kBsPartials - 1;
    constexpr int PSHIFT = 2;  // log2(kBsPartials)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    const uint32_t smem_a = smem_base;
    const uint32_t smem_b = smem_base + STAGES * L::kAStage;
    // One tcgen05.commit per K block: done[i] (i = running K-block count mod 12) says "that block has been multiplied",
    // which frees its shared-memory stage for the producer and publishes its partial to the rescale warps at once.
    const uint32_t bar_full = smem_base + L::kBarOffset;
    const uint32_t bar_done = bar_full + STAGES * 8;
    const uint32_t bar_pempty = bar_done + kBsDone * 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 4);

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;
    const int total_work = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) ptx::mbar_init(bar_full + s * 8, 1);
        for (int d = 0; d < kBsDone; ++d) ptx::mbar_init(bar_done + d * 8, 1);
        for (int a = 0; a < kBsPartials; ++a) ptx::mbar_init(bar_pempty + a * 8, kBsEpilogueWarps);
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        if (p.c_tma_ok) ptx::prefetch_tensormap(&tmap_c);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            uint32_t stage = 0;
            uint32_t blk = 0;               // running K-block count
            uint32_t prev = kBsDone - STAGES, prev_phase = 1;  // done[] slot of block blk - STAGES and its parity
            bool ok = true;
            for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
                int m_blk, n_blk;
                bs_decode(w, p, m_blk, n_blk);
                for (int kb = 0; kb < p.kb_total; ++kb, ++blk) {
                    // the stage is free once the block that used it last (blk - STAGES) has been multiplied, and the
                    // partial this block goes into (blk % P) once the rescale warps have drained block blk - P
                    if (!wait_bounded(bar_done + prev * 8, prev_phase, abort_flag, p.status, ROLE_PRODUCER, kb)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = bar_full + stage * 8;
                    ptx::mbar_arrive_expect_tx(full, L::kAStage + L::kBStage);
                    ptx::tma_load_2d(smem_a + stage * L::kAStage, &tmap_a, full, kb * BK, m_blk * kBM);
                    ptx::tma_load_2d(smem_b + stage * L::kBStage, &tmap_b, full, kb * BK, n_blk * BN);
                    if (++prev == kBsDone) {
                        prev = 0;
                        prev_phase ^= 1u;
                    }
                    if (++stage == STAGES) stage = 0;
                }
            }
        }
    } else if (warp == 1 || warp == kBsIssuerB) {
        // ------------------------------------------------------------ MMA issuers: one partial per K block; warp 1
        // takes the even blocks and warp kBsIssuerB the odd ones. Blocks go into different partials, so their MMAs
        // are independent, and each tcgen05.commit tracks the MMAs of its own thread only.
        const uint32_t my_parity = warp == 1 ? 0u : 1u;
        if (ptx::elect_one()) {
            uint32_t stage = 0, phase = 0;
            uint32_t blk = 0;   // running K-block count: partial buffer blk % P
            uint32_t slot = 0;  // blk % 12
            bool ok = true;
            for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
                for (int kb = 0; kb < p.kb_total; ++kb, ++blk) {
                    const uint32_t buf = blk & PMASK;
                    if ((blk & 1u) == my_parity) {
                        // the partial was drained four blocks ago, so it is normally free already (one try_wait)
                        if (!wait_bounded(bar_pempty + buf * 8, ((blk >> PSHIFT) & 1u) ^ 1u, abort_flag, p.status, ROLE_MMA,
                                          -1 - kb) ||
                            !wait_bounded(bar_full + stage * 8, phase, abort_flag, p.status, ROLE_MMA, kb)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint64_t a_desc = ptx::make_kmajor_sw128_desc(smem_a + stage * L::kAStage);
                        const uint64_t b_desc = ptx::make_kmajor_sw128_desc(smem_b + stage * L::kBStage);
                        const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            ptx::umma_ss<ptx::KIND_F8>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc, k > 0 ? 1u : 0u);
                        ptx::tc_commit(bar_done + slot * 8);
                    }
                    if (++slot == kBsDone) slot = 0;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ rescale + accumulate + store (warps 2..9)
        const int quad = warp & 3;              // tensor-memory lane quadrant
        const int half = (warp - 2) >> 2;       // which 64 of the tile's 128 columns
        constexpr int CPW = kBsColsPerWarp;
        uint32_t blk = 0;
        uint32_t slot = 0, slot_phase = 0;  // done[] slot of block blk and its parity
        bool ok = true;
        for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
            int m_blk, n_blk;
            bs_decode(w, p, m_blk, n_blk);
            const int row0 = m_blk * kBM + quad * 32;
            const int row = row0 + lane;
            const bool row_ok = row < p.M;
            float acc[CPW];
#pragma unroll
            for (int j = 0; j < CPW; ++j) acc[j] = 0.0f;
            // scales are fetched one K block ahead so that their latency never sits between a partial and its FMAs
            float sa_next = row_ok ? __ldg(p.a_scale + row) : 0.0f;
            float sb_next = __ldg(p.b_scale + n_blk);
            for (int kb = 0; kb < p.kb_total; ++kb, ++blk) {
                const uint32_t buf = blk & PMASK;
                const float sa = sa_next, sb = sb_next;
                if (kb + 1 < p.kb_total) {
                    sa_next = row_ok ? __ldg(p.a_scale + static_cast<long long>(kb + 1) * p.M + row) : 0.0f;
                    sb_next = __ldg(p.b_scale + static_cast<long long>(kb + 1) * p.n_scale_blocks + n_blk);
                }
                if (!wait_bounded(bar_done + slot * 8, slot_phase, abort_flag, p.status, ROLE_EPILOGUE, kb)) {
                    ok = false;
                    break;
                }
                if (++slot == kBsDone) {
                    slot = 0;
                    slot_phase ^= 1u;
                }
                ptx::tc_fence_after();
                const float s = sa * sb;
                const uint32_t t_addr =
                    tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN + half * CPW;
                uint32_t v0[32], v1[32];
                ptx::tmem_ld_32x32b_x32(t_addr, v0);
                ptx::tmem_ld_32x32b_x32(t_addr + 32, v1);
                ptx::tmem_ld_wait();
                // the partial is in registers: hand the buffer back before the arithmetic
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_pempty + buf * 8);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    acc[j] = fmaf(__uint_as_float(v0[j]), s, acc[j]);
                    acc[32 + j] = fmaf(__uint_as_float(v1[j]), s, acc[32 + j]);
                }
            }
            if (!ok) break;
            // ---- round and store this warp's 32 rows x 64 columns
            constexpr int OB = OutBytes<OUT>::value;
            constexpr int CW = 128 / OB;  // columns per 128-byte chunk
#pragma unroll
            for (int c = 0; c < CPW / CW; ++c) {
                const int n0 = n_blk * BN + half * CPW + c * CW;
                if (n0 >= p.N) break;
                uint32_t u[32];
                if constexpr (OUT == OUT_F32) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) u[j] = __float_as_uint(acc[c * 32 + j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if constexpr (OUT == OUT_BF16) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                            u[j] = *reinterpret_cast<uint32_t*>(&h);
                        } else {
                            __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
                            u[j] = *reinterpret_cast<uint32_t*>(&h);
                        }
                    }
                }
                if (p.c_tma_ok) {
                    if (row0 < p.M) {
                        // one 4 KB staging buffer per warp: the previous store must have read it
                        if (lane == 0) ptx::tma_store_wait_read<0>();
                        __syncwarp();
                        const uint32_t stage_base = smem_base + L::kOutOffset + (warp - 2) * 4096;
                        const uint32_t row_addr = stage_base + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            ptx::st_shared_v4(row_addr + static_cast<uint32_t>((j ^ (lane & 7)) * 16), u[4 * j],
                                              u[4 * j + 1], u[4 * j + 2], u[4 * j + 3]);
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (ptx::elect_one()) {
                            ptx::tma_store_3d(&tmap_c, stage_base, n0, row0, 0);
                            ptx::tma_store_commit();
                        }
                    }
                } else if (row_ok) {
                    // unaligned C: predicated element stores
                    uint8_t* dst = reinterpret_cast<uint8_t*>(p.C) + (static_cast<long long>(row) * p.ldc + n0) * OB;
#pragma unroll
                    for (int j = 0; j < CW; ++j) {
                        if (n0 + j < p.N) {
                            if constexpr (OB == 4) reinterpret_cast<uint32_t*>(dst)[j] = u[j];
                            else reinterpret_cast<uint16_t*>(dst)[j] =
                                static_cast<uint16_t>((j & 1) ? (u[j >> 1] >> 16) : (u[j >> 1] & 0xffffu));
                        }
                    }
                }
            }
        }
        if (lane == 0) ptx::tma_store_wait_read<0>();
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(20000);
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int OUT>
cudaError_t launch_bs(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const BlockScaleParams& p,
                      int grid, cudaStream_t stream) {
    auto kernel = fp8_blockscale_kernel<OUT>;
    constexpr int smem = BsSmem::kDynamicBytes;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_pdl(kernel, dim3(grid), dim3(kBsThreads), smem, stream, ta, tb, tc, p);
}

}  // namespace

cudaError_t launch_fp8_blockscale(int out_kind, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                                  const BlockScaleParams& p, int grid, cudaStream_t stream) {
    switch (out_kind) {
        case OUT_F32: return launch_bs<OUT_F32>(ta, tb, tc, p, grid, stream);
        case OUT_BF16: return launch_bs<OUT_BF16>(ta, tb, tc, p, grid, stream);
        case OUT_F16: return launch_bs<OUT_F16>(ta, tb, tc, p, grid, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace qgemm
