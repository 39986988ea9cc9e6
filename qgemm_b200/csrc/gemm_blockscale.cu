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
// reference does per K tile in registers. After the last block the registers are rounded once and
// stored (64 or 128 contiguous bytes per row and warp).
//
// Barriers: full[stage] (TMA bytes landed), done[blk % 12] (one tcgen05.commit per K block: the block has been
// multiplied, which both frees its stage and publishes its partial), pempty[partial] (all sixteen rescale warps
// have the partial in registers). Loads run the whole ring ahead; the MMA issuer waits for a free partial.
//
// What bounds the kernel is the latency of one drain (wake on done[], tcgen05.ld, wait, hand the partial back), not its
// arithmetic: a rescale warp that drains one block per round trip spends about 500 cycles per block, twice the 256
// cycles the tensor cores need for it. So each rescale warp drains TWO blocks per round trip (both loads in flight
// before the one tcgen05.wait::ld), and the 128 columns of a tile are spread over four warps per lane quadrant
// (32 columns each) so that two blocks' worth of registers fit.
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
constexpr int kBsEpilogueWarps = 16;                     // four warps per tensor-memory lane quadrant
constexpr int kBsFirstRescaleWarp = 4;                   // warps 0..3: producer, MMA issuer and two idle warps (one
                                                         // warpgroup, so that it can give its registers away)
constexpr int kBsThreads = 32 * (kBsFirstRescaleWarp + kBsEpilogueWarps);
constexpr int kBsRegsService = 24;                       // registers per thread after setmaxnreg: service warps ...
constexpr int kBsRegsRescale = 120;                      // ... and rescale warps (per SM sub-partition: 24 + 4 x 120 <= 512)
constexpr int kBsColsPerWarp = kBsBN / 4;                // each of the four warps of a quadrant takes 32 columns

struct BsSmem {
    static constexpr int kAStage = 128 * 128;
    static constexpr int kBStage = kBsBN * 128;
    static constexpr int kTiles = kBsStages * (kAStage + kBStage);
    static constexpr int kBarOffset = kTiles;  // full[S], done[12], pempty[P]
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
                      const BlockScaleParams p) {
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
    // The wait for a free partial is the producer's (a load is only issued once the partial its block will be
    // multiplied into has been handed back), so full[stage] stands for both and the issuing thread waits once per
    // block; measured 8-10 % faster than the issuer waiting for the partial itself.
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

    // The sixteen rescale warps hold two K blocks of partial sums plus their accumulators in registers; the four
    // service warps need next to none. Each warpgroup resizes its register allocation accordingly.
    // (The resize sits at the head of each group's own branch: after a join the compiler would have to assume the
    // smaller of the two budgets.)
    if (warp < kBsFirstRescaleWarp) {
      ptx::setmaxnreg_dec<kBsRegsService>();
      if (warp == 0) {
        // ------------------------------------------------------------ TMA producer: runs the whole ring ahead
        if (ptx::elect_one()) {
            uint32_t stage = 0;
            uint32_t prev = kBsDone - STAGES, prev_phase = 1;  // done[] slot of block blk - STAGES and its parity
            bool ok = true;
            for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
                int m_blk, n_blk;
                bs_decode(w, p, m_blk, n_blk);
                for (int kb = 0; kb < p.kb_total; ++kb) {
                    // the stage is free once the block that used it last (blk - STAGES) has been multiplied
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
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer: one partial per K block
        if (ptx::elect_one()) {
            uint32_t stage = 0, phase = 0;
            uint32_t blk = 0;   // running K-block count: partial buffer blk % P
            uint32_t slot = 0;  // blk % 12
            bool ok = true;
            for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
                for (int kb = 0; kb < p.kb_total; ++kb, ++blk) {
                    const uint32_t buf = blk & PMASK;
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
                    if (++slot == kBsDone) slot = 0;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
      }
    } else {
        ptx::setmaxnreg_inc<kBsRegsRescale>();
        // ------------------------------------------------------------ rescale + accumulate + store (warps 4..19)
        // This branch lives within kBsRegsRescale registers with 96 of them holding data (32 accumulators and two
        // blocks of 32 partial sums), so everything else is kept to a few words: the done[] slot and its parity are
        // derived from the running block count, tile coordinates are decoded again where they are needed.
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) +
                               ((warp - kBsFirstRescaleWarp) >> 2) * kBsColsPerWarp;
        uint32_t blk = 0;  // running K-block count: partial blk % 4, done[] slot blk % 12 with parity (blk / 12) & 1
        bool ok = true;
#pragma unroll 1
        for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
            const float* sa_ptr;
            const float* sb_ptr;
            {
                int m_blk, n_blk;
                bs_decode(w, p, m_blk, n_blk);
                const int row = m_blk * kBM + (warp & 3) * 32 + lane;
                sa_ptr = p.a_scale + (row < p.M ? row : 0);
                sb_ptr = p.b_scale + n_blk;
            }
            float acc[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0.0f;
            // two K blocks per round trip: both partials are requested before the one wait
#pragma unroll 1
            for (int pairs = p.kb_total >> 1; pairs > 0; --pairs, blk += 2) {
                const float s0 = __ldg(sa_ptr) * __ldg(sb_ptr);
                const float s1 = __ldg(sa_ptr + p.M) * __ldg(sb_ptr + p.n_scale_blocks);
                sa_ptr += 2 * static_cast<long long>(p.M);
                sb_ptr += 2 * p.n_scale_blocks;
                uint32_t v0[32], v1[32];
                if (!wait_bounded(bar_done + (blk % kBsDone) * 8, (blk / kBsDone) & 1u, abort_flag, p.status,
                                  ROLE_EPILOGUE, static_cast<int>(blk))) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                ptx::tmem_ld_32x32b_x32(t_row + (blk & PMASK) * BN, v0);
                if (!wait_bounded(bar_done + ((blk + 1) % kBsDone) * 8, ((blk + 1) / kBsDone) & 1u, abort_flag, p.status,
                                  ROLE_EPILOGUE, static_cast<int>(blk + 1))) {
                    ok = false;
                    ptx::tmem_ld_wait();
                    break;
                }
                ptx::tc_fence_after();
                ptx::tmem_ld_32x32b_x32(t_row + ((blk + 1) & PMASK) * BN, v1);
                ptx::tmem_ld_wait();
                // both partials are in registers: hand the buffers back before the arithmetic
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(bar_pempty + (blk & PMASK) * 8);
                    ptx::mbar_arrive(bar_pempty + ((blk + 1) & PMASK) * 8);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(v0[j]), s0, acc[j]);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(v1[j]), s1, acc[j]);
            }
            if (ok && (p.kb_total & 1)) {  // odd block count: the last one on its own
                const float s0 = __ldg(sa_ptr) * __ldg(sb_ptr);
                uint32_t v0[32];
                if (!wait_bounded(bar_done + (blk % kBsDone) * 8, (blk / kBsDone) & 1u, abort_flag, p.status,
                                  ROLE_EPILOGUE, static_cast<int>(blk))) {
                    ok = false;
                } else {
                    ptx::tc_fence_after();
                    ptx::tmem_ld_32x32b_x32(t_row + (blk & PMASK) * BN, v0);
                    ptx::tmem_ld_wait();
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar_pempty + (blk & PMASK) * 8);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(v0[j]), s0, acc[j]);
                    ++blk;
                }
            }
            if (!ok) break;
            // ---- round and store this warp's 32 rows x 32 columns: one rounding, straight from registers (64 or
            // 128 contiguous bytes per row; once per tile, against kb_total drains)
            int m_blk, n_blk;
            bs_decode(w, p, m_blk, n_blk);
            const int row = m_blk * kBM + (warp & 3) * 32 + lane;
            const int n0 = n_blk * BN + ((warp - kBsFirstRescaleWarp) >> 2) * kBsColsPerWarp;
            if (row < p.M && n0 < p.N) {
                uint32_t bits[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) bits[j] = __float_as_uint(acc[j]);
                store_chunk<ptx::KIND_F8, OUT>(reinterpret_cast<uint8_t*>(p.C), p.ldc, row, n0, min(32, p.N - n0),
                                               p.c_vec_ok != 0, bits, 1.0f);
            }
        }
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
cudaError_t launch_bs(const CUtensorMap& ta, const CUtensorMap& tb, const BlockScaleParams& p, int grid,
                      cudaStream_t stream) {
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
    return launch_pdl(kernel, dim3(grid), dim3(kBsThreads), smem, stream, ta, tb, p);
}

}  // namespace

cudaError_t launch_fp8_blockscale(int out_kind, const CUtensorMap& ta, const CUtensorMap& tb, const BlockScaleParams& p,
                                  int grid, cudaStream_t stream) {
    switch (out_kind) {
        case OUT_F32: return launch_bs<OUT_F32>(ta, tb, p, grid, stream);
        case OUT_BF16: return launch_bs<OUT_BF16>(ta, tb, p, grid, stream);
        case OUT_F16: return launch_bs<OUT_F16>(ta, tb, p, grid, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace qgemm
