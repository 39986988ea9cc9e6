// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M,N] = A[M,K] x B^T   with A K-major ([M,K] row-major) and B K-major ([N,K] row-major).
//
// One CTA per SM loops over output tiles (128 x BN) in a grouped order that keeps the set of
// concurrently processed tiles compact in (m, n) so their A/B panels are shared through L2. Inside
// the CTA three roles run concurrently:
//   warp 0 (one elected lane)  TMA producer: fills a STAGES-deep ring of 128-byte-swizzled
//                              shared-memory tiles, signalling `full[stage]` by transaction bytes;
//   warp 1 (one elected lane)  MMA issuer: tcgen05.mma from shared-memory descriptors into one of
//                              two tensor-memory accumulators, releasing ring slots with
//                              tcgen05.commit -> `empty[stage]` and publishing a finished tile
//                              with tcgen05.commit -> `tmem_full[acc]`;
//   warps 2..5                 epilogue: tcgen05.ld of their 32-lane quadrant, scale + down-cast,
//                              global stores, then `tmem_empty[acc]` so that the mainloop of the
//                              next tile overlaps the epilogue of this one.
//
// This replaces the reference's thread-block-per-tile WMMA / mma.sync kernels
// (src/gemm/sm80_gemm_kernel_v1.cu:73-173 ... src/gemm/sm89_gemm_kernel_v5.cu:133-270) and its
// gmem->smem loaders (src/include/gemm_utils.cuh:61-274). Unlike those it honours lda/ldb/ldc and
// takes any M, N, K >= 1: out-of-range parts of a tile are zero-filled by TMA on the way in and
// masked on the way out.
//
// Every mbarrier wait is bounded: when a wait runs out the CTA records where in `status`, raises a
// shared abort flag that makes every role leave its loop, lets copies in flight land, frees its
// tensor memory and returns, so the context stays usable.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace qgemm {

enum : int { OUT_F32 = 0, OUT_BF16 = 1, OUT_F16 = 2, OUT_RAW32 = 3 };

struct GemmParams {
    void* C;                 // output matrix, or the split-K partial workspace
    long long ldc;           // leading dimension of C in elements
    long long split_stride;  // elements between consecutive split-K slabs (unused when splits == 1)
    int M, N, K;
    int m_tiles, n_tiles, splits;
    int kb_total;      // number of 128-byte K blocks covering K
    int kb_per_split;  // K blocks per split (every split is non-empty)
    int group_m;       // tile rows per scheduling group
    uint32_t idesc;    // tcgen05 instruction descriptor
    const float* scale_a;  // device scalars (may be null = 1.0)
    const float* scale_b;
    int* status;   // device status words: [0] code, [1] cta, [2] role, [3] stage/tile
    int c_vec_ok;  // C base and ldc allow 16-byte vector stores
    int c_tma_ok;  // the C tensor map is valid: the epilogue stores through shared memory + TMA
    int b_mn_major;  // B is read in place as [K,N] row-major (N contiguous): tmap_b is over [K rows, N cols]
    int n_extra_dst;  // further copies of C written by the same epilogue (CTA-pair kernel only, see ExtraDst)
    // Last-wave split (CTA-pair kernel, splits == 1): work items [0, tail_begin) are whole tiles; item
    // tail_begin + u is K slice (u % tail_slices) of tile number tail_begin + u / tail_slices, whose 32-bit partial
    // sums go to 256 x 256 slot (u / tail_slices) of a [tail_slices][slots * 256][256] scratch array instead of C
    // (see tail_split in capi.cu). tail_begin == 0: no such items. total_work counts both kinds.
    int tail_begin;
    int tail_slices;
    int tail_kb_per_slice;
    // K range dealt out evenly (CTA-pair kernel, splits == 1, no last-wave split): the sk_tiles * kb_total K blocks of
    // all tiles, laid end to end in tile order, are cut into sk_parts equal runs; run r is the blocks [r * U / parts,
    // (r + 1) * U / parts). A run covers the end of one tile, whole tiles and the start of another; work item w is
    // piece (w / sk_parts) of run (w % sk_parts), so a launch of sk_parts clusters gives every cluster one run. A piece
    // that is a whole tile is stored to C as usual; the others (at most the first and the last of a run) store 32-bit
    // partial sums to scratch slot [run] if they begin the run, else [sk_parts + run], and splitk_reduce_runs_kernel
    // adds up each tile's pieces in run order. 0 = off.
    int sk_parts;
    int sk_tiles;
    int total_work;
    int tile_offset;  // added to the tile number by decode_tile (the pass that sums the slices locates slot i with it)
    // Balanced column tiling (lone-CTA kernel, K-major B, one wave): instead of n_tiles equal tiles of BN columns,
    // the N / 16 sixteen-column units are dealt out over n_tiles tiles, tile n getting bal_units units, the first
    // bal_wide tiles one more, so that a problem with fewer equal tiles than SMs still gives every SM a tile (and
    // the same share of B to pull from HBM). bal_units == 0: equal tiles. Widths never exceed the kernel's BN.
    int bal_units;
    int bal_wide;
    // Single-wave problems whose K loop is a little longer than the ring (one tile per CTA): before the dependency wait,
    // while the predecessor in the stream is still running, the CTA asks for its B tile to be brought into L2. 0 = off.
    int prefetch_b;
    // K-grouped loads (lone-CTA kernel, K-major A and B, K a whole number of 128-byte blocks): kgroup > 1 makes tmap_a
    // and tmap_b three-dimensional views [128 bytes][rows][K blocks] of the operands, and one TMA instruction brings
    // kgroup consecutive K blocks of a tile into kgroup consecutive ring slots, completing on the first slot's barrier.
    // The TMA unit retires small boxes at a fixed rate per instruction (about 120 cycles each on B200, whatever their
    // size up to several KB), which bounds a skinny problem's 2 KB + 8 KB stages; fewer, larger boxes lift that.
    int kgroup;
    int early_groups;  // groups of loads the producer issues ahead of the CTA-wide barrier (lone-CTA kernel), 0 = none
    int test_skip_kb;  // failure-detection test hook: the producer leaves out the loads of this K block (-1 = none),
                       // so the consumer's bounded wait runs out and the kernel returns through its error path
};

// Tensor maps of further destinations that receive the same output tiles as C: the same [M, N] block at the
// same leading dimension in other buffers, typically the matching column block of every peer GPU's full
// matrix, so that a column-sharded GEMM leaves the gathered matrix on every GPU without a separate all-gather.
// Only stores go there; nothing is ever loaded from a peer.
constexpr int kMaxExtraDst = 7;
struct ExtraDst {
    CUtensorMap map[kMaxExtraDst];
};
struct NoExtraDst {
    int unused;
};

constexpr int kBM = 128;
constexpr int kGemmThreads = 192;
constexpr long long kWaitLimitCycles = 2000000000LL;  // about one second

enum : int { ROLE_PRODUCER = 1, ROLE_MMA = 2, ROLE_EPILOGUE = 3 };
enum : int { DEV_ERR_WAIT_TIMEOUT = 1 };

__device__ __forceinline__ void record_error(int* status, int code, int role, int where) {
    if (status != nullptr && atomicCAS(&status[0], 0, code) == 0) {
        status[1] = static_cast<int>(blockIdx.x);
        status[2] = role;
        status[3] = where;
    }
}

// Returns false when the wait was abandoned (its own limit, or another role's abort). `peer_abort` (CTA-pair
// kernels; 0 = none) is the cluster address of the other CTA's abort flag, raised together with this CTA's.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                             int role, int where, uint32_t peer_abort = 0) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
        if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    // An epilogue warp legitimately waits for a whole mainloop, and when a load or an MMA goes missing its wait
    // starts before the wait that is really stuck: give it twice the limit so the report names the stuck role.
    const long long limit = (role == ROLE_EPILOGUE) ? 2 * kWaitLimitCycles : kWaitLimitCycles;
    uint32_t it = 0;
#pragma unroll 1
    while (!ptx::mbar_try_wait(bar, parity)) {
        if ((++it & 0xffu) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                if (peer_abort != 0) ptx::st_shared_cluster_u32(peer_abort, 1u);
                record_error(status, DEV_ERR_WAIT_TIMEOUT, role, where);
                return false;
            }
        }
    }
    return true;
}

// Diagnostic build only (-DQGEMM_STAMPS): SM cycle counter at points of the lone-CTA kernel's timeline, for the first
// and the last CTA of the grid, read back with qgemm_debug_stamps. Compiled out otherwise.
#ifdef QGEMM_STAMPS
static __device__ long long g_stamps[2][16];
#define QGEMM_STAMP(i)                                                                \
    do {                                                                              \
        if (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1) g_stamps[blockIdx.x == 0 ? 0 : 1][i] = clock64(); \
    } while (0)
#else
#define QGEMM_STAMP(i) \
    do {               \
    } while (0)
#endif

struct TileCoord {
    int m_blk, n_blk, split;
};

// Work item -> tile. Splits of one tile are adjacent; tiles are grouped `group_m` tile-rows at a
// time and walked column by column inside the group (the reference's GROUP_SIZE_M idea,
// src/gemm/sm80_gemm_kernel_v3.cu:170-184, counted here in tile rows, not elements).
__device__ __forceinline__ TileCoord decode_tile(int w, const GemmParams& p) {
    TileCoord t;
    int tile = w / p.splits;
    t.split = w - tile * p.splits;
    tile += p.tile_offset;
    int group_sz = p.group_m * p.n_tiles;
    int g = tile / group_sz;
    int first_m = g * p.group_m;
    int gm = min(p.m_tiles - first_m, p.group_m);
    int r = tile - g * group_sz;
    t.n_blk = r / gm;
    t.m_blk = first_m + (r - t.n_blk * gm);
    return t;
}

// Column origin and width of tile column n_blk (see GemmParams::bal_units).
__device__ __forceinline__ void tile_columns(const GemmParams& p, int n_blk, int bn, int& col0, int& width) {
    if (p.bal_units > 0) {
        col0 = (n_blk * p.bal_units + min(n_blk, p.bal_wide)) * 16;
        width = (p.bal_units + (n_blk < p.bal_wide ? 1 : 0)) * 16;
    } else {
        col0 = n_blk * bn;
        width = bn;
    }
}

// One work item of the CTA-pair kernel: a whole tile, one K slice of a last-wave tile, or one piece of a run
// (GemmParams::sk_parts; kb0 == kb1 marks an empty item).
struct WorkItem {
    TileCoord t;
    int kb0, kb1;  // K blocks [kb0, kb1)
    int slot;      // >= 0: partial sums of slice t.split go to this scratch slot; -1: an ordinary tile
};

// The run (see GemmParams::sk_parts) that holds K block x of the end-to-end order: the largest r with r * U / parts <= x.
__host__ __device__ __forceinline__ int run_of_block(long long x, int parts, long long total) {
    return static_cast<int>(((x + 1) * parts - 1) / total);
}

__device__ __forceinline__ WorkItem decode_work(int w, const GemmParams& p) {
    WorkItem it;
    if (p.sk_parts > 0) {
        const int run = w % p.sk_parts, piece = w / p.sk_parts;
        const long long total = static_cast<long long>(p.sk_tiles) * p.kb_total;
        const int start = static_cast<int>((run * total) / p.sk_parts);
        int pos = start;
        const int end = static_cast<int>(((run + 1) * total) / p.sk_parts);
        int tile = pos / p.kb_total;
        int pe = min(end, (tile + 1) * p.kb_total);
        for (int i = 0; i < piece && pos < end; ++i) {
            pos = pe;
            tile = pos / p.kb_total;
            pe = min(end, (tile + 1) * p.kb_total);
        }
        if (pos >= end) {  // this run has fewer pieces: an empty item, which every role passes over
            it.t = decode_tile(0, p);
            it.slot = -1;
            it.kb0 = it.kb1 = 0;
            return it;
        }
        it.t = decode_tile(tile, p);  // splits == 1: work item number == tile number
        it.kb0 = pos - tile * p.kb_total;
        it.kb1 = pe - tile * p.kb_total;
        if (it.kb0 == 0 && it.kb1 == p.kb_total) {
            it.slot = -1;
        } else {
            it.slot = pos == start ? run : p.sk_parts + run;
            it.t.split = 0;
        }
        return it;
    }
    if (p.tail_begin > 0 && w >= p.tail_begin) {
        const int u = w - p.tail_begin;
        it.slot = u / p.tail_slices;
        const int slice = u - it.slot * p.tail_slices;
        it.t = decode_tile(p.tail_begin + it.slot, p);  // splits == 1 here: work item number == tile number
        it.t.split = slice;
        it.kb0 = slice * p.tail_kb_per_slice;
        it.kb1 = min(p.kb_total, it.kb0 + p.tail_kb_per_slice);
    } else {
        it.t = decode_tile(w, p);
        it.slot = -1;
        it.kb0 = it.t.split * p.kb_per_split;
        it.kb1 = min(p.kb_total, it.kb0 + p.kb_per_split);
    }
    return it;
}

template <int OUT>
struct OutBytes {
    static constexpr int value = (OUT == OUT_BF16 || OUT == OUT_F16) ? 2 : 4;
};

// Writes 32 consecutive columns of one output row: scale, convert, store (16-byte vectors when the
// whole chunk is in range and aligned, predicated scalars otherwise).
template <int KIND, int OUT>
__device__ __forceinline__ void store_chunk(uint8_t* c_base, long long ldc, long long row, int n0, int n_valid,
                                            bool vec_ok, const uint32_t (&v)[32], float alpha) {
    if constexpr (OUT == OUT_RAW32) {
        uint32_t* dst = reinterpret_cast<uint32_t*>(c_base) + row * ldc + n0;
        if (vec_ok && n_valid == 32) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < n_valid) dst[j] = v[j];
        }
    } else {
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            float a = (KIND == ptx::KIND_I8) ? static_cast<float>(static_cast<int>(v[j])) : __uint_as_float(v[j]);
            f[j] = a * alpha;
        }
        if constexpr (OUT == OUT_F32) {
            float* dst = reinterpret_cast<float*>(c_base) + row * ldc + n0;
            if (vec_ok && n_valid == 32) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    reinterpret_cast<float4*>(dst)[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < n_valid) dst[j] = f[j];
            }
        } else {
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if constexpr (OUT == OUT_BF16) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                    pk[j] = *reinterpret_cast<uint32_t*>(&h);
                } else {
                    __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                    pk[j] = *reinterpret_cast<uint32_t*>(&h);
                }
            }
            uint16_t* dst = reinterpret_cast<uint16_t*>(c_base) + row * ldc + n0;
            if (vec_ok && n_valid == 32) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    reinterpret_cast<uint4*>(dst)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < n_valid) dst[j] = static_cast<uint16_t>((j & 1) ? (pk[j >> 1] >> 16) : (pk[j >> 1] & 0xffffu));
            }
        }
    }
}

// Shared-memory staging of the TMA-store epilogue: every epilogue warp owns two 4 KB buffers, each
// one 32-row x 128-byte box in the 128-byte-swizzled layout the C tensor map expects.
constexpr int kEpilogueStagingBytes = 4 * 2 * 4096;

// Drains one accumulator (this warp's 32 rows x BN columns) to C: tcgen05.ld -> scale/convert ->
// swizzled shared memory -> one TMA store per 128-byte-wide column chunk. The store clips rows and
// columns that fall outside C. `buf` alternates between the warp's two staging buffers.
template <int KIND, int OUT, int BN>
__device__ __forceinline__ void epilogue_tma(const CUtensorMap* tmap_c, uint32_t t_addr, int row0, int m_total,
                                             int n_base, int n_total, int split, uint32_t stage_base, int lane,
                                             float alpha, uint32_t& buf, const CUtensorMap* extra = nullptr,
                                             int n_extra = 0) {
    constexpr int OB = OutBytes<OUT>::value;
    constexpr int CW = 128 / OB;  // columns per chunk: 64 (16-bit out) or 32 (32-bit out)
    if (row0 >= m_total) return;  // this warp's 32 rows are all padding (warp-uniform)
#pragma unroll 1
    for (int c = 0; c < BN / CW; ++c) {
        const int n0 = n_base + c * CW;
        if (n0 >= n_total) break;  // warp-uniform
        uint32_t v[CW];
        ptx::tmem_ld_32x32b_x32(t_addr + c * CW, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        if constexpr (CW == 64) ptx::tmem_ld_32x32b_x32(t_addr + c * CW + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        // the buffer about to be overwritten was handed to a TMA store two chunks ago: wait until it was read
        if (ptx::elect_one()) ptx::tma_store_wait_read<1>();
        __syncwarp();
        ptx::tmem_ld_wait();
        uint32_t u[32];  // 8 sixteen-byte units of this row
        if constexpr (OUT == OUT_RAW32) {
#pragma unroll
            for (int j = 0; j < 32; ++j) u[j] = v[j];
        } else {
#pragma unroll
            for (int j = 0; j < CW; ++j) {
                const float a =
                    (KIND == ptx::KIND_I8) ? static_cast<float>(static_cast<int>(v[j])) : __uint_as_float(v[j]);
                v[j] = __float_as_uint(a * alpha);
            }
            if constexpr (OUT == OUT_F32) {
#pragma unroll
                for (int j = 0; j < 32; ++j) u[j] = v[j];
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if constexpr (OUT == OUT_BF16) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                        u[j] = *reinterpret_cast<uint32_t*>(&h);
                    } else {
                        __half2 h = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                        u[j] = *reinterpret_cast<uint32_t*>(&h);
                    }
                }
            }
        }
        const uint32_t row_addr = stage_base + buf * 4096u + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            ptx::st_shared_v4(row_addr + static_cast<uint32_t>((j ^ (lane & 7)) * 16), u[4 * j], u[4 * j + 1],
                              u[4 * j + 2], u[4 * j + 3]);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (ptx::elect_one()) {  // one lane, named so that the compiler keeps the TMA operands in uniform registers
            ptx::tma_store_3d(tmap_c, stage_base + buf * 4096u, n0, row0, split);
            // the same staged box goes to every further destination; one bulk group covers them all
            for (int d = 0; d < n_extra; ++d) ptx::tma_store_3d(extra + d, stage_base + buf * 4096u, n0, row0, split);
            ptx::tma_store_commit();
        }
        buf ^= 1u;
    }
}

// AM = rows of A actually loaded per stage (128, or 64 / 32 when M is that small: the MMA still reads 128 rows,
// the rest being whatever follows in shared memory, which only reaches accumulator rows that are never stored).
// ONE = the CTA is launched for exactly one tile: the epilogue's staging buffers then lie over the start of the ring
// (idle once the tile's last MMA has completed) instead of behind it, and the 32 KB saved hold one more stage -- for
// one wave of tiles what a CTA can have in flight, divided by the latency of a load, is what sets its pace.
template <int BN, int STAGES, int AM = kBM, bool ONE = false>
struct GemmSmem {
    static constexpr int kAStage = AM * 128;
    static constexpr int kBStage = BN * 128;
    static constexpr int kTiles = STAGES * (kAStage + kBStage);
    static_assert(!ONE || kTiles >= kEpilogueStagingBytes, "the staging buffers fit over the ring");
    static constexpr int kOutOffset = ONE ? 0 : kTiles;          // epilogue staging: 4 warps x 2 buffers x 4 KB
    static constexpr int kBarOffset = kTiles + (ONE ? 0 : kEpilogueStagingBytes);  // full[STAGES], empty[STAGES], tfull[2], tempty[2]
    static constexpr int kMiscOffset = kBarOffset + (2 * STAGES + 4) * 8;  // tmem base, abort flag
    static constexpr int kTotal = kMiscOffset + 16;
    static constexpr int kDynamicBytes = kTotal + 1024;          // slack for the 1024-byte alignment
};

template <int KIND, int BN, int STAGES, int OUT, int AM = kBM, bool ONE = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
    using L = GemmSmem<BN, STAGES, AM, ONE>;
    static_assert(STAGES * L::kAStage + (kBM - AM) * 128 <= L::kTiles, "the MMA's 128-row read of A stays inside the tile area");
    constexpr int ELT = (KIND == ptx::KIND_F16) ? 2 : 1;
    constexpr int BK = 128 / ELT;  // elements per 128-byte K block
    constexpr uint32_t TMEM_COLS = 2 * BN;
    static_assert(TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns");
    static_assert(BN % 32 == 0 && BN <= 256, "tile N");

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
    const int total_work = p.m_tiles * p.n_tiles * p.splits;
    if (threadIdx.x == 0) QGEMM_STAMP(0);
    // The successor in the stream may start its own set-up now (it waits for this grid's completion before it touches
    // global memory): every thread says so at once, so that no warp's later work delays it.
    ptx::pdl_launch_dependents();

    // The loads of one K block of one tile into ring slot `stage`.
    auto load_stage = [&](const TileCoord& t, int col0, int width, int kb, uint32_t stage) {
        const uint32_t full = bar_full + stage * 8;
        if (kb == p.test_skip_kb) {
            // test hook: this slot is never filled, so the MMA issuer's wait on it runs out
        } else if (p.bal_units > 0) {
            // tile of `width` columns: tmap_b's box has the narrow tiles' rows, and tmap_c (no TMA store in this
            // mode, see the epilogue) is the same B with a box sixteen rows taller for the wide tiles
            ptx::mbar_arrive_expect_tx(full, L::kAStage + width * 128);
            ptx::tma_load_2d(smem_a + stage * L::kAStage, &tmap_a, full, kb * BK, t.m_blk * kBM);
            ptx::tma_load_2d(smem_b + stage * L::kBStage, width == p.bal_units * 16 ? &tmap_b : &tmap_c, full, kb * BK,
                             col0);
        } else if (p.b_mn_major) {
            ptx::mbar_arrive_expect_tx(full, L::kAStage + L::kBStage);
            ptx::tma_load_2d(smem_a + stage * L::kAStage, &tmap_a, full, kb * BK, t.m_blk * kBM);
            // one box per 128-byte chunk of N: [BK rows of K] x [CHUNK columns]
            constexpr int CHUNK = 128 / ELT;
#pragma unroll
            for (int j = 0; j < BN / CHUNK; ++j)
                ptx::tma_load_2d(smem_b + stage * L::kBStage + j * (BK * 128), &tmap_b, full, col0 + j * CHUNK,
                                 kb * BK);
        } else {
            ptx::mbar_arrive_expect_tx(full, L::kAStage + L::kBStage);
            ptx::tma_load_2d(smem_a + stage * L::kAStage, &tmap_a, full, kb * BK, t.m_blk * kBM);
            ptx::tma_load_2d(smem_b + stage * L::kBStage, &tmap_b, full, kb * BK, col0);
        }
    };
    if (warp == 0) {  // the barriers are set up by the lanes of one warp side by side
        static_assert(STAGES <= 32, "one lane per ring slot");
        if (lane < STAGES) {
            ptx::mbar_init(bar_full + lane * 8, 1);
            ptx::mbar_init(bar_empty + lane * 8, 1);
        }
        if (lane < 2) {
            ptx::mbar_init(bar_tfull + lane * 8, 1);
            ptx::mbar_init(bar_tempty + lane * 8, 4);
        }
        if (lane == 0) *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        if (p.c_tma_ok || p.bal_units > 0) ptx::prefetch_tensormap(&tmap_c);
    }
    if (p.prefetch_b && warp == 2 && static_cast<int>(blockIdx.x) < total_work) {
        // B does not wait for the predecessor: a hint into L2 is harmless even if B were still being written
        const TileCoord t = decode_tile(blockIdx.x, p);
        int col0, width;
        tile_columns(p, t.n_blk, BN, col0, width);
        const int kb0 = t.split * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        for (int kb = kb0 + lane; kb < kb1; kb += 32) ptx::tma_prefetch_l2_2d(&tmap_b, kb * BK, col0);
    }
    // This CTA's first tile is decoded here, while the predecessor in the stream may still be running: the integer
    // divisions of decode_tile would otherwise sit between the predecessor's end and the first load (a skinny problem
    // is one tile per CTA, and its whole body is a few microseconds).
    const TileCoord first_tile =
        static_cast<int>(blockIdx.x) < total_work ? decode_tile(blockIdx.x, p) : TileCoord{0, 0, 0};
    // Likewise everything else the producer needs for its first loads: read from the parameters (constant memory, a
    // miss on first touch) and computed now, so that only the loads themselves follow the dependency wait.
    const int group = p.kgroup > 1 ? p.kgroup : 1;
    const int first_kb0 = first_tile.split * p.kb_per_split;
    const int first_kb1 = min(p.kb_total, first_kb0 + p.kb_per_split);
    int first_col0, first_width;
    tile_columns(p, first_tile.n_blk, BN, first_col0, first_width);
    const int skip_kb = p.test_skip_kb;
    // The loads of `group` K blocks starting at kb into ring slots stage .. stage + group - 1.
    auto load_group = [&](const TileCoord& t, int col0, int width, int kb, uint32_t stage) {
        if (group == 1) {
            load_stage(t, col0, width, kb, stage);
        } else if (!(skip_kb >= kb && skip_kb < kb + group)) {  // test hook: a group never filled
            // one instruction per operand (blocks past the end of K are zero-filled by the copy and never multiplied)
            const uint32_t full = bar_full + stage * 8;
            ptx::mbar_arrive_expect_tx(full, group * (L::kAStage + L::kBStage));
            ptx::tma_load_3d(smem_a + stage * L::kAStage, &tmap_a, full, 0, t.m_blk * kBM, kb);
            ptx::tma_load_3d(smem_b + stage * L::kBStage, &tmap_b, full, 0, col0, kb);
        }
    };
    // The producer (lane 0 of warp 0) does not wait for the rest of the CTA: its barriers are ready (its own warp set
    // them up), the ring is empty, so as soon as the predecessor in the stream is done it sends the first tile's first
    // loads on their way and only then joins the barrier below. Tensor-memory allocation and the barrier itself then
    // overlap the first bytes' flight from HBM (about a microsecond for cold operands) instead of preceding it. Two
    // groups only: issuing a whole ring-full takes longer than that flight (the TMA unit accepts only so many boxes at
    // a time), and the MMA issuer, held at the barrier meanwhile, would start late. The loop state is carried over
    // into the producer's main loop.
    uint32_t prod_stage = 0, prod_phase = 0, prod_filled = 0;
    int prod_kb = first_kb0;
    if (warp == 0) {
        __syncwarp();  // the other lanes' barrier set-up
        // elect_one() names the same lane every time for a full warp, and lets the compiler keep the TMA operands in
        // uniform registers (a plain lane test does not, and the one-block-per-load path issues a fifth slower)
        if (static_cast<int>(blockIdx.x) < total_work && ptx::elect_one()) {
            ptx::pdl_wait();
            QGEMM_STAMP(1);
            while (prod_kb < first_kb1 && prod_filled < static_cast<uint32_t>(min(STAGES, p.early_groups * group))) {
                load_group(first_tile, first_col0, first_width, prod_kb, prod_stage);
                if (prod_kb == first_kb0) QGEMM_STAMP(2);
                if (prod_kb + group >= first_kb1) QGEMM_STAMP(3);
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
    // From here on every thread may touch global memory: the predecessor's results are needed (and must not be
    // overwritten early).
    ptx::pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            uint32_t stage = prod_stage, phase = prod_phase;
            uint32_t filled = prod_filled;  // ring slots handed out so far: the first STAGES are free without asking
            bool ok = true;
            for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
                const bool first = w == static_cast<int>(blockIdx.x);
                const TileCoord t = first ? first_tile : decode_tile(w, p);
                int kb0 = prod_kb, kb1 = first_kb1, col0 = first_col0, width = first_width;  // the first tile: resumed
                if (!first) {
                    kb0 = t.split * p.kb_per_split;
                    kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                    tile_columns(p, t.n_blk, BN, col0, width);
                }
                const int G = group;
                for (int kb = kb0; kb < kb1; kb += G) {
                    if (filled >= static_cast<uint32_t>(STAGES) &&
                        !wait_bounded(bar_empty + stage * 8, phase ^ 1u, abort_flag, p.status, ROLE_PRODUCER, kb)) {
                        ok = false;
                        break;
                    }
                    if (filled < static_cast<uint32_t>(STAGES)) filled += G;
                    load_group(t, col0, width, kb, stage);
                    if (kb + G >= kb1) QGEMM_STAMP(3);
                    stage += G;
                    if (stage >= STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            uint32_t stage = 0, phase = 0;
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x, ++it) {
                const TileCoord t = (w == static_cast<int>(blockIdx.x)) ? first_tile : decode_tile(w, p);
                const int kb0 = t.split * p.kb_per_split;
                const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                const uint32_t acc = it & 1u;
                const uint32_t acc_phase = (it >> 1) & 1u;
                if (!wait_bounded(bar_tempty + acc * 8, acc_phase ^ 1u, abort_flag, p.status, ROLE_MMA, -1)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                uint32_t idesc = p.idesc;
                if (p.bal_units > 0) {  // the instruction's N is this tile's width
                    int col0, width;
                    tile_columns(p, t.n_blk, BN, col0, width);
                    idesc = (idesc & ~(0x3fu << 17)) | (static_cast<uint32_t>(width >> 3) << 17);
                }
                const int G = p.kgroup > 1 ? p.kgroup : 1;
                for (int kb = kb0; kb < kb1; kb += G) {
                    if (!wait_bounded(bar_full + stage * 8, phase, abort_flag, p.status, ROLE_MMA, kb)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    if (kb == kb0) QGEMM_STAMP(4);
                    if (kb + G >= kb1) QGEMM_STAMP(5);
                    const int blocks = min(G, kb1 - kb);  // the K blocks of this barrier: slots stage .. stage + blocks - 1
                    for (int j = 0; j < blocks; ++j) {
                        const uint64_t a_desc = ptx::make_kmajor_sw128_desc(smem_a + (stage + j) * L::kAStage);
                        const uint64_t b_desc =
                            p.b_mn_major ? ptx::make_mnmajor_sw128_desc(smem_b + (stage + j) * L::kBStage, BK * 128)
                                         : ptx::make_kmajor_sw128_desc(smem_b + (stage + j) * L::kBStage);
                        // K step of one MMA in 16-byte units: 32 bytes inside a K-major row, or (32 / ELT) rows of
                        // 128 bytes for an MN-major tile
                        const uint32_t b_step = p.b_mn_major ? static_cast<uint32_t>((32 / ELT) * 128 / 16) : 2u;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per 128-byte block
                            ptx::umma_ss<KIND>(d_tmem, a_desc + 2u * k, b_desc + b_step * k, idesc,
                                               (kb + j > kb0 || k > 0) ? 1u : 0u);
                        }
                    }
                    ptx::tc_commit(bar_empty + stage * 8);
                    stage += G;
                    if (stage >= STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) ptx::tc_commit(bar_tfull + acc * 8);
                QGEMM_STAMP(6);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3;  // tensor-memory lane quadrant this warp may read
        float alpha = 1.0f;
        if constexpr (OUT != OUT_RAW32) {
            if (p.scale_a != nullptr) alpha *= __ldg(p.scale_a);
            if (p.scale_b != nullptr) alpha *= __ldg(p.scale_b);
        }
        uint32_t it = 0;
        uint32_t out_buf = 0;
        for (int w = blockIdx.x; w < total_work; w += gridDim.x, ++it) {
            const TileCoord t = (w == static_cast<int>(blockIdx.x)) ? first_tile : decode_tile(w, p);
            const uint32_t acc = it & 1u;
            const uint32_t acc_phase = (it >> 1) & 1u;
            if (!wait_bounded(bar_tfull + acc * 8, acc_phase, abort_flag, p.status, ROLE_EPILOGUE, w)) break;
            ptx::tc_fence_after();
            if (warp == 2 && lane == 0) QGEMM_STAMP(7);
            const long long row = static_cast<long long>(t.m_blk) * kBM + quad * 32 + lane;
            uint8_t* c_base = reinterpret_cast<uint8_t*>(p.C) +
                              static_cast<long long>(t.split) * p.split_stride * OutBytes<OUT>::value;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
            if (p.bal_units > 0) {
                // balanced tiles end at any multiple of 16 columns: registers -> global, clipped at the tile's end;
                // a warp whose 32 rows are all beyond M has nothing to read or store
                int col0, width;
                tile_columns(p, t.n_blk, BN, col0, width);
                const int n_end = min(p.N, col0 + width);
                if (t.m_blk * kBM + quad * 32 < p.M) {
#pragma unroll 1
                    for (int c = 0; c < BN / 32; ++c) {
                        const int n0 = col0 + c * 32;
                        if (n0 >= n_end) break;  // warp-uniform
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(t_addr + c * 32, v);
                        ptx::tmem_ld_wait();
                        if (row < p.M)
                            store_chunk<KIND, OUT>(c_base, p.ldc, row, n0, min(32, n_end - n0), p.c_vec_ok != 0, v, alpha);
                    }
                }
            } else if (p.c_tma_ok) {
                epilogue_tma<KIND, OUT, BN>(&tmap_c, t_addr, t.m_blk * kBM + quad * 32, p.M, t.n_blk * BN, p.N, t.split,
                                            smem_base + L::kOutOffset + (warp - 2) * 8192, lane, alpha, out_buf);
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int n0 = t.n_blk * BN + c * 32;
                    if (n0 >= p.N) break;  // warp-uniform
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(t_addr + c * 32, v);
                    ptx::tmem_ld_wait();
                    if (row < p.M)
                        store_chunk<KIND, OUT>(c_base, p.ldc, row, n0, min(32, p.N - n0), p.c_vec_ok != 0, v, alpha);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_tempty + acc * 8);
        }
        // the staging buffers must have been read by every TMA store before the CTA (and its shared memory) goes away;
        // the global writes themselves complete with the grid
        if (lane == 0) ptx::tma_store_wait_read<0>();
        if (warp == 2 && lane == 0) QGEMM_STAMP(8);
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) QGEMM_STAMP(9);
    if (*abort_flag != 0) {
        // Let TMA copies and MMAs that were already issued finish before the memory they touch
        // is released.
        for (int i = 0; i < 64; ++i) __nanosleep(20000);
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace qgemm
