// Host side of libqgemm.so: argument validation, per-device scratch, TMA tensor maps, tile /
// split-K selection, kernel launches, and the extern "C" entry points declared in include/qgemm.h.
//
// Takes over the role of the reference's launch_bf16_kernel_v{1..5} host templates (grid / block /
// shared-memory arithmetic and the launch, e.g. src/gemm/sm80_gemm_kernel_v4.cu:333-355) and of its
// divisibility-based tile dispatch (src/mix_gemm/hip_mix_gemm_kernel.cpp:442-505), with shape
// heuristics at run time instead of compile-time constexpr configs (src/include/gemm_config.h:30-36).
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "gemm_launch.cuh"
#include "qgemm_internal.h"

namespace qgemm {

namespace {

constexpr int kMaxDevices = 64;

struct DeviceState {
    bool init = false;
    int sm_count = 0;
    int cc_major = 0;
    void* ws = nullptr;
    size_t ws_bytes = 0;
    void* ws_i4 = nullptr;  // int4 operands widened to int8: [A | B]
    size_t ws_i4_bytes = 0;
    int* status = nullptr;
};

std::mutex g_mutex;
DeviceState g_dev[kMaxDevices];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_state(DeviceState** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return QGEMM_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return QGEMM_ERR_UNSUPPORTED;
    DeviceState& s = g_dev[dev];
    if (!s.init) {
        if (cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return QGEMM_ERR_CUDA;
        if (cudaDeviceGetAttribute(&s.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
            return QGEMM_ERR_CUDA;
        if (s.cc_major != 10) return QGEMM_ERR_UNSUPPORTED;  // tcgen05 / tensor memory are sm_100 features
        if (cudaMalloc(&s.status, 64) != cudaSuccess) return QGEMM_ERR_CUDA;
        if (cudaMemset(s.status, 0, 64) != cudaSuccess) return QGEMM_ERR_CUDA;
        s.init = true;
    }
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || fn == nullptr)
            return QGEMM_ERR_CUDA;
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = &s;
    return QGEMM_OK;
}

int ensure_buffer(void** buf, size_t* cap, size_t bytes) {
    if (bytes <= *cap) return QGEMM_OK;
    // Growing: earlier launches may still be using the old buffer.
    if (cudaDeviceSynchronize() != cudaSuccess) return QGEMM_ERR_CUDA;
    if (*buf != nullptr) cudaFree(*buf);
    *buf = nullptr;
    *cap = 0;
    const size_t rounded = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    if (cudaMalloc(buf, rounded) != cudaSuccess) {
        (void)cudaGetLastError();
        return QGEMM_ERR_WORKSPACE;
    }
    *cap = rounded;
    return QGEMM_OK;
}

int ensure_workspace(DeviceState& s, size_t bytes) { return ensure_buffer(&s.ws, &s.ws_bytes, bytes); }

// ---------------------------------------------------------------- tensor maps
struct MapKey {
    const void* ptr;
    uint64_t rows, cols, ld;
    uint32_t box_rows, dtype;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
               dtype == o.dtype;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = reinterpret_cast<uint64_t>(k.ptr);
        auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
        mix(k.rows);
        mix(k.cols);
        mix(k.ld);
        mix(k.box_rows);
        mix(k.dtype);
        return static_cast<size_t>(h);
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// K-major operand [rows, cols=K] with leading dimension ld (elements); box = 128 bytes of K x box_rows,
// 128-byte swizzle, zero fill outside the tensor. kgroup > 1 (cols a whole number of 128-byte blocks): the
// three-dimensional view [128 bytes][rows][K blocks] with a box of kgroup K blocks, which lands in shared memory as
// kgroup consecutive [box_rows][128 bytes] tiles (see GemmParams::kgroup).
int make_operand_map(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, int in_dtype, uint32_t box_rows,
                     CUtensorMap* out, uint32_t kgroup = 1) {
    const MapKey key{ptr, rows, cols, ld, box_rows, static_cast<uint32_t>(in_dtype) + 1000u * kgroup};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
        *out = it->second;
        return QGEMM_OK;
    }
    CUtensorMapDataType dt;
    uint32_t es;
    switch (in_dtype) {
        case QGEMM_DTYPE_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; es = 2; break;
        case QGEMM_DTYPE_FP16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; es = 2; break;
        default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; es = 1; break;
    }
    CUtensorMap m;
    CUresult r;
    if (kgroup > 1) {
        const cuuint64_t dims[3] = {128u / es, rows, cols * es / 128u};
        const cuuint64_t strides[2] = {ld * es, 128u};
        const cuuint32_t box[3] = {128u / es, box_rows, kgroup};
        const cuuint32_t estr[3] = {1, 1, 1};
        r = g_encode(&m, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const cuuint64_t dims[2] = {cols, rows};
        const cuuint64_t strides[1] = {ld * es};
        const cuuint32_t box[2] = {128u / es, box_rows};
        const cuuint32_t estr[2] = {1, 1};
        r = g_encode(&m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return QGEMM_ERR_CUDA;
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, m);
    *out = m;
    return QGEMM_OK;
}

// Output [splits][M][N] (splits == 1 for the final C) with leading dimension ld and slab stride
// M*ld, elements of 2 or 4 bytes; box = 128 bytes of N x 32 rows x 1 slab, 128-byte swizzle. Stores
// through it are clipped at N, at M (per slab) and at the slab count.
int make_output_map(void* ptr, uint64_t M, uint64_t N, uint64_t ld, uint64_t splits, int out_kind, CUtensorMap* out) {
    const MapKey key{ptr, M, N, ld, static_cast<uint32_t>(splits), static_cast<uint32_t>(100 + out_kind)};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
        *out = it->second;
        return QGEMM_OK;
    }
    CUtensorMapDataType dt;
    uint32_t es;
    switch (out_kind) {
        case OUT_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; es = 4; break;
        case OUT_RAW32: dt = CU_TENSOR_MAP_DATA_TYPE_INT32; es = 4; break;
        case OUT_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; es = 2; break;
        default: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; es = 2; break;
    }
    const cuuint64_t dims[3] = {N, M, splits};
    const cuuint64_t strides[2] = {ld * es, M * ld * es};
    const cuuint32_t box[3] = {128u / es, 32u, 1u};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap m;
    const CUresult r = g_encode(&m, dt, 3, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return QGEMM_ERR_CUDA;
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, m);
    *out = m;
    return QGEMM_OK;
}

// ---------------------------------------------------------------- configuration
struct Config {
    int bn, splits, kb_per_split, group_m;
    bool pair;  // two CTAs per 256x256 tile (bn is then 256 and tiles are counted in 256-row units)
    bool wide;  // pair with 512x256 tiles, both accumulators of a CTA in use (gemm_sm100_2cta_wide.cuh)
    int am;     // rows of A loaded per stage (128; 64, 32 or 16 with the lone-CTA kernels when M is that small)
    // Balanced column tiling (GemmParams::bal_units): bal_tiles tile columns of bal_units (+1 for the first
    // bal_wide) sixteen-column units instead of ceil(N / bn) equal ones. bal_tiles == 0: equal tiles.
    int bal_tiles, bal_units, bal_wide;
    // K slices handled inside one launch by clusters of this many CTAs (gemm_sm100_kcluster.cuh); 0 = the slices are
    // separate work items whose partial sums go through scratch and splitk_reduce_kernel.
    int kcluster;
};

int env_int(const char* name) {
    const char* v = std::getenv(name);
    return v ? std::atoi(v) : 0;
}

// The QGEMM_* tuning variables are read once, when the library is loaded (and again by qgemm_reload_env): the
// launch path of a microsecond-scale kernel does not scan the environment.
EnvSettings read_env() {
    EnvSettings e;
    e.tile_n = env_int("QGEMM_TILE_N");
    e.split_k = env_int("QGEMM_SPLIT_K");
    e.group_m = env_int("QGEMM_GROUP_M");
    e.cta_pair = env_int("QGEMM_CTA_PAIR");
    e.relayout_b = env_int("QGEMM_RELAYOUT_B");
    e.max_ctas = env_int("QGEMM_MAX_CTAS");
    e.direct_store = env_int("QGEMM_DIRECT_STORE");
    e.full_a_tile = env_int("QGEMM_FULL_A_TILE");
    const char* tail = std::getenv("QGEMM_TAIL_SPLIT");
    e.tail_split_off = (tail != nullptr && tail[0] == '0') ? 1 : 0;
    e.even_runs = env_int("QGEMM_EVEN_RUNS") > 0 ? 1 : 0;  // 1: the K range of all 256 x 256 pair tiles dealt out evenly
    e.balance = env_int("QGEMM_BALANCE") > 0 ? 1 : 0;
    const char* pf = std::getenv("QGEMM_PREFETCH");
    e.prefetch_off = (pf != nullptr && pf[0] == '0') ? 1 : 0;
    e.prefetch_force = (pf != nullptr && pf[0] == '1') ? 1 : 0;  // experiments: hints wherever the kernel can issue them
    const char* kc = std::getenv("QGEMM_KCLUSTER");
    e.kcluster_off = (kc != nullptr && kc[0] == '0') ? 1 : 0;
    e.kcluster_pair_off = (kc != nullptr && kc[0] == '1') ? 1 : 0;  // 1: the lone-CTA form only, not the CTA-pair form
    const char* eg = std::getenv("QGEMM_EARLY_GROUPS");  // experiments: loads issued ahead of the CTA-wide barrier
    e.early_groups = eg != nullptr ? std::max(0, std::atoi(eg)) : -1;
    const char* ot = std::getenv("QGEMM_ONE_TILE");  // 0: never the one-tile-per-CTA kernel variants
    e.one_tile_off = (ot != nullptr && ot[0] == '0') ? 1 : 0;
    e.kgroup = std::max(0, env_int("QGEMM_KGROUP"));  // 0 = the library's choice, 1 = off, 2 / 4 / 8 = K blocks per load
    e.host_bands = std::max(0, env_int("QGEMM_HOST_BANDS"));
    e.host_bands_n = std::max(0, env_int("QGEMM_HOST_BANDS_N"));
    return e;
}
EnvSettings g_env = read_env();

// One-shot test hook (qgemm_test_arm_skip_load): the next GEMM launched by this process leaves out the loads of
// this K block. -1 = not armed.
int g_test_skip_kb = -1;

// Last-wave split of the CTA-pair kernel. T tiles on S clusters run as T / S full waves plus a last wave of
// R = T % S tiles that keeps only R clusters busy for a whole tile's duration. When R is small, the K range of
// each of those R tiles is cut into `slices` pieces so that R * slices <= S clusters share them: the last wave
// then lasts about 1 / slices of a tile. The slices are further work items of the same persistent launch; their
// 32-bit partial sums go to 256 x 256 scratch slots, and a small second kernel adds them up in slice order (a
// fixed order, so results are reproducible; int8 stays exact), scales and casts.
// Taken only when few clusters would be busy in the last wave (R <= S / 4) and the K blocks saved outweigh the
// partial-sum traffic and the second kernel (kTailOverhead, in the units of estimate()). Measured on B200: bf16
// 2560 x 2048 x 4096 (80 tiles on 74 clusters) 61 -> 51 us; with R = 34 (4096^3) the split gains nothing, because
// the part runs at its power cap and a half-empty last wave simply runs at a higher clock.
constexpr double kPairTimePerKb = 0.93;
constexpr double kPair128TimePerKb = 0.45;  // 256 x 128 pair tiles against 0.56 for a lone 128 x 128 tile
constexpr double kTailOverhead = 16.0;
bool tail_split(long long tiles, int clusters, int kb_total, int* tail_tiles, int* slices, int* kb_per_slice,
                double t_kb = kPairTimePerKb) {
    if (clusters <= 0 || tiles <= clusters) return false;
    const int r = static_cast<int>(tiles % clusters);
    if (r == 0 || 4 * r > clusters) return false;
    const int want = std::min(clusters / r, std::min(kb_total / 4, 16));  // at least 4 K blocks per slice
    if (want < 2) return false;
    const int kbps = (kb_total + want - 1) / want;
    if ((kb_total - kbps) * t_kb <= kTailOverhead) return false;
    *tail_tiles = r;
    *kb_per_slice = kbps;
    *slices = (kb_total + kbps - 1) / kbps;
    return *slices >= 2;
}

// The K range dealt out evenly over the clusters (GemmParams::sk_parts): T tiles of 256 x 256 on S clusters that are not a
// whole number of waves then take T / S tile times of main loop instead of ceil(T / S). Built, exact (tests/
// test_even_runs_gpu.py) and measured on B200, it does not pay and is therefore taken only with QGEMM_EVEN_RUNS=1: every
// cluster has two partial tiles of 256 KB of 32-bit sums to store and the pass that adds them up reads 39 MB, together
// 15-20 us, more than the idle SMs cost (us, whole tiles / even runs: FP8 768 x 3328 x 8192 25.8 / 32.2, 2048^3 10.9 / 29.7,
// 4096^3 51.6 / 74.1; BF16 768 x 3328 x 8192 45.7 / 47.3, 1024 x 2048 x 8192 31.2 / 38.1); on many waves the runs also
// break the tile order that keeps neighbouring tiles in L2 together (FP8 8192^3 345 / 545).
// `pieces_out` = the most pieces a tile can have.
bool even_runs_time(long long tiles, int clusters, int kb_total, double* t_out, int* pieces_out) {
    if (g_env.even_runs <= 0 || clusters <= 0 || tiles <= 0 || tiles % clusters == 0) return false;
    const long long total = tiles * kb_total;
    const long long per_run = total / clusters;
    if (per_run < 8) return false;  // runs of fewer than eight K blocks: set-up and drain outweigh them
    *t_out = 0.0;  // asked for: before all else
    *pieces_out = static_cast<int>((kb_total + per_run - 1) / per_run) + 1;
    return true;
}

// Estimated duration in units of "one 128-byte K block of a 128x256 tile" (about 0.27 us at peak).
// `pair` = CTA pairs on 256x256 tiles (half as many schedulable units, a third fewer bytes per flop).
// `in_cluster` = the K slices of a tile run on the CTAs of one cluster and are added up through distributed shared
// memory (gemm_sm100_kcluster.cuh): no slabs in global memory, no second kernel.
constexpr double kClusterReduceCost = 2.0;
constexpr double kPairClusterReduceCost = 3.0;  // a pair's CTA has 128 x 128 partial sums to put through shared memory
double estimate(int bn, bool pair, int splits, size_t M, size_t N, int kb_total, int sms, int* kbps_out,
                bool allow_tail = false, bool in_cluster = false) {
    const int tile_m = pair ? kPairTileM : kBM;
    const int mt = static_cast<int>((M + tile_m - 1) / tile_m);
    const int nt = static_cast<int>((N + bn - 1) / bn);
    const int kbps = (kb_total + splits - 1) / splits;
    const int real_splits = (kb_total + kbps - 1) / kbps;
    const long long units = static_cast<long long>(mt) * nt * real_splits;
    const int slots = pair ? std::max(1, sms / 2) : sms;
    const long long waves = (units + slots - 1) / slots;
    // time per K block of one unit, and pipeline fill + epilogue drain per unit
    double t_kb, fill;
    if (pair && bn == 128) { t_kb = kPair128TimePerKb; fill = 7.0; }
    else if (pair) { t_kb = kPairTimePerKb; fill = 6.0; }
    else if (bn == 256) { t_kb = 1.0; fill = 6.0; }
    else if (bn == 128) { t_kb = 0.56; fill = 4.5; }   // narrower tiles re-read A relatively more often
    else { t_kb = 0.33; fill = 4.0; }
    double t = static_cast<double>(waves) * (kbps * t_kb + fill);
    int tt = 0, ts = 0, tk = 0;
    if (pair && real_splits == 1 && allow_tail && tail_split(units, slots, kb_total, &tt, &ts, &tk, t_kb))
        t = static_cast<double>(waves - 1) * (kbps * t_kb + fill) + (tk * t_kb + fill) + kTailOverhead;
    else if (pair && bn == kPairTileN && real_splits == 1 && allow_tail) {
        double te = 0.0;
        int pieces = 0;
        if (even_runs_time(units, slots, kb_total, &te, &pieces)) t = te;
    }
    if (real_splits > 1 && in_cluster) {
        // full 128-row tiles have four times the partial sums of a 32-row problem to put through shared memory
        // (measured: FP8 1024 x 512 x 2048 in two slices 6.9 us against 6.0 unsplit, so the split must not be taken there)
        t += pair ? kPairClusterReduceCost : (M > 64 ? 2.0 * kClusterReduceCost : kClusterReduceCost);
    } else if (real_splits > 1) {
        // partial slabs are written once and read once by the second pass (~1.75 MB per unit of time)
        const double slab_bytes = static_cast<double>(real_splits) * M * N * 4.0;
        t += 12.0 + 2.0 * slab_bytes / 1.75e6;
    }
    *kbps_out = kbps;
    return t;
}

// Clusters of `slices` CTAs that run at once: what the device reports, or, without a device (planning queries on a
// machine without a GPU), seven eighths of SMs / slices -- a GPC's SM count is rarely a multiple of the cluster size.
int kcluster_capacity(int slices, int sms) {
    const int n = kcluster_max_clusters(slices);
    return n > 0 ? n : (sms / slices) * 7 / 8;
}

Config choose_config(size_t M, size_t N, int kb_total, int sms, const qgemm_tuning_t* tuning, int min_bn = 64,
                     bool allow_tail = false, int elem_bytes = 1, bool allow_balance = false,
                     bool allow_kcluster = false, bool allow_pair128 = false) {
    int want_bn = tuning ? tuning->tile_n : 0;
    int want_split = tuning ? tuning->split_k : 0;
    int want_group = tuning ? tuning->group_m : 0;
    int want_pair = tuning ? tuning->cta_pair : 0;
    if (!want_bn) want_bn = g_env.tile_n;
    if (!want_split) want_split = g_env.split_k;
    if (!want_group) want_group = g_env.group_m;
    if (!want_pair) want_pair = g_env.cta_pair;

    Config best{256, 1, kb_total, 16, false, false, kBM, 0, 0, 0, 0};
    double best_t = 1e300;
    struct Cand { int bn; bool pair; };
    const Cand cands[] = {{256, true}, {128, true}, {256, false}, {128, false}, {64, false}};
    for (const Cand& c : cands) {
        if (c.pair && (want_pair < 0 || (want_bn && want_bn != c.bn))) continue;
        // 256 x 128 pair tiles: K-major B in memory, one destination, not with the 512 x 256 override, and (unless
        // the caller asks for them) only when all tiles run in one wave -- that is where they were measured against one
        // wave of lone 128 x 128 tiles (us, graph replay over cold operands): BF16 1024 x 2048 x 8192 31.5 / 35.5, 2048 x
        // 1024 x 4096 16.8 / 17.8, 1280 x 1280 x 4096 15.8 / 17.9; FP8 1024 x 2048 x 8192 17.4 / 18.3, 1536 x 1536 x 6144
        // 14.5 / 15.0; over several waves the 256 x 256 pairs win (FP8 4096^3 56.0 against 67.2). One wave and a short
        // last one whose tiles are cut into K slices (tail_split) counts as one wave: such a problem has about 40 tiles of
        // 256 x 256, which leave half the SMs idle. Measured (BF16, planner before / with this form, us): 768 x 3328 x 8192
        // 45.7 / 37.6, 512 x 4864 x 8192 45.1 / 37.8, 1280 x 2048 x 8192 45.8 / 39.3, 1024 x 2560 x 4096 28.0 / 23.9,
        // 512 x 5120 x 5120 30.5 / 28.1; FP8 768 x 3328 x 8192 25.7 / 23.4, 512 x 4864 x
        // 8192 25.4 / 22.9, 1280 x 2048 x 8192 25.6 / 24.6. The gain is far from the factor the idle SMs suggest: per K
        // block a CTA of a 256 x 128 pair moves 56 KB through its shared memory (24 KB in by TMA, 32 KB read by the tensor
        // cores) for 256 cycles of tensor work, a ceiling of 58 % of the tensor pipe (ncu: 54-55 %).
        if (c.pair && c.bn == 128) {
            if (!allow_pair128 || want_pair == 2) continue;
            const long long tiles128 = static_cast<long long>((M + kPairTileM - 1) / kPairTileM) *
                                       static_cast<long long>((N + 127) / 128);
            int tt = 0, ts = 0, tk = 0;
            // With a single row of tiles (M <= 256) whose 256 x 256 tiles fit one wave, those keep the choice: every
            // 256 x 128 tile re-reads the same 256 rows of A (BF16 256 x 10240 x 4096 26.4 us against 28.5, 256 x 11008 x
            // 4096 25.8 against 28.7).
            const long long m_tiles = static_cast<long long>((M + kPairTileM - 1) / kPairTileM);
            const long long tiles256 = m_tiles * static_cast<long long>((N + kPairTileN - 1) / kPairTileN);
            const bool tail_fits = allow_tail && !want_split && tiles128 > sms / 2 && tiles128 < sms &&
                                   (m_tiles >= 2 || tiles256 > sms / 2) &&
                                   tail_split(tiles128, sms / 2, kb_total, &tt, &ts, &tk, kPair128TimePerKb);
            if (!(want_pair > 0 && want_bn == 128) && tiles128 > sms / 2 && !tail_fits) continue;
        }
        if (!c.pair && want_pair > 0) continue;
        if (want_bn && c.bn != want_bn) continue;
        if (c.bn < min_bn) continue;
        const int max_split = want_split ? want_split : std::min(kb_total, 16);
        for (int s = want_split ? want_split : 1; s <= max_split; ++s) {
            if (s > kb_total) break;
            int kbps = 0;
            const double t = estimate(c.bn, c.pair, s, M, N, kb_total, sms, &kbps, allow_tail && !want_split);
            if (!want_split && s > 1 && kbps < 2) continue;
            if (t < best_t) {
                best_t = t;
                best.bn = c.bn;
                best.pair = c.pair;
                best.kb_per_split = kbps;
                best.splits = (kb_total + kbps - 1) / kbps;
                best.kcluster = 0;
            }
            // The same slices inside one launch: 2, 4 or 8 non-empty slices of 64- or 128-wide tiles, as many clusters as the
            // device runs at once (one wave), K-major B, no CTA cap, balanced tiling not switched on. With 64 rows or fewer
            // the 128-wide tile only in four or eight slices (or when the caller asks for it): against 64-wide tiles in half as
            // many slices, the same number of CTAs each pull a quarter fewer bytes (A is shared by twice the columns). Measured
            // over 240 skinny shapes (time of the 128-wide form / the 64-wide one, median): 4 against 2 slices 0.94, 8 against 4
            // 0.91 (BF16) and 0.94 (FP8), with FP8 16 x 3072 x 16384 15.1 -> 12.6 us; 2 slices against one wave of unsplit
            // 64-wide tiles 0.98-0.99 with a spread of +-10 %, so that form is left out. Measured on B200 against the two-launch form at
            // the same split (graph replay over cold operands, us): FP8 32 x 2048 x 8192 7.5 / 8.7, 128 x 2048 x 16384
            // 11.6 / 12.9, 128 x 1024 x 4096 6.1 / 6.9; BF16 32 x 2048 x 8192 10.1 / 11.7, 256 x 1024 x 8192 10.9 / 12.4.
            // CTA pairs on 256 x 128 tiles likewise (gemm_sm100_2cta_kcluster.cuh): 2 or 4 pairs per cluster.
            const bool lone_ok = !c.pair && (c.bn == 64 || (c.bn == 128 && (M > 64 || want_bn == 128 || s >= 4))) &&
                                 (s == 2 || s == 4 || s == 8);
            const bool pair_ok = c.pair && c.bn == 128 && (s == 2 || s == 4) && g_env.kcluster_pair_off == 0;
            if (allow_kcluster && g_env.kcluster_off == 0 && g_env.balance == 0 && (lone_ok || pair_ok) &&
                (kb_total + kbps - 1) / kbps == s && !(tuning && tuning->max_ctas != 0) && g_env.max_ctas == 0) {
                const int tm = c.pair ? kPairTileM : kBM;
                const long long tiles =
                    static_cast<long long>((M + tm - 1) / tm) * static_cast<long long>((N + c.bn - 1) / c.bn);
                if (tiles <= kcluster_capacity(c.pair ? 2 * s : s, sms)) {
                    int kbps2 = 0;
                    const double tc = estimate(c.bn, c.pair, s, M, N, kb_total, sms, &kbps2, false, true);
                    if (tc < best_t) {
                        best_t = tc;
                        best.bn = c.bn;
                        best.pair = c.pair;
                        best.kb_per_split = kbps2;
                        best.splits = s;
                        best.kcluster = s;
                    }
                }
            }
        }
    }
    if (best_t == 1e300) {  // an override asked for something infeasible (e.g. split_k > K blocks)
        best.pair = want_pair > 0;
        best.bn = best.pair ? 256 : ((want_bn == 128 || want_bn == 64) ? want_bn : 256);
        best.splits = 1;
        best.kb_per_split = kb_total;
    }
    // Fewer equal tiles than SMs (skinny M: 16 x 7168 x 2048 has 112 tiles of 64 columns for 148 SMs): deal the
    // sixteen-column units of N out over as many tile columns as there are SMs per tile row, so that every SM pulls
    // the same share of B. Off unless QGEMM_BALANCE=1: measured on B200 (FP8, N = 7168, K = 2048, graph replay over
    // cold operands) it does not pay -- M = 16: 6.62 us either way (the streaming phase of a CTA shortens by 12 %, but
    // with every SM taken the successor's CTAs can no longer start their set-up early); M = 64 and 256: 7.9 vs 6.8 and
    // 11.1 vs 8.1 us, because every further tile column re-reads A from L2 and the tiles' odd widths rule out the
    // TMA-store epilogue. Only for a K-major B, one split, widths up to 128 columns, no explicit tile override.
    if (allow_balance && !best.pair && best.splits == 1 && want_bn == 0 && want_split == 0 && g_env.balance != 0 &&
        !(tuning && tuning->max_ctas != 0) && g_env.max_ctas == 0) {
        const int m_tiles = static_cast<int>((M + kBM - 1) / kBM);
        const long long units = static_cast<long long>((N + 15) / 16);
        const long long cur_tiles = static_cast<long long>((N + best.bn - 1) / best.bn);
        const long long slots = sms / std::max(1, m_tiles);
        if (cur_tiles * m_tiles < sms && slots >= 1) {
            const long long n_ctas = std::max<long long>(1, std::min<long long>(slots, units / 2));  // >= 32 columns
            const long long u = units / n_ctas, r = units % n_ctas;
            const long long wmax = (u + (r > 0 ? 1 : 0)) * 16;
            if (n_ctas > cur_tiles && wmax <= 128) {
                best.bal_tiles = static_cast<int>(n_ctas);
                best.bal_units = static_cast<int>(u);
                best.bal_wide = static_cast<int>(r);
                best.bn = wmax <= 64 ? 64 : 128;
            }
        }
    }
    // Rows of A loaded per stage. The lone-CTA kernels load only the rows that exist, rounded up to 16 / 32 / 64 (the
    // MMA still reads 128 rows; what lies behind the loaded ones only reaches accumulator rows that are never stored):
    // the stages get smaller, so more of them fit and more bytes are in flight, and, what weighs more, the TMA unit
    // does not zero-fill rows beyond M -- with 16 rows or fewer in a 128-row box that fill, not the memory system, sets
    // the pace. Measured on B200 (graph replay over cold operands, us; full box / existing rows): 128-wide tiles FP8
    // 16 x 11008 x 4096 18.0 / 11.2, 1 x 11008 x 4096 18.9 / 11.1, 32 rows 11.7 / 11.2; 256-wide tiles BF16 1 x 28672 x
    // 8192 117.2 / 76.5, 8 x 28672 x 4096 54.5 / 38.7, FP8 1 x 32768 x 8192 54.0 / 43.5, 24 x 28672 x 4096 28.3 / 21.1,
    // BF16 32 x 11008 x 8192 (three K slices) 35.4 / 33.7. With 256-wide tiles 64 rows leave the stage count at four, so
    // that form keeps the full box there.
    best.am = kBM;
    if (!best.pair && g_env.full_a_tile == 0) {
        if (best.bn == 64 || best.bn == 128) best.am = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : kBM));
        else if (best.bn == 256) best.am = M <= 16 ? 16 : (M <= 32 ? 32 : kBM);
    }
    // Tile rows per scheduling group: as many as keep the group's A panel (rows x K bytes) near 32 MiB, so that
    // it stays in L2 while the B panels stream past it.
    // 512 x 256 tiles per CTA pair instead of 256 x 256: a quarter fewer operand bytes from L2 per flop (clock, on a
    // power-capped part) against an epilogue that is no longer hidden behind the next tile. Measured on B200 at 8192^3:
    // bf16 +5 % sustained (1383 against 1314 TFLOP/s; the library GEMM 1371), int8 and fp8 -3 to -14 % (their
    // mainloop per tile is half as long, so the exposed epilogue weighs double), bf16 4096^3 -4 % (two waves of 128
    // tiles), 8192 x 4096 x 8192 -5 % (3.5 waves), 6144 x 7168 x 8192 -1 % (4.5 waves), 8192 x 8192 x 4096 -1 %,
    // 8192 x 8192 x 6144 +1 %, 16384 x 8192 x 8192 +2 %, 8192 x 8192 x 16384 +6 %. So: 16-bit inputs, at least six
    // waves of wide tiles, K deep enough (96 K blocks = 6144 elements). The gain is clock under the power cap: a
    // single launch on an idle GPU is not power-limited and runs faster on the 256 x 256 pairs.
    const long long wide_tiles = static_cast<long long>((M + kWideTileM - 1) / kWideTileM) *
                                 static_cast<long long>((N + kWideTileN - 1) / kWideTileN);
    const bool auto_wide = want_pair == 0 && elem_bytes == 2 && kb_total >= 96 && wide_tiles >= 6ll * (sms / 2);
    best.wide = (want_pair == 2 || auto_wide) && best.pair && best.bn == 256 && best.splits == 1;
    const long long panel_rows = (32ll << 20) / (static_cast<long long>(kb_total) * 128);
    const int tile_m = best.wide ? kWideTileM : (best.pair ? kPairTileM : kBM);
    const int auto_group = static_cast<int>(std::max<long long>(4, std::min<long long>(4096, panel_rows / tile_m)));
    best.group_m = want_group > 0 ? want_group : auto_group;
    return best;
}

struct TypeInfo {
    int kind;       // ptx::KIND_*
    int elem_bytes;
    uint32_t fmt;   // tcgen05 operand format code
    uint32_t cfmt;  // accumulator format code
    bool acc_int;
};

bool type_info(int in_dtype, TypeInfo* t) {
    switch (in_dtype) {
        case QGEMM_DTYPE_BF16: *t = {ptx::KIND_F16, 2, 1u, 1u, false}; return true;
        case QGEMM_DTYPE_FP16: *t = {ptx::KIND_F16, 2, 0u, 1u, false}; return true;
        case QGEMM_DTYPE_INT8: *t = {ptx::KIND_I8, 1, 1u, 2u, true}; return true;
        case QGEMM_DTYPE_FP8_E4M3: *t = {ptx::KIND_F8, 1, 0u, 1u, false}; return true;
        default: return false;
    }
}

int out_kind_of(int out_dtype) {
    switch (out_dtype) {
        case QGEMM_DTYPE_FP32: return OUT_F32;
        case QGEMM_DTYPE_BF16: return OUT_BF16;
        case QGEMM_DTYPE_FP16: return OUT_F16;
        case QGEMM_DTYPE_INT32: return OUT_RAW32;
        default: return -1;
    }
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Plan {
    TypeInfo ti;
    int out_kind;
    int kb_total;
    Config cfg;
    size_t ld_relayout;     // elements; leading dimension of the relaid-out B
    size_t relayout_bytes;  // 0 when B is already K-major
    size_t ldw;             // leading dimension of split-K partial slabs (elements)
    size_t partial_bytes;   // 0 when splits == 1 and there is no last-wave split
    int tail_tiles;         // last-wave split (see tail_split): tiles of the last wave, 0 = off
    int tail_slices;
    int tail_kb_per_slice;
    int kgroup;             // K blocks per TMA instruction (GemmParams::kgroup), 1 = one block per load
    int even_runs;          // clusters the K range of all tiles is dealt out over (GemmParams::sk_parts), 0 = off
    int even_pieces;        // the most pieces a tile has then (depth of the scratch array)
};

// K-grouped loads (GemmParams::kgroup): the lone-CTA kernels on K-major operands whose K is a whole number of 128-byte
// blocks; by default two blocks per TMA instruction with the 64-wide tile. Measured on B200 (graph replay over cold
// operands, us; 1 / 2 / 4 / 8 blocks per instruction): FP8 16 x 7168 x 2048 6.70 / 6.19 / 6.57 / 6.78, BF16 16 x 7168 x
// 2048 10.13 / 8.73 / 8.94 / 9.67, FP8 1024 x 1024 x 4096 10.25 / 8.87 / 10.43 / 13.09, BF16 1024^3 6.78 / 6.14 / 6.75 /
// 7.74: two halve the instruction count, more make the barriers too coarse for the pipeline. With the 128-wide tile
// (16 KB boxes, six stages) it does not pay: FP8 256 x 7168 x 2048 8.08 / 8.41 -- except where its A box is a 2 KB one
// (16 rows, ten stages, lone-CTA and in-cluster kernel alike): FP8 16 x 11008 x 4096
// 11.15 / 10.74, 16 x 9728 x 4096 11.08 / 10.39, 16 x 12288 x 2048 8.01 / 7.52, BF16 16 x 9728 x 4096 18.8 / 17.4; with 32
// rows nothing (FP8 32 x 10240 x 8192 19.17 / 19.12), with the 256-wide tile nothing (14.17 / 14.17).
int choose_kgroup(const Config& cfg, bool b_direct, size_t K, int elem_bytes) {
    if (cfg.pair || b_direct || cfg.bal_tiles != 0 || (K * elem_bytes) % 128 != 0) return 1;
    const int stages = std::min(16, (192 * 1024) / ((cfg.am + cfg.bn) * 128));
    const bool by_default = cfg.bn == 64 || (cfg.bn == 128 && cfg.am <= 16);
    int g = g_env.kgroup > 0 ? g_env.kgroup : (by_default ? 2 : 1);
    if (cfg.bn == 128 && cfg.kcluster != 0 && cfg.am != 16) g = 1;  // there the in-cluster kernel's ring has stages + 1 slots
    if (g != 2 && g != 4 && g != 8) g = 1;
    while (g > 1 && stages % g != 0) g /= 2;
    return g;
}

int make_plan(int in_dtype, int out_dtype, int b_layout, size_t M, size_t N, size_t K, int sms,
              const qgemm_tuning_t* tuning, Plan* p, bool b_direct = false, bool allow_tail = true,
              bool allow_balance = true) {
    if (!type_info(in_dtype, &p->ti)) return QGEMM_ERR_UNSUPPORTED;
    p->out_kind = out_kind_of(out_dtype);
    if (p->out_kind < 0) return QGEMM_ERR_UNSUPPORTED;
    if (p->out_kind == OUT_RAW32 && in_dtype != QGEMM_DTYPE_INT8) return QGEMM_ERR_UNSUPPORTED;
    if (b_layout != QGEMM_B_ROW_MAJOR && b_layout != QGEMM_B_K_MAJOR) return QGEMM_ERR_INVALID_ARG;
    if (M > 0x7fffff00ull || N > 0x7fffff00ull || K > 0x7fffff00ull) return QGEMM_ERR_INVALID_ARG;
    const size_t kblk = 128 / p->ti.elem_bytes;
    p->kb_total = static_cast<int>((K + kblk - 1) / kblk);
    // an 8-bit B read in place comes in 128-column chunks: no 64-wide tiles then
    // The last-wave split is the library's own choice: any explicit split-K, CTA cap or store-path override
    // (argument or environment) turns it off, and so does QGEMM_TAIL_SPLIT=0.
    allow_tail = allow_tail && !(tuning && (tuning->split_k != 0 || tuning->max_ctas != 0)) &&
                 g_env.split_k == 0 && g_env.max_ctas == 0 && g_env.direct_store == 0 && g_env.tail_split_off == 0;
    p->cfg = choose_config(M, N, std::max(p->kb_total, 1), sms, tuning,
                           (b_direct && p->ti.elem_bytes == 1) ? 128 : 64, allow_tail, p->ti.elem_bytes,
                           allow_balance && !b_direct, !b_direct, !b_direct && allow_balance);
    p->ld_relayout = round_up(K, 16 / p->ti.elem_bytes);
    p->relayout_bytes =
        (b_layout == QGEMM_B_ROW_MAJOR && !b_direct) ? round_up(N * p->ld_relayout * p->ti.elem_bytes, 256) : 0;
    p->ldw = round_up(N, 4);
    p->partial_bytes = (p->cfg.splits > 1 && p->cfg.kcluster == 0) ? static_cast<size_t>(p->cfg.splits) * M * p->ldw * 4 : 0;
    p->tail_tiles = p->tail_slices = p->tail_kb_per_slice = 0;
    p->kgroup = choose_kgroup(p->cfg, b_direct, K, p->ti.elem_bytes);
    if (allow_tail && p->cfg.pair && !p->cfg.wide && p->cfg.splits == 1) {
        const long long tiles = static_cast<long long>((M + kPairTileM - 1) / kPairTileM) *
                                static_cast<long long>((N + p->cfg.bn - 1) / p->cfg.bn);
        if (tail_split(tiles, sms / 2, p->kb_total, &p->tail_tiles, &p->tail_slices, &p->tail_kb_per_slice,
                       p->cfg.bn == kPairTileN ? kPairTimePerKb : kPair128TimePerKb))
            p->partial_bytes = static_cast<size_t>(p->tail_slices) * p->tail_tiles * kPairTileM * p->cfg.bn * 4;
        else
            p->tail_tiles = 0;
    }
    p->even_runs = p->even_pieces = 0;
    if (allow_tail && p->tail_tiles == 0 && p->cfg.pair && p->cfg.bn == kPairTileN && !p->cfg.wide && p->cfg.splits == 1 &&
        p->cfg.kcluster == 0) {
        const long long tiles = static_cast<long long>((M + kPairTileM - 1) / kPairTileM) *
                                static_cast<long long>((N + kPairTileN - 1) / kPairTileN);
        double t = 0.0;
        int pieces = 0;
        if (tiles < (1 << 20) && even_runs_time(tiles, sms / 2, p->kb_total, &t, &pieces)) {
            p->even_runs = sms / 2;
            p->even_pieces = pieces;
            p->partial_bytes = static_cast<size_t>(2) * p->even_runs * kPairTileM * kPairTileN * 4;  // two slots per run
        }
    }
    return QGEMM_OK;
}

// The caller holds g_mutex (scratch, tensor-map cache and the kernels' per-device set-up flags have one owner).
int gemm_dispatch_locked(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B,
                         size_t ldb, const float* scale_a, const float* scale_b, void* C, size_t ldc, size_t M,
                         size_t N, size_t K, const qgemm_tuning_t* tuning, cudaStream_t stream,
                         void* const* extra_dsts = nullptr, int n_extra = 0) {
    if (n_extra < 0 || n_extra > kMaxExtraDst || (n_extra > 0 && extra_dsts == nullptr)) return QGEMM_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return QGEMM_OK;
    if (C == nullptr || ldc < N) return QGEMM_ERR_INVALID_ARG;
    for (int d = 0; d < n_extra; ++d)
        if (extra_dsts[d] == nullptr) return QGEMM_ERR_INVALID_ARG;
    // Several destinations: the CTA-pair kernel's shared-memory + TMA-store epilogue is the one that fans a
    // tile out, one K pass per tile.
    qgemm_tuning_t multi_tuning;
    if (n_extra > 0) {
        std::memset(&multi_tuning, 0, sizeof(multi_tuning));
        if (tuning) multi_tuning = *tuning;
        multi_tuning.tile_n = 0;
        multi_tuning.split_k = 1;
        multi_tuning.cta_pair = 1;
        tuning = &multi_tuning;
    }
    if (K > 0 && (A == nullptr || B == nullptr || lda < K)) return QGEMM_ERR_INVALID_ARG;
    if (K > 0 && ldb < (b_layout == QGEMM_B_K_MAJOR ? K : N)) return QGEMM_ERR_INVALID_ARG;

    DeviceState* st = nullptr;
    int rc = get_state(&st);
    if (rc != QGEMM_OK) return rc;

    // A row-major B whose rows TMA can address is fed to the tensor cores in place (MN-major operand).
    TypeInfo ti0;
    if (!type_info(in_dtype, &ti0)) return QGEMM_ERR_UNSUPPORTED;
    const bool want_relayout = (tuning && tuning->relayout_b > 0) || g_env.relayout_b > 0;
    const bool b_direct = b_layout == QGEMM_B_ROW_MAJOR && !want_relayout && K > 0 &&
                          reinterpret_cast<uintptr_t>(B) % 16 == 0 && (ldb * ti0.elem_bytes) % 16 == 0;
    Plan plan;
    rc = make_plan(in_dtype, out_dtype, b_layout, M, N, K, st->sm_count, tuning, &plan, b_direct, n_extra == 0,
                   n_extra == 0);
    if (rc != QGEMM_OK) return rc;
    if (plan.out_kind == OUT_RAW32 && (scale_a != nullptr || scale_b != nullptr)) return QGEMM_ERR_INVALID_ARG;
    const int out_bytes = (plan.out_kind == OUT_BF16 || plan.out_kind == OUT_F16) ? 2 : 4;

    if (K == 0) {  // empty sum: C = 0
        for (int d = 0; d < n_extra; ++d)
            if (cudaMemset2DAsync(extra_dsts[d], ldc * out_bytes, 0, N * out_bytes, M, stream) != cudaSuccess)
                return QGEMM_ERR_CUDA;
        return cudaMemset2DAsync(C, ldc * out_bytes, 0, N * out_bytes, M, stream) == cudaSuccess ? QGEMM_OK
                                                                                                  : QGEMM_ERR_CUDA;
    }
    if (n_extra > 0) {
        if (!plan.cfg.pair || plan.cfg.splits != 1) return QGEMM_ERR_UNSUPPORTED;
        if ((ldc * out_bytes) % 16 != 0 || reinterpret_cast<uintptr_t>(C) % 16 != 0) return QGEMM_ERR_ALIGNMENT;
        for (int d = 0; d < n_extra; ++d)
            if (reinterpret_cast<uintptr_t>(extra_dsts[d]) % 16 != 0) return QGEMM_ERR_ALIGNMENT;
    }

    const int es = plan.ti.elem_bytes;
    if (reinterpret_cast<uintptr_t>(A) % 16 != 0 || (lda * es) % 16 != 0) return QGEMM_ERR_ALIGNMENT;
    if (b_layout == QGEMM_B_K_MAJOR && (reinterpret_cast<uintptr_t>(B) % 16 != 0 || (ldb * es) % 16 != 0))
        return QGEMM_ERR_ALIGNMENT;

    rc = ensure_workspace(*st, plan.relayout_bytes + plan.partial_bytes);
    if (rc != QGEMM_OK) return rc;

    const void* b_kmajor = B;
    size_t ldb_k = ldb;
    if (b_layout == QGEMM_B_ROW_MAJOR && !b_direct) {
        // B arrives N-major: relayout to K-major [N, K] in scratch (rows = K, cols = N on the way in).
        rc = transpose_launch(B, st->ws, K, N, ldb, plan.ld_relayout, es, stream);
        if (rc != QGEMM_OK) return rc;
        b_kmajor = st->ws;
        ldb_k = plan.ld_relayout;
    }

    // The wide pair kernel stores through TMA only: without a C it can address that way, take the 256 x 256 pairs.
    if (plan.cfg.wide && (n_extra > 0 || reinterpret_cast<uintptr_t>(C) % 16 != 0 || (ldc * out_bytes) % 16 != 0 ||
                          g_env.direct_store != 0))
        plan.cfg.wide = false;
    const Config& cfg = plan.cfg;
    const uint32_t kgroup = static_cast<uint32_t>(plan.kgroup);
    CUtensorMap ta, tb;
    rc = make_operand_map(A, M, K, lda, in_dtype, cfg.wide ? 256u : static_cast<uint32_t>(cfg.am), &ta, kgroup);
    if (rc != QGEMM_OK) return rc;
    if (b_direct)  // [K rows, N columns]; one box = 128 bytes of N x one 128-byte K block of rows
        rc = make_operand_map(B, K, N, ldb, in_dtype, 128u / static_cast<uint32_t>(es), &tb);
    else
        rc = make_operand_map(b_kmajor, N, K, ldb_k, in_dtype,
                              cfg.pair ? static_cast<uint32_t>(cfg.bn / 2) : (cfg.bal_tiles > 0 ? static_cast<uint32_t>(cfg.bal_units * 16)
                                                                   : static_cast<uint32_t>(cfg.bn)), &tb, kgroup);
    if (rc != QGEMM_OK) return rc;

    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.K = static_cast<int>(K);
    const int tile_m = cfg.wide ? kWideTileM : (cfg.pair ? kPairTileM : kBM);
    p.m_tiles = static_cast<int>((M + tile_m - 1) / tile_m);
    p.n_tiles = cfg.bal_tiles > 0 ? cfg.bal_tiles : static_cast<int>((N + cfg.bn - 1) / cfg.bn);
    p.bal_units = cfg.bal_tiles > 0 ? cfg.bal_units : 0;
    p.bal_wide = cfg.bal_tiles > 0 ? cfg.bal_wide : 0;
    p.splits = cfg.kcluster > 0 ? 1 : cfg.splits;  // in-cluster slices are not work items
    p.kb_total = plan.kb_total;
    p.kb_per_split = cfg.kb_per_split;
    p.group_m = cfg.group_m;
    p.idesc = ptx::make_idesc(plan.ti.cfmt, plan.ti.fmt, plan.ti.fmt, static_cast<uint32_t>(cfg.wide ? kPairTileM : tile_m),
                              static_cast<uint32_t>(cfg.bn), b_direct ? 1u : 0u);
    p.b_mn_major = b_direct ? 1 : 0;
    p.test_skip_kb = take_test_skip_kb();
    p.kgroup = static_cast<int>(kgroup);
    p.early_groups = g_env.early_groups >= 0 ? g_env.early_groups : 2;
    p.status = st->status;

    int launch_out = plan.out_kind;
    uint8_t* partials = static_cast<uint8_t*>(st->ws) + plan.relayout_bytes;
    if (cfg.splits > 1 && cfg.kcluster == 0) {
        p.C = partials;
        p.ldc = static_cast<long long>(plan.ldw);
        p.split_stride = static_cast<long long>(M) * static_cast<long long>(plan.ldw);
        p.c_vec_ok = 1;
        launch_out = OUT_RAW32;
    } else {
        p.C = C;
        p.ldc = static_cast<long long>(ldc);
        p.split_stride = 0;
        p.scale_a = scale_a;
        p.scale_b = scale_b;
        p.c_vec_ok = (reinterpret_cast<uintptr_t>(C) % 16 == 0) && ((ldc * out_bytes) % 16 == 0);
    }

    // The epilogue goes through shared memory + TMA stores when the destination qualifies for a tensor map.
    CUtensorMap tc;
    std::memset(&tc, 0, sizeof(tc));
    if (cfg.bal_tiles > 0) {
        // balanced tiles store from registers; the third tensor-map slot carries B with the wide tiles' box instead
        rc = make_operand_map(b_kmajor, N, K, ldb_k, in_dtype, static_cast<uint32_t>((cfg.bal_units + 1) * 16), &tc);
        if (rc != QGEMM_OK) return rc;
    } else if (p.c_vec_ok && (n_extra > 0 || g_env.direct_store == 0)) {
        const int map_rc = make_output_map(p.C, M, N, static_cast<uint64_t>(p.ldc), static_cast<uint64_t>(p.splits),
                                           launch_out, &tc);
        p.c_tma_ok = (map_rc == QGEMM_OK) ? 1 : 0;
    }
    ExtraDst extra;
    if (n_extra > 0) {
        if (!p.c_tma_ok) return QGEMM_ERR_CUDA;
        std::memset(&extra, 0, sizeof(extra));
        for (int d = 0; d < n_extra; ++d) {
            rc = make_output_map(extra_dsts[d], M, N, static_cast<uint64_t>(ldc), 1, launch_out, &extra.map[d]);
            if (rc != QGEMM_OK) return rc;
        }
        p.n_extra_dst = n_extra;
    }
    const ExtraDst* extra_arg = n_extra > 0 ? &extra : nullptr;

    const long long work = static_cast<long long>(p.m_tiles) * p.n_tiles * p.splits;
    if (work > 0x7fffffffLL) return QGEMM_ERR_UNSUPPORTED;
    int grid = static_cast<int>(std::min<long long>(work, st->sm_count));
    int cap = tuning ? tuning->max_ctas : 0;
    if (!cap) cap = g_env.max_ctas;
    if (cap > 0) grid = std::min(grid, cap);

    // One tile per CTA, B K-major in memory, and a K loop a little longer than the ring (so that the loads cannot all be
    // in flight at once): let the CTAs pull B towards L2 ahead of the dependency wait. Measured on B200 (FP8, graph
    // replay over cold operands): 256 x 7168 x 2048 (6 stages for 16 K blocks) 7.86 -> 7.19 us; where the whole K loop
    // fits in the ring it changes nothing (16 / 64 x 7168 x 2048: 6.31 -> 6.24, 6.48 -> 6.42 us) or costs a little
    // (1024^3 5.42 -> 5.63 us). For a long K loop the burst of hints gets in the way of the loads themselves and the
    // kernel runs at half speed or worse (FP8 1024 x 2048 x 8192, 64 K blocks: 18.0 us without, 34.3 with; 2048 x 1024 x
    // 4096: 10.6 / 17.8; the same for K slices, BF16 32 x 2048 x 8192 in four: 11.7 / 15.1), hence the upper limit of
    // 16 K blocks and no hints for K slices. With the 64-wide tile (8 or more stages) it does not pay either (FP8
    // 128 x 8192 x 2048: 6.89 us without, 7.37 with): 128-wide tiles only.
    {
        const int stages = std::min(16, (192 * 1024) / ((cfg.am + cfg.bn) * 128));
        const bool can = !cfg.pair && !b_direct && cfg.bal_tiles == 0 && cfg.kcluster == 0 && kgroup == 1 &&
                         work <= st->sm_count;
        if (can && (g_env.prefetch_force != 0 || (cfg.splits == 1 && cfg.bn == 128 && cfg.kb_per_split > stages &&
                                                  cfg.kb_per_split <= 16 && g_env.prefetch_off == 0)))
            p.prefetch_b = 1;
    }

    // One 128-wide tile per CTA: the kernel variant whose staging buffers lie over the ring, with a seventh stage.
    const bool one_tile = g_env.one_tile_off == 0 && !cfg.pair && cfg.kcluster == 0 && cfg.bn == 128 && cfg.am == kBM && cfg.bal_tiles == 0 &&
                          kgroup == 1 && work == static_cast<long long>(grid);
    cudaError_t e;
    const bool tail = cfg.pair && !cfg.wide && plan.tail_tiles > 0 && p.c_tma_ok && n_extra == 0;
    const bool even_runs = cfg.pair && !cfg.wide && !tail && plan.even_runs > 0 && p.c_tma_ok && n_extra == 0 && cfg.bn == kPairTileN;
    p.total_work = static_cast<int>(work);
    if (cfg.kcluster > 0 && cfg.pair) {
        switch (plan.ti.kind) {
            case ptx::KIND_F16: e = launch_gemm_pair_kcluster_f16(launch_out, cfg.kcluster, ta, tb, p, static_cast<int>(work), stream); break;
            case ptx::KIND_I8: e = launch_gemm_pair_kcluster_i8(launch_out, cfg.kcluster, ta, tb, p, static_cast<int>(work), stream); break;
            default: e = launch_gemm_pair_kcluster_f8(launch_out, cfg.kcluster, ta, tb, p, static_cast<int>(work), stream); break;
        }
    } else if (cfg.wide) {
        if (!p.c_tma_ok) return QGEMM_ERR_CUDA;
        int clusters = static_cast<int>(std::min<long long>(work, st->sm_count / 2));
        if (cap > 0) clusters = std::min(clusters, std::max(1, cap / 2));
        switch (plan.ti.kind) {
            case ptx::KIND_F16: e = launch_gemm_wide_f16(launch_out, ta, tb, tc, p, clusters, stream); break;
            case ptx::KIND_I8: e = launch_gemm_wide_i8(launch_out, ta, tb, tc, p, clusters, stream); break;
            default: e = launch_gemm_wide_f8(launch_out, ta, tb, tc, p, clusters, stream); break;
        }
    } else if (cfg.pair) {
        CUtensorMap tws;
        std::memset(&tws, 0, sizeof(tws));
        if (tail) {
            // whole tiles first, then the last wave's tiles as K slices whose partial sums go to scratch slots
            p.tail_begin = static_cast<int>(work) - plan.tail_tiles;
            p.tail_slices = plan.tail_slices;
            p.tail_kb_per_slice = plan.tail_kb_per_slice;
            p.total_work = p.tail_begin + plan.tail_tiles * plan.tail_slices;
            rc = make_output_map(partials, static_cast<uint64_t>(plan.tail_tiles) * kPairTileM, static_cast<uint64_t>(cfg.bn),
                                 static_cast<uint64_t>(cfg.bn), static_cast<uint64_t>(plan.tail_slices), OUT_RAW32, &tws);
            if (rc != QGEMM_OK) return rc;
        }
        if (even_runs) {
            // every cluster one run of K blocks across tile boundaries; a run's partial first and last tile go to its two scratch slots
            p.sk_parts = plan.even_runs;
            p.sk_tiles = static_cast<int>(work);
            const long long per_run = (work * p.kb_total + plan.even_runs - 1) / plan.even_runs;
            p.total_work = plan.even_runs * (static_cast<int>((per_run + p.kb_total - 1) / p.kb_total) + 1);
            rc = make_output_map(partials, static_cast<uint64_t>(2 * plan.even_runs) * kPairTileM, kPairTileN, kPairTileN, 1,
                                 OUT_RAW32, &tws);
            if (rc != QGEMM_OK) return rc;
        }
        int clusters = static_cast<int>(std::min<long long>(p.total_work, st->sm_count / 2));
        if (cap > 0) clusters = std::min(clusters, std::max(1, cap / 2));
        switch (plan.ti.kind) {
            case ptx::KIND_F16: e = launch_gemm_pair_f16(cfg.bn, launch_out, ta, tb, tc, tws, extra_arg, p, clusters, stream, g_env.one_tile_off == 0); break;
            case ptx::KIND_I8: e = launch_gemm_pair_i8(cfg.bn, launch_out, ta, tb, tc, tws, extra_arg, p, clusters, stream, g_env.one_tile_off == 0); break;
            default: e = launch_gemm_pair_f8(cfg.bn, launch_out, ta, tb, tc, tws, extra_arg, p, clusters, stream, g_env.one_tile_off == 0); break;
        }
    } else if (cfg.kcluster > 0) {
        switch (plan.ti.kind) {
            case ptx::KIND_F16: e = launch_gemm_kcluster_f16(cfg.bn, launch_out, cfg.am, cfg.kcluster, ta, tb, p, static_cast<int>(work), stream); break;
            case ptx::KIND_I8: e = launch_gemm_kcluster_i8(cfg.bn, launch_out, cfg.am, cfg.kcluster, ta, tb, p, static_cast<int>(work), stream); break;
            default: e = launch_gemm_kcluster_f8(cfg.bn, launch_out, cfg.am, cfg.kcluster, ta, tb, p, static_cast<int>(work), stream); break;
        }
    } else {
        switch (plan.ti.kind) {
            case ptx::KIND_F16: e = launch_gemm_f16(cfg.bn, launch_out, cfg.am, ta, tb, tc, p, grid, stream, one_tile); break;
            case ptx::KIND_I8: e = launch_gemm_i8(cfg.bn, launch_out, cfg.am, ta, tb, tc, p, grid, stream, one_tile); break;
            default: e = launch_gemm_f8(cfg.bn, launch_out, cfg.am, ta, tb, tc, p, grid, stream, one_tile); break;
        }
    }
    if (e != cudaSuccess) return QGEMM_ERR_CUDA;

    if (tail) {
        // the K slices of the last-wave tiles are in scratch: add them up in slice order, scale, cast, store
        GemmParams tiles = p;
        tiles.tile_offset = p.tail_begin;
        rc = splitk_reduce_tiles_launch(partials, plan.tail_tiles, plan.tail_slices, plan.ti.acc_int, C,
                                        static_cast<long long>(ldc), p.M, p.N, plan.out_kind, scale_a, scale_b, tiles,
                                        cfg.bn, stream);
        if (rc != QGEMM_OK) return rc;
    }

    if (even_runs) {
        GemmParams tiles = p;
        tiles.tile_offset = 0;
        rc = splitk_reduce_runs_launch(partials, plan.ti.acc_int, C, static_cast<long long>(ldc), p.M, p.N, plan.out_kind,
                                       scale_a, scale_b, tiles, stream);
        if (rc != QGEMM_OK) return rc;
    }

    if (cfg.splits > 1 && cfg.kcluster == 0) {
        rc = splitk_reduce_launch(partials, p.split_stride, p.ldc, cfg.splits, plan.ti.acc_int, C,
                                  static_cast<long long>(ldc), p.M, p.N, plan.out_kind, scale_a, scale_b, stream);
        if (rc != QGEMM_OK) return rc;
    }
    return QGEMM_OK;
}

int gemm_dispatch(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B, size_t ldb,
                  const float* scale_a, const float* scale_b, void* C, size_t ldc, size_t M, size_t N, size_t K,
                  const qgemm_tuning_t* tuning, cudaStream_t stream, void* const* extra_dsts = nullptr,
                  int n_extra = 0) {
    std::lock_guard<std::mutex> lock(g_mutex);
    return gemm_dispatch_locked(in_dtype, out_dtype, b_layout, A, lda, B, ldb, scale_a, scale_b, C, ldc, M, N, K, tuning,
                                stream, extra_dsts, n_extra);
}

// Packed int4 operands: widen both to int8 in their own scratch, then the int8 path (exact int32 sums). The
// lock is held from the moment the scratch pointer is taken until everything that uses it has been enqueued, so
// that another thread's larger int4 call cannot reallocate it in between.
int int4_dispatch(int out_dtype, int b_layout, const void* A, size_t lda, const void* B, size_t ldb,
                  const float* scale_a, const float* scale_b, void* C, size_t ldc, size_t M, size_t N, size_t K,
                  const qgemm_tuning_t* tuning, cudaStream_t stream) {
    if (b_layout != QGEMM_B_K_MAJOR) return QGEMM_ERR_UNSUPPORTED;  // two values share a byte along K only
    if (M == 0 || N == 0) return QGEMM_OK;
    if ((K & 1) || (lda & 1) || (ldb & 1)) return QGEMM_ERR_INVALID_ARG;
    if (K > 0 && (A == nullptr || B == nullptr || lda < K || ldb < K)) return QGEMM_ERR_INVALID_ARG;
    if (M > 0x7fffff00ull || N > 0x7fffff00ull || K > 0x7fffff00ull) return QGEMM_ERR_INVALID_ARG;
    const size_t ldu = round_up(std::max<size_t>(K, 1), 16);
    const size_t a_bytes = round_up(M * ldu, 256), b_bytes = round_up(N * ldu, 256);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState* st = nullptr;
    int rc = get_state(&st);
    if (rc != QGEMM_OK) return rc;
    rc = ensure_buffer(&st->ws_i4, &st->ws_i4_bytes, a_bytes + b_bytes);
    if (rc != QGEMM_OK) return rc;
    int8_t* a8 = static_cast<int8_t*>(st->ws_i4);
    int8_t* b8 = a8 + a_bytes;
    rc = unpack_int4_launch(A, lda, a8, ldu, M, K, stream);
    if (rc != QGEMM_OK) return rc;
    rc = unpack_int4_launch(B, ldb, b8, ldu, N, K, stream);
    if (rc != QGEMM_OK) return rc;
    return gemm_dispatch_locked(QGEMM_DTYPE_INT8, out_dtype, QGEMM_B_K_MAJOR, a8, ldu, b8, ldu, scale_a, scale_b, C, ldc, M, N,
                         K, tuning, stream);
}

int blockscale_dispatch(int out_dtype, int a_layout, int b_layout, const void* A, size_t lda, const void* B,
                        size_t ldb, const float* a_scale, const float* b_scale, void* C, size_t ldc, size_t M, size_t N,
                        size_t K, cudaStream_t stream) {
    if (M == 0 || N == 0) return QGEMM_OK;
    if (A == nullptr || B == nullptr || C == nullptr || a_scale == nullptr || b_scale == nullptr || K == 0)
        return QGEMM_ERR_INVALID_ARG;
    if (a_layout != QGEMM_A_ROW_MAJOR && a_layout != QGEMM_A_COL_MAJOR) return QGEMM_ERR_INVALID_ARG;
    if (b_layout != QGEMM_B_ROW_MAJOR && b_layout != QGEMM_B_K_MAJOR) return QGEMM_ERR_INVALID_ARG;
    if (lda < (a_layout == QGEMM_A_ROW_MAJOR ? K : M) || ldb < (b_layout == QGEMM_B_K_MAJOR ? K : N) || ldc < N)
        return QGEMM_ERR_INVALID_ARG;
    if (M > 0x7fffff00ull || N > 0x7fffff00ull || K > 0x7fffff00ull) return QGEMM_ERR_INVALID_ARG;
    const int out_kind = out_kind_of(out_dtype);
    if (out_kind != OUT_F32 && out_kind != OUT_BF16 && out_kind != OUT_F16) return QGEMM_ERR_UNSUPPORTED;
    const int out_bytes = (out_kind == OUT_F32) ? 4 : 2;

    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState* st = nullptr;
    int rc = get_state(&st);
    if (rc != QGEMM_OK) return rc;

    // Operands that arrive M-major / N-major are relaid out to K-major scratch: [A' | B'].
    const size_t ldk = round_up(K, 16);
    const size_t a_bytes = (a_layout == QGEMM_A_COL_MAJOR) ? round_up(M * ldk, 256) : 0;
    const size_t b_bytes = (b_layout == QGEMM_B_ROW_MAJOR) ? round_up(N * ldk, 256) : 0;
    rc = ensure_workspace(*st, a_bytes + b_bytes);
    if (rc != QGEMM_OK) return rc;
    const void* a_k = A;
    size_t lda_k = lda;
    if (a_layout == QGEMM_A_COL_MAJOR) {
        rc = transpose_launch(A, st->ws, K, M, lda, ldk, 1, stream);  // in: [K rows][M cols] -> out [M][K]
        if (rc != QGEMM_OK) return rc;
        a_k = st->ws;
        lda_k = ldk;
    } else if (reinterpret_cast<uintptr_t>(A) % 16 != 0 || lda % 16 != 0) {
        return QGEMM_ERR_ALIGNMENT;
    }
    const void* b_k = B;
    size_t ldb_k = ldb;
    if (b_layout == QGEMM_B_ROW_MAJOR) {
        void* dst = static_cast<uint8_t*>(st->ws) + a_bytes;
        rc = transpose_launch(B, dst, K, N, ldb, ldk, 1, stream);
        if (rc != QGEMM_OK) return rc;
        b_k = dst;
        ldb_k = ldk;
    } else if (reinterpret_cast<uintptr_t>(B) % 16 != 0 || ldb % 16 != 0) {
        return QGEMM_ERR_ALIGNMENT;
    }

    CUtensorMap ta, tb, tc;
    rc = make_operand_map(a_k, M, K, lda_k, QGEMM_DTYPE_FP8_E4M3, kBM, &ta);
    if (rc != QGEMM_OK) return rc;
    rc = make_operand_map(b_k, N, K, ldb_k, QGEMM_DTYPE_FP8_E4M3, 128u, &tb);
    if (rc != QGEMM_OK) return rc;

    BlockScaleParams p;
    std::memset(&p, 0, sizeof(p));
    p.C = C;
    p.ldc = static_cast<long long>(ldc);
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.K = static_cast<int>(K);
    p.m_tiles = static_cast<int>((M + kBM - 1) / kBM);
    p.n_tiles = static_cast<int>((N + 127) / 128);
    p.kb_total = static_cast<int>((K + 127) / 128);
    p.n_scale_blocks = p.n_tiles;
    p.group_m = g_env.group_m > 0
                    ? g_env.group_m
                    : static_cast<int>(std::max<long long>(4, std::min<long long>(4096, (16ll << 20) / (128ll * p.kb_total * kBM))));
    p.idesc = ptx::make_idesc(1u, 0u, 0u, kBM, 128u);
    p.a_scale = a_scale;
    p.b_scale = b_scale;
    p.status = st->status;
    std::memset(&tc, 0, sizeof(tc));
    if (reinterpret_cast<uintptr_t>(C) % 16 == 0 && (ldc * out_bytes) % 16 == 0 && g_env.direct_store == 0)
        p.c_tma_ok = make_output_map(C, M, N, ldc, 1, out_kind, &tc) == QGEMM_OK ? 1 : 0;

    const long long work = static_cast<long long>(p.m_tiles) * p.n_tiles;
    if (work > 0x7fffffffLL) return QGEMM_ERR_UNSUPPORTED;
    const int grid = static_cast<int>(std::min<long long>(work, st->sm_count));
    return launch_fp8_blockscale(out_kind, ta, tb, tc, p, grid, stream) == cudaSuccess ? QGEMM_OK : QGEMM_ERR_CUDA;
}

}  // namespace

std::mutex& dispatch_mutex() { return g_mutex; }
int take_test_skip_kb() {
    const int kb = g_test_skip_kb;
    g_test_skip_kb = -1;
    return kb;
}
const EnvSettings& env_settings() { return g_env; }

}  // namespace qgemm

// ------------------------------------------------------------------------------------ C-ABI
using namespace qgemm;

extern "C" {

int qgemm_gemm_ex(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B, size_t ldb,
                  const float* scale_a, const float* scale_b, void* C, size_t ldc, size_t M, size_t N, size_t K,
                  const qgemm_tuning_t* tuning, qgemm_stream_t stream) {
    if (in_dtype == QGEMM_DTYPE_INT4)
        return int4_dispatch(out_dtype, b_layout, A, lda, B, ldb, scale_a, scale_b, C, ldc, M, N, K, tuning,
                             static_cast<cudaStream_t>(stream));
    return gemm_dispatch(in_dtype, out_dtype, b_layout, A, lda, B, ldb, scale_a, scale_b, C, ldc, M, N, K, tuning,
                         reinterpret_cast<cudaStream_t>(stream));
}

int qgemm_gemm(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B, size_t ldb,
               void* C, size_t ldc, size_t M, size_t N, size_t K, qgemm_stream_t stream) {
    const bool ok = ((in_dtype == QGEMM_DTYPE_BF16 || in_dtype == QGEMM_DTYPE_FP16) &&
                     (out_dtype == QGEMM_DTYPE_FP32 || out_dtype == QGEMM_DTYPE_BF16 || out_dtype == QGEMM_DTYPE_FP16)) ||
                    ((in_dtype == QGEMM_DTYPE_INT8 || in_dtype == QGEMM_DTYPE_INT4) && out_dtype == QGEMM_DTYPE_INT32);
    if (!ok) return QGEMM_ERR_UNSUPPORTED;
    return qgemm_gemm_ex(in_dtype, out_dtype, b_layout, A, lda, B, ldb, nullptr, nullptr, C, ldc, M, N, K, nullptr, stream);
}

int qgemm_mix_gemm(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B, size_t ldb,
                   const float* scale_a, const float* scale_b, void* C, size_t ldc, size_t M, size_t N, size_t K,
                   qgemm_stream_t stream) {
    if (out_dtype != QGEMM_DTYPE_FP32 && out_dtype != QGEMM_DTYPE_BF16 && out_dtype != QGEMM_DTYPE_FP16)
        return QGEMM_ERR_UNSUPPORTED;
    return qgemm_gemm_ex(in_dtype, out_dtype, b_layout, A, lda, B, ldb, scale_a, scale_b, C, ldc, M, N, K, nullptr, stream);
}

int qgemm_gemm_multi_dst(int in_dtype, int out_dtype, int b_layout, const void* A, size_t lda, const void* B,
                         size_t ldb, const float* scale_a, const float* scale_b, void* const* C_dsts, int n_dsts,
                         size_t ldc, size_t M, size_t N, size_t K, qgemm_stream_t stream) {
    if (C_dsts == nullptr || n_dsts < 1 || n_dsts > QGEMM_MAX_DSTS) return QGEMM_ERR_INVALID_ARG;
    static_assert(QGEMM_MAX_DSTS == kMaxExtraDst + 1, "destination limit");
    if (n_dsts == 1)
        return gemm_dispatch(in_dtype, out_dtype, b_layout, A, lda, B, ldb, scale_a, scale_b, C_dsts[0], ldc, M, N, K,
                             nullptr, static_cast<cudaStream_t>(stream));
    return gemm_dispatch(in_dtype, out_dtype, b_layout, A, lda, B, ldb, scale_a, scale_b, C_dsts[0], ldc, M, N, K,
                         nullptr, static_cast<cudaStream_t>(stream), C_dsts + 1, n_dsts - 1);
}

int qgemm_fp8_block_scaled_gemm(int out_dtype, int a_layout, int b_layout, const void* A, size_t lda, const void* B,
                                size_t ldb, const float* a_scale, const float* b_scale, void* C, size_t ldc, size_t M,
                                size_t N, size_t K, qgemm_stream_t stream) {
    return blockscale_dispatch(out_dtype, a_layout, b_layout, A, lda, B, ldb, a_scale, b_scale, C, ldc, M, N, K,
                               reinterpret_cast<cudaStream_t>(stream));
}

int qgemm_quantize(int in_dtype, int out_dtype, const void* in, size_t ld_in, void* out, size_t ld_out,
                   float* scale_out, float* amax_out, size_t rows, size_t cols, qgemm_stream_t stream) {
    return quantize_launch(in_dtype, out_dtype, in, ld_in, out, ld_out, scale_out, amax_out, rows, cols,
                           reinterpret_cast<cudaStream_t>(stream));
}

int qgemm_transpose(const void* in, void* out, size_t rows, size_t cols, size_t ld_in, size_t ld_out,
                    size_t elem_bytes, qgemm_stream_t stream) {
    return transpose_launch(in, out, rows, cols, ld_in, ld_out, elem_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int qgemm_workspace_reserve(size_t bytes) {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState* st = nullptr;
    int rc = get_state(&st);
    if (rc != QGEMM_OK) return rc;
    return ensure_workspace(*st, bytes);
}

size_t qgemm_workspace_bytes(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    return g_dev[dev].ws_bytes;
}

size_t qgemm_workspace_query(int in_dtype, int b_layout, size_t M, size_t N, size_t K, const qgemm_tuning_t* tuning) {
    if (M == 0 || N == 0 || K == 0) return 0;
    int sms = 148;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_dev[dev].init)
            sms = g_dev[dev].sm_count;
    }
    Plan plan;
    size_t widened = 0;
    if (in_dtype == QGEMM_DTYPE_INT4) {  // both operands widened to int8, then the int8 path
        const size_t ldu = round_up(K, 16);
        widened = round_up(M * ldu, 256) + round_up(N * ldu, 256);
        in_dtype = QGEMM_DTYPE_INT8;
    }
    const int out = (in_dtype == QGEMM_DTYPE_INT8) ? QGEMM_DTYPE_INT32 : QGEMM_DTYPE_FP32;
    if (make_plan(in_dtype, out, b_layout, M, N, K, sms, tuning, &plan) != QGEMM_OK) return 0;
    return plan.relayout_bytes + plan.partial_bytes + widened;
}

int qgemm_plan_query(int in_dtype, int out_dtype, int b_layout, size_t M, size_t N, size_t K,
                     const qgemm_tuning_t* tuning, int* out6) {
    if (out6 == nullptr) return QGEMM_ERR_INVALID_ARG;
    int sms = 148;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_dev[dev].init)
            sms = g_dev[dev].sm_count;
    }
    Plan plan;
    const int rc = make_plan(in_dtype == QGEMM_DTYPE_INT4 ? QGEMM_DTYPE_INT8 : in_dtype, out_dtype, b_layout, M, N,
                             std::max<size_t>(K, 1), sms, tuning, &plan);
    if (rc != QGEMM_OK) return rc;
    out6[0] = plan.cfg.wide ? kWideTileM : (plan.cfg.pair ? kPairTileM : kBM);
    out6[1] = plan.cfg.bn;
    out6[2] = plan.cfg.pair ? 2 : 1;
    out6[3] = plan.cfg.splits;
    out6[4] = plan.tail_tiles;
    out6[5] = plan.tail_slices;
    return QGEMM_OK;
}

int qgemm_plan_query_ex(int in_dtype, int out_dtype, int b_layout, size_t M, size_t N, size_t K,
                        const qgemm_tuning_t* tuning, int* out, int n_out) {
    if (out == nullptr || n_out < 0) return QGEMM_ERR_INVALID_ARG;
    int sms = 148;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_dev[dev].init)
            sms = g_dev[dev].sm_count;
    }
    Plan plan;
    const int rc = make_plan(in_dtype == QGEMM_DTYPE_INT4 ? QGEMM_DTYPE_INT8 : in_dtype, out_dtype, b_layout, M, N,
                             std::max<size_t>(K, 1), sms, tuning, &plan);
    if (rc != QGEMM_OK) return rc;
    const Config& c = plan.cfg;
    const int tile_m = c.wide ? kWideTileM : (c.pair ? kPairTileM : kBM);
    const long long tiles_n = c.bal_tiles > 0 ? c.bal_tiles : static_cast<long long>((N + c.bn - 1) / c.bn);
    long long ctas = static_cast<long long>((M + tile_m - 1) / tile_m) * tiles_n * c.splits * (c.pair ? 2 : 1);
    if (plan.even_runs > 0) ctas = 2LL * plan.even_runs;  // one run of K blocks per cluster, whatever the number of tiles
    const int vals[QGEMM_PLAN_FIELDS] = {
        tile_m, c.bn, c.pair ? 2 : 1, c.splits, plan.tail_tiles, plan.tail_slices, c.bal_tiles,
        c.bal_tiles > 0 ? c.bal_units * 16 : c.bn, c.am, static_cast<int>(std::min<long long>(ctas, sms)), c.kcluster,
        plan.kgroup};
    for (int i = 0; i < n_out && i < QGEMM_PLAN_FIELDS; ++i) out[i] = vals[i];
    return QGEMM_OK;
}

int qgemm_device_status(int* out4) {
    std::lock_guard<std::mutex> lock(g_mutex);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return QGEMM_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return QGEMM_ERR_UNSUPPORTED;
    if (cudaDeviceSynchronize() != cudaSuccess) return QGEMM_ERR_CUDA;
    // Two sets of status words exist per device: the library's own (allocated with its first GEMM on the device) and
    // those of the allocation-free entry point (part of the loaded module). Both are read and cleared; neither is
    // created here, so a process that only ever uses the allocation-free entry point still allocates nothing.
    int host[4] = {0, 0, 0, 0};
    if (g_dev[dev].init) {
        if (cudaMemcpy(host, g_dev[dev].status, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess)
            return QGEMM_ERR_CUDA;
        if (host[0] != 0 && cudaMemset(g_dev[dev].status, 0, 64) != cudaSuccess) return QGEMM_ERR_CUDA;
    }
    int fixed[4] = {0, 0, 0, 0};
    const int rc = static_status_fetch(fixed);
    if (rc != QGEMM_OK) return rc;
    if (host[0] == 0 && fixed[0] != 0) std::memcpy(host, fixed, sizeof(host));
    if (out4 != nullptr) std::memcpy(out4, host, sizeof(host));
    return host[0] != 0 ? QGEMM_ERR_DEVICE_TIMEOUT : QGEMM_OK;
}

int qgemm_reload_env(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_env = read_env();
    return QGEMM_OK;
}

int qgemm_test_arm_skip_load(int k_block) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_test_skip_kb = k_block < 0 ? -1 : k_block;
    return QGEMM_OK;
}

int qgemm_shutdown(void) {
    host_path_shutdown();
    std::lock_guard<std::mutex> lock(g_mutex);
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) return QGEMM_ERR_CUDA;
    for (int d = 0; d < kMaxDevices; ++d) {
        DeviceState& s = g_dev[d];
        if (!s.init) continue;
        cudaSetDevice(d);
        cudaDeviceSynchronize();
        if (s.ws) cudaFree(s.ws);
        if (s.ws_i4) cudaFree(s.ws_i4);
        if (s.status) cudaFree(s.status);
        s = DeviceState();
    }
    cudaSetDevice(cur);
    g_maps.clear();
    return QGEMM_OK;
}

const char* qgemm_status_string(int status) {
    switch (status) {
        case QGEMM_OK: return "ok";
        case QGEMM_ERR_INVALID_ARG: return "invalid argument";
        case QGEMM_ERR_UNSUPPORTED: return "unsupported dtype combination or device";
        case QGEMM_ERR_ALIGNMENT: return "operand not 16-byte aligned (base or leading dimension)";
        case QGEMM_ERR_CUDA: return "CUDA call failed";
        case QGEMM_ERR_WORKSPACE: return "scratch memory unavailable";
        case QGEMM_ERR_DEVICE_TIMEOUT: return "a kernel abandoned a bounded wait";
        default: return "unknown status";
    }
}

int qgemm_version(void) { return 100; }

}  // extern "C"
