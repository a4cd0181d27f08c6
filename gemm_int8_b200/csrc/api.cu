// C ABI of the library: argument validation, TMA descriptor construction, per-shape dispatch and
// kernel launches.  No libtorch, no device allocation, no synchronisation on the compute path.
#include "../../include/gemm_int8_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <mutex>

#include "k_blockwise.cuh"
#include "k_dense.cuh"
#include "k_quant.cuh"
#include "k_smallm.cuh"
#include "k_dense_splitk.cuh"

namespace {

using namespace gi8;

constexpr int kMaxDevices = 64;
constexpr int64_t kMaxK = 131072;  // |acc| <= 128*128*K must stay below 2^31 (no saturation modelled)

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define GI8_CUDA(call)                                                                               \
    do {                                                                                             \
        cudaError_t e_ = (call);                                                                     \
        if (e_ != cudaSuccess) return fail(GI8_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

// Kernel status word: one instance per device (module-scope device variable).
__device__ uint32_t g_kernel_status;

enum Variant : int { VAR_AUTO = 0, VAR_DENSE_BN256, VAR_DENSE_BN128, VAR_DENSE_BN64, VAR_SMALLM, VAR_SMALLM_CLUSTER, VAR_PAIR };
const char* const kVariantNames[] = {"auto", "dense_bn256", "dense_bn128", "dense_bn64", "smallm", "smallm_cluster", "pair"};
constexpr int kNumVariants = 7;
std::atomic<int> g_forced_variant{VAR_AUTO};

// Tuning knobs from the environment (not part of the ABI; every combination gives bit-identical results).  They are
// read once, when the library is first used, and again only when gi8_reload_env() is called: nothing on the launch
// path calls getenv.
//   GEMM_INT8_GROUP_M    = 1..64   row-blocks per rasterisation band (default: fitted to K)
//   GEMM_INT8_TMA_STORE  = 0       bf16 epilogues store from registers instead of through shared memory + TMA
//   GEMM_INT8_PDL        = 0       no programmatic dependent launch anywhere (small-M kernels, second launches of a GEMM)
//   GEMM_INT8_SPLITS     = n       small-M kernels: number of K splits
//   GEMM_INT8_BW_HALVES  = 1 | 2   blockwise 256-wide tile: MMAs with N = 256, or two column halves with N = 128 (default:
//                                  N = 256 for the one-CTA tile, column halves for the two-CTA tile)
//   GEMM_INT8_BW_ISSUERS = 1 | 2   blockwise kernel without column halves: MMA-issuing threads (default: one for the
//                                  256-wide tile, two for the narrower ones, whose MMAs are issue bound)
//   GEMM_INT8_TAIL_SPLIT = 0 | 1 | 2   never / when the cost model says so (default) / whenever possible hand the last wave
//                                  of a tile grid to a second launch: the split-K kernel (dense entry points; also a whole
//                                  thin grid), narrower tiles over the remaining columns (blockwise entry point)
// and one promise by the host rather than a knob:
//   GEMM_INT8_STATIC_WEIGHTS = 1   the weight operand of the small-M path is not written by the work that directly
//                                  precedes the call in its stream: its first tiles may be requested early
struct Knobs {
    int group_m = 0;
    bool tma_store = true;
    bool pdl = true;
    int splits = 0;
    int bw_halves = 0;   // 0: column halves for the two-CTA tile, N = 256 MMAs for the one-CTA 256-wide tile
    int bw_issuers = 0;  // 0: one for the 256-wide tile, two for the narrower ones
    // The caller promises that the weight operand of the small-M path is not written by the kernel that precedes the
    // call in its stream (weights quantised ahead of time): its first tiles are then requested before that kernel ends.
    bool static_weights = false;
    int tail_split = 1;  // dense kernels: 0 never split K, 1 when the model says it pays, 2 whenever it is possible
};
Knobs g_knobs;
std::once_flag g_knobs_once;

void load_knobs()
{
    Knobs k;
    if (const char* e = getenv("GEMM_INT8_GROUP_M")) {
        const int v = atoi(e);
        if (v >= 1 && v <= 64) k.group_m = v;
    }
    if (const char* e = getenv("GEMM_INT8_TMA_STORE")) k.tma_store = e[0] != '0';
    if (const char* e = getenv("GEMM_INT8_PDL")) k.pdl = e[0] != '0';
    if (const char* e = getenv("GEMM_INT8_SPLITS")) k.splits = atoi(e);
    if (const char* e = getenv("GEMM_INT8_BW_HALVES")) k.bw_halves = atoi(e) == 1 ? 1 : atoi(e) == 2 ? 2 : 0;
    if (const char* e = getenv("GEMM_INT8_BW_ISSUERS")) k.bw_issuers = atoi(e) == 2 ? 2 : atoi(e) == 1 ? 1 : 0;
    if (const char* e = getenv("GEMM_INT8_TAIL_SPLIT")) k.tail_split = atoi(e) == 0 ? 0 : atoi(e) == 2 ? 2 : 1;
    if (const char* e = getenv("GEMM_INT8_STATIC_WEIGHTS")) k.static_weights = e[0] == '1';
    g_knobs = k;
}

const Knobs& knobs()
{
    std::call_once(g_knobs_once, load_knobs);
    return g_knobs;
}

struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    uint32_t* status = nullptr;
    bool attr_set[64] = {};
};

std::mutex g_mutex;
DeviceState g_dev[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_device_state(DeviceState** out)
{
    int dev = 0;
    GI8_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(GI8_ERR_UNSUPPORTED_DEVICE, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        int major = 0, minor = 0;
        GI8_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        GI8_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
        if (major != 10)
            return fail(GI8_ERR_UNSUPPORTED_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev,
                        major, minor);
        GI8_CUDA(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
        void* sym = nullptr;
        GI8_CUDA(cudaGetSymbolAddress(&sym, g_kernel_status));
        st.status = static_cast<uint32_t*>(sym);
        if (!g_encode) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            GI8_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
            if (q != cudaDriverEntryPointSuccess || !fn)
                return fail(GI8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
        st.ready = true;
    }
    *out = &st;
    return GI8_OK;
}

// ---------------------------------------------------------------------------------------------------
// Tensor-map cache.  A tensor map is a pure function of (base pointer, extents, row stride, box, element type), so a
// map built once can be reused for every later call with the same key -- a decode loop calls with the same weight
// pointers thousands of times, and encoding two to ten maps per call is a measurable part of a 6 us kernel.  A stale
// entry cannot be wrong: the same key always encodes to the same descriptor, whatever happened to the memory since.
// 4-way set-associative, 256 sets, guarded by g_mutex; replacement is round-robin within the set.
// ---------------------------------------------------------------------------------------------------
struct MapKey {
    const void* base;
    uint64_t d0, d1, stride_bytes;
    uint32_t box0, box1, kind;  // kind: 0 = int8 operand, 1 = bf16 output, 2 = fp32 output
    bool operator==(const MapKey& o) const
    {
        return base == o.base && d0 == o.d0 && d1 == o.d1 && stride_bytes == o.stride_bytes && box0 == o.box0 &&
               box1 == o.box1 && kind == o.kind;
    }
};
struct MapEntry {
    MapKey key{};
    bool valid = false;
    CUtensorMap map;
};
constexpr int kMapSets = 256, kMapWays = 4;
MapEntry g_map_cache[kMapSets][kMapWays];
uint8_t g_map_next[kMapSets] = {};

int cached_map(CUtensorMap* out, const MapKey& key)
{
    uint64_t h = reinterpret_cast<uintptr_t>(key.base) * 0x9E3779B97F4A7C15ull;
    h ^= (key.d0 * 0xC2B2AE3D27D4EB4Full) ^ (key.d1 * 0x165667B19E3779F9ull) ^ (key.box1 * 0x27D4EB2Full) ^ key.kind;
    const int set = static_cast<int>((h >> 40) % kMapSets);
    std::lock_guard<std::mutex> lock(g_mutex);
    for (int w = 0; w < kMapWays; ++w)
        if (g_map_cache[set][w].valid && g_map_cache[set][w].key == key) {
            *out = g_map_cache[set][w].map;
            return GI8_OK;
        }
    cuuint64_t dims[2] = {key.d0, key.d1};
    cuuint64_t strides[1] = {key.stride_bytes};
    cuuint32_t box[2] = {key.box0, key.box1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r;
    if (key.kind == 0)
        r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(key.base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    else if (key.kind == 2)
        r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(key.base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    else
        r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(key.base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, key.box0 == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GI8_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    MapEntry& e = g_map_cache[set][g_map_next[set]];
    g_map_next[set] = static_cast<uint8_t>((g_map_next[set] + 1) % kMapWays);
    e.key = key, e.map = *out, e.valid = true;
    return GI8_OK;
}

// Tensor map over a row-major int8 matrix [rows, K]: dimension 0 = K (contiguous), dimension 1 = rows.
// Box = 128 bytes of K x box_rows rows, 128-byte swizzle, out-of-range elements read as zero.
int make_operand_map(CUtensorMap* map, const int8_t* base, int64_t rows, int64_t K, int box_rows)
{
    MapKey key{base, static_cast<uint64_t>(K), static_cast<uint64_t>(rows), static_cast<uint64_t>(K),
               static_cast<uint32_t>(kBK), static_cast<uint32_t>(box_rows), 0u};
    return cached_map(map, key);
}

int check_common(const void* x, const void* y, const void* out, int64_t M, int64_t N, int64_t K, int out_align)
{
    if (M < 0 || N < 0 || K < 0) return fail(GI8_ERR_INVALID_ARGUMENT, "negative dimension (M=%lld N=%lld K=%lld)",
                                             (long long)M, (long long)N, (long long)K);
    if (M > INT32_MAX - 256 || N > INT32_MAX - 256)
        return fail(GI8_ERR_UNSUPPORTED_SHAPE, "M and N must be below 2^31 - 256");
    if (K >= kMaxK) return fail(GI8_ERR_UNSUPPORTED_SHAPE, "K=%lld: K must be below %lld", (long long)K, (long long)kMaxK);
    if (K % 16 != 0) return fail(GI8_ERR_UNSUPPORTED_SHAPE, "K=%lld: K must be a multiple of 16", (long long)K);
    if (M == 0 || N == 0) return GI8_OK;
    if (!out) return fail(GI8_ERR_INVALID_ARGUMENT, "null output pointer");
    if (reinterpret_cast<uintptr_t>(out) % out_align) return fail(GI8_ERR_MISALIGNED, "output pointer must be %d-byte aligned", out_align);
    if (K == 0) return GI8_OK;
    if (!x || !y) return fail(GI8_ERR_INVALID_ARGUMENT, "null operand pointer");
    if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(y) % 16)
        return fail(GI8_ERR_MISALIGNED, "x and y must be 16-byte aligned");
    return GI8_OK;
}

// ---------------------------------------------------------------------------------------------------
// Dispatch: picks the tile form for the dense/blockwise kernels (replaces the reference's five-branch shape table,
// csrc/kernels/gemm.cu:136-161).  Model: the persistent grid runs ceil(tiles / slots) waves, and a wave costs the
// form's cycles per K block, fitted on B200 from device-timed runs (8192^3, 2048 x 11008 x 4096, 128..512 x 8192 x
// 8192 and the reference benchmark's layer shapes, timed back to back):
//   dense      256 x 256 two-CTA tile (74 slots) 580 | 128 x 256: 655 | 128 x 128: 465 | 128 x 64: 330
//   blockwise  128 x 256 (N = 256 MMAs, one issuer): 950 | 256 x 256 two-CTA tile (column halves): 920, but only
//              ahead on long runs (16384 x 57344 x 8192: 8.72 against 9.00 ms; 16384 x 8192 x 28672: 4.63 against
//              4.85 ms; level at 8192^3; behind below that), hence its minimum number of waves
//              | 128 x 128: 650 | 128 x 64: 490
// The table is data: kDenseForms / kBlockwiseForms below.  The narrow tiles cost more per column (the tensor-core instruction is issue
// bound below N = 128, and the per-K-block hand-overs do not shrink with the tile) and only pay when the wide tile
// would leave most SMs without work.
// ---------------------------------------------------------------------------------------------------
struct TileForm {
    int bn;
    bool pair;
    double kblock_cycles;
    int min_waves;  // the form is considered only for grids of at least this many waves
};
constexpr TileForm kDenseForms[] = {{256, true, 580.0, 0}, {256, false, 655.0, 0}, {128, false, 465.0, 0}, {64, false, 330.0, 0}};
constexpr TileForm kBlockwiseForms[] = {{256, true, 920.0, 20}, {256, false, 950.0, 0}, {128, false, 650.0, 0}, {64, false, 490.0, 0}};

int pick_bn(int64_t M, int64_t N, int sms, bool blockwise, bool* pair = nullptr, double* cost_per_kb = nullptr)
{
    if (pair) *pair = false;
    const TileForm* forms = blockwise ? kBlockwiseForms : kDenseForms;
    const int n_forms = 4;
    int best = 256;
    double best_cost = 1e300;
    for (int i = 0; i < n_forms; ++i) {
        const TileForm& f = forms[i];
        if (f.pair && !pair) continue;  // the caller has no two-CTA form
        const int tile_m = f.pair ? 2 * kBM : kBM;
        const int64_t tiles = ((M + tile_m - 1) / tile_m) * ((N + f.bn - 1) / f.bn);
        const int64_t slots = f.pair ? sms / 2 : sms;
        const int64_t waves = (tiles + slots - 1) / slots;
        if (waves < f.min_waves) continue;
        // (a wave also pays a fixed part per tile: prologue, epilogue, tile turnover -- about 20 K blocks' worth at
        // K = 4096; the model only ranks forms for one K, so it enters as a small constant)
        const double cost = static_cast<double>(waves) * (f.kblock_cycles + 16.0);
        if (cost < best_cost - 1e-9) {
            best_cost = cost, best = f.bn;
            if (pair) *pair = f.pair;
        }
    }
    if (cost_per_kb) *cost_per_kb = best_cost;
    return best;
}

// Rasterisation band height in row-blocks: the band's slice of x (group_m x 128 x K bytes) is kept near 16 MB so
// that it stays in L2 while the band sweeps over y (fitted on 8192^3, 16384^3 and the K = 4096 layer shapes).
int pick_group_m(int64_t K)
{
    if (knobs().group_m) return knobs().group_m;
    int64_t g = (16ll << 20) / (kBM * (K > 0 ? K : 1));
    if (g < 4) g = 4;
    if (g > 32) g = 32;
    return static_cast<int>(g);
}

// A blockwise tile cannot split K (the accumulation order is part of the result), so a grid of W full waves plus a few
// tiles would pay W + 1 waves.  Where the full waves are whole column bands (W x SMs divisible by the row-block count),
// the columns are split instead: the first launch covers the columns of the W full waves with 128 x 256 tiles, a second
// launch covers the rest with the widest narrower tile that fits one wave -- more CTAs, each costing less per K block
// (cycles of kBlockwiseForms).  The second launch reads nothing the first writes, so it is released as the first one's
// CTAs leave (programmatic dependent launch without a wait before its work; it waits before it ends, see
// BlockwiseParams::pdl_role).  kColumnSplitFixedCycles: set-up and epilogue of the second kernel's CTAs.  Measured on
// B200, L2-cold: 512 x 10240 x 8192 (160 tiles) 75.8 -> 66.6 us, 512 x 57344 x 8192 256 -> 243, 2048 x 10240 x 8192 204 -> 196.
constexpr double kColumnSplitFixedCycles = 10000.0;  // measured: a lone 64-wide launch of 64 K blocks takes 5 us more than its K blocks
struct ColumnSplit {
    bool use;
    int64_t n1;   // columns of the first launch (a multiple of 256)
    int bn_tail;  // tile width of the second launch
};

ColumnSplit plan_column_split(int64_t M, int64_t N, int64_t K, int sms)
{
    ColumnSplit c{};
    if (knobs().tail_split == 0) return c;
    const int64_t tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + 255) / 256;
    const int64_t tiles = tiles_m * tiles_n;
    const int64_t W = tiles / sms, rest = tiles - W * sms;
    if (W == 0 || rest == 0 || (W * sms) % tiles_m != 0) return c;
    const int64_t n1 = (W * sms / tiles_m) * 256;
    const int64_t nt = N - n1;
    if (n1 <= 0 || nt <= 0) return c;
    const int kb = static_cast<int>((K + kBK - 1) / kBK);
    double best = 1e300;
    for (int i = 0; i < 4; ++i) {
        const TileForm& f = kBlockwiseForms[i];
        if (f.pair || f.bn == 256) continue;
        if (tiles_m * ((nt + f.bn - 1) / f.bn) > sms) continue;  // one wave
        if (f.kblock_cycles < best) best = f.kblock_cycles, c.bn_tail = f.bn;
    }
    if (c.bn_tail == 0) return c;
    const double form = kBlockwiseForms[1].kblock_cycles + 16.0;
    const double now = static_cast<double>(W + 1) * form * kb;
    const double split = (static_cast<double>(W) * form + best + 16.0) * kb + kColumnSplitFixedCycles;
    if (knobs().tail_split == 1 && split >= 0.98 * now) return c;
    c.use = true, c.n1 = n1;
    return c;
}

template <typename Kernel>
int ensure_smem(DeviceState* st, int slot, Kernel kernel, size_t bytes)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!st->attr_set[slot]) {
        GI8_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
        st->attr_set[slot] = true;
    }
    return GI8_OK;
}

// Tensor map over the bf16 output [M, N] (row stride ldo elements) for the epilogue's TMA stores: boxes of 32 rows x
// box_cols columns, 64-byte swizzle (32 columns) or 128-byte swizzle (64 columns).
int make_output_map(CUtensorMap* map, void* out, int64_t M, int64_t N, int64_t ldo, int box_cols = 32)
{
    MapKey key{out, static_cast<uint64_t>(N), static_cast<uint64_t>(M), static_cast<uint64_t>(ldo) * 2,
               static_cast<uint32_t>(box_cols), 32u, 1u};
    return cached_map(map, key);
}

template <int BN, int STAGES, int EPI>
int launch_dense(DeviceState* st, int slot, const int8_t* x, const int8_t* y, DenseParams p, cudaStream_t stream)
{
    constexpr size_t kStoreStage = 4 * 2 * 2048;  // four epilogue warps x two 32 x 64-byte blocks
    constexpr size_t smem = static_cast<size_t>(STAGES) * (kBM + BN) * kBK + kStoreStage + 1024;
    auto kernel = dense_gemm_kernel<BN, STAGES, EPI>;
    if (int rc = ensure_smem(st, slot, kernel, smem)) return rc;
    CUtensorMap mx, my, mo;
    if (int rc = make_operand_map(&mx, x, p.M, p.K, kBM)) return rc;
    if (int rc = make_operand_map(&my, y, p.N, p.K, BN)) return rc;
    // bf16 epilogues store through TMA when the output rows are 16-byte aligned
    p.tma_store = (EPI != EPI_RAW_I32) && p.vec_ok && knobs().tma_store;
    if (p.tma_store) {
        if (int rc = make_output_map(&mo, p.out, p.M, p.N, p.ldo)) return rc;
    } else {
        mo = mx;  // unused by the kernel
    }
    p.tiles_m = (p.M + kBM - 1) / kBM;
    p.tiles_n = (p.N + BN - 1) / BN;
    p.group_m = pick_group_m(p.K);
    const int64_t tiles = p.tile_end > 0 ? p.tile_end : static_cast<int64_t>(p.tiles_m) * p.tiles_n;
    const int grid = static_cast<int>(tiles < st->sm_count ? tiles : st->sm_count);
    kernel<<<grid, kDenseThreads, smem, stream>>>(mx, my, mo, p);
    GI8_CUDA(cudaGetLastError());
    return GI8_OK;
}

// Two-CTA form of the dense kernel: 256 x 256 tiles, one CTA pair (2 x 1 x 1 cluster) per tile.
template <int EPI>
int launch_dense_pair(DeviceState* st, int slot, const int8_t* x, const int8_t* y, DenseParams p, cudaStream_t stream)
{
    constexpr int BN = 256, STAGES = 6;
    constexpr size_t kStoreStage = 4 * 2 * 2048;
    constexpr size_t smem = static_cast<size_t>(STAGES) * (kBM + BN / 2) * kBK + kStoreStage + 1024;
    auto kernel = dense_gemm_kernel<BN, STAGES, EPI, true>;
    if (int rc = ensure_smem(st, slot, kernel, smem)) return rc;
    CUtensorMap mx, my, mo;
    if (int rc = make_operand_map(&mx, x, p.M, p.K, kBM)) return rc;
    if (int rc = make_operand_map(&my, y, p.N, p.K, BN / 2)) return rc;
    p.tma_store = (EPI != EPI_RAW_I32) && p.vec_ok && knobs().tma_store;
    if (p.tma_store) {
        if (int rc = make_output_map(&mo, p.out, p.M, p.N, p.ldo)) return rc;
    } else {
        mo = mx;  // unused by the kernel
    }
    p.tiles_m = (p.M + 2 * kBM - 1) / (2 * kBM);
    p.tiles_n = (p.N + BN - 1) / BN;
    p.group_m = pick_group_m(p.K) / 2 > 0 ? pick_group_m(p.K) / 2 : 1;
    const int64_t tiles = p.tile_end > 0 ? p.tile_end : static_cast<int64_t>(p.tiles_m) * p.tiles_n;
    const int pairs = static_cast<int>(tiles < st->sm_count / 2 ? tiles : st->sm_count / 2);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(kDenseThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    GI8_CUDA(cudaLaunchKernelEx(&cfg, kernel, mx, my, mo, p));
    return GI8_OK;
}

// Split-K launch for tiles [tile_begin, tile_begin + units / halves) of the grid described by p (tiles_m, tiles_n,
// group_m as the main launch set them).
template <int EPI>
int launch_dense_splitk(DeviceState* st, int slot, const int8_t* x, const int8_t* y, const DenseParams& p,
                        const SplitKParams& q, cudaStream_t stream)
{
    constexpr size_t smem = static_cast<size_t>(kSplitKStages) * (kBM + kSplitKBN) * kBK + 1024;
    auto kernel = dense_splitk_kernel<EPI>;
    if (int rc = ensure_smem(st, slot, kernel, smem)) return rc;
    CUtensorMap mx, my;
    if (int rc = make_operand_map(&mx, x, p.M, p.K, kBM)) return rc;
    if (int rc = make_operand_map(&my, y, p.N, p.K, kSplitKBN)) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(q.units * q.splits, 1, 1);
    cfg.blockDim = dim3(kDenseThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = q.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = q.after_main ? 2 : 1;
    GI8_CUDA(cudaLaunchKernelEx(&cfg, kernel, mx, my, p, q));
    return GI8_OK;
}

// The last wave of a persistent grid costs as much as a full one however few tiles it holds.  When it is thin -- or
// the whole grid is -- its tiles can go to the split-K kernel instead: `units` 128 x 256 tiles times S K-splits, S the
// largest of 8, 4, 2 that keeps units x S CTAs within the machine and at least two K blocks per split.  Cost model
// in the units of the tile-form table (cycles per K block): split if
//   (waves - 1) x form + kb / S x 655 + fixed < what would run instead.
// The fixed part was fitted on B200 (L2-cold runs): 16000 cycles when the split-K launch is the only one (its ramp-up
// on cold operands, two cluster barriers, 128 KB of partials per CTA through distributed shared memory, stores of 8
// bytes per thread), 20000 when it follows a main launch.  The split-K launch reads nothing the main launch writes:
// it is released by programmatic dependent launch as the main launch's CTAs leave, does not wait before its work, and
// waits for the main grid before it ends (a fully dependent second launch had measured 26000).  With these numbers a
// thin last wave moves only when one wave is long (1024 x 14336 x K: level at K = 4096, 90 -> 82 us at 8192, 167 -> 143
// at 16384), and a thin grid when K is long against its tile count (256 x 4096 x 28672: 62 -> 41 us; 512 x 4096 x 14336
// and 128 x 8192 x 8192: level, left alone).  A split must promise at least 1 % of the whole run.
constexpr double kSplitKBlockCycles = 655.0;   // one-CTA 128 x 256 tile
constexpr double kTailFixedAlone = 16000.0;
constexpr double kTailFixedAfterMain = 20000.0;
struct TailPlan {
    bool use;
    int tile_end;  // tiles left to the main launch
    SplitKParams q;
};

// `now_per_kb` >= 0: the cost (per K block) of what would run instead, when that is not the form whose grid is split.
TailPlan plan_tail(int64_t M, int64_t N, int64_t K, bool pair, double form_cycles, int sms, double now_per_kb = -1.0)
{
    TailPlan t{};
    if (knobs().tail_split == 0) return t;
    const int tile_m = pair ? 2 * kBM : kBM;
    const int64_t tiles = ((M + tile_m - 1) / tile_m) * ((N + 255) / 256);
    const int64_t slots = pair ? sms / 2 : sms;
    const int64_t waves = (tiles + slots - 1) / slots;
    const int64_t rest = tiles - (waves - 1) * slots;       // tiles of the last wave
    const int64_t units = rest * (pair ? 2 : 1);
    const int kb = static_cast<int>((K + kBK - 1) / kBK);
    int S = 0;
    for (int c = 8; c >= 2; c /= 2)
        if (units * c <= sms && kb / c >= 2) {
            S = c;
            break;
        }
    if (S == 0) return t;
    const int kbs = (kb + S - 1) / S;
    const double now = now_per_kb >= 0.0 ? now_per_kb * kb : static_cast<double>(waves) * kb * (form_cycles + 16.0);
    const double split = static_cast<double>(waves - 1) * kb * (form_cycles + 16.0) + kbs * kSplitKBlockCycles + (waves > 1 ? kTailFixedAfterMain : kTailFixedAlone);
    if (knobs().tail_split == 1 && split >= 0.99 * now) return t;
    t.use = true;
    t.tile_end = static_cast<int>((waves - 1) * slots);
    t.q.tile_begin = t.tile_end;
    t.q.units = static_cast<int>(units);
    t.q.splits = S;
    t.q.kb_per_split = kbs;
    t.q.pair_grid = pair ? 1 : 0;
    return t;
}

// The automatic choice for the dense entry points: tile form, and whether (part of) its grid goes to the split-K kernel.
// A narrow-tile choice (few tiles) is also weighed against splitting the whole one-CTA 256-wide grid.
struct DenseChoice {
    int bn;
    bool pair;
    TailPlan tail;
};

DenseChoice choose_dense(int64_t M, int64_t N, int64_t K, int sms)
{
    DenseChoice c{};
    double cost = 0.0;
    c.bn = pick_bn(M, N, sms, false, &c.pair, &cost);
    if (c.bn == 256) {
        c.tail = plan_tail(M, N, K, c.pair, c.pair ? kDenseForms[0].kblock_cycles : kDenseForms[1].kblock_cycles, sms);
    } else {
        const TailPlan t = plan_tail(M, N, K, false, kDenseForms[1].kblock_cycles, sms, cost);
        if (t.use && t.tile_end == 0) c.bn = 256, c.pair = false, c.tail = t;
    }
    return c;
}

template <int EPI>
int dispatch_dense(DeviceState* st, const int8_t* x, const int8_t* y, DenseParams p, cudaStream_t stream)
{
    const int forced = g_forced_variant;
    int bn;
    bool pair = false;
    TailPlan t{};
    switch (forced) {
        case VAR_PAIR: bn = 256, pair = true; break;
        case VAR_DENSE_BN256: bn = 256; break;
        case VAR_DENSE_BN128: bn = 128; break;
        case VAR_DENSE_BN64: bn = 64; break;
        default: {
            const DenseChoice c = choose_dense(p.M, p.N, p.K, st->sm_count);
            bn = c.bn, pair = c.pair, t = c.tail;
        }
    }
    // A forced 256-wide form still hands its last wave to the split-K kernel when that is forced too (tests).
    if (forced != VAR_AUTO && bn == 256 && knobs().tail_split == 2)
        t = plan_tail(p.M, p.N, p.K, pair, pair ? kDenseForms[0].kblock_cycles : kDenseForms[1].kblock_cycles, st->sm_count);
    if constexpr (EPI != EPI_RAW_I32) {
        if (t.use && p.vec_ok) {
            DenseParams pm = p;
            pm.tile_end = t.tile_end;
            // (GEMM_INT8_PDL=0: the split-K launch is an ordinary, fully dependent second launch)
            pm.pdl_role = knobs().pdl ? 1 : 0;
            t.q.after_main = (t.tile_end > 0 && knobs().pdl) ? 1 : 0;
            DenseParams pt = p;  // the grid description the split-K kernel numbers its tiles by
            pt.tiles_m = static_cast<int>((p.M + (pair ? 2 * kBM : kBM) - 1) / (pair ? 2 * kBM : kBM));
            pt.tiles_n = static_cast<int>((p.N + 255) / 256);
            pt.group_m = pair ? (pick_group_m(p.K) / 2 > 0 ? pick_group_m(p.K) / 2 : 1) : pick_group_m(p.K);
            if (t.tile_end > 0) {
                if (int rc = pair ? launch_dense_pair<EPI>(st, 45 + EPI, x, y, pm, stream)
                                  : launch_dense<256, 4, EPI>(st, EPI * 3 + 0, x, y, pm, stream))
                    return rc;
            }
            return launch_dense_splitk<EPI>(st, 60 + (EPI == EPI_ALPHA_BF16 ? 0 : 1), x, y, pt, t.q, stream);
        }
    }
    if (pair) return launch_dense_pair<EPI>(st, 45 + EPI, x, y, p, stream);
    if (bn == 256) return launch_dense<256, 4, EPI>(st, EPI * 3 + 0, x, y, p, stream);
    if (bn == 128) return launch_dense<128, 6, EPI>(st, EPI * 3 + 1, x, y, p, stream);
    return launch_dense<64, 8, EPI>(st, EPI * 3 + 2, x, y, p, stream);
}

// K == 0: the product is all zeros; written with a plain memset-equivalent kernel.
__global__ void fill_zero_kernel(uint8_t* out, int64_t bytes)
{
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < bytes;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i] = 0;
}

int zero_output(void* out, int64_t bytes, cudaStream_t stream)
{
    fill_zero_kernel<<<148, 256, 0, stream>>>(static_cast<uint8_t*>(out), bytes);
    GI8_CUDA(cudaGetLastError());
    return GI8_OK;
}

// ---------------------------------------------------------------------------------------------------
// Small-M plan: token tile MT, number of K splits and pipeline depth.  Fitted on B200 with device-timed CUDA-graph
// replays over HBM-cold weights (M in {1,16,64} x {4096x4096, 14336x4096, 4096x14336}): few weight tiles want the
// largest cluster (8 splits: 32 tiles -> 256 CTAs), many weight tiles want one or two; for M >= 16 the reduction
// costs more than a second split gains (measured again with the one-barrier reduction: the same choices win).  Two CTAs
// fit one SM (about 100 KB of shared memory each).
// ---------------------------------------------------------------------------------------------------
struct SmallMPlan {
    bool use;
    int mt, splits, kb_per_split, tiles_n;
    int64_t scratch_bytes, total_bytes;
};

constexpr int kSmallMMaxM = 64;  // the automatic dispatch sends M <= 64 to the small-M kernel

SmallMPlan plan_smallm(int64_t M, int64_t N, int64_t K, int sms, bool forced, int max_splits = 1 << 30)
{
    SmallMPlan pl{};
    pl.use = (M >= 1) && (forced ? M <= 128 : M <= kSmallMMaxM) && K > 0 && N > 0;
    if (!pl.use) return pl;
    pl.mt = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    pl.tiles_n = static_cast<int>((N + kSmallMTileN - 1) / kSmallMTileN);
    const int kb_total = static_cast<int>((K + kBK - 1) / kBK);
    const int slots = 2 * sms;
    int splits = slots / pl.tiles_n;
    if (splits < 1) splits = 1;
    if (splits <= 2) splits = 1;  // many weight tiles already fill the machine; a second split only adds a reduction
    if (splits > kb_total / 2) splits = kb_total / 2 > 0 ? kb_total / 2 : 1;
    if (splits > max_splits) splits = max_splits;
    if (const int v = knobs().splits) {  // tuning override
        if (v >= 1 && v <= max_splits && v <= kb_total) splits = v;
    }
    pl.kb_per_split = (kb_total + splits - 1) / splits;
    pl.splits = (kb_total + pl.kb_per_split - 1) / pl.kb_per_split;
    pl.scratch_bytes = pl.splits > 1 ? static_cast<int64_t>(pl.tiles_n) * pl.mt * kSmallMTileN * 4 : 0;
    pl.total_bytes = pl.splits > 1 ? pl.scratch_bytes + ((static_cast<int64_t>(pl.tiles_n) * 4 + 15) / 16) * 16 : 0;
    return pl;
}

template <int MT, int STAGES>
int launch_smallm(DeviceState* st, int slot, const int8_t* x, const int8_t* w, SmallMParams p, const SmallMPlan& pl,
                  cudaStream_t stream)
{
    constexpr size_t stage = kSmallMTileN * kBK + ((MT * kBK + 1023) / 1024) * 1024;
    constexpr size_t smem = STAGES * stage + 1024;
    auto kernel = smallm_gemm_kernel<MT, STAGES>;
    if (int rc = ensure_smem(st, slot, kernel, smem)) return rc;
    CUtensorMap mw, mx;
    if (int rc = make_operand_map(&mw, w, p.N, p.K, kSmallMTileN)) return rc;
    if (int rc = make_operand_map(&mx, x, p.M, p.K, MT)) return rc;
    dim3 grid(pl.tiles_n, pl.splits);
    kernel<<<grid, kSmallMThreads, smem, stream>>>(mw, mx, p);
    GI8_CUDA(cudaGetLastError());
    return GI8_OK;
}

constexpr int kMaxClusterSplits = 8;  // portable thread-block cluster size

// RECV: room behind the pipeline buffers for the partial sums the cluster peers send (needed when splits > 1).
template <int MT, int STAGES, bool RECV>
int launch_smallm_cluster(DeviceState* st, int slot, const int8_t* x, const int8_t* w, SmallMParams p,
                          const SmallMPlan& pl, cudaStream_t stream)
{
    constexpr size_t stage = kSmallMTileN * kBK + ((MT * kBK + 1023) / 1024) * 1024;
    constexpr size_t smem = STAGES * stage + (RECV ? (MT + kMaxClusterSplits) * kSmallMTileN * 4 : 0) + 1024;
    static_assert(smem <= 227 * 1024, "shared memory per CTA");
    auto kernel = smallm_cluster_kernel<MT, STAGES>;
    if (int rc = ensure_smem(st, slot, kernel, smem)) return rc;
    CUtensorMap mw, mx;
    if (int rc = make_operand_map(&mw, w, p.N, p.K, kSmallMTileN)) return rc;
    if (int rc = make_operand_map(&mx, x, p.M, p.K, MT)) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pl.tiles_n, pl.splits, 1);
    cfg.blockDim = dim3(kSmallMThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = pl.splits;
    attr[0].val.clusterDim.z = 1;
    // Programmatic dependent launch: this kernel's set-up overlaps the tail of the previous kernel in the stream
    // (it waits with griddepcontrol.wait before its first global access).
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = knobs().pdl ? 2 : 1;
    GI8_CUDA(cudaLaunchKernelEx(&cfg, kernel, mw, mx, p));
    return GI8_OK;
}

// ---------------------------------------------------------------------------------------------------
// Fixed scratch for gi8_matmul_scaled_static.  In host code the name below is only a handle for the
// runtime, not a device address: the address a kernel can use comes from cudaGetSymbolAddress, looked up
// once per device (each device has its own copy of the array) and cached here.
// ---------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[GI8_STATIC_SCRATCH_BYTES];
void* g_static_scratch_ptr[kMaxDevices] = {};

int get_static_scratch(void** out)
{
    int dev = 0;
    GI8_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(GI8_ERR_UNSUPPORTED_DEVICE, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_static_scratch_ptr[dev]) {
        void* ptr = nullptr;
        GI8_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));  // device `dev` is current here
        if (!ptr) return fail(GI8_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the static scratch");
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return GI8_OK;
}

}  // namespace

// Exercises the bounded-wait error path without faulting or hanging anything: warp 1 waits (1 ms limit) on a barrier
// that nobody ever arrives on, gives up, records ERR_TIMEOUT_EPILOGUE and raises the CTA's abort flag; warp 0 waits
// on a second such barrier with the ordinary limit and must leave early because of the flag.  The kernel then
// returns normally and the context stays usable.
__global__ void wait_timeout_selftest_kernel(uint32_t* status)
{
    __shared__ __align__(8) uint64_t bar_never[2];
    __shared__ volatile uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        gi8::mbar_init(&bar_never[0], 1);
        gi8::mbar_init(&bar_never[1], 1);
        gi8::fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 32) {
        if (!gi8::wait_or_abort(&bar_never[0], 0, &abort_flag, 1000000ull))
            gi8::raise_error(status, &abort_flag, gi8::ERR_TIMEOUT_EPILOGUE);
    } else if (threadIdx.x == 0) {
        // returns false within microseconds of the flag being raised, long before its own 250 ms limit
        if (gi8::wait_or_abort(&bar_never[1], 0, &abort_flag)) gi8::raise_error(status, &abort_flag, gi8::ERR_TIMEOUT_PRODUCER);
    }
    __syncthreads();
}

// out[i] = bf16( ((parts[0][i] + parts[1][i]) + parts[2][i]) + ... ): the partial accumulators of a K-sharded GEMM
// summed in the order of the parts (fp32, round to nearest each step) and cast once.  HBM-bound: n_parts * 4 + 2
// bytes per element, 16-byte loads, grid-stride over a grid of 16 CTAs per SM.
template <bool VEC>
__global__ void sum_parts_bf16_kernel(const float* __restrict__ parts, int n_parts, int64_t part_stride,
                                      uint16_t* __restrict__ out, int64_t count)
{
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if constexpr (VEC) {
        for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count / 4; i += step) {
            float4 a = *reinterpret_cast<const float4*>(parts + 4 * i);
            for (int r = 1; r < n_parts; ++r) {
                const float4 b = *reinterpret_cast<const float4*>(parts + r * part_stride + 4 * i);
                a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
            }
            *reinterpret_cast<uint2*>(out + 4 * i) = make_uint2(gi8::pack_bf16x2(a.x, a.y), gi8::pack_bf16x2(a.z, a.w));
        }
    } else {
        for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count; i += step) {
            float a = parts[i];
            for (int r = 1; r < n_parts; ++r) a += parts[r * part_stride + i];
            out[i] = gi8::to_bf16_bits(a);
        }
    }
}

template <typename T>
static int launch_hadamard_quant(const T* in, int8_t* q, float* scales, int64_t M, int K, int KB, int H, cudaStream_t s)
{
    const int threads = H / 4 < kQuantThreads ? H / 4 : kQuantThreads;
    const int e = H / threads;
    const size_t smem = threads > 32 ? sizeof(float) * H : 0;
    const float norm = static_cast<float>(pow(static_cast<double>(H), -0.5));
    const int64_t blocks = M * (K / H);
    if (blocks > INT32_MAX) return fail(GI8_ERR_UNSUPPORTED_SHAPE, "too many rotation blocks");
    const int grid = static_cast<int>(blocks);
    switch (e) {
        case 4: hadamard_quantize_token_block_kernel<T, 4><<<grid, threads, smem, s>>>(in, q, scales, K, KB, H, norm); break;
        case 8: hadamard_quantize_token_block_kernel<T, 8><<<grid, threads, smem, s>>>(in, q, scales, K, KB, H, norm); break;
        case 16: hadamard_quantize_token_block_kernel<T, 16><<<grid, threads, smem, s>>>(in, q, scales, K, KB, H, norm); break;
        default: hadamard_quantize_token_block_kernel<T, 32><<<grid, threads, smem, s>>>(in, q, scales, K, KB, H, norm); break;
    }
    GI8_CUDA(cudaGetLastError());
    return GI8_OK;
}

extern "C" {

int gi8_version(void) { return 100; }

const char* gi8_last_error(void) { return g_err; }

int gi8_force_variant(const char* name)
{
    if (!name || !*name) {
        g_forced_variant = VAR_AUTO;
        return GI8_OK;
    }
    for (int i = 0; i < kNumVariants; ++i)
        if (!strcmp(name, kVariantNames[i])) {
            g_forced_variant = i;
            return GI8_OK;
        }
    return fail(GI8_ERR_INVALID_ARGUMENT, "unknown variant '%s'", name);
}

const char* gi8_pick_variant(int kind, int64_t M, int64_t N, int64_t K)
{
    int sms = 148;
    DeviceState* st = nullptr;
    if (get_device_state(&st) == GI8_OK) sms = st->sm_count;
    const int forced = g_forced_variant;
    if (forced != VAR_AUTO) return kVariantNames[forced];
    if (kind == 1 && plan_smallm(M, N, K, sms, false).use) return "smallm_cluster";
    if (kind == 2) {
        bool pair = false;
        const int bn = pick_bn(M, N, sms, true, &pair);
        if (bn == 256 && !pair && N % 8 == 0) {
            const ColumnSplit c = plan_column_split(M, N, K, sms);
            if (c.use) return c.bn_tail == 128 ? "blockwise_bn256+columns_bn128" : "blockwise_bn256+columns_bn64";
        }
        return pair ? "blockwise_pair" : bn == 256 ? "blockwise_bn256" : bn == 128 ? "blockwise_bn128" : "blockwise_bn64";
    }
    const DenseChoice c = choose_dense(M, N, K, sms);
    const bool pair = c.pair;
    const int bn = c.bn;
    if (c.tail.use) {
        static const char* const names[2][2][4] = {
            {{"", "dense_bn256+splitk2", "dense_bn256+splitk4", "dense_bn256+splitk8"}, {"", "splitk2", "splitk4", "splitk8"}},
            {{"", "pair+splitk2", "pair+splitk4", "pair+splitk8"}, {"", "splitk2", "splitk4", "splitk8"}}};
        const int si = c.tail.q.splits == 2 ? 1 : c.tail.q.splits == 4 ? 2 : 3;
        return names[pair ? 1 : 0][c.tail.tile_end > 0 ? 0 : 1][si];
    }
    return pair ? "pair" : bn == 256 ? "dense_bn256" : bn == 128 ? "dense_bn128" : "dense_bn64";
}

int gi8_reload_env(void)
{
    knobs();  // make sure the one-time load has happened, then load again
    std::lock_guard<std::mutex> lock(g_mutex);
    load_knobs();
    return GI8_OK;
}

int gi8_device_check(void)
{
    uint32_t code = 0;
    if (int rc = gi8_device_status(&code)) return rc;
    if (code)
        return fail(GI8_ERR_DEVICE_TIMEOUT, "a kernel gave up a bounded wait: role %u (1 producer, 2 MMA issuer, 3 epilogue, "
                    "4 drain, 5 reduction) in CTA %u; the results of that launch are invalid", code & 0xff, code >> 8);
    return GI8_OK;
}

int gi8_selftest_wait_timeout(void* stream)
{
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    wait_timeout_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(st->status);
    GI8_CUDA(cudaGetLastError());
    return GI8_OK;
}

int gi8_device_status(uint32_t* code)
{
    if (!code) return fail(GI8_ERR_INVALID_ARGUMENT, "null code pointer");
    GI8_CUDA(cudaDeviceSynchronize());
    uint32_t v = 0, zero = 0;
    GI8_CUDA(cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof(v)));
    if (v) GI8_CUDA(cudaMemcpyToSymbol(g_kernel_status, &zero, sizeof(zero)));
    *code = v;
    return GI8_OK;
}

int gi8_matmul(const int8_t* x, const int8_t* y, void* out, int64_t M, int64_t N, int64_t K, float alpha, void* stream)
{
    if (int rc = check_common(x, y, out, M, N, K, 2)) return rc;
    if (M == 0 || N == 0) return GI8_OK;
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) return zero_output(out, M * N * 2, s);
    DenseParams p{};
    p.out = out, p.status = st->status, p.ldo = N, p.M = (int)M, p.N = (int)N, p.K = (int)K, p.alpha = alpha;
    p.vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (N % 8 == 0);
    return dispatch_dense<EPI_ALPHA_BF16>(st, x, y, p, s);
}

int gi8_matmul_i32(const int8_t* x, const int8_t* y, int32_t* out, int64_t M, int64_t N, int64_t K, void* stream)
{
    if (int rc = check_common(x, y, out, M, N, K, 4)) return rc;
    if (M == 0 || N == 0) return GI8_OK;
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) return zero_output(out, M * N * 4, s);
    DenseParams p{};
    p.out = out, p.status = st->status, p.ldo = N, p.M = (int)M, p.N = (int)N, p.K = (int)K, p.alpha = 1.0f;
    p.vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (N % 4 == 0);
    return dispatch_dense<EPI_RAW_I32>(st, x, y, p, s);
}

int64_t gi8_matmul_scaled_workspace_bytes(int64_t M, int64_t N, int64_t K)
{
    if (g_forced_variant != VAR_SMALLM) return 0;  // only the scratch variant needs a workspace
    // The plan depends on the SM count, so the device is initialised here: the size returned is the size the launch
    // will ask for.
    int sms = 148;
    DeviceState* st = nullptr;
    if (get_device_state(&st) == GI8_OK) sms = st->sm_count;
    const SmallMPlan pl = plan_smallm(M, N, K, sms, true);
    return pl.use ? pl.total_bytes : 0;
}

int gi8_matmul_scaled(const int8_t* x, const int8_t* y, const float* sx, const float* sw, void* out, int64_t M,
                      int64_t N, int64_t K, void* workspace, int64_t workspace_bytes, void* stream)
{
    if (int rc = check_common(x, y, out, M, N, K, 2)) return rc;
    if (M == 0 || N == 0) return GI8_OK;
    if (!sx || !sw) return fail(GI8_ERR_INVALID_ARGUMENT, "null scale pointer");
    if (reinterpret_cast<uintptr_t>(sx) % 4 || reinterpret_cast<uintptr_t>(sw) % 4)
        return fail(GI8_ERR_MISALIGNED, "scale pointers must be 4-byte aligned");
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) return zero_output(out, M * N * 2, s);
    const int forced = g_forced_variant;
    if (forced == VAR_AUTO || forced == VAR_SMALLM_CLUSTER) {
        const SmallMPlan pl = plan_smallm(M, N, K, st->sm_count, forced == VAR_SMALLM_CLUSTER, kMaxClusterSplits);
        if (pl.use) {
            SmallMParams q{};
            q.out = out, q.sx = sx, q.sw = sw, q.status = st->status, q.ldo = N;
            q.M = (int)M, q.N = (int)N, q.K = (int)K, q.kb_per_split = pl.kb_per_split, q.splits = pl.splits;
            q.static_w = knobs().static_weights && knobs().pdl;
            // Pipeline depth: two CTAs share an SM (about 100 KB each, the receive area of a cluster CTA included).  A
            // deeper pipeline with one CTA per SM measured slower even for grids of at most one CTA per SM: the next
            // kernel's CTAs could no longer move in beside the running ones, and its set-up no longer overlapped.
            if (pl.splits > 1) {
                switch (pl.mt) {
                    case 16: return launch_smallm_cluster<16, 5, true>(st, 48, x, y, q, pl, s);
                    case 32: return launch_smallm_cluster<32, 4, true>(st, 49, x, y, q, pl, s);
                    case 64: return launch_smallm_cluster<64, 3, true>(st, 50, x, y, q, pl, s);
                    default: return launch_smallm_cluster<128, 3, true>(st, 51, x, y, q, pl, s);
                }
            } else {
                switch (pl.mt) {
                    case 16: return launch_smallm_cluster<16, 6, false>(st, 52, x, y, q, pl, s);
                    case 32: return launch_smallm_cluster<32, 5, false>(st, 53, x, y, q, pl, s);
                    case 64: return launch_smallm_cluster<64, 4, false>(st, 54, x, y, q, pl, s);
                    default: return launch_smallm_cluster<128, 3, true>(st, 51, x, y, q, pl, s);
                }
            }
        }
    }
    if (forced == VAR_SMALLM) {
        const SmallMPlan pl = plan_smallm(M, N, K, st->sm_count, true);
        if (pl.use) {
            SmallMParams q{};
            q.out = out, q.sx = sx, q.sw = sw, q.status = st->status, q.ldo = N;
            q.M = (int)M, q.N = (int)N, q.K = (int)K, q.kb_per_split = pl.kb_per_split, q.splits = pl.splits;
            if (pl.splits > 1) {
                if (!workspace || workspace_bytes < pl.total_bytes)
                    return fail(GI8_ERR_WORKSPACE, "this shape needs %lld bytes of zero-filled workspace, got %lld",
                                (long long)pl.total_bytes, (long long)workspace_bytes);
                if (reinterpret_cast<uintptr_t>(workspace) % 16)
                    return fail(GI8_ERR_MISALIGNED, "workspace must be 16-byte aligned");
                q.scratch = static_cast<int32_t*>(workspace);
                q.counters = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(workspace) + pl.scratch_bytes);
            }
            switch (pl.mt) {
                case 16: return launch_smallm<16, 6>(st, 24, x, y, q, pl, s);
                case 32: return launch_smallm<32, 5>(st, 25, x, y, q, pl, s);
                case 64: return launch_smallm<64, 4>(st, 26, x, y, q, pl, s);
                default: return launch_smallm<128, 3>(st, 27, x, y, q, pl, s);
            }
        }
    }
    DenseParams p{};
    p.out = out, p.sx = sx, p.sw = sw, p.status = st->status, p.ldo = N, p.M = (int)M, p.N = (int)N, p.K = (int)K;
    p.alpha = 1.0f;
    p.vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (N % 8 == 0);
    return dispatch_dense<EPI_ROWCOL_BF16>(st, x, y, p, s);
}

int gi8_matmul_scaled_static(const int8_t* x, const int8_t* y, const float* sx, const float* sw, void* out, int64_t M,
                             int64_t N, int64_t K, void* stream)
{
    if (int rc = check_common(x, y, out, M, N, K, 2)) return rc;
    if (M == 0 || N == 0) return GI8_OK;
    if (M > 128)
        return fail(GI8_ERR_UNSUPPORTED_SHAPE, "gi8_matmul_scaled_static covers M <= 128 only (got M=%lld); use "
                    "gi8_matmul_scaled", (long long)M);
    if (!sx || !sw) return fail(GI8_ERR_INVALID_ARGUMENT, "null scale pointer");
    if (reinterpret_cast<uintptr_t>(sx) % 4 || reinterpret_cast<uintptr_t>(sw) % 4)
        return fail(GI8_ERR_MISALIGNED, "scale pointers must be 4-byte aligned");
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) return zero_output(out, M * N * 2, s);
    const SmallMPlan pl = plan_smallm(M, N, K, st->sm_count, true);
    if (pl.total_bytes > GI8_STATIC_SCRATCH_BYTES)
        return fail(GI8_ERR_UNSUPPORTED_SHAPE, "this shape needs %lld bytes of scratch but the static scratch holds "
                    "%lld (GI8_STATIC_SCRATCH_BYTES); use gi8_matmul_scaled with a caller-owned workspace",
                    (long long)pl.total_bytes, (long long)GI8_STATIC_SCRATCH_BYTES);
    SmallMParams q{};
    q.out = out, q.sx = sx, q.sw = sw, q.status = st->status, q.ldo = N;
    q.M = (int)M, q.N = (int)N, q.K = (int)K, q.kb_per_split = pl.kb_per_split, q.splits = pl.splits;
    if (pl.splits > 1) {
        void* base = nullptr;
        if (int rc = get_static_scratch(&base)) return rc;
        // The array holds the previous call's leftovers: clear the part this call accumulates into.
        GI8_CUDA(cudaMemsetAsync(base, 0, static_cast<size_t>(pl.total_bytes), s));
        q.scratch = static_cast<int32_t*>(base);
        q.counters = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(base) + pl.scratch_bytes);
    }
    switch (pl.mt) {
        case 16: return launch_smallm<16, 6>(st, 24, x, y, q, pl, s);
        case 32: return launch_smallm<32, 5>(st, 25, x, y, q, pl, s);
        case 64: return launch_smallm<64, 4>(st, 26, x, y, q, pl, s);
        default: return launch_smallm<128, 3>(st, 27, x, y, q, pl, s);
    }
}

static int check_quant(const void* in, int in_dtype, const int8_t* q, const float* scales, int64_t M, int64_t K)
{
    if (M < 0 || K < 0) return fail(GI8_ERR_INVALID_ARGUMENT, "negative dimension");
    if (in_dtype != 0 && in_dtype != 1) return fail(GI8_ERR_INVALID_ARGUMENT, "in_dtype must be 0 (fp32) or 1 (bf16)");
    if (M == 0 || K == 0) return GI8_OK;
    if (!in || !q || !scales) return fail(GI8_ERR_INVALID_ARGUMENT, "null pointer");
    if (M > INT32_MAX || K > INT32_MAX - 1024) return fail(GI8_ERR_UNSUPPORTED_SHAPE, "dimension too large");
    const int64_t mult = in_dtype == 0 ? 4 : 8;
    if (K % mult) return fail(GI8_ERR_UNSUPPORTED_SHAPE, "K=%lld must be a multiple of %lld for this input type",
                              (long long)K, (long long)mult);
    if (reinterpret_cast<uintptr_t>(in) % 16 || reinterpret_cast<uintptr_t>(q) % 8 || reinterpret_cast<uintptr_t>(scales) % 4)
        return fail(GI8_ERR_MISALIGNED, "in must be 16-byte aligned, q 8-byte and scales 4-byte aligned");
    return GI8_OK;
}

int gi8_quantize_token_block(const void* in, int in_dtype, int8_t* q, float* scales, int64_t M, int64_t K, void* stream)
{
    if (int rc = check_quant(in, in_dtype, q, scales, M, K)) return rc;
    if (M == 0 || K == 0) return GI8_OK;
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int KB = static_cast<int>((K + 127) / 128);
    // A warp takes eight 128-wide blocks per iteration: eight loads of 32 lanes x 16 bytes (fp32) or four (bf16).
    const int64_t per_warp = kQuantBlocksPerItem;
    const int64_t warps = M * ((KB + per_warp - 1) / per_warp);  // one work item per warp and iteration
    if (warps >= (int64_t(1) << 32)) return fail(GI8_ERR_UNSUPPORTED_SHAPE, "too many quantisation blocks");
    int64_t blocks = (warps + kQuantThreads / 32 - 1) / (kQuantThreads / 32);
    const int64_t cap = static_cast<int64_t>(st->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    if (in_dtype == 0)
        quantize_token_block_kernel<float><<<static_cast<int>(blocks), kQuantThreads, 0, s>>>(
            static_cast<const float*>(in), q, scales, M, static_cast<int>(K), KB);
    else
        quantize_token_block_kernel<__nv_bfloat16><<<static_cast<int>(blocks), kQuantThreads, 0, s>>>(
            static_cast<const __nv_bfloat16*>(in), q, scales, M, static_cast<int>(K), KB);
    GI8_CUDA(cudaGetLastError());
    return GI8_OK;
}

int gi8_hadamard_quantize_token_block(const void* in, int in_dtype, int8_t* q, float* scales, int64_t M, int64_t K,
                                      int64_t had_block, void* stream)
{
    if (int rc = check_quant(in, in_dtype, q, scales, M, K)) return rc;
    if (had_block < 128 || had_block > 8192 || (had_block & (had_block - 1)))
        return fail(GI8_ERR_UNSUPPORTED_SHAPE, "rotation block %lld must be a power of two in [128, 8192]", (long long)had_block);
    if (K % had_block)
        return fail(GI8_ERR_UNSUPPORTED_SHAPE, "K=%lld must be a multiple of the rotation block %lld", (long long)K,
                    (long long)had_block);
    if (M == 0 || K == 0) return GI8_OK;
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int KB = static_cast<int>(K / 128);
    if (in_dtype == 0)
        return launch_hadamard_quant(static_cast<const float*>(in), q, scales, M, static_cast<int>(K), KB,
                                     static_cast<int>(had_block), s);
    return launch_hadamard_quant(static_cast<const __nv_bfloat16*>(in), q, scales, M, static_cast<int>(K), KB,
                                 static_cast<int>(had_block), s);
}

int gi8_quantize_token(const void* in, int in_dtype, int8_t* q, float* scales, int64_t M, int64_t K, void* stream)
{
    if (int rc = check_quant(in, in_dtype, q, scales, M, K)) return rc;
    if (M == 0 || K == 0) return GI8_OK;
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int64_t blocks = M;
    const int64_t cap = static_cast<int64_t>(st->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (in_dtype == 0)
        quantize_token_row_kernel<float><<<static_cast<int>(blocks), kQuantThreads, 0, s>>>(static_cast<const float*>(in), q,
                                                                                         scales, M, static_cast<int>(K));
    else
        quantize_token_row_kernel<__nv_bfloat16><<<static_cast<int>(blocks), kQuantThreads, 0, s>>>(
            static_cast<const __nv_bfloat16*>(in), q, scales, M, static_cast<int>(K));
    GI8_CUDA(cudaGetLastError());
    return GI8_OK;
}

// gather != nullptr: the N-sharded form.  This GEMM's [M,N] result is columns [col0, col0 + N) of an [M, n_total]
// matrix, and the epilogue writes every block into all n_out such matrices (gather[i]: this rank's own and every
// peer's, the latter through mapped peer memory) instead of `out`.
static int blockwise_impl(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw, int64_t ld_sw,
                          void* out, int64_t M, int64_t N, int64_t K, void* stream, void* const* gather, int n_out,
                          int64_t n_total, int64_t col0, bool out_f32 = false, int force_bn = 0, int pdl_role = 0,
                          int scatter_me = -1)
{
    // scatter_me >= 0: `gather` holds the n_out ranks' receive areas of the K-sharded reduce-scatter form
    const bool scatter = scatter_me >= 0;
    if (gather) out = gather[0];
    if (int rc = check_common(x, y, out, M, N, K, out_f32 ? 4 : 2)) return rc;
    if (M == 0 || N == 0) return GI8_OK;
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) return zero_output(out, M * N * (out_f32 ? 4 : 2), s);
    const int64_t KB = (K + kBK - 1) / kBK;
    if (!sa || !sw) return fail(GI8_ERR_INVALID_ARGUMENT, "null scale pointer");
    if (ld_sa < KB || ld_sw < KB)
        return fail(GI8_ERR_INVALID_ARGUMENT, "scale row strides (%lld, %lld) must be at least ceil(K/128) = %lld",
                    (long long)ld_sa, (long long)ld_sw, (long long)KB);
    if (reinterpret_cast<uintptr_t>(sa) % 4 || reinterpret_cast<uintptr_t>(sw) % 4)
        return fail(GI8_ERR_MISALIGNED, "scale pointers must be 4-byte aligned");
    // The kernels index the scale arrays with 32-bit element offsets.
    if (M * ld_sa >= (int64_t(1) << 31) || ((N + 127) / 128) * ld_sw >= (int64_t(1) << 31))
        return fail(GI8_ERR_INVALID_ARGUMENT, "scale arrays of 2^31 or more elements are not supported");
    BlockwiseParams p{};
    p.out = out, p.sa = sa, p.sw = sw, p.status = st->status, p.ldo = N, p.ld_sa = ld_sa, p.ld_sw = ld_sw;
    p.M = (int)M, p.N = (int)N, p.K = (int)K;
    p.vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (N % 8 == 0);
    p.out_f32 = out_f32 ? 1 : 0;
    p.n_out = 1, p.out_col0 = 0;
    p.scale_vec = (KB % 4 == 0) && (ld_sa % 4 == 0) && (ld_sw % 4 == 0) && reinterpret_cast<uintptr_t>(sa) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(sw) % 16 == 0;
    const int forced = g_forced_variant;
    int bn;
    bool pair = false;
    switch (forced) {
        case VAR_DENSE_BN256: bn = 256; break;
        case VAR_DENSE_BN128: bn = 128; break;
        case VAR_DENSE_BN64: bn = 64; break;
        case VAR_PAIR: bn = 256, pair = true; break;
        default: bn = pick_bn(M, N, st->sm_count, true, &pair);
    }
    if (force_bn) bn = force_bn, pair = false;
    if (scatter && bn == 64) bn = 128;  // a 32 x 32 fp32 box needs the 4 KB staging block of the wider tiles
    p.pdl_role = pdl_role;
    // The epilogue's TMA-store boxes are 64 columns wide for the 256- and 128-wide tiles and 32 for the 64-wide one.
    // A box is clipped at the edge of the tensor map, i.e. of the whole [M, n_total] matrix, not at the edge of this
    // GEMM's column slice: a slice that starts or ends inside a box (and is not the last one) would overwrite its
    // neighbour's columns, so such slices take the narrow tile, whose boxes the slice contract (multiples of 32)
    // always fits.
    if (gather && !scatter && (col0 % 64 != 0 || (N % 64 != 0 && col0 + N != n_total))) bn = 64, pair = false;
    const int box_cols = blockwise_store_cols(bn);
    CUtensorMap mx, my;
    if (int rc = make_operand_map(&mx, x, M, K, kBM)) return rc;
    if (int rc = make_operand_map(&my, y, N, K, pair ? bn / 2 : bn)) return rc;
    const int tile_m = pair ? 2 * kBM : kBM;
    p.tiles_m = (int)((M + tile_m - 1) / tile_m);
    p.tiles_n = (int)((N + bn - 1) / bn);
    p.group_m = pick_group_m(p.K);
    if (pair) p.group_m = p.group_m / 2 > 0 ? p.group_m / 2 : 1;
    const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
    const int slots = pair ? st->sm_count / 2 : st->sm_count;
    const int grid = static_cast<int>(tiles < slots ? tiles : slots) * (pair ? 2 : 1);
    OutputMaps mo{};
    if (scatter) {
        // one fp32 map per rank over its receive area [n_out * R, N], boxes of 32 rows x 32 columns
        const int64_t R = M / n_out;
        for (int i = 0; i < n_out; ++i) {
            MapKey key{gather[i], static_cast<uint64_t>(N), static_cast<uint64_t>(n_out * R), static_cast<uint64_t>(N) * 4, 32u, 32u, 2u};
            if (int rc = cached_map(&mo.m[i], key)) return rc;
        }
        p.scatter_ranks = n_out, p.scatter_rows = static_cast<int>(R), p.scatter_me = scatter_me;
        // rank r starts with (about) its own rows: tiles are numbered band by band over the row blocks
        p.tile_rot = static_cast<int>(tiles * scatter_me / n_out);
        p.tma_store = 0, p.n_out = n_out;
    } else if (gather) {
        for (int i = 0; i < n_out; ++i)
            if (int rc = make_output_map(&mo.m[i], gather[i], M, n_total, n_total, box_cols)) return rc;
        p.tma_store = 1, p.n_out = n_out, p.out_col0 = static_cast<int>(col0);
    } else {
        p.tma_store = p.vec_ok && knobs().tma_store && !out_f32;  // the fp32 form stores from registers
        if (p.tma_store)
            if (int rc = make_output_map(&mo.m[0], out, M, N, N, box_cols)) return rc;
    }
#define GI8_LAUNCH_BW(BN_, ST_, SPLIT_, NISS_, PAIR_, SLOT_)                                  \
    do {                                                                                      \
        constexpr size_t smem = blockwise_smem_bytes(BN_, ST_, PAIR_);                        \
        auto kernel = blockwise_gemm_kernel<BN_, ST_, SPLIT_, NISS_, PAIR_>;                  \
        if (int rc = ensure_smem(st, SLOT_, kernel, smem)) return rc;                         \
        cudaLaunchConfig_t cfg{};                                                             \
        cfg.gridDim = dim3(grid, 1, 1);                                                       \
        cfg.blockDim = dim3(kBlockwiseThreads, 1, 1);                                         \
        cfg.dynamicSmemBytes = smem;                                                          \
        cfg.stream = s;                                                                       \
        cudaLaunchAttribute attr[2];                                                          \
        attr[0].id = cudaLaunchAttributeClusterDimension;                                     \
        attr[0].val.clusterDim.x = PAIR_ ? 2 : 1;                                             \
        attr[0].val.clusterDim.y = 1;                                                         \
        attr[0].val.clusterDim.z = 1;                                                         \
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;                      \
        attr[1].val.programmaticStreamSerializationAllowed = 1;                               \
        cfg.attrs = attr;                                                                     \
        cfg.numAttrs = pdl_role == 2 ? 2 : 1;                                                 \
        GI8_CUDA(cudaLaunchKernelEx(&cfg, kernel, mx, my, mo, p));                            \
    } while (0)
    const bool two = knobs().bw_issuers == 2 || (knobs().bw_issuers == 0 && bn < 256);
    const bool halves = knobs().bw_halves == 2 || (knobs().bw_halves == 0 && pair);
    if (pair) {
        if (halves) GI8_LAUNCH_BW(256, 4, 2, 2, true, 21);
        else if (two) GI8_LAUNCH_BW(256, 4, 1, 2, true, 22);
        else GI8_LAUNCH_BW(256, 4, 1, 1, true, 23);
    } else if (bn == 256) {
        if (halves) GI8_LAUNCH_BW(256, 4, 2, 2, false, 13);
        else if (two) GI8_LAUNCH_BW(256, 4, 1, 2, false, 15);
        else GI8_LAUNCH_BW(256, 4, 1, 1, false, 16);
    } else if (bn == 128) {
        if (two) GI8_LAUNCH_BW(128, 6, 1, 2, false, 17);
        else GI8_LAUNCH_BW(128, 6, 1, 1, false, 18);
    } else {
        if (two) GI8_LAUNCH_BW(64, 8, 1, 2, false, 19);
        else GI8_LAUNCH_BW(64, 8, 1, 1, false, 20);
    }
#undef GI8_LAUNCH_BW
    return GI8_OK;
}

int gi8_matmul_blockwise(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw,
                         int64_t ld_sw, void* out, int64_t M, int64_t N, int64_t K, void* stream)
{
    if (g_forced_variant == VAR_AUTO && M > 0 && N > 0 && K > 0 && out && reinterpret_cast<uintptr_t>(out) % 16 == 0 && N % 8 == 0) {
        DeviceState* st;
        if (int rc = get_device_state(&st)) return rc;
        bool pair = false;
        if (pick_bn(M, N, st->sm_count, true, &pair) == 256 && !pair) {
            const ColumnSplit c = plan_column_split(M, N, K, st->sm_count);
            if (c.use) {
                // both launches write through a tensor map of the whole [M, N] matrix, each its own columns
                void* outs[1] = {out};
                const bool pdl = knobs().pdl;  // GEMM_INT8_PDL=0: two ordinary launches, one after the other
                if (int rc = blockwise_impl(x, y, sa, ld_sa, sw, ld_sw, nullptr, M, c.n1, K, stream, outs, 1, N, 0, false, 256, pdl ? 1 : 0))
                    return rc;
                return blockwise_impl(x, y + c.n1 * K, sa, ld_sa, sw ? sw + (c.n1 / 128) * ld_sw : sw, ld_sw, nullptr, M, N - c.n1, K,
                                      stream, outs, 1, N, c.n1, false, c.bn_tail, pdl ? 2 : 0);
            }
        }
    }
    return blockwise_impl(x, y, sa, ld_sa, sw, ld_sw, out, M, N, K, stream, nullptr, 1, N, 0);
}

int gi8_matmul_blockwise_f32(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw,
                             int64_t ld_sw, float* out, int64_t M, int64_t N, int64_t K, void* stream)
{
    return blockwise_impl(x, y, sa, ld_sa, sw, ld_sw, out, M, N, K, stream, nullptr, 1, N, 0, true);
}

int gi8_sum_parts_bf16(const float* parts, int n_parts, int64_t part_stride, void* out_bf16, int64_t count, void* stream)
{
    if (n_parts < 1 || n_parts > 64 || count < 0 || part_stride < count)
        return fail(GI8_ERR_INVALID_ARGUMENT, "n_parts must be in [1, 64] and part_stride at least count");
    if (count == 0) return GI8_OK;
    if (!parts || !out_bf16) return fail(GI8_ERR_INVALID_ARGUMENT, "null pointer");
    if (reinterpret_cast<uintptr_t>(parts) % 4 || reinterpret_cast<uintptr_t>(out_bf16) % 2)
        return fail(GI8_ERR_MISALIGNED, "parts must be 4-byte and out 2-byte aligned");
    DeviceState* st;
    if (int rc = get_device_state(&st)) return rc;
    const bool vec = reinterpret_cast<uintptr_t>(parts) % 16 == 0 && reinterpret_cast<uintptr_t>(out_bf16) % 8 == 0 &&
                     part_stride % 4 == 0 && count % 4 == 0;
    const int64_t items = vec ? count / 4 : count;
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = static_cast<int64_t>(st->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    if (vec)
        sum_parts_bf16_kernel<true><<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            parts, n_parts, part_stride, static_cast<uint16_t*>(out_bf16), count);
    else
        sum_parts_bf16_kernel<false><<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            parts, n_parts, part_stride, static_cast<uint16_t*>(out_bf16), count);
    GI8_CUDA(cudaGetLastError());
    return GI8_OK;
}

int gi8_matmul_blockwise_allgather(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw,
                                   int64_t ld_sw, void* const* outs, int n_outs, int64_t M, int64_t N, int64_t K,
                                   int64_t n_total, int64_t col0, void* stream)
{
    if (!outs || n_outs < 1 || n_outs > kMaxOutputs)
        return fail(GI8_ERR_INVALID_ARGUMENT, "n_outs must be in [1, %d]", kMaxOutputs);
    for (int i = 0; i < n_outs; ++i)
        if (!outs[i] || reinterpret_cast<uintptr_t>(outs[i]) % 16)
            return fail(GI8_ERR_MISALIGNED, "output %d is null or not 16-byte aligned", i);
    if (col0 < 0 || N < 0 || col0 + N > n_total || n_total % 8 || col0 % 32 || (N % 32 && col0 + N != n_total))
        return fail(GI8_ERR_UNSUPPORTED_SHAPE, "column slice [%lld, %lld) of %lld: n_total must be a multiple of 8, the "
                    "slice must start at a multiple of 32 and end at one (or at n_total)", (long long)col0,
                    (long long)(col0 + N), (long long)n_total);
    if (M > 0 && N > 0 && K == 0) return fail(GI8_ERR_UNSUPPORTED_SHAPE, "K must be positive for the gathering form");
    return blockwise_impl(x, y, sa, ld_sa, sw, ld_sw, nullptr, M, N, K, stream, outs, n_outs, n_total, col0);
}

int gi8_matmul_blockwise_f32_scatter(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw,
                                     int64_t ld_sw, void* const* recv, int n_ranks, int my_rank, int64_t M, int64_t N,
                                     int64_t K, void* stream)
{
    if (!recv || n_ranks < 1 || n_ranks > kMaxOutputs || my_rank < 0 || my_rank >= n_ranks)
        return fail(GI8_ERR_INVALID_ARGUMENT, "n_ranks must be in [1, %d] and my_rank below it", kMaxOutputs);
    for (int i = 0; i < n_ranks; ++i)
        if (!recv[i] || reinterpret_cast<uintptr_t>(recv[i]) % 16)
            return fail(GI8_ERR_MISALIGNED, "receive area %d is null or not 16-byte aligned", i);
    if (M <= 0 || N <= 0 || K <= 0 || M % n_ranks || (M / n_ranks) % 32 || N % 4)
        return fail(GI8_ERR_UNSUPPORTED_SHAPE, "the scattering form needs M a multiple of 32 x n_ranks (M=%lld, n_ranks=%d), "
                    "N a multiple of 4 and K > 0", (long long)M, n_ranks);
    return blockwise_impl(x, y, sa, ld_sa, sw, ld_sw, nullptr, M, N, K, stream, recv, n_ranks, N, 0, true, 0, 0, my_rank);
}

// Peer buffers for the gathering form: plain cudaMalloc allocations (an IPC handle names a whole allocation) and the
// CUDA IPC calls, so that a host without its own peer-memory plumbing can map every rank's output matrix.
int gi8_peer_alloc(void** ptr, int64_t bytes)
{
    if (!ptr || bytes <= 0) return fail(GI8_ERR_INVALID_ARGUMENT, "bad peer allocation request");
    GI8_CUDA(cudaMalloc(ptr, static_cast<size_t>(bytes)));
    return GI8_OK;
}

int gi8_peer_free(void* ptr)
{
    GI8_CUDA(cudaFree(ptr));
    return GI8_OK;
}

int gi8_peer_export(void* ptr, void* handle64)
{
    if (!ptr || !handle64) return fail(GI8_ERR_INVALID_ARGUMENT, "null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
    GI8_CUDA(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), ptr));
    return GI8_OK;
}

int gi8_peer_import(const void* handle64, void** ptr)
{
    if (!ptr || !handle64) return fail(GI8_ERR_INVALID_ARGUMENT, "null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    GI8_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return GI8_OK;
}

int gi8_peer_release(void* ptr)
{
    GI8_CUDA(cudaIpcCloseMemHandle(ptr));
    return GI8_OK;
}

}  // extern "C"
