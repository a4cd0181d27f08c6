// Blockwise-dequantised W8A8 GEMM for sm_100a:
//   out[m,n] = bf16( sum_kb fp32(P[m,n,kb]) * (sa[m,kb] * sw[n/128,kb]) ),  kb ascending, one fused
//   multiply-add per K block (128 wide), P = exact int32 partial dot product of the block.
// There is no such path in the reference (its epilogue applies one scalar, csrc/kernels/gemm.cu:96); the
// semantics are those of the CPU oracle's blockwise restatement.
//
// Structure (one persistent CTA per SM, 640 threads = 5 warpgroups):
//   warpgroup 0 control: warp 0 TMA producer (as in the dense kernel); warps 1 and 3 MMA issuers taking alternate
//               K blocks -- per K block, four tcgen05.mma kind::i8 that overwrite one of NBUF = 512 / BN
//               tensor-memory partial buffers, then ONE commit that both frees the pipeline stage and publishes
//               the partial; warp 2 allocates tensor memory; the group gives most of its registers back
//               (setmaxnreg.dec).
//   warps 4..19 promotion (16 warps, setmaxnreg.inc): tcgen05.ld the int32 partial, hand the buffer back to the
//               MMA warp as soon as the loads have landed in registers, then convert to fp32 and fma with the
//               block's scale into fp32 register accumulators.  Warp w owns TMEM lane quarter (w % 4) and column
//               quarter ((w - 4) / 4) of the tile; a column quarter never straddles a 128-wide weight-scale
//               block.  At the end of the tile the same warps cast to bf16 and store.
//
// What bounds it (measured with cycle counters in a tuning build, 128 x 256 tile): the tensor core needs ~750 cycles
// per K block; ONE issuing thread needed ~240-580 cycles for the four MMAs plus ~170 per commit, in series with its
// two waits (hence two issuers and a single commit); the promotion warps need ~1230 cycles per K block -- 512
// tensor-memory loads and 2 x 256 arithmetic warp-instructions per scheduler at ~0.65 instructions per cycle
// (cvt.rn.f32.s32 issues at half rate) -- and are the bound that remains.
#pragma once

#include "k_dense.cuh"

namespace gi8 {

constexpr int kBlockwiseThreads = 640;
constexpr int kPromoWarps = 16;
constexpr int kPromoRegs = 112;   // registers per promotion thread after setmaxnreg.inc
constexpr int kControlRegs = 32;  // registers per control-warpgroup thread after setmaxnreg.dec
constexpr int kLaunchRegs = 96;   // registers per thread at launch: 65536 / 640 rounded down to a multiple of 8
// setmaxnreg.inc can only take what setmaxnreg.dec gave back inside the same CTA (the pool is the CTA's launch
// allocation); an unbalanced pair blocks in hardware for ever.
static_assert(kPromoWarps * (kPromoRegs - kLaunchRegs) <= 4 * (kLaunchRegs - kControlRegs), "setmaxnreg pool unbalanced");

// How a promotion warp turns an int32 partial P (|P| <= 128 * 128 * 128 = 2^21) into fp32 and accumulates it.
// All variants produce bit-identical results: fp32(P) is exact in each, and the packed f32x2 instructions round
// each half like the scalar ones.
enum Promotion : int {
    PROMO_MAGIC = 0,     // integer add of 0x4B400000, fp32 subtract of 12582912.0, fma
    PROMO_MAGIC_X2 = 1,  // same, with add.f32x2 / fma.f32x2 on register pairs
    PROMO_I2F = 2,       // cvt.rn.f32.s32, fma
    PROMO_ABLATE_HANDSHAKE = 3,  // measurement only (wrong results): buffers are handed straight back
    PROMO_ABLATE_LOAD = 4,       // measurement only (wrong results): tensor-memory loads, no arithmetic
    PROMO_ABLATE_SCALES = 5,     // measurement only (wrong results): full arithmetic with a constant scale, no scale loads
    PROMO_ABLATE_MATH = 6,       // measurement only (wrong results): scale loads and tensor-memory loads, no arithmetic
    PROMO_ABLATE_FMA_ONLY = 7,   // measurement only (wrong results): one fma per element on the raw bits, no conversion
    PROMO_ABLATE_CVT_ONLY = 8,   // measurement only (wrong results): one cvt per element, folded with xor
    // The partial buffers hold 0x4B400000 before the MMAs, which all accumulate: the tensor core delivers the bit
    // pattern of fp32 (12582912 + P) and no integer instruction is left -- add.f32x2 of -12582912 and fma.f32x2,
    // one issue slot per element instead of two.  The promotion warps write the constant back (tcgen05.st) behind
    // every load.
    PROMO_BIAS_X2 = 9,
};

constexpr uint32_t kMagicBits = 0x4B400000u;  // fp32 12582912.0 = 1.5 * 2^23: adding an integer |P| < 2^22 to the
constexpr float kMagicF32 = 12582912.0f;      // bit pattern adds P to the value exactly

struct BlockwiseParams {
    void* out;        // bf16 [M,N], leading dimension ldo
    const float* sa;  // [M, KB], row stride ld_sa
    const float* sw;  // [ceil(N/128), KB], row stride ld_sw
    uint32_t* status;
    int64_t ldo, ld_sa, ld_sw;
    int M, N, K;
    int tiles_m, tiles_n;
    int vec_ok;  // out is 16-byte aligned and ldo % 8 == 0
    int group_m; // row-blocks per rasterisation band
    int tma_store;  // stage 32 x 32 bf16 blocks in shared memory and write them with TMA stores
    int n_out;      // number of output matrices the TMA-store epilogue writes every block to (1, or the ranks of an
                    // N-sharded group: each rank's full [M, N_total] matrix, peers through mapped peer memory)
    int out_col0;   // column of this GEMM's first output column in those matrices
};

constexpr int kMaxOutputs = 8;
struct OutputMaps {
    CUtensorMap m[kMaxOutputs];
};

GI8_DEVICE uint64_t pack_f32x2(uint32_t lo_bits, uint32_t hi_bits)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo_bits), "r"(hi_bits));
    return r;
}

GI8_DEVICE void unpack_f32x2(uint64_t v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

GI8_DEVICE uint64_t add_f32x2(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

GI8_DEVICE uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// acc{0,1} += (fp32 bits v{0,1} - 12582912) * t as one add.f32x2 and one fma.f32x2, kept together so that no more
// than one intermediate pair is live at a time.
GI8_DEVICE void promote_biased_pair(uint32_t v0, uint32_t v1, float t, float& acc0, float& acc1)
{
    asm volatile(
        "{\n\t"
        ".reg .b64 pv, pn, pt, pa;\n\t"
        "mov.b64 pv, {%2, %3};\n\t"
        "mov.b64 pn, {%5, %5};\n\t"
        "mov.b64 pt, {%4, %4};\n\t"
        "mov.b64 pa, {%0, %1};\n\t"
        "add.rn.f32x2 pv, pv, pn;\n\t"
        "fma.rn.f32x2 pa, pv, pt, pa;\n\t"
        "mov.b64 {%0, %1}, pa;\n\t"
        "}\n"
        : "+f"(acc0), "+f"(acc1)
        : "r"(v0), "r"(v1), "f"(t), "f"(-kMagicF32));
}

template <int N>
GI8_DEVICE void setmaxnreg_inc()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

template <int N>
GI8_DEVICE void setmaxnreg_dec()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

#ifdef GI8_ENABLE_ABLATIONS
// Tuning builds: per-CTA cycle counters (MMA thread: 0 wait-empty-buffer, 1 wait-stage, 2 issue, 3 commits, 4 count;
// promotion warp 4: 5 wait-partial, 6 rest of the K block, 7 count).
__device__ unsigned long long g_bw_dbg[148 * 8];
#define GI8_BW_DBG(slot, v) atomicAdd(&g_bw_dbg[blockIdx.x * 8 + (slot)], (unsigned long long)(v))
#define GI8_BW_CLOCK() clock64()
#else
#define GI8_BW_DBG(slot, v) ((void)0)
#define GI8_BW_CLOCK() 0ll
#endif

// Makes a 32-bit value opaque to the optimiser at this point, so that later uses read the register instead of
// recomputing the value.
#define GI8_PIN(v) asm volatile("" : "+r"(v))

enum PartialPipe : int { PIPE_X16_DOUBLE = 0, PIPE_X32_DOUBLE = 1, PIPE_X32_SINGLE = 2, PIPE_X16_SINGLE = 3 };

// SPLIT = 2 (BN = 256 only): the MMAs of a K block are issued as two column halves (N = 128 each), each half with
// its own commit and its own hand-back barrier.  The eight promotion warps of the first half then start half an
// MMA time earlier and run out of phase with those of the second half, and the time from "partial buffer handed
// back" to "next partial published" -- which, with two buffers, bounds the K-block period together with the
// promotion time -- shrinks by the MMA time of the other half.
// STORE_W: columns of one TMA-store box of the epilogue.  32: 32 rows x 64 bytes, 64-byte swizzle (2 KB of staging
// per promotion warp).  64 (needs 64 columns per warp, i.e. BN = 256): 32 rows x 128 bytes, 128-byte swizzle (4 KB
// per warp) -- half as many stores with rows twice as long, which is what stores that cross NVLink want.
template <int BN, int STAGES, int PROMO, int PIPE = PIPE_X16_DOUBLE, int SPLIT = 1, int STORE_W = 32>
__global__ void __launch_bounds__(kBlockwiseThreads, 1)
blockwise_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                      const __grid_constant__ OutputMaps outs, const BlockwiseParams p)
{
    static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
    static_assert(SPLIT == 1 || (SPLIT == 2 && BN == 256), "column halves only for the 256-wide tile");
    static_assert(STORE_W == 32 || (STORE_W == 64 && BN == 256), "wide store boxes need 64 columns per warp");
    constexpr int NBUF = 512 / BN;  // partial buffers in tensor memory (2, 4 or 8)
    constexpr int NSUB = BN / SPLIT;  // N of one MMA
    constexpr int CW = BN / 4;      // columns per promotion warp (64, 32 or 16)
    constexpr bool kPacked = PROMO == PROMO_MAGIC_X2;
    constexpr bool kBias = PROMO == PROMO_BIAS_X2;
    // (With double-buffered loads the biased mode works but spills: the write-back stores at several places make
    // the compiler copy the constant registers.)
    constexpr uint32_t kBytesA = kBM * kBK;
    constexpr uint32_t kBytesB = BN * kBK;
    constexpr uint32_t kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdesc = make_idesc_i8(kBM, NSUB, false);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // Behind the pipeline stages: one 32-row x 64-byte staging block per promotion warp for TMA stores (its
    // address is recomputed where it is used, to keep it out of the promotion loop's registers).

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    // bar_done[s]: the MMAs of the K block that used stage s have completed -- the stage may be reloaded (the
    // producer waits on it) AND the K block's partial is complete in tensor memory (the promotion warps wait on it).
    // One tcgen05.commit per K block serves both.
    __shared__ __align__(8) uint64_t bar_done[SPLIT][STAGES];
    __shared__ __align__(8) uint64_t bar_part_empty[SPLIT][NBUF];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            for (int h = 0; h < SPLIT; ++h) mbar_init(&bar_done[h][s], 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            for (int h = 0; h < SPLIT; ++h) mbar_init(&bar_part_empty[h][b], kPromoWarps / SPLIT);
        }
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_y);
    }
    if (warp == 2) {
        tmem_alloc(&tmem_base_slot, kTmemCols);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    // Promotion warps in the biased mode: eight registers that hold the constant for the write-back stores.
    [[maybe_unused]] uint32_t m8[8];
    if constexpr (kBias) {
        // Every partial buffer starts out holding the constant in all 128 lanes x 512 columns.
        if (warp >= 4) {
            uint32_t init8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) init8[j] = kMagicBits;
            const uint32_t base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(((warp - 4) >> 2) * 128);
#pragma unroll 1
            for (int c = 0; c < 128; c += 8) tmem_st_32x32b_x8(base + c, init8);
            tmem_st_wait();
            // Read the constant back (before any MMA can run): a tensor-memory load leaves its eight results in
            // consecutive registers, which is what the stores in the K loop want as their source -- with eight
            // independently defined registers the compiler copies them together again for every store.
            tmem_ld_32x32b_x8(base, m8);
            tmem_ld_wait();
        }
        tcgen05_fence_before_sync();
        __syncthreads();
        tcgen05_fence_after_sync();
    }

    if (warp < 4) {
        setmaxnreg_dec<kControlRegs>();
        if (warp == 0) {
            // -------------------------------------------------------------- TMA producer
            if (lane == 0) {
                uint32_t it = 0;
                bool ok = true;
                for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                    int mb, nb;
                    tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        bool freed = wait_or_abort(&bar_done[0][s], ph ^ 1, &abort_flag);
                        if (SPLIT == 2 && freed) freed = wait_or_abort(&bar_done[SPLIT - 1][s], ph ^ 1, &abort_flag);
                        if (!freed) {
                            raise_error(p.status, &abort_flag, ERR_TIMEOUT_PRODUCER);
                            ok = false;
                            break;
                        }
                        uint8_t* sa_tile = smem + s * kStageBytes;
                        mbar_arrive_expect_tx(&bar_full[s], kStageBytes);
                        tma_load_2d(sa_tile, &map_x, &bar_full[s], kb * kBK, mb * kBM);
                        tma_load_2d(sa_tile + kBytesA, &map_y, &bar_full[s], kb * kBK, nb * BN);
                    }
                }
                const uint32_t armed = it < STAGES ? it : STAGES;
                for (uint32_t j = 0; j < armed; ++j) {
                    const uint32_t i2 = it - 1 - j;
                    if (!mbar_wait(&bar_full[i2 % STAGES], (i2 / STAGES) & 1)) {
                        raise_error(p.status, &abort_flag, ERR_TIMEOUT_DRAIN);
                        break;
                    }
                }
            }
        } else if (warp == 1 || warp == 3) {
            // -------------------------------------------------------------- MMA issuers
            // Issuing the four MMAs of a K block and committing them costs one thread several hundred cycles
            // (more when its scheduler is busy with promotion warps), which is of the order of the tensor-core
            // time of the block itself.  Two threads on different schedulers therefore take alternate K blocks:
            // each owns the tensor-memory buffers of its parity, so no ordering between the two is needed.
            // (With an odd number of stages the two issuers share every stage; see the extra wait below.)
            static_assert(NBUF % 2 == 0, "K blocks of one parity must map to partial buffers of that parity");
            if (lane == 0) {
                const uint32_t parity = warp == 1 ? 0u : 1u;
                int my_tiles = 0;
                for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) ++my_tiles;
                const uint32_t total = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(num_kb);
                for (uint32_t it = parity; it < total; it += 2) {
                    const uint32_t s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    const uint32_t buf = it % NBUF;
                    const uint32_t bph = (it / NBUF) & 1;
                    // The operands first (they land long before the partial buffer is free) and everything that
                    // can be prepared, so that nothing but the MMAs stands between the buffer hand-back and the
                    // tensor core.
                    [[maybe_unused]] const long long c0 = GI8_BW_CLOCK();
                    if constexpr (STAGES % 2 != 0) {
                        // Odd stage count: this thread's K blocks do not return to a stage with alternating parity
                        // (stage 0 serves K blocks 0, 3, 6, ...: this thread sees only every second of its phases), and
                        // a parity wait cannot tell phase k from phase k - 2.  Observing the other issuer's K block
                        // first makes the thread see every phase of every stage in order.
                        if (it >= 1 && !wait_or_abort(&bar_full[(it - 1) % STAGES], ((it - 1) / STAGES) & 1, &abort_flag)) {
                            raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                            break;
                        }
                    }
                    const bool w1 = wait_or_abort(&bar_full[s], ph, &abort_flag);
                    const uint32_t tmem_d = tmem_base + buf * BN;
                    const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                    const uint64_t da = make_smem_desc_k128(a_addr);
                    const uint64_t db = make_smem_desc_k128(a_addr + kBytesA);
                    [[maybe_unused]] const long long c1 = GI8_BW_CLOCK();
                    [[maybe_unused]] long long c2 = 0, c3 = 0;
                    bool issued = w1;
#pragma unroll
                    for (int h = 0; h < SPLIT && issued; ++h) {
                        if (!wait_or_abort(&bar_part_empty[h][buf], bph ^ 1, &abort_flag)) {
                            issued = false;
                            break;
                        }
                        if (h == 0) c2 = GI8_BW_CLOCK();
                        tcgen05_fence_after_sync();
                        // Half h: rows h * NSUB.. of the weight tile (NSUB rows of 128 bytes: 16-byte units in
                        // the descriptor's address field) into columns h * NSUB.. of the partial buffer.
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k)
                            umma_i8(tmem_d + h * NSUB, da + 2 * k, db + (h * NSUB * kBK) / 16 + 2 * k, kIdesc, (kBias || k != 0) ? 1u : 0u);
                        if (h == SPLIT - 1) c3 = GI8_BW_CLOCK();
                        umma_commit(&bar_done[h][s]);
                    }
                    if (!issued) {
                        raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                        break;
                    }
                    GI8_BW_DBG(1, c1 - c0);
                    GI8_BW_DBG(0, c2 - c1);
                    GI8_BW_DBG(2, c3 - c2);
                    GI8_BW_DBG(3, GI8_BW_CLOCK() - c3);
                    GI8_BW_DBG(4, 1);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue warps
        setmaxnreg_inc<kPromoRegs>();
        const int quarter = warp & 3;
        const int cg = (warp - 4) >> 2;   // column quarter of the tile
        // Tensor-memory address of this warp's lanes and first column in partial buffer 0 (buffer b is b * BN
        // columns further).  GI8_PIN keeps such loop-invariant values in a register: left alone, the compiler
        // re-derives them from %tid.x inside the K loop -- a dozen integer instructions per use, in a loop whose
        // bound is instruction issue.
        uint32_t tm_warp = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(cg * CW);
        GI8_PIN(tm_warp);
        // Barriers of this warp's column half, as shared-memory addresses.
        const int half = SPLIT == 2 ? cg >> 1 : 0;
        uint32_t bar_done_h = smem_u32(&bar_done[half][0]);
        uint32_t bar_empty_h = smem_u32(&bar_part_empty[half][0]);
        if constexpr (SPLIT == 2) {
            GI8_PIN(bar_done_h);
            GI8_PIN(bar_empty_h);
        }
        // How a warp's CW columns of a K block travel from tensor memory to registers:
        //   PIPE_X16_DOUBLE  16-column loads into two alternating register sets; while one set is converted the
        //                    next load (the first of the next K block after the last) is in flight.
        //   PIPE_X32_DOUBLE  the same with 32-column loads (needs CW == 32: 32 accumulators + 2 x 32 registers).
        //   PIPE_X32_SINGLE  32-column loads into one register set, load -> wait -> convert; the latency is
        //                    covered by the other warps of the scheduler only.
        constexpr int kChunk = (PIPE == PIPE_X16_DOUBLE || PIPE == PIPE_X16_SINGLE) ? 16 : 32;  // columns per load
        constexpr bool kDouble = PIPE == PIPE_X16_DOUBLE || PIPE == PIPE_X32_DOUBLE;
        constexpr int NC = CW / kChunk;                             // chunks per K block per warp
        static_assert(CW % kChunk == 0 && (!kDouble || NC == 1 || NC % 2 == 0), "chunk registers alternate statically");
        uint32_t it = 0;                    // running K-block counter, as in the MMA warp
        bool ok = true;

        uint32_t va[kChunk], vb[kDouble ? kChunk : 1];

        [[maybe_unused]] long long dbg_t = GI8_BW_CLOCK();
        const int first_tile = blockIdx.x;

        auto load_chunk = [&](uint32_t taddr, uint32_t (&v)[kChunk]) {
            if constexpr (kChunk == 16) tmem_ld_32x32b_x16(taddr, v);
            else tmem_ld_32x32b_x32(taddr, v);
        };
        // Waits for the partial of K block `kblock` (running index); false on every lane if any lane gave up.
        // The common case is one successful test; the branch to the bounded spin is taken on a vote, which makes
        // it warp-uniform (no reconvergence bookkeeping in the loop).
        auto wait_partial = [&](uint32_t kblock) {
            const uint32_t bar = bar_done_h + (kblock % STAGES) * 8;
            const uint32_t parity = (kblock / STAGES) & 1;
            bool got = mbar_try_wait_addr(bar, parity);
            if (!__all_sync(0xffffffffu, got)) {
                got = wait_or_abort_addr(bar, parity, &abort_flag);
                if (!got && lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                got = __all_sync(0xffffffffu, got);
                if (!got) return false;
            }
            tcgen05_fence_after_sync();
            return true;
        };
        // The whole partial buffer of K block `kblock` is in registers: hand it back to the MMA issuers.
        auto release_partial = [&](uint32_t kblock) {
            tcgen05_fence_before_sync();
            __syncwarp();
            mbar_arrive_elected_addr(bar_empty_h + (kblock % NBUF) * 8);
        };

        for (int tile = first_tile; tile < num_tiles && ok; tile += gridDim.x) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
            const int row = mb * kBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const int col_base = nb * BN + cg * CW;  // first output column of this warp
            // A column quarter lies inside one 128-wide weight-scale block (CW divides 128, col_base % CW == 0).
            const bool cols_ok = col_base < p.N;
            // 32-bit element offsets (the scale arrays are far smaller than 2^31 elements) instead of two pointers.
            uint32_t sa_off = static_cast<uint32_t>(row_ok ? row : 0) * static_cast<uint32_t>(p.ld_sa);
            uint32_t sw_off = static_cast<uint32_t>(cols_ok ? col_base / 128 : 0) * static_cast<uint32_t>(p.ld_sw);
            GI8_PIN(sa_off);
            GI8_PIN(sw_off);

            // The tile's first K block (no load is carried over from the previous tile: the epilogue then runs
            // without a chunk in flight, which it has no registers for).
            if (!wait_partial(it)) {
                ok = false;
                break;
            }
            if constexpr (kDouble) load_chunk(tm_warp + (it % NBUF) * BN, va);
            [[maybe_unused]] auto store_magic = [&](uint32_t taddr) {
#pragma unroll
                for (int jj = 0; jj < kChunk; jj += 8) tmem_st_32x32b_x8(taddr + jj, m8);
            };

            float acc[CW];
#pragma unroll
            for (int j = 0; j < CW; ++j) acc[j] = 0.0f;

            // Scales are loaded kScaleDepth K blocks before their use (an L2 hit takes longer than one K block);
            // set j serves the K blocks with kb % kScaleDepth == j, statically, through unrolling.
            constexpr int kScaleDepth = (kDouble && NC > 1) ? 1 : (BN == 256 ? 2 : (kDouble ? 2 : 4));
            float sa_q[kScaleDepth], sw_q[kScaleDepth];
#pragma unroll
            for (int j = 0; j < kScaleDepth; ++j) {
                if (j < num_kb) {
                    sa_q[j] = __ldg(p.sa + (sa_off + j));
                    sw_q[j] = __ldg(p.sw + (sw_off + j));
                }
            }
            if constexpr (kDouble) {
                tmem_ld_wait();
                if constexpr (kBias) store_magic(tm_warp + (it % NBUF) * BN);
            }

            float t = 0.0f;
            // Scale of K block kb (fp32 product, round to nearest) and the loads for the next one.
            auto scale_from_set = [&](int kb, int j) {
                t = sa_q[j] * sw_q[j];
                if constexpr (PROMO == PROMO_ABLATE_SCALES) t = 0.5f;
                if (PROMO != PROMO_ABLATE_SCALES && kb + kScaleDepth < num_kb) {
                    sa_q[j] = __ldg(p.sa + (sa_off + kb + kScaleDepth));
                    sw_q[j] = __ldg(p.sw + (sw_off + kb + kScaleDepth));
                }
            };
            auto consume = [&](const uint32_t (&v)[kChunk], int c) {
                if constexpr (PROMO == PROMO_ABLATE_HANDSHAKE) return;
                if constexpr (PROMO == PROMO_ABLATE_LOAD) {
                    acc[c] = __uint_as_float(__float_as_uint(acc[c]) ^ v[0] ^ v[kChunk - 1]);
                    return;
                }
                if constexpr (PROMO == PROMO_ABLATE_MATH) {
                    acc[c] = __uint_as_float(__float_as_uint(acc[c]) ^ v[0] ^ v[kChunk - 1]) + t;
                    return;
                }
#pragma unroll
                for (int j = 0; j < kChunk; j += 2) {
                    if constexpr (PROMO == PROMO_ABLATE_FMA_ONLY) {
                        acc[c + j] = fmaf(__uint_as_float(v[j]), t, acc[c + j]);
                        acc[c + j + 1] = fmaf(__uint_as_float(v[j + 1]), t, acc[c + j + 1]);
                    } else if constexpr (PROMO == PROMO_ABLATE_CVT_ONLY) {
                        acc[c + j] = __int2float_rn(static_cast<int32_t>(v[j]) + __float_as_int(acc[c + j]));
                        acc[c + j + 1] = __int2float_rn(static_cast<int32_t>(v[j + 1]) + __float_as_int(acc[c + j + 1]));
                    } else if constexpr (kBias) {
                        promote_biased_pair(v[j], v[j + 1], t, acc[c + j], acc[c + j + 1]);
                    } else if constexpr (kPacked) {
                        const uint64_t neg2 = pack_f32x2(__float_as_uint(-kMagicF32), __float_as_uint(-kMagicF32));
                        const uint64_t t2 = pack_f32x2(__float_as_uint(t), __float_as_uint(t));
                        const uint64_t pf = add_f32x2(pack_f32x2(v[j] + kMagicBits, v[j + 1] + kMagicBits), neg2);
                        const uint64_t a2 = fma_f32x2(
                            pf, t2, pack_f32x2(__float_as_uint(acc[c + j]), __float_as_uint(acc[c + j + 1])));
                        unpack_f32x2(a2, acc[c + j], acc[c + j + 1]);
                    } else if constexpr (PROMO == PROMO_I2F || PROMO == PROMO_ABLATE_SCALES) {
                        acc[c + j] = fmaf(__int2float_rn(static_cast<int32_t>(v[j])), t, acc[c + j]);
                        acc[c + j + 1] = fmaf(__int2float_rn(static_cast<int32_t>(v[j + 1])), t, acc[c + j + 1]);
                    } else {
                        acc[c + j] = fmaf(__uint_as_float(v[j] + kMagicBits) - kMagicF32, t, acc[c + j]);
                        acc[c + j + 1] = fmaf(__uint_as_float(v[j + 1] + kMagicBits) - kMagicF32, t, acc[c + j + 1]);
                    }
                }
            };
            // Double-buffered step: chunk c of K block kb has landed in `cur` (and, in the biased mode, the
            // constant has been written back over it).  Start the next chunk's load into `nxt` -- the first chunk
            // of the next K block after the last one -- then do this chunk's arithmetic; the buffer is handed
            // back after the last chunk's arithmetic, when the write-back stores have long completed.
            auto chunk_step = [&](const uint32_t (&cur)[kChunk], uint32_t (&nxt)[kChunk], int kb, int c) {
                const bool last_chunk = c + 1 == NC;
                const bool have_next = !last_chunk || kb + 1 < num_kb;
                uint32_t next_addr = tm_warp + (it % NBUF) * BN + (c + 1) * kChunk;
                if (last_chunk && have_next) {
                    [[maybe_unused]] const long long w0 = GI8_BW_CLOCK();
                    if (warp == 4 && lane == 0) { GI8_BW_DBG(6, w0 - dbg_t); }
                    ok = wait_partial(it + 1);
                    dbg_t = GI8_BW_CLOCK();
                    if (warp == 4 && lane == 0) { GI8_BW_DBG(5, dbg_t - w0); GI8_BW_DBG(7, 1); }
                    next_addr = tm_warp + ((it + 1) % NBUF) * BN;
                }
                const bool in_flight = have_next && ok;
                if (in_flight) load_chunk(next_addr, nxt);
                consume(cur, c * kChunk);
                if (last_chunk) {
                    if constexpr (kBias) tmem_st_wait();
                    release_partial(it);
                    ++it;
                }
                if (in_flight) {
                    tmem_ld_wait();
                    if constexpr (kBias) store_magic(next_addr);
                }
            };

            if constexpr (!kDouble) {
                bool tile_done = false;
                for (int kb = 0; !tile_done && ok;) {
#pragma unroll
                    for (int j = 0; j < kScaleDepth; ++j) {
                        scale_from_set(kb, j);
                        const uint32_t taddr = tm_warp + (it % NBUF) * BN;
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            load_chunk(taddr + c * kChunk, va);
                            tmem_ld_wait();
                            if constexpr (kBias) {
#pragma unroll
                                for (int jj = 0; jj < kChunk; jj += 8) tmem_st_32x32b_x8(taddr + c * kChunk + jj, m8);
                                if (c + 1 == NC) tmem_st_wait();
                            }
                            if (c + 1 == NC) release_partial(it);
                            consume(va, c * kChunk);
                        }
                        ++it;
                        if (++kb == num_kb) {
                            tile_done = true;
                            break;
                        }
                        [[maybe_unused]] const long long w0 = GI8_BW_CLOCK();
                        if (warp == 4 && lane == 0) { GI8_BW_DBG(6, w0 - dbg_t); }
                        if (!wait_partial(it)) {
                            ok = false;
                            break;
                        }
                        dbg_t = GI8_BW_CLOCK();
                        if (warp == 4 && lane == 0) { GI8_BW_DBG(5, dbg_t - w0); GI8_BW_DBG(7, 1); }
                    }
                }
            } else if constexpr (NC == 1) {
                // One chunk per K block: the register sets (and the scale sets) alternate from K block to K block.
                for (int kb = 0; kb < num_kb && ok; kb += 2) {
                    scale_from_set(kb, 0);
                    chunk_step(va, vb, kb, 0);
                    if (kb + 1 < num_kb && ok) {
                        scale_from_set(kb + 1, 1);
                        chunk_step(vb, va, kb + 1, 0);
                    }
                }
            } else {
                for (int kb = 0; kb < num_kb && ok; ++kb) {
                    scale_from_set(kb, 0);
#pragma unroll
                    for (int c = 0; c < NC; c += 2) {
                        chunk_step(va, vb, kb, c);  // NC is even: even chunks in va, odd chunks in vb
                        chunk_step(vb, va, kb, c + 1);
                    }
                }
            }
            if (!ok) break;

            bool stored = false;
            if constexpr (CW >= 32) {
                if (p.tma_store) {
                    stored = true;
                    // 32 x 32 blocks through 64-byte-swizzled shared memory and TMA stores (rows >= M and columns >= N
                    // are clipped by the hardware); see the dense kernel's epilogue for the layout.  The tile's
                    // coordinates are derived again from an opaque copy of the tile index so that they do not occupy
                    // registers across the promotion loop.
                    int tile_again = tile, mb2, nb2;
                    asm volatile("" : "+r"(tile_again));
                    tile_coords(tile_again, p.tiles_m, p.tiles_n, mb2, nb2, p.group_m);
                    const int row0 = mb2 * kBM + quarter * 32;
                    const int col_base = nb2 * BN + cg * CW;
                    if constexpr (STORE_W == 64) {
                        if (row0 < p.M && col_base < p.N) {
                            const uint32_t stg = ((smem_u32(smem_raw) + 1023u) & ~1023u) + STAGES * kStageBytes + (warp - 4) * 4096;
                            if (lane == 0) tma_store_wait_read<0>();
                            __syncwarp();
                            // row = lane: eight 16-byte chunks, chunk index xor (row % 8) (the 128-byte swizzle)
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const int cq = q ^ (lane & 7);
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * 128 + cq * 16),
                                             "r"(pack_bf16x2(acc[8 * q], acc[8 * q + 1])),
                                             "r"(pack_bf16x2(acc[8 * q + 2], acc[8 * q + 3])),
                                             "r"(pack_bf16x2(acc[8 * q + 4], acc[8 * q + 5])),
                                             "r"(pack_bf16x2(acc[8 * q + 6], acc[8 * q + 7]))
                                             : "memory");
                            }
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                for (int o = 0; o < p.n_out; ++o)
                                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                                     reinterpret_cast<uint64_t>(&outs.m[o])),
                                                 "r"(stg), "r"(p.out_col0 + col_base), "r"(row0)
                                                 : "memory");
                                tma_store_commit();
                            }
                        }
                    } else if (row0 < p.M && col_base < p.N) {
                        const uint32_t stg = ((smem_u32(smem_raw) + 1023u) & ~1023u) + STAGES * kStageBytes + (warp - 4) * 2048;
#pragma unroll
                        for (int c = 0; c < CW; c += 32) {
                            if (col_base + c >= p.N) break;
                            if (lane == 0) tma_store_wait_read<0>();
                            __syncwarp();
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int cq = q ^ ((lane >> 1) & 3);
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * 64 + cq * 16),
                                             "r"(pack_bf16x2(acc[c + 8 * q], acc[c + 8 * q + 1])),
                                             "r"(pack_bf16x2(acc[c + 8 * q + 2], acc[c + 8 * q + 3])),
                                             "r"(pack_bf16x2(acc[c + 8 * q + 4], acc[c + 8 * q + 5])),
                                             "r"(pack_bf16x2(acc[c + 8 * q + 6], acc[c + 8 * q + 7]))
                                             : "memory");
                            }
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                // one store per output matrix (the local one, and in an N-sharded group every
                                // peer's, through its mapped memory: plain unicast TMA stores)
                                for (int o = 0; o < p.n_out; ++o)
                                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                                     reinterpret_cast<uint64_t>(&outs.m[o])),
                                                 "r"(stg), "r"(p.out_col0 + col_base + c), "r"(row0)
                                                 : "memory");
                                tma_store_commit();
                            }
                        }
                    }
                }
            }
            if (!stored && row_ok && cols_ok) {
                uint16_t* dst = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col_base;
                if (col_base + CW <= p.N && p.vec_ok) {
#pragma unroll
                    for (int j = 0; j < CW; j += 8)
                        *reinterpret_cast<uint4*>(dst + j) =
                            make_uint4(pack_bf16x2(acc[j], acc[j + 1]), pack_bf16x2(acc[j + 2], acc[j + 3]),
                                       pack_bf16x2(acc[j + 4], acc[j + 5]), pack_bf16x2(acc[j + 6], acc[j + 7]));
                } else {
#pragma unroll
                    for (int j = 0; j < CW; ++j)
                        if (col_base + j < p.N) dst[j] = to_bf16_bits(acc[j]);
                }
            }
            __syncwarp();
        }
        if (lane == 0) tma_store_wait_all<0>();  // stores read this CTA's shared memory: finish before exit
    }

    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        __syncwarp();
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace gi8
