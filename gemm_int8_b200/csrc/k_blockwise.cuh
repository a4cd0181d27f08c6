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
#else
#define GI8_BW_DBG(slot, v) ((void)0)
#endif

template <int BN, int STAGES, int PROMO>
__global__ void __launch_bounds__(kBlockwiseThreads, 1)
blockwise_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                      const __grid_constant__ CUtensorMap map_out, const BlockwiseParams p)
{
    static_assert(BN == 128 || BN == 256, "BN must be 128 or 256");
    constexpr int NBUF = 512 / BN;  // partial buffers in tensor memory (2 or 4)
    constexpr int CW = BN / 4;      // columns per promotion warp (64 or 32)
    constexpr bool kPacked = PROMO == PROMO_MAGIC_X2;
    constexpr uint32_t kBytesA = kBM * kBK;
    constexpr uint32_t kBytesB = BN * kBK;
    constexpr uint32_t kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdesc = make_idesc_i8(kBM, BN, false);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // Behind the pipeline stages: one 32-row x 64-byte staging block per promotion warp for TMA stores (its
    // address is recomputed where it is used, to keep it out of the promotion loop's registers).

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    // bar_done[s]: the MMAs of the K block that used stage s have completed -- the stage may be reloaded (the
    // producer waits on it) AND the K block's partial is complete in tensor memory (the promotion warps wait on it).
    // One tcgen05.commit per K block serves both.
    __shared__ __align__(8) uint64_t bar_done[STAGES];
    __shared__ __align__(8) uint64_t bar_part_empty[NBUF];
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
            mbar_init(&bar_done[s], 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(&bar_part_empty[b], kPromoWarps);
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
                        if (!wait_or_abort(&bar_done[s], ph ^ 1, &abort_flag)) {
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
            // each owns the tensor-memory buffers and pipeline stages of its parity, so no ordering between the
            // two is needed.
            static_assert(STAGES % 2 == 0 && NBUF % 2 == 0, "K blocks of one parity must map to stages/buffers of that parity");
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
                    const long long c0 = clock64();
                    const bool w1 = wait_or_abort(&bar_part_empty[buf], bph ^ 1, &abort_flag);
                    const long long c1 = clock64();
                    if (!w1 || !wait_or_abort(&bar_full[s], ph, &abort_flag)) {
                        raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                        break;
                    }
                    const long long c2 = clock64();
                    tcgen05_fence_after_sync();
                    const uint32_t tmem_d = tmem_base + buf * BN;
                    const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                    const uint64_t da = make_smem_desc_k128(a_addr);
                    const uint64_t db = make_smem_desc_k128(a_addr + kBytesA);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k)
                        umma_i8(tmem_d, da + 2 * k, db + 2 * k, kIdesc, k != 0 ? 1u : 0u);
                    const long long c3 = clock64();
                    umma_commit(&bar_done[s]);
                    GI8_BW_DBG(0, c1 - c0);
                    GI8_BW_DBG(1, c2 - c1);
                    GI8_BW_DBG(2, c3 - c2);
                    GI8_BW_DBG(3, clock64() - c3);
                    GI8_BW_DBG(4, 1);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue warps
        setmaxnreg_inc<kPromoRegs>();
        const int quarter = warp & 3;
        const int cg = (warp - 4) >> 2;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        constexpr int kChunk = 16;          // columns per tensor-memory load
        constexpr int NC = CW / kChunk;     // chunks per K block per warp (4 or 2, even)
        static_assert(NC % 2 == 0, "the two chunk registers alternate statically");
        uint32_t it = 0;                    // running K-block counter, as in the MMA warp
        bool ok = true;

        // Software pipeline over 16-column chunks that runs ACROSS K blocks: while chunk c is converted and
        // accumulated, the load of the next chunk -- the first chunk of the next K block when c is the last --
        // is already in flight, so neither the tensor-memory load latency nor the hand-over to the MMA warp sits
        // in front of the arithmetic.  A buffer is handed back as soon as its last chunk is in registers.
        uint32_t va[kChunk], vb[kChunk];
        long long dbg_t = clock64();
        const int first_tile = blockIdx.x;

        for (int tile = first_tile; tile < num_tiles && ok; tile += gridDim.x) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
            const int row = mb * kBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const int col_base = nb * BN + cg * CW;  // first output column of this warp
            // A column quarter lies inside one 128-wide weight-scale block (CW divides 128, col_base % CW == 0).
            const bool cols_ok = col_base < p.N;
            const float* sa_row = p.sa + static_cast<int64_t>(row_ok ? row : 0) * p.ld_sa;
            const float* sw_row = p.sw + static_cast<int64_t>(cols_ok ? col_base / 128 : 0) * p.ld_sw;

            // First chunk of the tile's first K block (not issued from the previous tile's last chunk: the
            // epilogue then runs without a chunk in flight, which it has no registers for).
            if (!wait_or_abort(&bar_done[it % STAGES], (it / STAGES) & 1, &abort_flag)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after_sync();
            tmem_ld_32x32b_x16(tmem_base + lane_base + (it % NBUF) * BN + cg * CW, va);

            float acc[CW];
#pragma unroll
            for (int j = 0; j < CW; ++j) acc[j] = 0.0f;

            float sa_next = __ldg(sa_row);
            float sw_next = __ldg(sw_row);
            tmem_ld_wait();
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                float t = sa_next * sw_next;  // fp32, round to nearest: the scale of this K block
                if constexpr (PROMO == PROMO_ABLATE_SCALES) t = 0.5f;
                if (PROMO != PROMO_ABLATE_SCALES && kb + 1 < num_kb) {
                    sa_next = __ldg(sa_row + kb + 1);
                    sw_next = __ldg(sw_row + kb + 1);
                }
                const uint32_t taddr = tmem_base + lane_base + (it % NBUF) * BN + cg * CW;

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

#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    // Chunk c of this K block is in va (c even) or vb (c odd) and has landed.
                    bool in_flight = false;
                    if (c + 1 < NC) {
                        if (c & 1) tmem_ld_32x32b_x16(taddr + (c + 1) * kChunk, va);
                        else tmem_ld_32x32b_x16(taddr + (c + 1) * kChunk, vb);
                        in_flight = true;
                    } else {
                        // Last chunk: the whole buffer is in registers -> hand it back, then start on the next
                        // K block (possibly the next tile's first) before doing this chunk's arithmetic.
                        tcgen05_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bar_part_empty[it % NBUF]);
                        const bool have_next = kb + 1 < num_kb;
                        if (have_next) {
                            const uint32_t nit = it + 1;
                            const long long w0 = clock64();
                            if (warp == 4 && lane == 0) { GI8_BW_DBG(6, w0 - dbg_t); }
                            if (!wait_or_abort(&bar_done[nit % STAGES], (nit / STAGES) & 1, &abort_flag)) {
                                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                                ok = false;
                            }
                            ok = __all_sync(0xffffffffu, ok);
                            dbg_t = clock64();
                            if (warp == 4 && lane == 0) { GI8_BW_DBG(5, dbg_t - w0); GI8_BW_DBG(7, 1); }
                            if (ok) {
                                tcgen05_fence_after_sync();
                                tmem_ld_32x32b_x16(tmem_base + lane_base + (nit % NBUF) * BN + cg * CW, va);
                                in_flight = true;
                            }
                        }
                    }
                    if (c & 1) consume(vb, c * kChunk);
                    else consume(va, c * kChunk);
                    if (in_flight) tmem_ld_wait();
                }
                if (!ok) break;
            }
            if (!ok) break;

            if (p.tma_store) {
                // 32 x 32 blocks through 64-byte-swizzled shared memory and TMA stores (rows >= M and columns >= N
                // are clipped by the hardware); see the dense kernel's epilogue for the layout.  The tile's
                // coordinates are derived again from an opaque copy of the tile index so that they do not occupy
                // registers across the promotion loop.
                int tile_again = tile, mb2, nb2;
                asm volatile("" : "+r"(tile_again));
                tile_coords(tile_again, p.tiles_m, p.tiles_n, mb2, nb2, p.group_m);
                const int row0 = mb2 * kBM + quarter * 32;
                const int col_base = nb2 * BN + cg * CW;
                if (row0 < p.M && col_base < p.N) {
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
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                             reinterpret_cast<uint64_t>(&map_out)),
                                         "r"(stg), "r"(col_base + c), "r"(row0)
                                         : "memory");
                            tma_store_commit();
                        }
                    }
                }
            } else if (row_ok && cols_ok) {
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
