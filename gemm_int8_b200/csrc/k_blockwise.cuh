// Blockwise-dequantised W8A8 GEMM for sm_100a:
//   out[m,n] = bf16( sum_kb fp32(P[m,n,kb]) * (sa[m,kb] * sw[n/128,kb]) ),  kb ascending, one fused
//   multiply-add per K block (128 wide), P = exact int32 partial dot product of the block.
// There is no such path in the reference (its epilogue applies one scalar, csrc/kernels/gemm.cu:96); the
// semantics are those of the CPU oracle's blockwise restatement.
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer (as in the dense kernel).
//   warp 1      MMA issuer: per K block, four tcgen05.mma kind::i8 that OVERWRITE one of two tensor-memory
//               partial buffers (accumulate disabled on the first), then a commit to that buffer's barrier.
//   warps 2..9  promotion: tcgen05.ld the int32 partial, convert to fp32, fma with the block's scale into
//               fp32 register accumulators while the MMA warp already fills the other buffer.  Warp w owns
//               TMEM lane quarter (w % 4) and column half ((w - 2) / 4) of the tile; a column half never
//               straddles a 128-wide weight-scale block.  At the end of the tile the same warps cast to
//               bf16 and store.
#pragma once

#include "k_dense.cuh"

namespace gi8 {

constexpr int kBlockwiseThreads = 320;

// How a promotion warp turns an int32 partial P (|P| <= 128 * 128 * 128 = 2^21) into fp32 and accumulates it.
// All three produce bit-identical results: fp32(P) is exact, and the packed f32x2 instructions round each
// half like the scalar ones.
enum Promotion : int {
    PROMO_MAGIC = 0,     // per element: integer add of 0x4B400000, fp32 subtract of 12582912.0, fma
    PROMO_MAGIC_X2 = 1,  // same, with add.f32x2 / fma.f32x2 on register pairs (half the fp32 instructions)
    PROMO_BIAS_X2 = 2,   // the TMEM buffer is pre-filled with 0x4B400000 and the MMA accumulates onto it, so the
                         // value read back is already the float 12582912 + P: only the packed subtract and fma
                         // remain; the warp re-fills the buffer (tcgen05.st) before handing it back
};

constexpr uint32_t kMagicBits = 0x4B400000u;  // fp32 12582912.0 = 1.5 * 2^23: adding an integer |P| < 2^22 to the
constexpr float kMagicF32 = 12582912.0f;      // bit pattern adds P to the value exactly

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

// Stores one 32-bit value to N consecutive TMEM columns (N = 8 or 16) of the warp's 32 lanes.
template <int N>
GI8_DEVICE void tmem_fill_32x32b(uint32_t taddr, uint32_t v)
{
    if constexpr (N == 16) {
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(v)
            : "memory");
    } else {
        static_assert(N == 8, "fill width");
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(v)
                     : "memory");
    }
}

template <int N>
GI8_DEVICE void tmem_ld_chunk(uint32_t taddr, uint32_t (&r)[N])
{
    if constexpr (N == 16) tmem_ld_32x32b_x16(taddr, r);
    else tmem_ld_32x32b_x8(taddr, r);
}

GI8_DEVICE void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

struct BlockwiseParams {
    void* out;        // bf16 [M,N], leading dimension ldo
    const float* sa;  // [M, KB], row stride ld_sa
    const float* sw;  // [ceil(N/128), KB], row stride ld_sw
    uint32_t* status;
    int64_t ldo, ld_sa, ld_sw;
    int M, N, K;
    int tiles_m, tiles_n;
    int vec_ok;  // out is 16-byte aligned and ldo % 8 == 0
};

template <int BN, int STAGES, int PROMO>
__global__ void __launch_bounds__(kBlockwiseThreads, 1)
blockwise_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                      const BlockwiseParams p)
{
    static_assert(BN == 128 || BN == 256, "BN must be 128 or 256");
    constexpr int CW = BN / 2;  // columns per promotion warp
    constexpr int kLd = CW > 64 ? 8 : 16;  // columns per tcgen05.ld; two chunks live at a time (register budget)
    constexpr bool kBias = PROMO == PROMO_BIAS_X2;
    constexpr uint32_t kBytesA = kBM * kBK;
    constexpr uint32_t kBytesB = BN * kBK;
    constexpr uint32_t kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512
    constexpr uint32_t kIdesc = make_idesc_i8(kBM, BN, false);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_part_full[2];
    __shared__ __align__(8) uint64_t bar_part_empty[2];
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
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_part_full[b], 1);
            mbar_init(&bar_part_empty[b], 8);
        }
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_y);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, kTmemCols);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int mb, nb;
                tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!wait_or_abort(&bar_empty[s], ph ^ 1, &abort_flag)) {
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
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0;  // running K-block counter: selects both the smem stage and the TMEM buffer
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    const uint32_t buf = it & 1;
                    const uint32_t bph = (it >> 1) & 1;
                    // kBias: the buffer's first hand-over is the promotion warps' initial fill (one extra phase)
                    if (!wait_or_abort(&bar_part_empty[buf], kBias ? bph : (bph ^ 1), &abort_flag) ||
                        !wait_or_abort(&bar_full[s], ph, &abort_flag)) {
                        raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after_sync();
                    const uint32_t tmem_d = tmem_base + buf * BN;
                    const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                    const uint64_t da = make_smem_desc_k128(a_addr);
                    const uint64_t db = make_smem_desc_k128(a_addr + kBytesA);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k)
                        umma_i8(tmem_d, da + 2 * k, db + 2 * k, kIdesc, (kBias || k != 0) ? 1u : 0u);
                    umma_commit(&bar_empty[s]);
                    umma_commit(&bar_part_full[buf]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue warps
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        uint32_t it = 0;
        bool ok = true;

        if constexpr (kBias) {
            // Pre-fill this warp's part of both partial buffers with the magic constant, then hand them over.
#pragma unroll
            for (int b = 0; b < 2; ++b) {
#pragma unroll
                for (int c = 0; c < CW; c += kLd) tmem_fill_32x32b<kLd>(tmem_base + lane_base + b * BN + half * CW + c, kMagicBits);
            }
            tmem_st_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bar_part_empty[0]);
                mbar_arrive(&bar_part_empty[1]);
            }
        }

        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb);
            const int row = mb * kBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const int col_base = nb * BN + half * CW;  // first output column of this warp
            // A column half lies inside one 128-wide weight-scale block (CW divides 128, col_base % CW == 0).
            const bool cols_ok = col_base < p.N;
            const float* sa_row = p.sa + static_cast<int64_t>(row_ok ? row : 0) * p.ld_sa;
            const float* sw_row = p.sw + static_cast<int64_t>(cols_ok ? col_base / 128 : 0) * p.ld_sw;

            // fp32 accumulators, two per 64-bit register pair: acc2[j] = {column 2j, column 2j + 1}
            uint64_t acc2[CW / 2];
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) acc2[j] = 0ull;

            float sa_next = __ldg(sa_row);
            float sw_next = __ldg(sw_row);
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const uint32_t buf = it & 1;
                const uint32_t bph = (it >> 1) & 1;
                const float t = sa_next * sw_next;  // fp32, round to nearest: the scale of this K block
                if (kb + 1 < num_kb) {
                    sa_next = __ldg(sa_row + kb + 1);
                    sw_next = __ldg(sw_row + kb + 1);
                }
                const uint64_t t2 = pack_f32x2(__float_as_uint(t), __float_as_uint(t));
                const uint64_t neg_magic2 = pack_f32x2(__float_as_uint(-kMagicF32), __float_as_uint(-kMagicF32));
                if (!wait_or_abort(&bar_part_full[buf], bph, &abort_flag)) {
                    if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                    ok = false;
                    break;
                }
                tcgen05_fence_after_sync();
                const uint32_t taddr = tmem_base + lane_base + buf * BN + half * CW;

                // Software pipeline over 16-column chunks: the load of chunk c + 1 is in flight while chunk c
                // is converted and accumulated.
                uint32_t va[kLd], vb[kLd];
                auto consume = [&](const uint32_t (&v)[kLd], int c) {
#pragma unroll
                    for (int j = 0; j < kLd; j += 2) {
                        if constexpr (PROMO == PROMO_MAGIC) {
                            float lo, hi;
                            unpack_f32x2(acc2[(c + j) / 2], lo, hi);
                            lo = fmaf(__uint_as_float(v[j] + kMagicBits) - kMagicF32, t, lo);
                            hi = fmaf(__uint_as_float(v[j + 1] + kMagicBits) - kMagicF32, t, hi);
                            acc2[(c + j) / 2] = pack_f32x2(__float_as_uint(lo), __float_as_uint(hi));
                        } else {
                            const uint32_t b0 = kBias ? v[j] : v[j] + kMagicBits;
                            const uint32_t b1 = kBias ? v[j + 1] : v[j + 1] + kMagicBits;
                            const uint64_t pf = add_f32x2(pack_f32x2(b0, b1), neg_magic2);  // exact fp32(P)
                            acc2[(c + j) / 2] = fma_f32x2(pf, t2, acc2[(c + j) / 2]);
                        }
                    }
                };
                tmem_ld_chunk<kLd>(taddr, va);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < CW; c += 2 * kLd) {
                    tmem_ld_chunk<kLd>(taddr + c + kLd, vb);
                    if constexpr (kBias) tmem_fill_32x32b<kLd>(taddr + c, kMagicBits);
                    consume(va, c);
                    tmem_ld_wait();
                    if (c + 2 * kLd < CW) tmem_ld_chunk<kLd>(taddr + c + 2 * kLd, va);
                    if constexpr (kBias) tmem_fill_32x32b<kLd>(taddr + c + kLd, kMagicBits);
                    consume(vb, c + kLd);
                    if (c + 2 * kLd < CW) tmem_ld_wait();
                }
                if constexpr (kBias) tmem_st_wait();
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_part_empty[buf]);
            }
            if (!ok) break;

            if (row_ok && cols_ok) {
                uint16_t* dst = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col_base;
                if (col_base + CW <= p.N && p.vec_ok) {
#pragma unroll
                    for (int j = 0; j < CW; j += 8) {
                        float f[8];
#pragma unroll
                        for (int q = 0; q < 4; ++q) unpack_f32x2(acc2[j / 2 + q], f[2 * q], f[2 * q + 1]);
                        *reinterpret_cast<uint4*>(dst + j) =
                            make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                                       pack_bf16x2(f[6], f[7]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < CW; j += 2) {
                        float lo, hi;
                        unpack_f32x2(acc2[j / 2], lo, hi);
                        if (col_base + j < p.N) dst[j] = to_bf16_bits(lo);
                        if (col_base + j + 1 < p.N) dst[j + 1] = to_bf16_bits(hi);
                    }
                }
            }
            __syncwarp();
        }
    }

    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace gi8
