// Blockwise-dequantised W8A8 GEMM, two-CTA form (same arithmetic and results as k_blockwise.cuh).
//
// Two CTAs on neighbouring SMs (a 2 x 1 x 1 cluster) share one 256 x 128 output tile: tcgen05.mma.cta_group::2
// (M = 256) is issued by the leader CTA's MMA thread and reads the A rows and half of the B rows from each
// CTA's own shared memory; each CTA keeps its 128 x 128 int32 partial in its own tensor memory.  Per CTA that is
//   * 6 KB of shared-memory operand traffic per instruction instead of 8 KB for a one-CTA 128 x 128 tile, so the
//     narrow tile no longer starves the tensor core, and
//   * four 128-column partial buffers instead of two 256-column ones, with only 32 columns per promotion warp:
//     a warp pulls its whole share with ONE tensor-memory load, hands the buffer back at once, and does the fp32
//     arithmetic off the MMA's critical path while the next K block's load is already in flight.
// No multicast anywhere: every TMA load is unicast into the issuing CTA's shared memory (signalling the leader's
// barrier, which .cta_group::2 permits), and the MMA thread commits to each CTA's barrier with its own unicast
// tcgen05.commit.
#pragma once

#include "k_blockwise.cuh"
#include "k_smallm.cuh"  // cluster helpers

namespace gi8 {

constexpr int kPairBM = 256;  // rows of the pair's tile (128 per CTA)

#ifdef GI8_ENABLE_ABLATIONS
// Tuning builds: per-CTA cycle counters of the control threads' waits.
__device__ unsigned long long g_pair_dbg[148 * 8];
#define GI8_DBG_ADD(slot, v) atomicAdd(&g_pair_dbg[blockIdx.x * 8 + (slot)], (unsigned long long)(v))
#else
#define GI8_DBG_ADD(slot, v) ((void)0)
#endif

template <int STAGES, int PROMO>
__global__ void __launch_bounds__(kBlockwiseThreads, 1)
blockwise_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                      const BlockwiseParams p)
{
    constexpr int BN = 128;          // columns of the pair's tile; each CTA holds all 128 for its 128 rows
    constexpr int NBUF = 512 / BN;   // 4 partial buffers in each CTA's tensor memory
    constexpr int CW = BN / 4;       // 32 columns per promotion warp
    constexpr uint32_t kBytesA = kBM * kBK;          // this CTA's 128 rows of x
    constexpr uint32_t kBytesB = (BN / 2) * kBK;     // this CTA's 64 of the tile's 128 rows of y
    constexpr uint32_t kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdesc = make_idesc_i8(kPairBM, BN, false);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    __shared__ __align__(8) uint64_t bar_full[STAGES];        // used in the leader: both CTAs' loads land here
    __shared__ __align__(8) uint64_t bar_empty[STAGES];       // per CTA: its stage may be overwritten
    __shared__ __align__(8) uint64_t bar_part_full[NBUF];     // per CTA: its partial buffer is complete
    __shared__ __align__(8) uint64_t bar_part_empty[NBUF];    // used in the leader: 32 promotion warps arrive
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();  // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_tiles = p.tiles_m * p.tiles_n;  // tiles_m counts 256-row tiles here
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(&bar_part_full[b], 1);
            mbar_init(&bar_part_empty[b], 2 * kPromoWarps);
        }
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_y);
    }
    if (warp == 2) {
        tmem_alloc_pair(&tmem_base_slot, kTmemCols);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anything signals them remotely
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp < 4) {
        setmaxnreg_dec<kControlRegs>();
        if (warp == 0) {
            // -------------------------------------------------------------- TMA producer (one per CTA)
            if (lane == 0) {
                uint32_t it = 0;
                bool ok = true;
                for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                    int mb, nb;
                    tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        const long long tw0 = clock64();
                        if (!wait_or_abort(&bar_empty[s], ph ^ 1, &abort_flag)) {
                            raise_error(p.status, &abort_flag, ERR_TIMEOUT_PRODUCER);
                            ok = false;
                            break;
                        }
                        GI8_DBG_ADD(0, clock64() - tw0);
                        uint8_t* sa_tile = smem + s * kStageBytes;
                        const uint32_t leader_full = map_to_cta(smem_u32(&bar_full[s]), 0);
                        // The leader arms its barrier for the bytes of BOTH CTAs; the peer only sends bytes.
                        if (rank == 0) mbar_arrive_expect_tx(&bar_full[s], 2 * kStageBytes);
                        tma_load_2d_pair(sa_tile, &map_x, leader_full, kb * kBK, mb * kPairBM + static_cast<int>(rank) * kBM);
                        tma_load_2d_pair(sa_tile + kBytesA, &map_y, leader_full, kb * kBK,
                                         nb * BN + static_cast<int>(rank) * (BN / 2));
                    }
                }
                // Drain: the leader's barrier completes only when both CTAs' bytes have landed.
                if (rank == 0) {
                    const uint32_t armed = it < STAGES ? it : STAGES;
                    for (uint32_t j = 0; j < armed; ++j) {
                        const uint32_t i2 = it - 1 - j;
                        if (!mbar_wait(&bar_full[i2 % STAGES], (i2 / STAGES) & 1)) {
                            raise_error(p.status, &abort_flag, ERR_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        } else if (warp == 1) {
            // -------------------------------------------------------------- MMA issuer (leader CTA only)
            if (lane == 0 && rank == 0) {
                uint32_t it = 0;
                bool ok = true;
                for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        const uint32_t buf = it % NBUF;
                        const uint32_t bph = (it / NBUF) & 1;
                        const long long tm0 = clock64();
                        const bool w1 = wait_or_abort(&bar_part_empty[buf], bph ^ 1, &abort_flag);
                        const long long tm1 = clock64();
                        if (!w1 || !wait_or_abort(&bar_full[s], ph, &abort_flag)) {
                            raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                            ok = false;
                            break;
                        }
                        const long long tm2 = clock64();
                        GI8_DBG_ADD(1, tm1 - tm0);
                        GI8_DBG_ADD(2, tm2 - tm1);
                        tcgen05_fence_after_sync();
                        const uint32_t tmem_d = tmem_base + buf * BN;
                        const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                        const uint64_t da = make_smem_desc_k128(a_addr);
                        const uint64_t db = make_smem_desc_k128(a_addr + kBytesA);
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k)
                            umma_i8_pair(tmem_d, da + 2 * k, db + 2 * k, kIdesc, k != 0 ? 1u : 0u);
                        const uint32_t e = smem_u32(&bar_empty[s]);
                        const uint32_t f = smem_u32(&bar_part_full[buf]);
                        const long long tm3 = clock64();
                        GI8_DBG_ADD(5, tm3 - tm2);
                        umma_commit_pair(map_to_cta(e, 0));
                        GI8_DBG_ADD(6, clock64() - tm3);
                        umma_commit_pair(map_to_cta(e, 1));
                        umma_commit_pair(map_to_cta(f, 0));
                        umma_commit_pair(map_to_cta(f, 1));
                        GI8_DBG_ADD(3, clock64() - tm2);
                        GI8_DBG_ADD(4, 1);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue warps
        setmaxnreg_inc<kPromoRegs>();
        const int quarter = warp & 3;
        const int cg = (warp - 4) >> 2;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        uint32_t va[CW], vb[CW];

        // Loads this warp's 32 columns of K block `i` and hands the buffer back to the leader's MMA thread.
        auto fetch = [&](uint32_t i, uint32_t (&v)[CW]) {
            const uint32_t buf = i % NBUF;
            if (!wait_or_abort(&bar_part_full[buf], (i / NBUF) & 1, &abort_flag)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            tcgen05_fence_after_sync();
            tmem_ld_32x32b_x32(tmem_base + lane_base + buf * BN + cg * CW, v);
        };
        auto release = [&](uint32_t i) {
            tmem_ld_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_part_empty[i % NBUF]), 0));
        };

        const bool any_tile = pair < num_tiles;
        if (any_tile) {
            fetch(0, va);
            if (ok) release(0);
        }

        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
            const int row = mb * kPairBM + static_cast<int>(rank) * kBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const int col_base = nb * BN + cg * CW;
            const bool cols_ok = col_base < p.N;
            const float* sa_row = p.sa + static_cast<int64_t>(row_ok ? row : 0) * p.ld_sa;
            const float* sw_row = p.sw + static_cast<int64_t>(cols_ok ? col_base / 128 : 0) * p.ld_sw;
            const bool last_tile = tile + num_pairs >= num_tiles;

            float acc[CW];
#pragma unroll
            for (int j = 0; j < CW; ++j) acc[j] = 0.0f;

            auto consume = [&](const uint32_t (&v)[CW], float t) {
#pragma unroll
                for (int j = 0; j < CW; ++j) {
                    if constexpr (PROMO == PROMO_I2F) {
                        acc[j] = fmaf(__int2float_rn(static_cast<int32_t>(v[j])), t, acc[j]);
                    } else {
                        acc[j] = fmaf(__uint_as_float(v[j] + kMagicBits) - kMagicF32, t, acc[j]);
                    }
                }
            };

            float sa_next = __ldg(sa_row);
            float sw_next = __ldg(sw_row);
            // Two K blocks per trip so that the two register sets alternate statically.
            for (int kb = 0; kb < num_kb && ok; kb += 2) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (kb + h >= num_kb) break;
                    const float t = sa_next * sw_next;  // fp32, round to nearest: the scale of this K block
                    if (kb + h + 1 < num_kb) {
                        sa_next = __ldg(sa_row + kb + h + 1);
                        sw_next = __ldg(sw_row + kb + h + 1);
                    }
                    const bool have_next = (kb + h + 1 < num_kb) || !last_tile;
                    // The current block is in va (h == 0) or vb (h == 1); start the next block's load first.
                    if (have_next) {
                        if (h == 0) fetch(it + 1, vb);
                        else fetch(it + 1, va);
                    }
                    if (h == 0) consume(va, t);
                    else consume(vb, t);
                    if (have_next && ok) release(it + 1);
                    ++it;
                    if (!ok) break;
                }
                if ((num_kb & 1) && kb + 2 > num_kb && ok) {
                    // Odd number of K blocks: the next tile's first block was loaded into vb; move it to va.
#pragma unroll
                    for (int j = 0; j < CW; ++j) va[j] = vb[j];
                }
            }
            if (!ok) break;

            if (row_ok && cols_ok) {
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
    }

    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves while the other may still read its shared memory or signal it
    if (warp == 2) {
        __syncwarp();
        tcgen05_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

}  // namespace gi8
