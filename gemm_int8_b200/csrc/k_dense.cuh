// Dense INT8 GEMM for sm_100a:  D[M,N] = epilogue( sum_k X[m,k] * Y[n,k] ),  X [M,K], Y [N,K] int8.
//
// Replaces the reference's CUTLASS Sm80 mma.sync instantiation (csrc/kernels/gemm.cu:46-65) and its
// LinearCombination epilogue (csrc/kernels/gemm.cu:59-63, 96).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: K-major 128-byte-wide tiles of X and Y into 128B-swizzled shared memory,
//               STAGES-deep ring guarded by full/empty mbarriers.
//   warp 1      MMA issuer: one thread issues tcgen05.mma kind::i8 (128 x BN x 32 per instruction),
//               int32 accumulators live in tensor memory; two accumulator buffers so the epilogue of
//               tile i overlaps the main loop of tile i+1.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp owns the 32-lane quarter warp_id % 4),
//               apply the epilogue in registers, store to global.
// Every mbarrier wait is bounded; on expiry the CTA records an error code and drains.
#pragma once

#include "ptx.cuh"

namespace gi8 {

constexpr int kBM = 128;       // rows of X per tile = UMMA M
constexpr int kBK = 128;       // int8 elements (= bytes) of K per pipeline stage = one swizzle row
constexpr int kUmmaK = 32;     // K per tcgen05.mma kind::i8
constexpr int kDenseThreads = 192;

enum Epilogue : int {
    EPI_ALPHA_BF16 = 0,   // bf16( fp32(acc) * alpha )                       reference semantics
    EPI_RAW_I32 = 1,      // int32 accumulators, for bit-exact checks
    EPI_ROWCOL_BF16 = 2,  // bf16( fp32(acc) * (sx[m] * sw[n]) )             per-token x per-channel
};

enum KernelError : uint32_t {
    ERR_NONE = 0,
    ERR_TIMEOUT_PRODUCER = 1,
    ERR_TIMEOUT_MMA = 2,
    ERR_TIMEOUT_EPILOGUE = 3,
    ERR_TIMEOUT_DRAIN = 4,
    ERR_TIMEOUT_REDUCE = 5,
};

struct DenseParams {
    void* out;            // bf16 [M,N] or int32 [M,N], row-major, leading dimension ldo (elements)
    const float* sx;      // [M]  (EPI_ROWCOL_BF16)
    const float* sw;      // [N]  (EPI_ROWCOL_BF16)
    uint32_t* status;     // device word, receives a KernelError on failure
    int64_t ldo;
    int M, N, K;
    int tiles_m, tiles_n;
    int vec_ok;           // out is 16-byte aligned and ldo keeps every row 16-byte aligned
    int group_m;          // row-blocks per rasterisation band
    int tma_store;        // bf16 epilogues: stage 32 x 32 blocks in shared memory and write them with TMA stores
    int tile_end;         // > 0: only tiles [0, tile_end) of the grid are computed here (the rest by the split-K launch)
    int pdl_role;         // 1: an independent launch over other output tiles follows: let it start as SMs free up
    float alpha;
};

// Records the first error of the grid and raises the CTA-wide abort flag.
GI8_DEVICE void raise_error(uint32_t* status, volatile uint32_t* abort_flag, uint32_t code)
{
    *abort_flag = 1;
    atomicCAS(status, 0u, code | (blockIdx.x << 8));
}

// Bounded wait that also gives up when another role of this CTA has aborted.
GI8_DEVICE bool wait_or_abort_addr(uint32_t bar_addr, uint32_t parity, volatile uint32_t* abort_flag,
                                   uint64_t limit_ns = GI8_WAIT_LIMIT_NS)
{
    if (mbar_try_wait_addr(bar_addr, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait_addr(bar_addr, parity)) return true;
        if ((++spins & 0x3f) == 0) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns) return false;
        }
    }
}

GI8_DEVICE bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                              uint64_t limit_ns = GI8_WAIT_LIMIT_NS)
{
    return wait_or_abort_addr(smem_u32(bar), parity, abort_flag, limit_ns);
}

// Maps a linear tile index to (m block, n block).  Tiles are walked in bands of kGroupM row-blocks so
// that the tiles resident at one time share X rows and Y rows in L2.
GI8_DEVICE void tile_coords(int tile, int tiles_m, int tiles_n, int& mb, int& nb, int kGroupM = 8)
{
    const int per_group = kGroupM * tiles_n;
    const int g = tile / per_group;
    const int first_m = g * kGroupM;
    const int rows = min(kGroupM, tiles_m - first_m);
    const int r = tile - g * per_group;
    mb = first_m + r % rows;
    nb = r / rows;
}

// PAIR: two CTAs on neighbouring SMs (a 2 x 1 x 1 cluster) share one 256 x BN tile.  The leader's MMA thread issues
// tcgen05.mma.cta_group::2 (M = 256), which reads each CTA's own 128 rows of x and each CTA's half of the BN rows
// of y from that CTA's shared memory, so a CTA loads (128 + BN/2) x 128 bytes per K block instead of (128 + BN) x 128
// -- a third less L2 traffic per MAC at BN = 256 -- and each CTA keeps the accumulators of its 128 rows in its own
// tensor memory.  Every TMA load is unicast into the issuing CTA's shared memory and signals the leader's barrier;
// the MMA thread commits to each CTA's barrier with its own unicast tcgen05.commit (no multicast anywhere).
template <int BN, int STAGES, int EPI, bool PAIR = false>
__global__ void __launch_bounds__(kDenseThreads, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                  const __grid_constant__ CUtensorMap map_out, const DenseParams p)
{
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN must be a multiple of 32 up to 256");
    constexpr uint32_t kBytesA = kBM * kBK;
    constexpr int kTileM = PAIR ? 2 * kBM : kBM;       // rows of the (pair's) tile
    constexpr int kRowsB = PAIR ? BN / 2 : BN;         // rows of y this CTA loads
    constexpr uint32_t kBytesB = kRowsB * kBK;
    constexpr uint32_t kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                 : (2 * BN <= 256) ? 256 : 512;
    constexpr uint32_t kIdesc = make_idesc_i8(kTileM, BN, false);

    extern __shared__ uint8_t smem_raw[];
    // 128B-swizzled tiles need 1024-byte alignment.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // Behind the pipeline stages: per epilogue warp two 32-row x 64-byte staging blocks for TMA stores.
    uint8_t* store_stage = smem + STAGES * kStageBytes;

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = p.tile_end > 0 ? p.tile_end : p.tiles_m * p.tiles_n;   // tiles_m counts kTileM-row tiles
    const int num_kb = (p.K + kBK - 1) / kBK;
    // PAIR: rank 0 is the leader (its bar_full and bar_acc_empty serve both CTAs); the pair is the scheduling unit.
    const uint32_t rank = PAIR ? cluster_cta_rank() : 0u;
    const int first_tile = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        if (p.pdl_role == 1) pdl_launch_dependents();
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_acc_full[b], 1);
            mbar_init(&bar_acc_empty[b], PAIR ? 8 : 4);
        }
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_y);
        if (p.tma_store) prefetch_tensormap(&map_out);
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            tmem_alloc_pair(&tmem_base_slot, kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(&tmem_base_slot, kTmemCols);
            tmem_relinquish_alloc_permit();
        }
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // both CTAs' barriers exist before anything signals them remotely
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    // The producer and the MMA issuer run their loops with the WHOLE warp (uniform control flow) and elect one lane
    // only around the TMA / MMA / commit instructions.  Inside an `if (lane == 0)` region the compiler treats
    // addresses and descriptors as per-thread values and moves them into uniform registers one by one for every
    // tcgen05.mma: four MMAs plus a commit then cost about 440 cycles to issue on an idle SM against about 200 in
    // this form, with 512 cycles of tensor-core work per K block.
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        uint32_t s = 0, ph = 0;  // stage and phase parity of the running K-block counter
        uint32_t armed = 0;
        bool ok = true;
        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!wait_or_abort(&bar_empty[s], ph ^ 1, &abort_flag)) {
                    if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_PRODUCER);
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    uint8_t* sa = smem + s * kStageBytes;
                    uint8_t* sb = sa + kBytesA;
                    if constexpr (PAIR) {
                        // The leader arms its barrier for the bytes of BOTH CTAs; the peer only sends bytes.
                        const uint32_t leader_full = map_to_cta(smem_u32(&bar_full[s]), 0);
                        if (rank == 0) mbar_arrive_expect_tx(&bar_full[s], 2 * kStageBytes);
                        tma_load_2d_pair(sa, &map_x, leader_full, kb * kBK, mb * kTileM + static_cast<int>(rank) * kBM);
                        tma_load_2d_pair(sb, &map_y, leader_full, kb * kBK, nb * BN + static_cast<int>(rank) * kRowsB);
                    } else {
                        mbar_arrive_expect_tx(&bar_full[s], kStageBytes);
                        tma_load_2d(sa, &map_x, &bar_full[s], kb * kBK, mb * kBM);
                        tma_load_2d(sb, &map_y, &bar_full[s], kb * kBK, nb * BN);
                    }
                }
                __syncwarp();
                if (armed < STAGES) ++armed;
                if (++s == STAGES) s = 0, ph ^= 1;
            }
        }
        // Drain: every armed stage must have landed before the CTA may exit (PAIR: the leader's barriers complete
        // only when both CTAs' bytes have landed; the peer leaves through the final cluster barrier).  (s, ph) is the
        // slot after the last armed one; walk backwards.
        if (PAIR && rank != 0) armed = 0;
        for (uint32_t j = 0; j < armed; ++j) {
            if (s == 0) s = STAGES, ph ^= 1;
            --s;
            if (!mbar_wait(&bar_full[s], ph)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_DRAIN);
                break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (rank == 0) {
            uint32_t s = 0, ph = 0;
            uint32_t local_tile = 0;
            bool ok = true;
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
                const uint32_t buf = local_tile & 1;
                const uint32_t acc_ph = (local_tile >> 1) & 1;
                if (!wait_or_abort(&bar_acc_empty[buf], acc_ph ^ 1, &abort_flag)) {
                    if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                    break;
                }
                tcgen05_fence_after_sync();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!wait_or_abort(&bar_full[s], ph, &abort_flag)) {
                        if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                    const uint64_t da = make_smem_desc_k128(a_addr);
                    const uint64_t db = make_smem_desc_k128(a_addr + kBytesA);
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k) {
                            // +2 in the start-address field = +32 bytes = one UMMA K step inside the swizzled row
                            if constexpr (PAIR) umma_i8_pair(tmem_d, da + 2 * k, db + 2 * k, kIdesc, (kb | k) != 0);
                            else umma_i8(tmem_d, da + 2 * k, db + 2 * k, kIdesc, (kb | k) != 0);
                        }
                        // frees the stage (in both CTAs) once these MMAs have read it
                        if constexpr (PAIR) {
                            umma_commit_pair(map_to_cta(smem_u32(&bar_empty[s]), 0));
                            umma_commit_pair(map_to_cta(smem_u32(&bar_empty[s]), 1));
                        } else {
                            umma_commit(&bar_empty[s]);
                        }
                    }
                    __syncwarp();
                    if (++s == STAGES) s = 0, ph ^= 1;
                }
                if (ok && elect_one()) {
                    if constexpr (PAIR) {
                        umma_commit_pair(map_to_cta(smem_u32(&bar_acc_full[buf]), 0));
                        umma_commit_pair(map_to_cta(smem_u32(&bar_acc_full[buf]), 1));
                    } else {
                        umma_commit(&bar_acc_full[buf]);
                    }
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32)
        uint32_t local_tile = 0;
        bool ok = true;
        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
            const uint32_t buf = local_tile & 1;
            const uint32_t acc_ph = (local_tile >> 1) & 1;
            if (!wait_or_abort(&bar_acc_full[buf], acc_ph, &abort_flag)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                ok = false;
                break;
            }
            tcgen05_fence_after_sync();
            const int row = mb * kTileM + static_cast<int>(rank) * kBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            float row_scale = 1.0f;
            if constexpr (EPI == EPI_ROWCOL_BF16) row_scale = row_ok ? __ldg(p.sx + row) : 0.0f;

#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the predicated stores
                tmem_ld_32x32b_x32(taddr + c, v);
                tmem_ld_wait();
                const int col0 = nb * BN + c;
                if (col0 >= p.N) continue;  // warp-uniform
                if constexpr (EPI == EPI_RAW_I32) {
                    if (!row_ok) continue;
                    int32_t* dst = static_cast<int32_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0;
                    if (col0 + 32 <= p.N && p.vec_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<uint4*>(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < p.N) dst[j] = static_cast<int32_t>(v[j]);
                    }
                } else {
                    float f[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float a = __int2float_rn(static_cast<int32_t>(v[j]));
                        if constexpr (EPI == EPI_ALPHA_BF16) {
                            f[j] = a * p.alpha;
                        } else {
                            const float cs = (col0 + j < p.N) ? __ldg(p.sw + col0 + j) : 0.0f;
                            f[j] = a * (row_scale * cs);
                        }
                    }
                    if (p.tma_store) {
                        // 32 rows x 32 bf16 of this warp go to shared memory in the 64-byte-swizzled layout the
                        // output tensor map expects (16-byte chunk index xor (row / 2) % 4: conflict-free), then one
                        // lane issues the TMA store; rows and columns beyond M and N are clipped by the hardware.
                        const int row0 = mb * kTileM + static_cast<int>(rank) * kBM + quarter * 32;
                        if (row0 < p.M) {
                            uint8_t* stg = store_stage + ((warp - 2) * 2 + ((c >> 5) & 1)) * 2048;
                            if (lane == 0) tma_store_wait_read<1>();  // the block staged two chunks ago has been read
                            __syncwarp();
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int cq = q ^ ((lane >> 1) & 3);
                                *reinterpret_cast<uint4*>(stg + lane * 64 + cq * 16) = make_uint4(
                                    pack_bf16x2(f[8 * q], f[8 * q + 1]), pack_bf16x2(f[8 * q + 2], f[8 * q + 3]),
                                    pack_bf16x2(f[8 * q + 4], f[8 * q + 5]), pack_bf16x2(f[8 * q + 6], f[8 * q + 7]));
                            }
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                tma_store_2d(&map_out, stg, col0, row0);
                                tma_store_commit();
                            }
                        }
                        continue;
                    }
                    if (!row_ok) continue;
                    uint16_t* dst = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0;
                    if (col0 + 32 <= p.N && p.vec_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8)
                            *reinterpret_cast<uint4*>(dst + j) =
                                make_uint4(pack_bf16x2(f[j], f[j + 1]), pack_bf16x2(f[j + 2], f[j + 3]),
                                           pack_bf16x2(f[j + 4], f[j + 5]), pack_bf16x2(f[j + 6], f[j + 7]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < p.N) dst[j] = to_bf16_bits(f[j]);
                    }
                }
            }
            // All of this warp's reads of the accumulator buffer are complete: hand it back.
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_acc_empty[buf]), 0));
                else mbar_arrive(&bar_acc_empty[buf]);
            }
        }
        // Outstanding TMA stores read this CTA's shared memory: they must have completed before it exits.
        if (lane == 0) tma_store_wait_all<0>();
    }

    tcgen05_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // neither CTA leaves while the other may still read or signal it
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after_sync();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
        else tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace gi8
