// Small-M (decode) W8A8 GEMM for sm_100a: a split-K weight-streaming kernel bounded by HBM bandwidth.
//   out[m,n] = bf16( fp32(acc[m,n]) * (sx[m] * sw[n]) ),  acc = sum_k X[m,k] * W[n,k]  (exact int32)
// The reference has no small-M path: M <= 64 falls into its 256 x 128 default tile (csrc/kernels/gemm.cu:156-161),
// where at least three quarters of every tile is padding.
//
// Operands are swapped relative to the dense kernel: the 128 rows of a WEIGHT tile fill the M = 128 side of
// tcgen05.mma, the (few) tokens are the N side (MT = 16..128 columns of tensor memory), so no tensor-core
// work is spent on padding and the CTA's shared memory is almost entirely weight bytes in flight.
// grid = (N / 128 weight tiles) x (SPLITS slices of K).  Each CTA streams its [128 x K/SPLITS] weight slab
// through a TMA ring, accumulates in TMEM, and
//   SPLITS == 1: scales and stores its tile directly;
//   SPLITS  > 1: adds its int32 partial into a zero-initialised scratch tile with integer reductions (integer
//                addition is associative, so the sum is exact and independent of arrival order), then bumps the
//                tile's arrival counter; the CTA that arrives last reads the total, applies the scales, stores
//                bf16 and writes the zeros back, leaving the scratch ready for the next call.
// No CTA ever waits for another CTA, so the grid cannot deadlock whatever the residency.
#pragma once

#include "k_dense.cuh"

namespace gi8 {

constexpr int kSmallMThreads = 192;
constexpr int kSmallMTileN = 128;  // weight rows per CTA = UMMA M

struct SmallMParams {
    void* out;          // bf16 [M,N], leading dimension ldo
    const float* sx;    // [M]
    const float* sw;    // [N]
    int32_t* scratch;   // [tiles_n][MT][128] int32 partial sums, zero on entry and on exit (SPLITS > 1)
    uint32_t* counters; // [tiles_n] arrival counters, zero on entry and on exit (SPLITS > 1)
    uint32_t* status;
    int64_t ldo;
    int M, N, K;
    int kb_per_split;   // K blocks (of 128) per split
    int splits;
    int static_w;       // weights are not written by the preceding kernel: their first tiles may be fetched before it ends
};

template <int MT, int STAGES>
__global__ void __launch_bounds__(kSmallMThreads)
smallm_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const SmallMParams p)
{
    static_assert(MT == 16 || MT == 32 || MT == 64 || MT == 128, "token tile must be 16, 32, 64 or 128");
    constexpr uint32_t kBytesW = kSmallMTileN * kBK;                      // 16 KiB
    constexpr uint32_t kBytesX = MT * kBK;                                // token tile
    constexpr uint32_t kBytesXPad = (kBytesX + 1023u) & ~1023u;          // keep every tile 1024-byte aligned
    constexpr uint32_t kStageBytes = kBytesW + kBytesXPad;
    constexpr uint32_t kTmemCols = MT < 32 ? 32 : MT;
    constexpr uint32_t kIdesc = make_idesc_i8(kSmallMTileN, MT, false);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t is_last_slot;
    __shared__ volatile uint32_t abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x;
    const int split = blockIdx.y;
    const int kb_total = (p.K + kBK - 1) / kBK;
    // K blocks are dealt round-robin to the splits (split s takes blocks s, s + splits, ...): at any moment the
    // CTAs that share a weight tile stream ADJACENT 128-byte pieces of every weight row, so the DRAM requests in
    // flight form runs of splits x STAGES x 128 contiguous bytes per row instead of isolated 128-byte pieces.
    const int kb_begin = split;
    const int kb_step = p.splits;
    const int num_kb = split < kb_total ? (kb_total - split + p.splits - 1) / p.splits : 0;

    if (warp == 0 && lane == 0) {
        // The producer thread initialises the barriers itself and starts the first loads before the rest of
        // the CTA has finished its set-up: the weight stream is the critical path.
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(&bar_acc_full, 1);
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_x);
        const uint64_t pol_w = l2_policy_evict_first();
        const uint64_t pol_x = l2_policy_evict_last();
        const int first = min(num_kb, STAGES);
        for (int i = 0; i < first; ++i) {
            uint8_t* sw_tile = smem + i * kStageBytes;
            mbar_arrive_expect_tx(&bar_full[i], kBytesW + kBytesX);
            tma_load_2d_hint(sw_tile, &map_w, &bar_full[i], (kb_begin + i * kb_step) * kBK, tile_n * kSmallMTileN, pol_w);
            tma_load_2d_hint(sw_tile + kBytesW, &map_x, &bar_full[i], (kb_begin + i * kb_step) * kBK, 0, pol_x);
        }
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
        // ------------------------------------------------------------------ TMA producer (remaining stages)
        if (lane == 0) {
            const uint64_t pol_w = l2_policy_evict_first();
            const uint64_t pol_x = l2_policy_evict_last();
            int issued = min(num_kb, STAGES);
            for (int i = STAGES; i < num_kb; ++i) {
                const uint32_t s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!wait_or_abort(&bar_empty[s], ph ^ 1, &abort_flag)) {
                    raise_error(p.status, &abort_flag, ERR_TIMEOUT_PRODUCER);
                    break;
                }
                uint8_t* sw_tile = smem + s * kStageBytes;
                mbar_arrive_expect_tx(&bar_full[s], kBytesW + kBytesX);
                tma_load_2d_hint(sw_tile, &map_w, &bar_full[s], (kb_begin + i * kb_step) * kBK, tile_n * kSmallMTileN, pol_w);
                tma_load_2d_hint(sw_tile + kBytesW, &map_x, &bar_full[s], (kb_begin + i * kb_step) * kBK, 0, pol_x);
                issued = i + 1;
            }
            const int armed = issued < STAGES ? issued : STAGES;
            for (int j = 0; j < armed; ++j) {
                const int i2 = issued - 1 - j;
                if (!mbar_wait(&bar_full[i2 % STAGES], (i2 / STAGES) & 1)) {
                    raise_error(p.status, &abort_flag, ERR_TIMEOUT_DRAIN);
                    break;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && num_kb > 0) {
            bool ok = true;
            for (int i = 0; i < num_kb; ++i) {
                const uint32_t s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!wait_or_abort(&bar_full[s], ph, &abort_flag)) {
                    raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                tcgen05_fence_after_sync();
                const uint32_t w_addr = smem_u32(smem + s * kStageBytes);
                const uint64_t dw = make_smem_desc_k128(w_addr);
                const uint64_t dx = make_smem_desc_k128(w_addr + kBytesW);
#pragma unroll
                for (int k = 0; k < kBK / kUmmaK; ++k) umma_i8(tmem_base, dw + 2 * k, dx + 2 * k, kIdesc, (i | k) != 0);
                umma_commit(&bar_empty[s]);
            }
            if (ok) umma_commit(&bar_acc_full);
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps (128 threads)
        const int quarter = warp & 3;
        const int n_local = quarter * 32 + lane;            // weight row inside the tile = TMEM lane
        const int n = tile_n * kSmallMTileN + n_local;
        const bool n_ok = n < p.N;
        const int et = threadIdx.x - 64;                    // 0..127 among the epilogue threads
        uint32_t v[MT];
        bool ok = true;
        if (num_kb > 0) {
            if (!wait_or_abort(&bar_acc_full, 0, &abort_flag)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                ok = false;
            }
            tcgen05_fence_after_sync();
            __syncwarp();
            if (ok) {
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
                for (int c = 0; c < MT; c += 16) {
                    uint32_t t16[16];
                    tmem_ld_32x32b_x16(taddr + c, t16);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[c + j] = t16[j];
                }
                tmem_ld_wait();
            }
        } else {
#pragma unroll
            for (int j = 0; j < MT; ++j) v[j] = 0;
        }

        uint16_t* out = static_cast<uint16_t*>(p.out);
        const float col_scale = n_ok ? __ldg(p.sw + n) : 0.0f;
        if (p.splits == 1) {
            if (ok && n_ok) {
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < p.M) {
                        const float t = __ldg(p.sx + m) * col_scale;
                        out[static_cast<int64_t>(m) * p.ldo + n] =
                            to_bf16_bits(__int2float_rn(static_cast<int32_t>(v[m])) * t);
                    }
            }
        } else {
            // Every epilogue thread executes both named barriers below whatever happened before, so a
            // failed wait in one warp can never strand the others.
            int32_t* tile_scratch = p.scratch + static_cast<int64_t>(tile_n) * MT * kSmallMTileN;
            if (ok && num_kb > 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < p.M) atomicAdd(tile_scratch + m * kSmallMTileN + n_local, static_cast<int32_t>(v[m]));
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (et == 0) {
                const uint32_t prev = atomicAdd(p.counters + tile_n, 1u);
                is_last_slot = (prev == static_cast<uint32_t>(p.splits - 1)) ? 1u : 0u;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (is_last_slot) {
                __threadfence();
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < p.M) {
                        int32_t* src = tile_scratch + m * kSmallMTileN + n_local;
                        const int32_t total = __ldcg(src);
                        __stcg(src, 0);
                        if (n_ok) {
                            const float t = __ldg(p.sx + m) * col_scale;
                            out[static_cast<int64_t>(m) * p.ldo + n] = to_bf16_bits(__int2float_rn(total) * t);
                        }
                    }
                if (et == 0) p.counters[tile_n] = 0;
            }
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

// ---------------------------------------------------------------------------------------------------
// Cluster variant: the SPLITS CTAs that share one weight tile form a thread-block cluster (1 x SPLITS x 1,
// SPLITS <= 8).  Token row m belongs to CTA m % SPLITS: every CTA sends its int32 partials of that row straight
// from registers into the owner's receive area (remote shared-memory stores, which do not stall the sender);
// after ONE cluster barrier each owner sums what it received from its own shared memory, applies the scales and
// stores bf16.  After that barrier nobody touches a peer's memory, so CTAs leave independently.  The receive
// area lies behind the pipeline buffers (a fast peer may send while the owner is still streaming weights).
// No global scratch, no atomics, and the sum is exact whatever the order.  The cluster barrier is a hardware
// barrier that every thread of every CTA reaches unconditionally.
// ---------------------------------------------------------------------------------------------------
template <int MT, int STAGES>
__global__ void __launch_bounds__(kSmallMThreads)
smallm_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const SmallMParams p)
{
    static_assert(MT == 16 || MT == 32 || MT == 64 || MT == 128, "token tile must be 16, 32, 64 or 128");
    constexpr uint32_t kBytesW = kSmallMTileN * kBK;
    constexpr uint32_t kBytesX = MT * kBK;
    constexpr uint32_t kBytesXPad = (kBytesX + 1023u) & ~1023u;
    constexpr uint32_t kStageBytes = kBytesW + kBytesXPad;
    constexpr uint32_t kTmemCols = MT < 32 ? 32 : MT;
    constexpr uint32_t kIdesc = make_idesc_i8(kSmallMTileN, MT, false);

    extern __shared__ uint8_t smem_raw[];
    // The dynamic shared window starts at the same offset in every CTA of the cluster, so the aligned base
    // (and with it the partial tile's address) is identical across peers.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;
    __shared__ float sx_s[MT];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x;
    const int split = blockIdx.y;            // == rank inside the (1 x SPLITS x 1) cluster
    const int kb_total = (p.K + kBK - 1) / kBK;
    // K blocks are dealt round-robin to the splits (split s takes blocks s, s + splits, ...): at any moment the
    // CTAs that share a weight tile stream ADJACENT 128-byte pieces of every weight row, so the DRAM requests in
    // flight form runs of splits x STAGES x 128 contiguous bytes per row instead of isolated 128-byte pieces.
    const int kb_begin = split;
    const int kb_step = p.splits;
    const int num_kb = split < kb_total ? (kb_total - split + p.splits - 1) / p.splits : 0;

    if (warp == 0 && lane == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(&bar_acc_full, 1);
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_x);
        pdl_launch_dependents();  // the next kernel may be scheduled as soon as SMs free up
        const uint64_t pol_w = l2_policy_evict_first();
        const uint64_t pol_x = l2_policy_evict_last();
        const int first = min(num_kb, STAGES);
        // Everything above overlapped the previous kernel's tail.  Reads of what that kernel may have written start
        // after the dependency wait; the weights, when the caller declared them static, are requested before it, so
        // that the first tiles are already on their way when the previous kernel ends.
        if (!p.static_w) pdl_wait();
        for (int i = 0; i < first; ++i) {
            uint8_t* sw_tile = smem + i * kStageBytes;
            mbar_arrive_expect_tx(&bar_full[i], kBytesW + kBytesX);
            tma_load_2d_hint(sw_tile, &map_w, &bar_full[i], (kb_begin + i * kb_step) * kBK, tile_n * kSmallMTileN, pol_w);
            if (!p.static_w)
                tma_load_2d_hint(sw_tile + kBytesW, &map_x, &bar_full[i], (kb_begin + i * kb_step) * kBK, 0, pol_x);
        }
        if (p.static_w) {
            pdl_wait();
            for (int i = 0; i < first; ++i)
                tma_load_2d_hint(smem + i * kStageBytes + kBytesW, &map_x, &bar_full[i], (kb_begin + i * kb_step) * kBK, 0, pol_x);
        }
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, kTmemCols);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    pdl_wait();  // every thread: scales are read and the output is written only after the previous kernel is done
    const uint32_t tmem_base = tmem_base_slot;
    // [sender][row of this owner][128] int32, behind the pipeline buffers
    int32_t* recv = reinterpret_cast<int32_t*>(smem + STAGES * kStageBytes);
    const uint32_t nranks = static_cast<uint32_t>(p.splits);
    const uint32_t my_rank = p.splits > 1 ? cluster_cta_rank() : 0u;
    const uint32_t rows_per_owner = (static_cast<uint32_t>(p.M) + nranks - 1) / nranks;
    float col_scale = 0.0f;  // of this thread's output column (epilogue warps)

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol_w = l2_policy_evict_first();
            const uint64_t pol_x = l2_policy_evict_last();
            int issued = min(num_kb, STAGES);
            for (int i = STAGES; i < num_kb; ++i) {
                const uint32_t s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!wait_or_abort(&bar_empty[s], ph ^ 1, &abort_flag)) {
                    raise_error(p.status, &abort_flag, ERR_TIMEOUT_PRODUCER);
                    break;
                }
                uint8_t* sw_tile = smem + s * kStageBytes;
                mbar_arrive_expect_tx(&bar_full[s], kBytesW + kBytesX);
                tma_load_2d_hint(sw_tile, &map_w, &bar_full[s], (kb_begin + i * kb_step) * kBK, tile_n * kSmallMTileN, pol_w);
                tma_load_2d_hint(sw_tile + kBytesW, &map_x, &bar_full[s], (kb_begin + i * kb_step) * kBK, 0, pol_x);
                issued = i + 1;
            }
            const int armed = issued < STAGES ? issued : STAGES;
            for (int j = 0; j < armed; ++j) {
                const int i2 = issued - 1 - j;
                if (!mbar_wait(&bar_full[i2 % STAGES], (i2 / STAGES) & 1)) {
                    raise_error(p.status, &abort_flag, ERR_TIMEOUT_DRAIN);
                    break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && num_kb > 0) {
            bool ok = true;
            for (int i = 0; i < num_kb; ++i) {
                const uint32_t s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!wait_or_abort(&bar_full[s], ph, &abort_flag)) {
                    raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                tcgen05_fence_after_sync();
                const uint32_t w_addr = smem_u32(smem + s * kStageBytes);
                const uint64_t dw = make_smem_desc_k128(w_addr);
                const uint64_t dx = make_smem_desc_k128(w_addr + kBytesW);
#pragma unroll
                for (int k = 0; k < kBK / kUmmaK; ++k) umma_i8(tmem_base, dw + 2 * k, dx + 2 * k, kIdesc, (i | k) != 0);
                umma_commit(&bar_empty[s]);
            }
            if (ok) umma_commit(&bar_acc_full);
        }
    } else {
        // epilogue warps: tensor memory -> global (one split) or -> the row owners' receive areas
        const int quarter = warp & 3;
        const int n_local = quarter * 32 + lane;
        const int n = tile_n * kSmallMTileN + n_local;
        // The scales are fetched while the weights stream, not between the last MMA and the stores.
        col_scale = n < p.N ? __ldg(p.sw + n) : 0.0f;
        {
            const int t = static_cast<int>(threadIdx.x) - 64;
            if (t < MT) sx_s[t] = t < p.M ? __ldg(p.sx + t) : 0.0f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        bool ok = true;
        if (num_kb > 0) {
            if (!wait_or_abort(&bar_acc_full, 0, &abort_flag)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below are warp-collective
            tcgen05_fence_after_sync();
        }
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t recv_mine = smem_u32(recv) + (my_rank * rows_per_owner * kSmallMTileN + n_local) * 4u;
        uint32_t owner = 0, row_local = 0;  // of token row c + j, kept incrementally
#pragma unroll
        for (int c = 0; c < MT; c += 16) {
            uint32_t t16[16];
            if (ok && num_kb > 0) {
                tmem_ld_32x32b_x16(taddr + c, t16);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) t16[j] = 0;
            }
            if (p.splits == 1) {
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c + j < p.M)
                            static_cast<uint16_t*>(p.out)[static_cast<int64_t>(c + j) * p.ldo + n] =
                                to_bf16_bits(__int2float_rn(static_cast<int32_t>(t16[j])) * (sx_s[c + j] * col_scale));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (c + j < p.M)
                        st_dsmem_u32(map_to_cta(recv_mine + row_local * (kSmallMTileN * 4u), owner), t16[j]);
                    if (++owner == nranks) owner = 0, ++row_local;
                }
            }
        }
    }

    tcgen05_fence_before_sync();
    if (p.splits > 1) {
        cluster_sync_all();  // every partial has landed in its owner's receive area
        if (warp >= 2) {
            const int n_local = (warp & 3) * 32 + lane;
            const int n = tile_n * kSmallMTileN + n_local;
            uint32_t row_local = 0;
            for (int m = static_cast<int>(my_rank); m < p.M; m += static_cast<int>(nranks), ++row_local) {
                int32_t total = 0;
                for (uint32_t r = 0; r < nranks; ++r)
                    total += recv[(r * rows_per_owner + row_local) * kSmallMTileN + n_local];
                if (n < p.N)
                    static_cast<uint16_t*>(p.out)[static_cast<int64_t>(m) * p.ldo + n] =
                        to_bf16_bits(__int2float_rn(total) * (sx_s[m] * col_scale));
            }
        }
    } else {
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace gi8
