// Split-K form of the dense INT8 GEMM for sm_100a, for the tiles that would otherwise run as a thin last wave (or as
// a grid far smaller than the machine): the S CTAs of a thread-block cluster (S x 1 x 1, S in {2, 4, 8}) share one
// 128 x 256 output tile, each accumulating a contiguous range of K blocks in its own tensor memory.  The int32
// partials are exact, so the sum does not depend on the order and the result is bit-identical to the unsplit
// kernel's.  The reference has no split-K (csrc/kernels/gemm.cu:136-161 picks a tile shape only).
//
// Reduction (no global scratch, no atomics): tile row m belongs to CTA m / (128 / S).  Once every CTA of the cluster
// has finished its MMAs (first cluster barrier: all pipeline buffers are idle), each CTA sends the rows of its
// partial to their owners' pipeline buffers with remote shared-memory stores, straight from the registers the
// tensor-memory loads fill; after the second cluster barrier each owner adds the S partials of its rows from its
// own shared memory, applies the epilogue and stores bf16.  Nobody touches a peer's memory after that barrier, so
// CTAs leave independently.  Both cluster barriers are hardware barriers that every thread of every CTA reaches
// unconditionally; every mbarrier wait is bounded.
//
// Receive layout in the owner's shared memory, in 16-byte units (four int32 of one row):
//   unit((sender, c4, r)) = (sender * 64 + c4) * R + r,   c4 = column / 4, r = row inside the owner's R = 128 / S rows
// so that the 32 lanes of a sending warp (consecutive rows) and the threads of the adding loop (consecutive r) touch
// consecutive units: no bank conflicts on either side.
#pragma once

#include "k_dense.cuh"

namespace gi8 {

constexpr int kSplitKBN = 256;
constexpr int kSplitKStages = 4;

struct SplitKParams {
    int tile_begin;     // first tile (in the numbering of the main launch's tile grid) this launch covers
    int units;          // 128-row output tiles covered = cluster count
    int splits;         // S
    int kb_per_split;   // K blocks per split (the last may get fewer, or none)
    int pair_grid;      // the numbering is that of 256-row (two-CTA) tiles: unit u is half u % 2 of tile u / 2
    int after_main;     // launched (with programmatic dependent launch) behind the main launch of the same GEMM: it
                        // reads nothing that launch writes and starts as SMs free up, but ends only after it
};

GI8_DEVICE void st_dsmem_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(kDenseThreads, 1)
dense_splitk_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                    const DenseParams p, const SplitKParams q)
{
    static_assert(EPI == EPI_ALPHA_BF16 || EPI == EPI_ROWCOL_BF16, "bf16 epilogues only");
    constexpr int BN = kSplitKBN, STAGES = kSplitKStages;
    constexpr uint32_t kBytesA = kBM * kBK;
    constexpr uint32_t kBytesB = BN * kBK;
    constexpr uint32_t kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kTmemCols = 256;
    constexpr uint32_t kIdesc = make_idesc_i8(kBM, BN, false);
    static_assert(STAGES * kStageBytes >= kBM * BN * 4, "the partial tile must fit in the pipeline buffers");

    extern __shared__ uint8_t smem_raw[];
    // The dynamic shared window starts at the same offset in every CTA of the cluster, so the aligned base (and
    // with it the receive area's address) is identical across peers.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile uint32_t abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t S = static_cast<uint32_t>(q.splits);
    const uint32_t rank = cluster_cta_rank();          // == blockIdx.x % S
    const int unit = static_cast<int>(blockIdx.x / S);

    int mb, nb;
    {
        const int tile = q.tile_begin + (q.pair_grid ? unit >> 1 : unit);
        tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
        if (q.pair_grid) mb = 2 * mb + (unit & 1);
    }
    // The lower half of a 256-row tile can lie wholly below M: the whole cluster leaves (same decision in every CTA).
    if (mb * kBM >= p.M) {
        if (q.after_main && threadIdx.x == 0) pdl_wait();
        return;
    }

    const int num_kb_total = (p.K + kBK - 1) / kBK;
    const int kb_begin = static_cast<int>(rank) * q.kb_per_split;
    const int num_kb = max(0, min(num_kb_total - kb_begin, q.kb_per_split));

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(&bar_acc_full, 1);
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

    bool acc_ok = num_kb > 0;  // epilogue warps: the accumulator holds this CTA's partial
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        uint32_t s = 0, ph = 0;
        int issued = 0;
        for (int i = 0; i < num_kb; ++i) {
            if (!wait_or_abort(&bar_empty[s], ph ^ 1, &abort_flag)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_PRODUCER);
                break;
            }
            if (elect_one()) {
                uint8_t* sa = smem + s * kStageBytes;
                mbar_arrive_expect_tx(&bar_full[s], kStageBytes);
                tma_load_2d(sa, &map_x, &bar_full[s], (kb_begin + i) * kBK, mb * kBM);
                tma_load_2d(sa + kBytesA, &map_y, &bar_full[s], (kb_begin + i) * kBK, nb * BN);
            }
            __syncwarp();
            issued = i + 1;
            if (++s == STAGES) s = 0, ph ^= 1;
        }
        // Drain: every armed stage must have landed before the buffers are reused or the CTA exits.
        const int armed = issued < STAGES ? issued : STAGES;
        for (int j = 0; j < armed; ++j) {
            const int i2 = issued - 1 - j;
            if (!mbar_wait(&bar_full[i2 % STAGES], (i2 / STAGES) & 1)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_DRAIN);
                break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int i = 0; i < num_kb; ++i) {
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
                for (int k = 0; k < kBK / kUmmaK; ++k) umma_i8(tmem_base, da + 2 * k, db + 2 * k, kIdesc, (i | k) != 0);
                umma_commit(&bar_empty[s]);
            }
            __syncwarp();
            if (++s == STAGES) s = 0, ph ^= 1;
        }
        if (ok && num_kb > 0 && elect_one()) umma_commit(&bar_acc_full);
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue warps: wait for the partial
        if (num_kb > 0) {
            // bar_acc_full completes only after every MMA has finished reading the pipeline buffers.
            if (!wait_or_abort(&bar_acc_full, 0, &abort_flag)) {
                if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                acc_ok = false;
            }
            acc_ok = __all_sync(0xffffffffu, acc_ok);  // the tensor-memory loads below are warp-collective
            tcgen05_fence_after_sync();
        }
    }

    // Every CTA of the cluster is done with its pipeline buffers (or has given up: it then sends zeros).
    __syncthreads();
    cluster_sync_all();

    const uint32_t R = static_cast<uint32_t>(kBM) / S;  // rows per owner
    const uint32_t recv = smem_u32(smem);
    if (warp >= 2) {
        const int quarter = warp & 3;
        const uint32_t m = static_cast<uint32_t>(quarter * 32 + lane);  // tile row = tensor-memory lane
        const uint32_t owner = m / R, r = m % R;
        const uint32_t dst0 = map_to_cta(recv + ((rank * 64u) * R + r) * 16u, owner);
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
            uint32_t v[32];
            if (acc_ok) {
                tmem_ld_32x32b_x32(taddr + c, v);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                st_dsmem_v4(dst0 + static_cast<uint32_t>(c / 4 + j) * R * 16u, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // every partial has landed in its owner's receive area

    if (warp >= 2) {
        const uint32_t tid = threadIdx.x - 64;  // 0..127
        const uint32_t items = R * 64u;         // (r, c4) pairs of this owner, r fastest
        for (uint32_t i = tid; i < items; i += 128) {
            const uint32_t r = i % R, c4 = i / R;
            int32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
            for (uint32_t s = 0; s < S; ++s) {
                const int4 t = *reinterpret_cast<const int4*>(smem + (((s * 64u + c4) * R + r) << 4));
                a0 += t.x, a1 += t.y, a2 += t.z, a3 += t.w;
            }
            const int row = mb * kBM + static_cast<int>(rank * R + r);
            const int col = nb * BN + static_cast<int>(c4 * 4);
            if (row >= p.M || col >= p.N) continue;
            float f0, f1, f2, f3;
            if constexpr (EPI == EPI_ALPHA_BF16) {
                f0 = __int2float_rn(a0) * p.alpha, f1 = __int2float_rn(a1) * p.alpha;
                f2 = __int2float_rn(a2) * p.alpha, f3 = __int2float_rn(a3) * p.alpha;
            } else {
                const float rs = __ldg(p.sx + row);
                f0 = __int2float_rn(a0) * (rs * __ldg(p.sw + col));
                f1 = col + 1 < p.N ? __int2float_rn(a1) * (rs * __ldg(p.sw + col + 1)) : 0.0f;
                f2 = col + 2 < p.N ? __int2float_rn(a2) * (rs * __ldg(p.sw + col + 2)) : 0.0f;
                f3 = col + 3 < p.N ? __int2float_rn(a3) * (rs * __ldg(p.sw + col + 3)) : 0.0f;
            }
            uint16_t* dst = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col;
            if (col + 4 <= p.N && p.vec_ok) {
                *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(f0, f1), pack_bf16x2(f2, f3));
            } else {
                dst[0] = to_bf16_bits(f0);
                if (col + 1 < p.N) dst[1] = to_bf16_bits(f1);
                if (col + 2 < p.N) dst[2] = to_bf16_bits(f2);
                if (col + 3 < p.N) dst[3] = to_bf16_bits(f3);
            }
        }
    }
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (q.after_main && threadIdx.x == 0) pdl_wait();  // the pair of launches completes as one
}

}  // namespace gi8
