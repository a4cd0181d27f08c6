// Blockwise-dequantised W8A8 GEMM for sm_100a:
//   out[m,n] = bf16( sum_kb fp32(P[m,n,kb]) * (sa[m,kb] * sw[n/128,kb]) ),  kb ascending, one fused
//   multiply-add per K block (128 wide), P = exact int32 partial dot product of the block.
// There is no such path in the reference (its epilogue applies one scalar, csrc/kernels/gemm.cu:96); the
// semantics are those of the CPU oracle's blockwise restatement.
//
// Structure (one persistent CTA per SM, 384 threads = 3 warpgroups):
//   warpgroup 0 control (setmaxnreg.dec): warp 0 TMA producer (as in the dense kernel); warp 1 (and warp 3 when
//               NISS == 2, taking alternate K blocks) MMA issuer -- per K block four tcgen05.mma kind::i8 with N = BN
//               (or 2 x 4 with N = 128 when SPLIT == 2) that overwrite one of NBUF = 512 / BN tensor-memory partial
//               buffers, then ONE commit per column half that both frees the pipeline stage and publishes the
//               partial; warp 2 allocates tensor memory.
//   warps 4..11 promotion (setmaxnreg.inc): warp w owns TMEM lane quarter (w % 4) and column half ((w - 4) / 4) of
//               the tile, i.e. 32 rows x BN/2 columns, whose fp32 accumulators it keeps in registers (as f32x2
//               pairs).  Per K block: tcgen05.ld the int32 partial in 32-column chunks, hand the buffer back after
//               the last load, cvt.rn.f32.s32 + fma.rn.f32x2 with the block's scale.  A column half never
//               straddles a 128-wide weight-scale block.  At the end of the tile the same warps cast to bf16 and
//               store through swizzled shared memory and TMA.
//
// Why eight fat warps (measured on B200 with a stand-alone loop of the same instructions, cycles per 128 x 256
// K block, tensor core busy in the background): a tcgen05.ld costs about one cycle per 32-lane column whatever its
// width and does not overlap the arithmetic of the same scheduler, so deeper load pipelines buy nothing; what
// counts is instructions issued.  16 warps x 64 columns with 16-column loads and a biased accumulator written
// back with tcgen05.st: 860-920.  8 warps x 128 columns, 32-column loads: biased accumulator with write-back 665-685
// (the stores alone cost 140), cvt + fma.f32x2 without any write-back 545-580, against 512 for the MMAs.
//
// Barrier protocol (every wait is a parity wait, so it must hold that a barrier cannot complete a second phase
// before the waiter has consumed the first; the comment at each barrier says what gates its next phase):
//   bar_full[s]        completed by the TMA bytes of K block `it` (s = it % STAGES).  Waiter: the issuer of K block
//                      `it`.  Next phase needs the producer to refill stage s, which needs bar_done[.][s] of K block
//                      `it`, which needs this issuer's commit: gated by the waiter.
//   bar_done[h][s]     completed by the issuer's commit for column half h of K block `it`.  Waiters: the producer
//                      (before refilling s; the next completion needs its own refill: gated) and the promotion warps
//                      of half h (the next completion is K block it + STAGES, whose MMAs need partial buffer
//                      (it + STAGES) % NBUF handed back by every warp of the half for K block it + STAGES - NBUF >= it:
//                      gated).
//   bar_part_empty[h][b]  completed by the arrivals of the promotion warps of half h after their last load of a
//                      K block in buffer b.  Waiter: the issuer of the next K block that uses b; the completion
//                      after that needs this issuer's MMAs: gated.
//   With two issuers, issuer j takes K blocks it % 2 == j, hence stages s % 2 == j and buffers b % 2 == j
//   (STAGES and NBUF are even): every barrier still has exactly one issuing waiter, which sees all its phases.
#pragma once

#include "k_dense.cuh"

namespace gi8 {

constexpr int kBlockwiseThreads = 384;
constexpr int kPromoWarps = 8;
constexpr int kPromoRegs = 224;   // registers per promotion thread after setmaxnreg.inc
constexpr int kControlRegs = 48;  // registers per control-warpgroup thread after setmaxnreg.dec
constexpr int kLaunchRegs = 168;  // registers per thread at launch: 65536 / 384 rounded down to a multiple of 8
// setmaxnreg.inc can only take what setmaxnreg.dec gave back inside the same CTA (the pool is the CTA's launch
// allocation); an unbalanced pair blocks in hardware for ever.
static_assert(kPromoWarps * (kPromoRegs - kLaunchRegs) <= 4 * (kLaunchRegs - kControlRegs), "setmaxnreg pool unbalanced");

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
    int tma_store;  // stage blocks of 32 rows in shared memory and write them with TMA stores
    int n_out;      // number of output matrices the TMA-store epilogue writes every block to (1, or the ranks of an
                    // N-sharded group: each rank's full [M, N_total] matrix, peers through mapped peer memory)
    int out_col0;   // column of this GEMM's first output column in those matrices
};

constexpr int kMaxOutputs = 8;
struct OutputMaps {
    CUtensorMap m[kMaxOutputs];
};

// Columns of one TMA-store box of the epilogue for a tile BN wide: 64 (32 rows x 128 bytes, 128-byte swizzle) when
// a promotion warp owns at least 64 columns, else 32 (32 rows x 64 bytes, 64-byte swizzle).
__host__ __device__ constexpr int blockwise_store_cols(int bn) { return bn / 2 >= 64 ? 64 : 32; }
__host__ __device__ constexpr size_t blockwise_smem_bytes(int bn, int stages)
{
    return static_cast<size_t>(stages) * (kBM + bn) * kBK + kPromoWarps * blockwise_store_cols(bn) * 64 + 1024;
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

// acc{lo,hi} += fp32(v0, v1) * t for a pair of int32 partials (|P| <= 128 * 128 * 128 = 2^21, so the conversion is
// exact) as two cvt.rn.f32.s32 and one fma.rn.f32x2; each half of the packed fma rounds like a scalar fmaf.
GI8_DEVICE void promote_pair(uint64_t& acc, uint32_t v0, uint32_t v1, uint64_t t2)
{
    asm volatile(
        "{\n\t"
        ".reg .b64 pv;\n\t"
        ".reg .f32 a, b;\n\t"
        "cvt.rn.f32.s32 a, %1;\n\t"
        "cvt.rn.f32.s32 b, %2;\n\t"
        "mov.b64 pv, {a, b};\n\t"
        "fma.rn.f32x2 %0, pv, %3, %0;\n\t"
        "}\n"
        : "+l"(acc)
        : "r"(v0), "r"(v1), "l"(t2));
}

GI8_DEVICE uint64_t splat_f32x2(float t)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(t));
    return r;
}

GI8_DEVICE void unpack_f32x2(uint64_t v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// Two packed pairs (four consecutive columns) -> two bf16x2 words.
GI8_DEVICE uint32_t pack_bf16x2_of(uint64_t pair)
{
    float lo, hi;
    unpack_f32x2(pair, lo, hi);
    return pack_bf16x2(lo, hi);
}

// Makes a 32-bit value opaque to the optimiser at this point, so that later uses read the register instead of
// recomputing the value.
#define GI8_PIN(v) asm volatile("" : "+r"(v))

// SPLIT = 2 (BN = 256 only): the MMAs of a K block are issued as two column halves (N = 128 each), each half with
// its own commit and its own hand-back barrier, so the four promotion warps of the first half start half an MMA
// time earlier.  NISS: number of MMA-issuing threads (1 or 2, alternate K blocks).
template <int BN, int STAGES, int SPLIT, int NISS>
__global__ void __launch_bounds__(kBlockwiseThreads, 1)
blockwise_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                      const __grid_constant__ OutputMaps outs, const BlockwiseParams p)
{
    static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
    static_assert(SPLIT == 1 || (SPLIT == 2 && BN == 256), "column halves only for the 256-wide tile");
    static_assert(NISS == 1 || NISS == 2, "one or two MMA issuers");
    constexpr int NBUF = 512 / BN;    // partial buffers in tensor memory (2, 4 or 8)
    constexpr int NSUB = BN / SPLIT;  // N of one MMA
    constexpr int CW = BN / 2;        // columns per promotion warp (128, 64 or 32)
    constexpr int NC = CW / 32;       // 32-column loads per K block and warp
    constexpr int STORE_W = blockwise_store_cols(BN);
    // Each issuer must own the stages and the partial buffers of its K blocks (see the protocol above): with an odd
    // count an issuer would meet a barrier only every second phase, which a parity wait cannot tell apart.
    static_assert(STAGES % NISS == 0 && NBUF % NISS == 0, "issuers must own their stages and partial buffers");
    // A promotion warp's parity wait on bar_done is safe only if the commit STAGES K blocks later needs a partial
    // buffer that the same warp hands back after the awaited K block (see the protocol above).
    static_assert(STAGES >= NBUF, "the stage ring must be at least as deep as the partial-buffer ring");
    constexpr uint32_t kBytesA = kBM * kBK;
    constexpr uint32_t kBytesB = BN * kBK;
    constexpr uint32_t kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdesc = make_idesc_i8(kBM, NSUB, false);
    constexpr uint32_t kStoreBytes = STORE_W * 64;  // one staging block per promotion warp: 32 rows x STORE_W bf16

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    __shared__ __align__(8) uint64_t bar_full[STAGES];
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

    if (warp < 4) {
        setmaxnreg_dec<kControlRegs>();
        // Both control roles run their loops with the WHOLE warp (uniform control flow) and elect one lane only
        // around the TMA / MMA / commit instructions themselves.  Inside an `if (lane == 0)` region the compiler
        // treats addresses and descriptors as per-thread values and moves them into uniform registers one by one for
        // every tcgen05.mma; measured on an otherwise idle SM, four MMAs plus a commit then cost 390-440 cycles to
        // issue against about 200 in this form -- with 512 cycles of tensor-core work per K block and two busy
        // promotion warps on the same scheduler, that difference decides whether the tensor core is kept fed.
        if (warp == 0) {
            // -------------------------------------------------------------- TMA producer
            uint32_t s = 0, ph = 0;  // stage and phase parity of the running K-block counter
            uint32_t armed = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int mb, nb;
                tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
                for (int kb = 0; kb < num_kb; ++kb) {
                    bool freed = wait_or_abort(&bar_done[0][s], ph ^ 1, &abort_flag);
                    if (SPLIT == 2 && freed) freed = wait_or_abort(&bar_done[SPLIT - 1][s], ph ^ 1, &abort_flag);
                    if (!freed) {
                        if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    if (elect_one()) {
                        uint8_t* sa_tile = smem + s * kStageBytes;
                        mbar_arrive_expect_tx(&bar_full[s], kStageBytes);
                        tma_load_2d(sa_tile, &map_x, &bar_full[s], kb * kBK, mb * kBM);
                        tma_load_2d(sa_tile + kBytesA, &map_y, &bar_full[s], kb * kBK, nb * BN);
                    }
                    __syncwarp();
                    if (armed < STAGES) ++armed;
                    if (++s == STAGES) s = 0, ph ^= 1;
                }
            }
            // Drain: every armed stage must have landed before the CTA may exit.  (s, ph) is the slot after the last
            // armed one; walk backwards over the armed stages.
            for (uint32_t j = 0; j < armed; ++j) {
                if (s == 0) s = STAGES, ph ^= 1;
                --s;
                if (!mbar_wait(&bar_full[s], ph)) {
                    if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_DRAIN);
                    break;
                }
            }
        } else if (warp == 1 || (NISS == 2 && warp == 3)) {
            // -------------------------------------------------------------- MMA issuer(s)
            const uint32_t first = (NISS == 2 && warp == 3) ? 1u : 0u;
            int my_tiles = 0;
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) ++my_tiles;
            const uint32_t total = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(num_kb);
            // stage / partial buffer of K block `it` and their phase parities, stepped by NISS without divisions
            uint32_t s = first, ph = 0, buf = first, bph = 0;
            for (uint32_t it = first; it < total; it += NISS) {
                // The operands first (they land long before the partial buffer is free), so that nothing but the
                // MMAs stands between the buffer hand-back and the tensor core.
                bool issued = wait_or_abort(&bar_full[s], ph, &abort_flag);
                const uint32_t tmem_d = tmem_base + buf * BN;
                const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                const uint64_t da = make_smem_desc_k128(a_addr);
                const uint64_t db = make_smem_desc_k128(a_addr + kBytesA);
#pragma unroll
                for (int h = 0; h < SPLIT && issued; ++h) {
                    if (!wait_or_abort(&bar_part_empty[h][buf], bph ^ 1, &abort_flag)) {
                        issued = false;
                        break;
                    }
                    tcgen05_fence_after_sync();
                    if (elect_one()) {
                        // Half h: rows h * NSUB.. of the weight tile (NSUB rows of 128 bytes: 16-byte units in
                        // the descriptor's address field) into columns h * NSUB.. of the partial buffer.  The
                        // first K step overwrites the buffer.
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k)
                            umma_i8(tmem_d + h * NSUB, da + 2 * k, db + (h * NSUB * kBK) / 16 + 2 * k, kIdesc, k != 0 ? 1u : 0u);
                        umma_commit(&bar_done[h][s]);
                    }
                    __syncwarp();
                }
                if (!issued) {
                    if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                    break;
                }
                s += NISS;
                if (s >= STAGES) s -= STAGES, ph ^= 1;
                buf += NISS;
                if (buf >= NBUF) buf -= NBUF, bph ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue warps
        setmaxnreg_inc<kPromoRegs>();
        const int quarter = warp & 3;
        const int cg = (warp - 4) >> 2;  // column half of the tile
        // Tensor-memory address of this warp's lanes and first column in partial buffer 0 (buffer b is b * BN
        // columns further).  GI8_PIN keeps such loop-invariant values in a register: left alone, the compiler
        // re-derives them from %tid.x inside the K loop, in a loop whose bound is instruction issue.
        uint32_t tm_warp = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(cg * CW);
        GI8_PIN(tm_warp);
        const int half = SPLIT == 2 ? cg : 0;
        uint32_t bar_done_h = smem_u32(&bar_done[half][0]);
        uint32_t bar_empty_h = smem_u32(&bar_part_empty[half][0]);
        GI8_PIN(bar_done_h);
        GI8_PIN(bar_empty_h);
        // Stage, partial buffer and barrier phase of the running K block (as in the MMA issuer), stepped without
        // divisions: byte offset of the stage's barrier, its parity, byte offset of the buffer's barrier, the
        // buffer's first column.
        uint32_t st_off = 0, st_par = 0, buf_off = 0, buf_col = 0;
        bool ok = true;

        // Waits for the partial of the running K block; false on every lane if any lane gave up.  The common case is
        // one successful test; the branch to the bounded spin is taken on a vote, which makes it warp-uniform.
        auto wait_partial = [&]() {
            const uint32_t bar = bar_done_h + st_off;
            bool got = mbar_try_wait_addr(bar, st_par);
            if (!__all_sync(0xffffffffu, got)) {
                got = wait_or_abort_addr(bar, st_par, &abort_flag);
                if (!got && lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                got = __all_sync(0xffffffffu, got);
                if (!got) return false;
            }
            tcgen05_fence_after_sync();
            return true;
        };
        // The whole partial buffer of the running K block is in registers: hand it back to the MMA issuer.
        auto release_partial = [&]() {
            tcgen05_fence_before_sync();
            __syncwarp();
            mbar_arrive_elected_addr(bar_empty_h + buf_off);
        };
        auto next_k_block = [&]() {
            st_off += 8;
            if (st_off == STAGES * 8) st_off = 0, st_par ^= 1;
            buf_off += 8, buf_col += BN;
            if (buf_off == NBUF * 8) buf_off = 0, buf_col = 0;
        };

        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m);
            const int row = mb * kBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const int col_base = nb * BN + cg * CW;  // first output column of this warp
            // A column half lies inside one 128-wide weight-scale block (CW divides 128, col_base % CW == 0).
            const bool cols_ok = col_base < p.N;
            // 32-bit element offsets (the scale arrays are far smaller than 2^31 elements) instead of two pointers.
            uint32_t sa_off = static_cast<uint32_t>(row_ok ? row : 0) * static_cast<uint32_t>(p.ld_sa);
            uint32_t sw_off = static_cast<uint32_t>(cols_ok ? col_base / 128 : 0) * static_cast<uint32_t>(p.ld_sw);
            GI8_PIN(sa_off);
            GI8_PIN(sw_off);

            uint64_t acc[CW / 2];  // fp32 accumulators of columns (2j, 2j + 1) as f32x2 pairs
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) acc[j] = 0ull;

            // Scales are loaded two K blocks before their use (an L2 hit takes about one K block); the two register
            // sets alternate statically through the unrolled loop below.
            float sa0 = 0.0f, sw0 = 0.0f, sa1 = 0.0f, sw1 = 0.0f;
            sa0 = __ldg(p.sa + sa_off);
            sw0 = __ldg(p.sw + sw_off);
            if (num_kb > 1) {
                sa1 = __ldg(p.sa + (sa_off + 1));
                sw1 = __ldg(p.sw + (sw_off + 1));
            }

            // One K block: wait for its partial, form the block's scale (fp32 product, round to nearest) and start
            // the loads of the scales two blocks on, then per 32-column chunk load, (after the last load) hand the
            // buffer back, convert and accumulate.
            auto k_block = [&](int kb, float& sa_r, float& sw_r) -> bool {
                if (!wait_partial()) return false;
                const uint64_t t2 = splat_f32x2(sa_r * sw_r);
                if (kb + 2 < num_kb) {
                    sa_r = __ldg(p.sa + (sa_off + kb + 2));
                    sw_r = __ldg(p.sw + (sw_off + kb + 2));
                }
                const uint32_t taddr = tm_warp + buf_col;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, v);
                    tmem_ld_wait();
                    if (c + 1 == NC) release_partial();
#pragma unroll
                    for (int j = 0; j < 16; ++j) promote_pair(acc[c * 16 + j], v[2 * j], v[2 * j + 1], t2);
                }
                next_k_block();
                return true;
            };
            for (int kb = 0; kb < num_kb; kb += 2) {
                if (!k_block(kb, sa0, sw0)) {
                    ok = false;
                    break;
                }
                if (kb + 1 < num_kb && !k_block(kb + 1, sa1, sw1)) {
                    ok = false;
                    break;
                }
            }
            if (!ok) break;

            if (p.tma_store) {
                // Blocks of 32 rows x STORE_W columns through swizzled shared memory and TMA stores (rows >= M and
                // columns beyond the tensor map are clipped by the hardware).  The tile's coordinates are derived
                // again from an opaque copy of the tile index so that they do not occupy registers across the
                // promotion loop.
                int tile_again = tile, mb2, nb2;
                asm volatile("" : "+r"(tile_again));
                tile_coords(tile_again, p.tiles_m, p.tiles_n, mb2, nb2, p.group_m);
                const int row0 = mb2 * kBM + quarter * 32;
                const int col0 = nb2 * BN + cg * CW;
                if (row0 < p.M) {
                    const uint32_t stg = ((smem_u32(smem_raw) + 1023u) & ~1023u) + STAGES * kStageBytes + (warp - 4) * kStoreBytes;
#pragma unroll
                    for (int b = 0; b < CW / STORE_W; ++b) {
                        if (col0 + b * STORE_W >= p.N) break;  // warp-uniform
                        if (lane == 0) tma_store_wait_read<0>();  // the previous block has been read out of the staging
                        __syncwarp();
                        // row = lane; 16-byte chunk q of the row goes to chunk q ^ (row % 8) (128-byte swizzle) or
                        // q ^ ((row / 2) % 4) (64-byte swizzle): conflict-free and what the tensor map expects.
#pragma unroll
                        for (int q = 0; q < STORE_W / 8; ++q) {
                            const int cq = STORE_W == 64 ? (q ^ (lane & 7)) : (q ^ ((lane >> 1) & 3));
                            const int a0 = b * (STORE_W / 2) + 4 * q;
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * (STORE_W * 2) + cq * 16),
                                         "r"(pack_bf16x2_of(acc[a0])), "r"(pack_bf16x2_of(acc[a0 + 1])),
                                         "r"(pack_bf16x2_of(acc[a0 + 2])), "r"(pack_bf16x2_of(acc[a0 + 3]))
                                         : "memory");
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            // one store per output matrix (the local one, and in an N-sharded group every peer's,
                            // through its mapped memory: plain unicast TMA stores)
                            for (int o = 0; o < p.n_out; ++o)
                                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                                 reinterpret_cast<uint64_t>(&outs.m[o])),
                                             "r"(stg), "r"(p.out_col0 + col0 + b * STORE_W), "r"(row0)
                                             : "memory");
                            tma_store_commit();
                        }
                    }
                }
            } else if (row_ok && cols_ok) {
                uint16_t* dst = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col_base;
                if (col_base + CW <= p.N && p.vec_ok) {
#pragma unroll
                    for (int j = 0; j < CW / 2; j += 4)
                        *reinterpret_cast<uint4*>(dst + 2 * j) = make_uint4(pack_bf16x2_of(acc[j]), pack_bf16x2_of(acc[j + 1]),
                                                                            pack_bf16x2_of(acc[j + 2]), pack_bf16x2_of(acc[j + 3]));
                } else {
#pragma unroll
                    for (int j = 0; j < CW / 2; ++j) {
                        float lo, hi;
                        unpack_f32x2(acc[j], lo, hi);
                        if (col_base + 2 * j < p.N) dst[2 * j] = to_bf16_bits(lo);
                        if (col_base + 2 * j + 1 < p.N) dst[2 * j + 1] = to_bf16_bits(hi);
                    }
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
