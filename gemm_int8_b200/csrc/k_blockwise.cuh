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
//   warps 4..11 promotion (setmaxnreg.inc): warp w owns TMEM lane quarter (w % 4) and BN/2 of the tile's columns
//               (with column halves: 64 columns of each half), i.e. 32 rows x BN/2 columns, whose fp32
//               accumulators it keeps in registers (as f32x2 pairs).  Per K block and half: tcgen05.ld the int32
//               partial in 32-column chunks, hand the half back after the last load, cvt.rn.f32.s32 +
//               fma.rn.f32x2 with the block's scale.  A warp's segment never straddles a 128-wide weight-scale
//               block.  At the end of the tile the same warps cast to bf16 and store through swizzled shared
//               memory and TMA.
//
// Why eight fat warps (measured on B200 with a stand-alone loop of the same instructions, cycles per 128 x 256
// K block, tensor core busy in the background): a tcgen05.ld costs about one cycle per 32-lane column whatever its
// width and does not overlap the arithmetic of the same scheduler, so deeper load pipelines buy nothing; what
// counts is instructions issued.  16 warps x 64 columns with 16-column loads and a biased accumulator written
// back with tcgen05.st: 860-920.  8 warps x 128 columns, 32-column loads: biased accumulator with write-back 665-685
// (the stores alone cost 140), cvt + fma.f32x2 without any write-back 545-580, against 512 for the MMAs.
// The same was measured in this kernel itself, with the column groups made a template parameter: twelve promotion
// warps (three per scheduler) on a 128 x 192 tile ran 15-20 % slower than eight on 128 x 256, sixteen (four per
// scheduler, 112 registers each, 16-column loads) 40-50 % slower -- every warp repeats the per-K-block bookkeeping
// (barrier test, hand-back, scale product, counters), and those instructions share the half-rate integer pipe
// with the conversions, which is the busiest unit (two cycles per cvt.rn.f32.s32: 512 of the K block's cycles).
//
// Barrier protocol (every wait is a parity wait, so it must hold that a barrier cannot complete a second phase
// before the waiter has consumed the first; the comment at each barrier says what gates its next phase):
//   bar_full[s]        completed by the TMA bytes of K block `it` (s = it % STAGES).  Waiter: the issuer of K block
//                      `it` (with column halves: both issuers, each of which visits every K block).  Next phase
//                      needs the producer to refill stage s, which needs bar_done[h][s] of K block `it` for every
//                      half h, i.e. every waiting issuer's own commit: gated by each waiter.
//   bar_done[h][s]     completed by the issuer's commit for column half h of K block `it`.  Waiters: the producer
//                      (before refilling s; the next completion needs its own refill: gated) and all promotion
//                      warps (the next completion is K block it + STAGES, whose MMAs need half h of partial buffer
//                      (it + STAGES) % NBUF handed back by every warp for K block it + STAGES - NBUF >= it: gated).
//   bar_part_empty[h][b]  completed by the arrivals of all eight promotion warps after their last load of half h of
//                      a K block in buffer b.  Waiter: the issuer of half h of the next K block that uses b; the
//                      completion after that needs this issuer's MMAs: gated.
//   Without column halves and with two issuers, issuer j takes K blocks it % 2 == j, hence stages s % 2 == j and
//   buffers b % 2 == j (STAGES and NBUF are even): every barrier still has exactly one issuing waiter, which sees
//   all its phases.
#pragma once

#include <type_traits>

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
    int scale_vec;  // ceil(K/128) % 4 == 0 and the rows of sa and sw are 16-byte aligned: scales are loaded four at a time
    int pdl_role;   // 0: none.  1: this launch is followed by an independent launch over other output columns: let it start
                    // as SMs free up (griddepcontrol.launch_dependents).  2: that second launch: it reads nothing the first
                    // one writes and therefore does not wait before working, but it waits for the first before it ends,
                    // so that the completion of the pair means the completion of both.
    int scatter_ranks;  // > 0: K-sharded reduce-scatter form.  The fp32 accumulators of tile rows [j R, (j + 1) R), R =
    int scatter_rows;   // scatter_rows, go to output matrix j (rank j's receive area, float [ranks, R, N], mapped peer
    int scatter_me;     // memory for j != me) at row block scatter_me, as 32 x 32 fp32 TMA-store boxes; R % 32 == 0
    int tile_rot;       // the tile sequence starts at this tile (and wraps): in the scattering form rank r starts with its
                        // own rows, so that at any moment the ranks send to different owners instead of all to the same
    int out_f32;    // store the fp32 accumulators themselves (out is float [M,N]) instead of their bf16 cast; the
                    // partial results of a K-sharded GEMM, and the bit-exact check of the accumulation order
};

constexpr int kMaxOutputs = 8;
struct OutputMaps {
    CUtensorMap m[kMaxOutputs];
};

// Columns of one TMA-store box of the epilogue for a tile BN wide: 64 (32 rows x 128 bytes, 128-byte swizzle) when
// a promotion warp owns at least 64 columns, else 32 (32 rows x 64 bytes, 64-byte swizzle).
__host__ __device__ constexpr int blockwise_store_cols(int bn) { return bn / 2 >= 64 ? 64 : 32; }
__host__ __device__ constexpr size_t blockwise_smem_bytes(int bn, int stages, bool pair = false)
{
    return static_cast<size_t>(stages) * (kBM + (pair ? bn / 2 : bn)) * kBK + kPromoWarps * blockwise_store_cols(bn) * 64 + 1024;
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
// The conversions write back into v0 and v1, which a tensor-memory load left in two consecutive registers: the
// packed operand of the fma is then that register pair as it stands.  Converting into fresh registers made the
// compiler add a move or two per pair to bring the results together (measured: 74 extra instructions per warp and
// K block next to 192 useful ones).
GI8_DEVICE void promote_pair(uint64_t& acc, uint32_t& v0, uint32_t& v1, uint64_t t2)
{
    asm volatile(
        "{\n\t"
        ".reg .b64 pv;\n\t"
        "cvt.rn.f32.s32 %1, %1;\n\t"
        "cvt.rn.f32.s32 %2, %2;\n\t"
        "mov.b64 pv, {%1, %2};\n\t"
        "fma.rn.f32x2 %0, pv, %3, %0;\n\t"
        "}\n"
        : "+l"(acc), "+r"(v0), "+r"(v1)
        : "l"(t2));
}

GI8_DEVICE uint64_t splat_f32x2(float t)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(t));
    return r;
}

// a * b (fp32, round to nearest) as a volatile statement: it keeps its place among the other volatile statements
// (tensor-memory loads, conversions).  The scales are loaded two K blocks before their use; written as plain C++ the
// compiler hoists the product up to the loads to save a register, and the warp then waits out the L2 latency right
// there (measured: 150 cycles per K block).
// Read-only global load as a volatile statement, for the same reason: the compiler may not sink it towards its use.
GI8_DEVICE float ldg_in_place(const float* p)
{
    float r;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(r) : "l"(p));
    return r;
}

GI8_DEVICE float4 ldg4_in_place(const float* p)
{
    float4 r;
    asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(p));
    return r;
}

GI8_DEVICE float mul_in_place(float a, float b)
{
    float r;
    asm volatile("mul.rn.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
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

// Position `tile` of the sequence that starts at tile `rot` and wraps at `n` (rot < n).
GI8_DEVICE int rotate_tile(int tile, int rot, int n)
{
    const int t = tile + rot;
    return t >= n ? t - n : t;
}

// Makes a 32-bit value opaque to the optimiser at this point, so that later uses read the register instead of
// recomputing the value.
#define GI8_PIN(v) asm volatile("" : "+r"(v))

// SPLIT = 2 (BN = 256 only): the MMAs of a K block are issued as two column halves (N = 128 each), each half by its
// own issuing thread, with its own commit and its own hand-back barrier, and EVERY promotion warp takes 64 columns of
// each half.  A half's partial buffer is then held for two loads and one chunk of arithmetic instead of four and
// three, and the tensor core refills one half while the warps read the other: with only two 256-column buffers in
// tensor memory the time a buffer is held, plus the latencies of the two hand-overs, is what bounds the K-block
// period (measured: 1000-1200 cycles per K block with contiguous 128-column ownership, where neither instruction
// issue (51 %) nor any pipe was saturated).
// SPLIT = 1: MMAs with N = BN; NISS issuing threads (1 or 2) take alternate K blocks.
// PAIR: two CTAs on neighbouring SMs (a 2 x 1 x 1 cluster) share one 256 x BN tile, as in the dense kernel: the
// leader's issuers run tcgen05.mma.cta_group::2 (M = 256), each CTA loads its own 128 rows of x and HALF of the BN
// rows of y, keeps the partials of its 128 rows in its own tensor memory and promotes them with its own eight warps.
// Per SM that is a third fewer operand bytes per K block (32 KB instead of 48 KB; four stages are used, six would fit
// and measured the same) and half the MMA instructions.  It matters because the 1-CTA kernel is bound by bytes in flight: with four
// 48 KB stages, one of them being read by the tensor core, 144 KB are in flight against an L2 latency of about 2000
// cycles under load -- 72 bytes per cycle, i.e. 670 cycles per 48 KB K block where the tensor core needs 512.  TMA
// loads are unicast into the issuing CTA's shared memory and signal the leader's barrier; the commits are two
// unicast tcgen05.commit (no multicast anywhere).
// An N = 128 two-CTA MMA (column halves) takes 64 rows of y from each CTA, so half h of the partial holds tile
// columns [64 h, 64 h + 64) and [128 + 64 h, 128 + 64 h + 64): a promotion warp's 64-column segment of half h is then
// tile columns cg * 128 + h * 64 .. (still contiguous and inside one weight-scale block).
template <int BN, int STAGES, int SPLIT, int NISS, bool PAIR = false>
__global__ void __launch_bounds__(kBlockwiseThreads, 1)
blockwise_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                      const __grid_constant__ OutputMaps outs, const BlockwiseParams p)
{
    static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
    static_assert(SPLIT == 1 || (SPLIT == 2 && BN == 256), "column halves only for the 256-wide tile");
    static_assert(NISS == 1 || NISS == 2, "one or two MMA issuers");
    static_assert(SPLIT == 1 || NISS == 2, "with column halves there is one issuer per half");
    constexpr int NBUF = 512 / BN;       // partial buffers in tensor memory (2, 4 or 8)
    constexpr int NSUB = BN / SPLIT;     // N of one MMA = columns of one half
    constexpr int CW = BN / 2;           // columns per promotion warp (128, 64 or 32) ...
    constexpr int SEGW = CW / SPLIT;     // ... as SPLIT segments of SEGW columns, one in each half
    constexpr int CHW = 32;              // columns per tensor-memory load (64 was measured: no gain)
    constexpr int NC = SEGW / CHW;       // loads per segment
    constexpr int STORE_W = blockwise_store_cols(BN);
    static_assert(SEGW % STORE_W == 0 && SEGW % 32 == 0, "segments are whole store boxes and whole loads");
    // SPLIT == 1: each issuer must own the stages and the partial buffers of its K blocks (see the protocol above):
    // with an odd count an issuer would meet a barrier only every second phase, which a parity wait cannot tell apart.
    static_assert(SPLIT == 2 || (STAGES % NISS == 0 && NBUF % NISS == 0), "issuers must own their stages and partial buffers");
    // A promotion warp's parity wait on bar_done is safe only if the commit STAGES K blocks later needs a partial
    // buffer that the same warp hands back after the awaited K block (see the protocol above).
    static_assert(STAGES >= NBUF, "the stage ring must be at least as deep as the partial-buffer ring");
    static_assert(!PAIR || BN == 256, "two-CTA tiles are 256 wide");
    constexpr int kTileM = PAIR ? 2 * kBM : kBM;  // rows of the (pair's) tile
    constexpr int kRowsB = PAIR ? BN / 2 : BN;    // rows of y this CTA loads
    constexpr uint32_t kBytesA = kBM * kBK;
    constexpr uint32_t kBytesB = kRowsB * kBK;
    constexpr uint32_t kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdesc = make_idesc_i8(kTileM, NSUB, false);
    // Tile column of the first column of segment (half h, column group cg), see above.
    constexpr int kSegStrideH = (PAIR && SPLIT == 2) ? SEGW : NSUB;
    constexpr int kSegStrideCg = (PAIR && SPLIT == 2) ? NSUB : SEGW;
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
    const int num_tiles = p.tiles_m * p.tiles_n;  // tiles_m counts kTileM-row tiles
    const int num_kb = (p.K + kBK - 1) / kBK;
    // PAIR: rank 0 is the leader (its bar_full and bar_part_empty serve both CTAs); the pair is the scheduling unit.
    const uint32_t rank = PAIR ? cluster_cta_rank() : 0u;
    const int first_tile = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        if (p.pdl_role == 1) pdl_launch_dependents();
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            for (int h = 0; h < SPLIT; ++h) mbar_init(&bar_done[h][s], 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            for (int h = 0; h < SPLIT; ++h) mbar_init(&bar_part_empty[h][b], PAIR ? 2 * kPromoWarps : kPromoWarps);
        }
        fence_barrier_init();
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_y);
    }
    if (warp == 2) {
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
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
                int mb, nb;
                tile_coords(rotate_tile(tile, p.tile_rot, num_tiles), p.tiles_m, p.tiles_n, mb, nb, p.group_m);
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
                        if constexpr (PAIR) {
                            // The leader arms its barrier for the bytes of BOTH CTAs; the peer only sends bytes.
                            const uint32_t leader_full = map_to_cta(smem_u32(&bar_full[s]), 0);
                            if (rank == 0) mbar_arrive_expect_tx(&bar_full[s], 2 * kStageBytes);
                            tma_load_2d_pair(sa_tile, &map_x, leader_full, kb * kBK, mb * kTileM + static_cast<int>(rank) * kBM);
                            tma_load_2d_pair(sa_tile + kBytesA, &map_y, leader_full, kb * kBK, nb * BN + static_cast<int>(rank) * kRowsB);
                        } else {
                            mbar_arrive_expect_tx(&bar_full[s], kStageBytes);
                            tma_load_2d(sa_tile, &map_x, &bar_full[s], kb * kBK, mb * kBM);
                            tma_load_2d(sa_tile + kBytesA, &map_y, &bar_full[s], kb * kBK, nb * BN);
                        }
                    }
                    __syncwarp();
                    if (armed < STAGES) ++armed;
                    if (++s == STAGES) s = 0, ph ^= 1;
                }
            }
            // Drain: every armed stage must have landed before the CTA may exit (PAIR: the leader's barriers complete
            // only when both CTAs' bytes have landed; the peer leaves through the final cluster barrier).  (s, ph) is
            // the slot after the last armed one; walk backwards over the armed stages.
            if (PAIR && rank != 0) armed = 0;
            for (uint32_t j = 0; j < armed; ++j) {
                if (s == 0) s = STAGES, ph ^= 1;
                --s;
                if (!mbar_wait(&bar_full[s], ph)) {
                    if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_DRAIN);
                    break;
                }
            }
        } else if ((warp == 1 || (NISS == 2 && warp == 3)) && rank == 0) {
            // -------------------------------------------------------------- MMA issuer(s) (PAIR: the leader's)
            const uint32_t me = warp == 1 ? 0u : 1u;
            // SPLIT == 2: issuer `me` issues column half `me` of EVERY K block.  SPLIT == 1: issuer `me` issues the
            // K blocks with it % NISS == me.
            constexpr uint32_t kStep = SPLIT == 2 ? 1u : static_cast<uint32_t>(NISS);
            const uint32_t first = SPLIT == 2 ? 0u : me;
            const uint32_t h = SPLIT == 2 ? me : 0u;
            int my_tiles = 0;
            for (int tile = first_tile; tile < num_tiles; tile += tile_step) ++my_tiles;
            const uint32_t total = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(num_kb);
            // stage / partial buffer of K block `it` and their phase parities, stepped without divisions
            uint32_t s = first, ph = 0, buf = first, bph = 0;
            uint64_t* const done_h = &bar_done[h][0];
            uint64_t* const empty_h = &bar_part_empty[h][0];
            for (uint32_t it = first; it < total; it += kStep) {
                // The operands first (they land long before the partial buffer is free), so that nothing but the
                // MMAs stands between the buffer hand-back and the tensor core.
                bool issued = wait_or_abort(&bar_full[s], ph, &abort_flag);
                // Half h: rows h * NSUB.. of the weight tile (PAIR: rows h * NSUB / 2.. of each CTA's half of it) into
                // columns h * NSUB.. of the partial buffer.
                const uint32_t tmem_d = tmem_base + buf * BN + h * NSUB;
                const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                const uint64_t da = make_smem_desc_k128(a_addr);
                const uint64_t db = make_smem_desc_k128(a_addr + kBytesA + h * (PAIR ? NSUB / 2 : NSUB) * kBK);
                issued = issued && wait_or_abort(&empty_h[buf], bph ^ 1, &abort_flag);
                if (!issued) {
                    if (lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_MMA);
                    break;
                }
                tcgen05_fence_after_sync();
                if (elect_one()) {
                    // The first K step overwrites the buffer.
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        if constexpr (PAIR) umma_i8_pair(tmem_d, da + 2 * k, db + 2 * k, kIdesc, k != 0 ? 1u : 0u);
                        else umma_i8(tmem_d, da + 2 * k, db + 2 * k, kIdesc, k != 0 ? 1u : 0u);
                    }
                    if constexpr (PAIR) {
                        umma_commit_pair(map_to_cta(smem_u32(&done_h[s]), 0));
                        umma_commit_pair(map_to_cta(smem_u32(&done_h[s]), 1));
                    } else {
                        umma_commit(&done_h[s]);
                    }
                }
                __syncwarp();
                s += kStep;
                if (s >= STAGES) s -= STAGES, ph ^= 1;
                buf += kStep;
                if (buf >= NBUF) buf -= NBUF, bph ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue warps
        setmaxnreg_inc<kPromoRegs>();
        const int quarter = warp & 3;
        const int cg = (warp - 4) >> 2;  // which SEGW columns of every half this warp owns
        // Tensor-memory address of this warp's lanes and first column in partial buffer 0 (buffer b is b * BN
        // columns further, half h another h * NSUB).  GI8_PIN keeps such loop-invariant values in a register: left
        // alone, the compiler re-derives them from %tid.x inside the K loop, in a loop whose bound is instruction
        // issue.
        uint32_t tm_warp = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(cg * SEGW);
        GI8_PIN(tm_warp);
        uint32_t bar_done_0 = smem_u32(&bar_done[0][0]);
        // (PAIR: the hand-back barriers are the leader's, addressed through the cluster window)
        uint32_t bar_empty_0 = PAIR ? map_to_cta(smem_u32(&bar_part_empty[0][0]), 0) : smem_u32(&bar_part_empty[0][0]);
        GI8_PIN(bar_done_0);
        GI8_PIN(bar_empty_0);
        // Stage, partial buffer and barrier phase of the running K block (as in the MMA issuer), stepped without
        // divisions: byte offset of the stage's barrier, its parity, byte offset of the buffer's barrier, the
        // buffer's first column.
        uint32_t st_off = 0, st_par = 0, buf_off = 0, buf_col = 0;
        bool ok = true;

        // Waits for half h of the partial of the running K block; false on every lane if any lane gave up.  The
        // barrier was already tested once, without blocking, before the arithmetic of the previous chunk
        // (`polled`, see poll_next): in the steady state the MMAs are ahead, the test has succeeded and its latency
        // lay under that arithmetic.  Otherwise the bounded wait runs; the branch is taken on a vote, which makes it
        // warp-uniform.
        bool polled = false;
        // (so, sp): byte offset of the stage's barrier in its ring and the parity awaited there.
        auto wait_partial = [&](int h, uint32_t so, uint32_t sp) {
            if (!__all_sync(0xffffffffu, polled)) {
                const uint32_t bar = bar_done_0 + h * (STAGES * 8) + so;
                bool got = wait_or_abort_addr(bar, sp, &abort_flag);
                if (!got && lane == 0) raise_error(p.status, &abort_flag, ERR_TIMEOUT_EPILOGUE);
                got = __all_sync(0xffffffffu, got);
                if (!got) return false;
            }
            tcgen05_fence_after_sync();
            return true;
        };
        // Tests the barrier of the partial that follows half h of the K block at (so, sp): the other half of the same
        // K block, or half 0 of the next K block (the stage ring runs on across tiles; after the last K block of the
        // last tile the test simply fails and is never looked at).
        auto poll_next = [&](int h, uint32_t so, uint32_t sp) {
            int hn = h + 1;
            if (hn == SPLIT) {
                hn = 0;
                so += 8;
                if (so == STAGES * 8) so = 0, sp ^= 1;
            }
            polled = mbar_test_wait_addr(bar_done_0 + hn * (STAGES * 8) + so, sp);
        };
        // This warp's columns of half h of the K block in the partial buffer whose barrier lies at byte offset bo are
        // in registers: one of the arrivals that hand the half back to its MMA issuer.
        auto release_partial = [&](int h, uint32_t bo) {
            tcgen05_fence_before_sync();
            __syncwarp();
            if constexpr (PAIR) {
                if (elect_one()) mbar_arrive_cluster(bar_empty_0 + h * (NBUF * 8) + bo);
            } else {
                mbar_arrive_elected_addr(bar_empty_0 + h * (NBUF * 8) + bo);
            }
        };
        auto next_k_block = [&]() {
            st_off += 8;
            if (st_off == STAGES * 8) st_off = 0, st_par ^= 1;
            buf_off += 8, buf_col += BN;
            if (buf_off == NBUF * 8) buf_off = 0, buf_col = 0;
        };
        // With four stages, two partial buffers and K blocks handled four at a time (the vector-scale path, whose K
        // block count is a multiple of four), every tile starts at stage 0 and buffer 0: the ring positions of the four
        // K blocks of a group are compile-time constants and only the parity, flipped once per group, lives in a
        // register.  That removes the counter arithmetic (about ten instructions per warp and K block on the integer
        // pipe, which the conversions keep busiest).
        constexpr bool kStaticRing = STAGES == 4 && NBUF == 2;

        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
            int mb, nb;
            tile_coords(rotate_tile(tile, p.tile_rot, num_tiles), p.tiles_m, p.tiles_n, mb, nb, p.group_m);
            const int row = mb * kTileM + static_cast<int>(rank) * kBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            // First output column of this warp's segment in half 0 (half h: kSegStrideH further).  A segment lies
            // inside one 128-wide weight-scale block (SEGW divides 128 and the segment starts at a multiple of it).
            const int col_base = nb * BN + cg * kSegStrideCg;
            // 32-bit element offsets (the scale arrays are far smaller than 2^31 elements) instead of pointers.
            uint32_t sa_off = static_cast<uint32_t>(row_ok ? row : 0) * static_cast<uint32_t>(p.ld_sa);
            uint32_t sw_off[SPLIT];
#pragma unroll
            for (int h = 0; h < SPLIT; ++h) {
                const int c = col_base + h * kSegStrideH;
                sw_off[h] = static_cast<uint32_t>(c < p.N ? c / 128 : 0) * static_cast<uint32_t>(p.ld_sw);
                GI8_PIN(sw_off[h]);
            }
            GI8_PIN(sa_off);

            uint64_t acc[CW / 2];  // fp32 accumulators as f32x2 pairs: segment h, columns (2j, 2j + 1) in acc[h * SEGW / 2 + j]
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) acc[j] = 0ull;

            // One K block with the scale products t[h] of its column halves: per half wait for the partial, then per
            // 32-column chunk load, (after the half's last load) hand the half back, convert and accumulate.
            // (Issuing the next chunk's load before this chunk's arithmetic was tried with 32- and with 16-column
            // chunks: no gain, the 32-column form spills.  64-column loads: no gain.  Sending a third of the pairs
            // through an integer multiply-add on the other pipe instead of cvt: no gain.  Leaving the grouping of
            // conversions and multiply-adds to the compiler (non-volatile statements): the same cycle count.  Writing
            // the conversions one to sixteen pairs ahead of their multiply-adds: the same times to within the run-to-run
            // spread -- the assembler schedules the block itself.  Sending every third to eighth pair through
            // multiply-add-pipe instructions only (integer multiply-add with the bias 0x4B400000, packed subtract,
            // packed fma), measured again after the barrier latencies had been hidden: 15-45 % slower on the one-CTA
            // form, 2-4 % faster on the two-CTA form with column halves.)
            // J >= 0: K block J of a group of four under kStaticRing; J < 0: the running counters.
            auto k_block = [&](const float (&t)[SPLIT], auto jc) -> bool {
                constexpr int J = decltype(jc)::value;
                const uint32_t so = J >= 0 ? static_cast<uint32_t>(J * 8) : st_off;
                const uint32_t sp = st_par;
                const uint32_t bo = J >= 0 ? static_cast<uint32_t>((J & 1) * 8) : buf_off;
                const uint32_t bc = J >= 0 ? static_cast<uint32_t>((J & 1) * BN) : buf_col;
#pragma unroll
                for (int h = 0; h < SPLIT; ++h) {
                    if (!wait_partial(h, so, sp)) return false;
                    const uint64_t t2 = splat_f32x2(t[h]);
                    const uint32_t taddr = tm_warp + bc + h * NSUB;
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        uint32_t v[CHW];
                        tmem_ld_32x32b_x32(taddr + c * CHW, v);
                        tmem_ld_wait();
                        if (c + 1 == NC) {
                            release_partial(h, bo);
                            poll_next(h, so, sp);
                        }
#pragma unroll
                        for (int q = 0; q < CHW / 2; ++q) promote_pair(acc[h * (SEGW / 2) + c * (CHW / 2) + q], v[2 * q], v[2 * q + 1], t2);
                    }
                }
                if constexpr (J < 0) next_k_block();
                else if constexpr (J == 3) st_par ^= 1;
                return true;
            };
            using Dyn = std::integral_constant<int, -1>;

            if (p.scale_vec) {
                // Scales of four K blocks per load (16 bytes per row): a quarter of the load instructions and of
                // the sectors touched (a token's scales of eight consecutive K blocks share one 32-byte sector, and
                // the 32 lanes of a warp read 32 different rows).  The next group is loaded before the current one
                // is used.  Needs ceil(K/128) % 4 == 0 and 16-byte aligned scale rows; the host checks.
                float4 sa_c = ldg4_in_place(p.sa + sa_off), sw_c[SPLIT];
#pragma unroll
                for (int h = 0; h < SPLIT; ++h) sw_c[h] = ldg4_in_place(p.sw + sw_off[h]);
                for (int kb = 0; kb < num_kb && ok; kb += 4) {
                    float4 sa_n = sa_c, sw_n[SPLIT];
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) sw_n[h] = sw_c[h];
                    if (kb + 4 < num_kb) {
                        sa_n = ldg4_in_place(p.sa + (sa_off + kb + 4));
#pragma unroll
                        for (int h = 0; h < SPLIT; ++h) sw_n[h] = ldg4_in_place(p.sw + (sw_off[h] + kb + 4));
                    }
                    float t[SPLIT];
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) t[h] = mul_in_place(sa_c.x, sw_c[h].x);
                    ok = k_block(t, std::integral_constant<int, kStaticRing ? 0 : -1>{});
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) t[h] = mul_in_place(sa_c.y, sw_c[h].y);
                    ok = ok && k_block(t, std::integral_constant<int, kStaticRing ? 1 : -1>{});
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) t[h] = mul_in_place(sa_c.z, sw_c[h].z);
                    ok = ok && k_block(t, std::integral_constant<int, kStaticRing ? 2 : -1>{});
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) t[h] = mul_in_place(sa_c.w, sw_c[h].w);
                    ok = ok && k_block(t, std::integral_constant<int, kStaticRing ? 3 : -1>{});
                    sa_c = sa_n;
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) sw_c[h] = sw_n[h];
                }
            } else {
                // Scales are loaded two K blocks before their use (an L2 hit takes about one K block); the two
                // register sets alternate statically through the unrolled loop below.
                float sa_q[2], sw_q[2][SPLIT];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    sa_q[j] = 0.0f;
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) sw_q[j][h] = 0.0f;
                    if (j < num_kb) {
                        sa_q[j] = ldg_in_place(p.sa + (sa_off + j));
#pragma unroll
                        for (int h = 0; h < SPLIT; ++h) sw_q[j][h] = ldg_in_place(p.sw + (sw_off[h] + j));
                    }
                }
                auto k_block_scalar = [&](int kb, int j) -> bool {
                    float t[SPLIT];
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) t[h] = mul_in_place(sa_q[j], sw_q[j][h]);
                    if (kb + 2 < num_kb) {
                        sa_q[j] = ldg_in_place(p.sa + (sa_off + kb + 2));
#pragma unroll
                        for (int h = 0; h < SPLIT; ++h) sw_q[j][h] = ldg_in_place(p.sw + (sw_off[h] + kb + 2));
                    }
                    return k_block(t, Dyn{});
                };
                for (int kb = 0; kb < num_kb && ok; kb += 2) {
                    ok = k_block_scalar(kb, 0);
                    if (ok && kb + 1 < num_kb) ok = k_block_scalar(kb + 1, 1);
                }
            }
            if (!ok) break;

            if (p.scatter_ranks > 0) {
                // fp32 accumulators, 32 rows x 32 columns per box (128-byte rows, 128-byte swizzle: the same staging
                // block as a 32 x 64 bf16 box), to the output matrix of the rank that owns these rows.
                int tile_again = tile, mb2, nb2;
                asm volatile("" : "+r"(tile_again));
                tile_coords(rotate_tile(tile_again, p.tile_rot, num_tiles), p.tiles_m, p.tiles_n, mb2, nb2, p.group_m);
                const int row0 = mb2 * kTileM + static_cast<int>(rank) * kBM + quarter * 32;
                if (row0 < p.M) {
                    const int owner = row0 / p.scatter_rows;   // warp-uniform; a 32-row block has one owner (R % 32 == 0)
                    const int dst_row0 = p.scatter_me * p.scatter_rows + (row0 - owner * p.scatter_rows);
                    const uint32_t stg = ((smem_u32(smem_raw) + 1023u) & ~1023u) + STAGES * kStageBytes + (warp - 4) * kStoreBytes;
#pragma unroll
                    for (int b = 0; b < CW / 32; ++b) {
                        const int col0 = nb2 * BN + cg * kSegStrideCg + (b / (SEGW / 32)) * kSegStrideH + (b % (SEGW / 32)) * 32;
                        if (col0 >= p.N) continue;  // warp-uniform
                        if (lane == 0) tma_store_wait_read<0>();
                        __syncwarp();
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const int cq = q ^ (lane & 7);
                            const int a0 = b * 16 + 2 * q;
                            asm volatile("st.shared.v2.b64 [%0], {%1, %2};" ::"r"(stg + lane * 128 + cq * 16), "l"(acc[a0]), "l"(acc[a0 + 1])
                                         : "memory");
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                             reinterpret_cast<uint64_t>(&outs.m[owner])),
                                         "r"(stg), "r"(col0), "r"(dst_row0)
                                         : "memory");
                            tma_store_commit();
                        }
                    }
                }
            } else if (p.tma_store) {
                // Blocks of 32 rows x STORE_W columns through swizzled shared memory and TMA stores (rows >= M and
                // columns beyond the tensor map are clipped by the hardware).  The tile's coordinates are derived
                // again from an opaque copy of the tile index so that they do not occupy registers across the
                // promotion loop.
                int tile_again = tile, mb2, nb2;
                asm volatile("" : "+r"(tile_again));
                tile_coords(rotate_tile(tile_again, p.tile_rot, num_tiles), p.tiles_m, p.tiles_n, mb2, nb2, p.group_m);
                const int row0 = mb2 * kTileM + static_cast<int>(rank) * kBM + quarter * 32;
                if (row0 < p.M) {
                    const uint32_t stg = ((smem_u32(smem_raw) + 1023u) & ~1023u) + STAGES * kStageBytes + (warp - 4) * kStoreBytes;
#pragma unroll
                    for (int b = 0; b < CW / STORE_W; ++b) {
                        // box b: segment b / (SEGW / STORE_W), box b % (SEGW / STORE_W) inside it
                        const int col0 = nb2 * BN + cg * kSegStrideCg + (b / (SEGW / STORE_W)) * kSegStrideH + (b % (SEGW / STORE_W)) * STORE_W;
                        if (col0 >= p.N) continue;  // warp-uniform
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
                                             "r"(stg), "r"(p.out_col0 + col0), "r"(row0)
                                             : "memory");
                            tma_store_commit();
                        }
                    }
                }
            } else if (p.out_f32) {
                if (row_ok) {
#pragma unroll
                    for (int h = 0; h < SPLIT; ++h) {
                        const int c0 = col_base + h * kSegStrideH;
                        if (c0 >= p.N) continue;
                        float* dst = static_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo + c0;
                        const uint64_t* a = acc + h * (SEGW / 2);
                        if (c0 + SEGW <= p.N && p.vec_ok) {
#pragma unroll
                            for (int j = 0; j < SEGW / 2; j += 2)
                                *reinterpret_cast<ulonglong2*>(dst + 2 * j) = make_ulonglong2(a[j], a[j + 1]);
                        } else {
#pragma unroll
                            for (int j = 0; j < SEGW / 2; ++j) {
                                float lo, hi;
                                unpack_f32x2(a[j], lo, hi);
                                if (c0 + 2 * j < p.N) dst[2 * j] = lo;
                                if (c0 + 2 * j + 1 < p.N) dst[2 * j + 1] = hi;
                            }
                        }
                    }
                }
            } else if (row_ok) {
#pragma unroll
                for (int h = 0; h < SPLIT; ++h) {
                    const int c0 = col_base + h * kSegStrideH;
                    if (c0 >= p.N) continue;
                    uint16_t* dst = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + c0;
                    const uint64_t* a = acc + h * (SEGW / 2);
                    if (c0 + SEGW <= p.N && p.vec_ok) {
#pragma unroll
                        for (int j = 0; j < SEGW / 2; j += 4)
                            *reinterpret_cast<uint4*>(dst + 2 * j) = make_uint4(pack_bf16x2_of(a[j]), pack_bf16x2_of(a[j + 1]),
                                                                                pack_bf16x2_of(a[j + 2]), pack_bf16x2_of(a[j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < SEGW / 2; ++j) {
                            float lo, hi;
                            unpack_f32x2(a[j], lo, hi);
                            if (c0 + 2 * j < p.N) dst[2 * j] = to_bf16_bits(lo);
                            if (c0 + 2 * j + 1 < p.N) dst[2 * j + 1] = to_bf16_bits(hi);
                        }
                    }
                }
            }
            __syncwarp();
        }
        if (lane == 0) tma_store_wait_all<0>();  // stores read this CTA's shared memory: finish before exit
    }

    tcgen05_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // neither CTA leaves while the other may still read or signal it
    if (warp == 2) {
        __syncwarp();
        tcgen05_fence_after_sync();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
        else tmem_dealloc(tmem_base, kTmemCols);
    }
    if (p.pdl_role == 2 && threadIdx.x == 0) pdl_wait();  // this grid ends only after the launch before it has ended
}

}  // namespace gi8
