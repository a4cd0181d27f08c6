/*
 * C ABI of libgemm_int8_b200.so -- the B200 (sm_100a) INT8 GEMM library.
 *
 * This is the drop-in boundary for the reference project's native layer.  The reference binds its
 * Python operator to C++ symbols that take torch::Tensor and are linked against libtorch
 * (csrc/kernels/include/gemm.h:6-10, csrc/kernels/bindings.cpp:10-38).  Here the same work is exposed
 * as plain C entry points: raw device pointers, sizes, a CUDA stream handle, an int status.  The caller
 * owns every buffer (inputs, output, scratch); the library allocates no device memory, launches on the
 * stream it is given and never synchronises, except where a function says otherwise.
 *
 * Conventions
 *   x    int8  [M,K] row-major, contiguous         (reference operand A, bindings.cpp:10, gemm.cu:76-79)
 *   y    int8  [N,K] row-major, contiguous         (reference operand B, "column-major K x N", gemm.cu:80-83)
 *   out  bf16  [M,N] row-major, contiguous         (reference result C,  bindings.cpp:23, gemm.cu:85-88)
 *   stream  a cudaStream_t passed as void* (NULL = the legacy default stream, which is what the
 *           reference launches on, gemm.cu:118)
 *   Requirements: x, y 16-byte aligned and K % 16 == 0 (the reference's CUTLASS alignment, which it
 *   reports as "cutlass cannot implement", gemm.cu:107-110); out 2-byte aligned (16-byte aligned and
 *   N % 8 == 0 selects vector stores; the reference requires N % 8 == 0).  M, N, K >= 0; K < 131072.
 *   Every entry point returns GI8_OK or an error code; gi8_last_error() gives the message.
 */
#ifndef GEMM_INT8_B200_H_
#define GEMM_INT8_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum gi8_status {
    GI8_OK = 0,
    GI8_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, bad leading dimension */
    GI8_ERR_UNSUPPORTED_SHAPE = 2, /* K % 16 != 0, K too large, size beyond a stated limit */
    GI8_ERR_MISALIGNED = 3,        /* a pointer violates the alignment stated above */
    GI8_ERR_CUDA = 4,              /* a CUDA runtime/driver call failed (message has the detail) */
    GI8_ERR_UNSUPPORTED_DEVICE = 5, /* the current device is not compute capability 10.0 */
    GI8_ERR_WORKSPACE = 6,         /* scratch buffer missing or too small */
    GI8_ERR_DEVICE_TIMEOUT = 7     /* a kernel reported a bounded wait that expired (gi8_device_status) */
};

/* Library version, major * 10000 + minor * 100 + patch. */
int gi8_version(void);

/* Message of the most recent failing call on the calling thread (never NULL). */
const char* gi8_last_error(void);

/*
 * out = bf16( fp32(x @ y^T) * alpha ).
 * Replaces int8_matmul_host / int8_matmul<Tile,Warp,Stages> (csrc/kernels/gemm.cu:22-162) as called
 * from the torch op int8_matmul(Tensor A, Tensor B, float alpha) (csrc/kernels/bindings.cpp:10-26).
 */
int gi8_matmul(const int8_t* x, const int8_t* y, void* out_bf16, int64_t M, int64_t N, int64_t K, float alpha,
               void* stream);

/*
 * acc = x @ y^T as raw int32 [M,N] (the accumulator the reference keeps in registers before its
 * epilogue, csrc/kernels/gemm.cu:33-37).  For bit-exact verification; out_i32 must be 4-byte aligned.
 */
int gi8_matmul_i32(const int8_t* x, const int8_t* y, int32_t* out_i32, int64_t M, int64_t N, int64_t K,
                   void* stream);

/*
 * out[m,n] = bf16( fp32(acc[m,n]) * (sx[m] * sw[n]) ), sx fp32 [M] per-token, sw fp32 [N] per output
 * channel.  No counterpart in the reference (its epilogue takes one scalar, gemm.cu:96).
 * Small-M shapes (M <= 64) run a split-K weight-streaming kernel.  By default its K slices are reduced
 * inside a thread-block cluster and no scratch is needed (gi8_matmul_scaled_workspace_bytes returns 0).
 * The "smallm" variant reduces through global scratch instead: `workspace` must then hold at least
 * gi8_matmul_scaled_workspace_bytes(M,N,K) bytes, 16-byte aligned, AND BE ZERO-FILLED before the first
 * call; the kernel leaves it zero-filled again on completion, so one zeroed buffer can be reused by
 * successive calls on the same stream.  Pass NULL/0 when that function returns 0.
 */
int gi8_matmul_scaled(const int8_t* x, const int8_t* y, const float* sx, const float* sw, void* out_bf16,
                      int64_t M, int64_t N, int64_t K, void* workspace, int64_t workspace_bytes, void* stream);

int64_t gi8_matmul_scaled_workspace_bytes(int64_t M, int64_t N, int64_t K);

/*
 * Blockwise-dequantised W8A8 GEMM:
 *   out[m,n] = bf16( sum over kb (ascending) of  fp32(P[m,n,kb]) * (sa[m,kb] * sw[n/128,kb]) )
 * accumulated with one fused multiply-add per K block; P is the exact int32 dot product over K block
 * kb (128 wide).  sa fp32 [M, ceil(K/128)] with row stride ld_sa; sw fp32 [ceil(N/128), ceil(K/128)]
 * with row stride ld_sw (strides in elements).  No counterpart in the reference.
 */
int gi8_matmul_blockwise(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw,
                         int64_t ld_sw, void* out_bf16, int64_t M, int64_t N, int64_t K, void* stream);

/*
 * Allocation-free variant of gi8_matmul_scaled for small token counts (M <= 128), same arithmetic and result.
 * It has no counterpart in the reference.
 *
 * Who it is for: hosts that may not allocate device memory around this call -- a serving runtime that handed
 * all of HBM to its own pool at start-up (a cudaMalloc there fails or fragments the pool), a decode loop that
 * cannot afford the device-wide synchronisation cudaMalloc/cudaFree imply, or a plain C caller that has no
 * device allocator to make the scratch buffer gi8_matmul_scaled asks for.  Here the split-K scratch lives in
 * a fixed GI8_STATIC_SCRATCH_BYTES array inside the library's device image (every GPU that loads the library
 * holds those bytes until the process exits); the caller passes only inputs and outputs, and the call
 * performs no cudaMalloc, cudaFree or other allocating routine.
 *
 * Limits and rules
 *   - M must be in [1, 128]; the scratch the shape needs, ceil(N/128) * MT * 512 + 4 * ceil(N/128) bytes
 *     (MT = M rounded up to 16, 32, 64 or 128), must fit GI8_STATIC_SCRATCH_BYTES.  Larger shapes are
 *     refused with GI8_ERR_UNSUPPORTED_SHAPE and a message naming both numbers; nothing is launched.
 *   - The first call on each device looks up the array's device address (once, with that device current).
 *     Make that first call outside any stream capture.
 *   - Every call on a device shares the one array, and the array keeps whatever the previous call left:
 *     the part a call uses is cleared on `stream` before its kernel runs.  Two calls whose GPU work can
 *     overlap (different streams, or different host threads on different streams) race on it -- serialise
 *     them on one stream or with events.
 */
#define GI8_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int gi8_matmul_scaled_static(const int8_t* x, const int8_t* y, const float* sx, const float* sw, void* out_bf16,
                             int64_t M, int64_t N, int64_t K, void* stream);

/*
 * gi8_matmul_blockwise with the fp32 accumulators themselves as the result (out_f32 float [M,N] row-major, 4-byte
 * aligned): the value gi8_matmul_blockwise would round to bf16.  No reference counterpart (the reference's epilogue
 * always casts, csrc/kernels/gemm.cu:59-63).  Two uses: the bit-exact check of the accumulation order, and the
 * partial result of a K-sharded (row-parallel) GEMM, whose per-rank partials are summed across ranks before the cast.
 */
int gi8_matmul_blockwise_f32(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw,
                             int64_t ld_sw, float* out_f32, int64_t M, int64_t N, int64_t K, void* stream);

/*
 * K-sharded (row-parallel) form with the reduce-scatter's data movement fused into the epilogue (no reference
 * counterpart; the reference is single-GPU): this rank holds a K slice of x, y and both scale arrays, computes the fp32
 * accumulators of the whole [M, N] output over its slice, and stores rows [j R, (j + 1) R), R = M / n_ranks, straight
 * into recv[j] + my_rank * R * N -- recv[j] being rank j's receive area, float [n_ranks, R, N], the caller's own
 * memory for j == my_rank and mapped peer memory otherwise (gi8_peer_*).  Only unicast TMA stores cross the links.
 * After a barrier across the ranks each rank calls gi8_sum_parts_bf16 over its receive area.  Needs M a multiple of
 * 32 * n_ranks, N a multiple of 4, n_ranks <= 8.
 */
int gi8_matmul_blockwise_f32_scatter(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw,
                                     int64_t ld_sw, void* const* recv, int n_ranks, int my_rank, int64_t M, int64_t N,
                                     int64_t K, void* stream);

/*
 * out[i] = bf16( ((parts[0][i] + parts[1][i]) + parts[2][i]) + ... ) for i < count, parts[r] = parts + r * part_stride:
 * the second step of a K-sharded GEMM -- the ranks' fp32 partials of one output slice, summed in the order given
 * (so the result does not depend on which rank finished first) and cast once.  No reference counterpart.
 * n_parts <= 64.
 */
int gi8_sum_parts_bf16(const float* parts, int n_parts, int64_t part_stride, void* out_bf16, int64_t count, void* stream);

/*
 * N-sharded form of gi8_matmul_blockwise with the all-gather fused into the epilogue (no reference counterpart; the
 * reference is single-GPU).  This rank holds rows [col0, col0 + N) of the weight (y [N,K], sw [ceil(N/128), ...]) and
 * computes columns [col0, col0 + N) of the full [M, n_total] result; every output block (32 rows x 64 columns, or
 * 32 x 32, see below) is written by TMA store into ALL `n_outs` matrices `outs[i]` (bf16 [M, n_total], row-major,
 * 16-byte aligned): this rank's own and every peer's, the peers' through pointers that map their memory into this
 * process (gi8_peer_import, or any other peer mapping the host already has).  The transfer over NVLink overlaps the
 * GEMM tile by tile; there is no separate collective and no permuting copy.  After the call has completed on every
 * rank (a barrier the host provides), every matrix holds the full result.  col0 and N must be multiples of 32 (N may
 * be ragged only at the end of n_total), n_total a multiple of 8, n_outs <= 8.  Slices whose start and end are
 * multiples of 64 (or end at n_total) use the wide tiles and 128-byte store rows, which is what NVLink wants; other
 * slices take a 64-wide tile with 32 x 32 boxes so that no store reaches into a neighbour's columns.  A matrix may be
 * overwritten by a peer as soon as that peer starts its next call: the host must not start call i + 1 on any rank
 * before every rank has finished reading the result of call i.  Plain unicast stores only (no multicast).
 */
int gi8_matmul_blockwise_allgather(const int8_t* x, const int8_t* y, const float* sa, int64_t ld_sa, const float* sw,
                                   int64_t ld_sw, void* const* outs, int n_outs, int64_t M, int64_t N, int64_t K,
                                   int64_t n_total, int64_t col0, void* stream);

/*
 * Peer buffers for gi8_matmul_blockwise_allgather, for hosts without peer-memory plumbing of their own:
 *   gi8_peer_alloc / gi8_peer_free     a device allocation of its own (cudaMalloc), which an IPC handle can name
 *   gi8_peer_export                    writes the allocation's 64-byte CUDA IPC handle
 *   gi8_peer_import / gi8_peer_release maps / unmaps another process's allocation from its handle (peer access is
 *                                      enabled on first use)
 * These allocate and map memory: call them at set-up time, not per GEMM.
 */
int gi8_peer_alloc(void** ptr, int64_t bytes);
int gi8_peer_free(void* ptr);
int gi8_peer_export(void* ptr, void* handle64);
int gi8_peer_import(const void* handle64, void** ptr);
int gi8_peer_release(void* ptr);

/*
 * Activation quantisers that feed the W8A8 entry points (the reference ships none; its benchmark only rounds and
 * clamps, benchmark.py:17-18).  Rule: s = amax / 127 (s = 1 where the block is all zero),
 * q = clamp(round_half_even(v / s), -127, 127).  `in` is row-major [M,K], fp32 (in_dtype 0) or bf16 (in_dtype 1),
 * 16-byte aligned rows (K % 8 == 0 for bf16, K % 4 == 0 for fp32); q int8 [M,K] 8-byte aligned.
 *   gi8_quantize_token_block : one scale per row per 128-wide K block, scales fp32 [M, ceil(K/128)]
 *   gi8_quantize_token       : one scale per row, scales fp32 [M]
 */
int gi8_quantize_token_block(const void* in, int in_dtype, int8_t* q, float* scales, int64_t M, int64_t K, void* stream);
int gi8_quantize_token(const void* in, int in_dtype, int8_t* q, float* scales, int64_t M, int64_t K, void* stream);

/*
 * gi8_quantize_token_block preceded, in the same kernel, by a normalised Walsh-Hadamard rotation along K in blocks
 * of `had_block` elements (the rotation the reference's README names as its use case, README.md:10; the reference
 * has no code for it).  Transform: in-place butterflies with strides 1, 2, 4, ... ascending, (a, b) -> (a + b, a - b)
 * in fp32, then one multiplication by fp32(had_block^-1/2); then the quantiser's rule per 128-wide block.
 * had_block: a power of two in [128, 8192] that divides K.  Other arguments as gi8_quantize_token_block.
 */
int gi8_hadamard_quantize_token_block(const void* in, int in_dtype, int8_t* q, float* scales, int64_t M, int64_t K,
                                      int64_t had_block, void* stream);

/*
 * Forces a kernel variant for the calling process (tuning and tests); NULL or "" restores the fitted
 * per-shape dispatch that replaces the reference's shape table (csrc/kernels/gemm.cu:136-161).
 * Names: "dense_bn256", "dense_bn128", "dense_bn64" (tile width of the dense and of the blockwise kernel), "smallm"
 * (split-K through global scratch), "smallm_cluster" (split-K through distributed shared memory), "pair" (256 x 256
 * two-CTA tiles with tcgen05.mma.cta_group::2, dense and blockwise), "auto".  Returns
 * GI8_ERR_INVALID_ARGUMENT for an unknown name.
 */
int gi8_force_variant(const char* name);

/* Name of the variant the dispatch would pick for (kind, M, N, K); kind: 0 plain, 1 scaled, 2 blockwise (whose names
 * read "blockwise_bn256", "blockwise_bn128", "blockwise_bn64", "blockwise_pair", and "blockwise_bn256+columns_bnW" where
 * the columns of the thin last wave go to a second launch with W-wide tiles).  For the dense kernels "+splitkS"
 * after a form's name means that the tiles of its last wave go to the split-K kernel with S splits, and "splitkS" alone
 * that the whole grid does. */
const char* gi8_pick_variant(int kind, int64_t M, int64_t N, int64_t K);

/*
 * Reads and clears the current device's kernel status word.  SYNCHRONISES the device.  *code is 0 when
 * every kernel since the last call ran to completion, else the first recorded failure
 * (low byte: 1 producer, 2 MMA, 3 epilogue, 4 drain, 5 reduce wait expired; upper bits: CTA index).
 */
int gi8_device_status(uint32_t* code);

/*
 * gi8_device_status as a status code: GI8_OK, or GI8_ERR_DEVICE_TIMEOUT (with the role and CTA in gi8_last_error) when
 * a kernel since the last check gave up one of its bounded waits -- the counterpart of the exceptions the reference
 * throws on a failed launch (csrc/kernels/gemm.cu:108-121).  SYNCHRONISES the device and clears the word.
 */
int gi8_device_check(void);

/*
 * Launches a one-CTA kernel whose only job is to let a bounded wait run out (a 1 ms wait on a barrier nobody arrives
 * on), so that hosts and tests can see the whole error path -- status word, gi8_device_check, a context that stays
 * usable -- without a faulting or hanging kernel.  No reference counterpart.
 */
int gi8_selftest_wait_timeout(void* stream);

/*
 * The GEMM_INT8_* tuning variables (tile band height, TMA-store epilogue, programmatic dependent launch, K splits,
 * blockwise MMA shape and issuer count, GEMM_INT8_TAIL_SPLIT = 0 / 1 / 2: never / when the cost model says so / whenever
 * possible give a thin last wave of a tile grid to a second launch -- the split-K kernel for the dense entry points,
 * narrower tiles over the remaining columns for the blockwise one) are read once, when the library is first used; this
 * reads them again.
 * GEMM_INT8_STATIC_WEIGHTS=1 (default 0) is a promise rather than a tuning: the weight operand of gi8_matmul_scaled's
 * small-M path is not written by the work that directly precedes the call in its stream (weights quantised ahead of
 * time), so the kernel may request its first weight tiles while that work is still finishing.  Activations, scales
 * and the output are touched only after it has ended, whatever the setting.
 * No reference counterpart (its tuning is compile-time, CMakeLists.txt:49-51).
 */
int gi8_reload_env(void);

#ifdef __cplusplus
}
#endif

#endif /* GEMM_INT8_B200_H_ */
