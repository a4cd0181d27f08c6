// Weight-streaming kernel for the fewest tokens (M <= 8) of the per-token x per-channel entry point:
//   out[m,n] = bf16( fp32( sum_k x[m,k] * w[n,k] ) * (sx[m] * sw[n]) )
// At these sizes the work is reading N*K weight bytes once; arithmetic intensity is M MACs per byte.  This kernel
// does that without tensor memory, TMA, barriers or a cluster reduction, to find out whether the fixed 3-4 us the
// tensor-core small-M kernels spend above their HBM time is their set-up.  It is not: measured on B200 this kernel
// needs the same fixed time (6.0 vs 6.5 us at M = 1 on a 17 MB weight, slower from M = 2 on), so it is a selectable
// variant ("gemv") and not part of the automatic dispatch.
//   * one warp per output channel n: the K bytes of w[n,:] are read with 16-byte loads, 512 contiguous bytes per
//     warp and load, kGemvUnroll loads in flight per lane;
//   * the tokens (M*K bytes) sit in shared memory, read with 16-byte loads at the same k;
//   * dp4a (four int8 MACs into int32, exact) -- 4*M per 16 weight bytes and lane, far below the integer rate at
//     the byte rate HBM delivers;
//   * warp shuffle reduction, then the same epilogue arithmetic as the other kernels (scales multiplied first).
// Integer sums are exact in any order, so the result is bit-identical to that of the tensor-core kernels.
#pragma once

#include "ptx.cuh"

namespace gi8 {

constexpr int kGemvThreads = 256;
constexpr int kGemvUnroll = 4;

struct GemvParams {
    const int8_t* x;   // [M,K]
    const int8_t* w;   // [N,K]
    const float* sx;   // [M]
    const float* sw;   // [N]
    uint16_t* out;     // bf16 [M,N], leading dimension ldo
    int64_t ldo;
    int M, N, K;       // K % 16 == 0
};

GI8_DEVICE int dp4a_s8(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int MT>
__global__ void __launch_bounds__(kGemvThreads)
gemv_scaled_kernel(const GemvParams p)
{
    extern __shared__ uint4 gemv_x[];  // MT rows of K bytes, as 16-byte chunks
    const int chunks = p.K / 16;       // 16-byte chunks per row
    pdl_wait();
    // stage the tokens (rows >= M are zero)
    for (int i = threadIdx.x; i < MT * chunks; i += kGemvThreads) {
        const int m = i / chunks, c = i - m * chunks;
        gemv_x[i] = m < p.M ? __ldg(reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(m) * p.K) + c)
                            : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int warps = gridDim.x * (kGemvThreads / 32);
    for (int n = blockIdx.x * (kGemvThreads / 32) + (threadIdx.x >> 5); n < p.N; n += warps) {
        const uint4* wrow = reinterpret_cast<const uint4*>(p.w + static_cast<int64_t>(n) * p.K);
        int acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0;
        for (int c0 = 0; c0 < chunks; c0 += 32 * kGemvUnroll) {
            uint4 wv[kGemvUnroll];
#pragma unroll
            for (int u = 0; u < kGemvUnroll; ++u) {
                const int c = c0 + u * 32 + lane;
                wv[u] = c < chunks ? ld_nc_na(wrow + c) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < kGemvUnroll; ++u) {
                const int c = c0 + u * 32 + lane;
                if (c < chunks) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint4 xv = gemv_x[m * chunks + c];
                        acc[m] = dp4a_s8(wv[u].x, xv.x, acc[m]);
                        acc[m] = dp4a_s8(wv[u].y, xv.y, acc[m]);
                        acc[m] = dp4a_s8(wv[u].z, xv.z, acc[m]);
                        acc[m] = dp4a_s8(wv[u].w, xv.w, acc[m]);
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
        }
        const float cs = __ldg(p.sw + n);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (lane == m && m < p.M) {
                const float f = __int2float_rn(acc[m]) * (__ldg(p.sx + m) * cs);
                p.out[static_cast<int64_t>(m) * p.ldo + n] = to_bf16_bits(f);
            }
        }
    }
}

}  // namespace gi8
