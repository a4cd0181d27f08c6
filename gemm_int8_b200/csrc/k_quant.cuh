// Activation quantisers: the step that feeds the W8A8 GEMMs.  The reference ships none (its benchmark only rounds
// and clamps, benchmark.py:17-18); these follow the package's torch quantisers bit for bit:
//     s = amax / 127  (s = 1 where the block is all zero),  q = clamp(rint(v / s), -127, 127)
// with IEEE division and round-half-even.  Both kernels are HBM-bound streams (5 bytes per fp32 element,
// 3 per bf16 element): every element is read once with 16-byte loads and written once.
#pragma once

#include <cuda_bf16.h>

#include "ptx.cuh"

namespace gi8 {

constexpr int kQuantThreads = 256;

GI8_DEVICE float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

GI8_DEVICE int quant_one(float v, float s)
{
    float t = rintf(__fdiv_rn(v, s));
    t = fminf(fmaxf(t, -127.0f), 127.0f);
    return static_cast<int>(t);
}

GI8_DEVICE uint32_t pack_i8x4(int a, int b, int c, int d)
{
    return (static_cast<uint32_t>(a) & 0xff) | ((static_cast<uint32_t>(b) & 0xff) << 8) |
           ((static_cast<uint32_t>(c) & 0xff) << 16) | ((static_cast<uint32_t>(d) & 0xff) << 24);
}

template <typename T>
GI8_DEVICE void load4(const T* p, bool ok, float (&v)[4]);

template <>
GI8_DEVICE void load4<float>(const float* p, bool ok, float (&v)[4])
{
    float4 f = ok ? __ldg(reinterpret_cast<const float4*>(p)) : make_float4(0.f, 0.f, 0.f, 0.f);
    v[0] = f.x, v[1] = f.y, v[2] = f.z, v[3] = f.w;
}

template <>
GI8_DEVICE void load4<__nv_bfloat16>(const __nv_bfloat16* p, bool ok, float (&v)[4])
{
    uint2 u = ok ? __ldg(reinterpret_cast<const uint2*>(p)) : make_uint2(0u, 0u);
    v[0] = __uint_as_float(u.x << 16), v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16), v[3] = __uint_as_float(u.y & 0xffff0000u);
}

// One warp per (row, 128-wide K block): lane l owns elements [4l, 4l + 4) of the block.
// a [M,K] (K % 4 == 0, rows 16-byte aligned) -> q int8 [M,K], s fp32 [M, ceil(K/128)].
template <typename T>
__global__ void __launch_bounds__(kQuantThreads)
quantize_token_block_kernel(const T* __restrict__ a, int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int K,
                            int KB)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = static_cast<int64_t>(gridDim.x) * (kQuantThreads / 32);
    const int64_t blocks_total = M * KB;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * (kQuantThreads / 32) + (threadIdx.x >> 5); b < blocks_total;
         b += warps_total) {
        const int64_t row = b / KB;
        const int kb = static_cast<int>(b - row * KB);
        const int col = kb * 128 + lane * 4;
        const bool ok = col < K;
        float v[4];
        load4<T>(a + row * K + col, ok, v);
        const float amax = warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
        const float sc = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
        if (lane == 0) s[row * KB + kb] = sc;
        if (ok)
            *reinterpret_cast<uint32_t*>(q + row * K + col) =
                pack_i8x4(quant_one(v[0], sc), quant_one(v[1], sc), quant_one(v[2], sc), quant_one(v[3], sc));
    }
}

// One CTA per row: per-token scale over the whole row (decode shapes).  The row is read twice (the second
// read hits L1/L2), keeping register use independent of K.
template <typename T>
__global__ void __launch_bounds__(kQuantThreads)
quantize_token_row_kernel(const T* __restrict__ a, int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int K)
{
    __shared__ float warp_amax[kQuantThreads / 32];
    __shared__ float row_scale;
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
        const T* src = a + row * K;
        float amax = 0.0f;
        for (int col = threadIdx.x * 4; col < K; col += kQuantThreads * 4) {
            float v[4];
            load4<T>(src + col, true, v);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
        }
        amax = warp_max(amax);
        if ((threadIdx.x & 31) == 0) warp_amax[threadIdx.x >> 5] = amax;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = 0.0f;
            for (int w = 0; w < kQuantThreads / 32; ++w) m = fmaxf(m, warp_amax[w]);
            const float sc = m > 0.0f ? __fdiv_rn(m, 127.0f) : 1.0f;
            row_scale = sc;
            s[row] = sc;
        }
        __syncthreads();
        const float sc = row_scale;
        for (int col = threadIdx.x * 4; col < K; col += kQuantThreads * 4) {
            float v[4];
            load4<T>(src + col, true, v);
            *reinterpret_cast<uint32_t*>(q + row * K + col) =
                pack_i8x4(quant_one(v[0], sc), quant_one(v[1], sc), quant_one(v[2], sc), quant_one(v[3], sc));
        }
        __syncthreads();
    }
}

}  // namespace gi8
