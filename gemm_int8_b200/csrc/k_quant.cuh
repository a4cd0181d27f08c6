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

// q = clamp(rint(v / s)) with the IEEE quotient, at the price of a multiplication for all but one element in
// several thousand: v * (1/s) is within 2^-16 of the correctly rounded quotient (|v / s| <= 127), so rounding it
// gives the same integer unless it lies within 2^-14 of a half-integer -- only then is the division carried out.
// `fast` is false for blocks whose scale is so small or large that 1/s overflows or loses accuracy.
struct QuantScale {
    float s, r;
    bool fast;
};

GI8_DEVICE QuantScale make_quant_scale(float amax)
{
    QuantScale qs;
    qs.s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    qs.fast = qs.s > 1e-30f && qs.s < 1e30f;
    qs.r = __fdiv_rn(1.0f, qs.s);
    return qs;
}

// The exact rule for one element.
GI8_DEVICE int quant_exact(float v, float s)
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

// Four elements -> four packed int8.  Fast path, full-rate instructions only: t0 = v * (1/s); adding 1.5 * 2^23
// rounds t0 to the nearest-even integer n in the low mantissa bits, whose low byte is the int8 result; subtracting
// the constant again gives n as a float for the half-integer test.  |n| <= 127 because |v| <= amax, so no clamp.
GI8_DEVICE uint32_t quant_pack4(float v0, float v1, float v2, float v3, const QuantScale& qs)
{
    constexpr float kMagic = 12582912.0f;
    const float t0 = v0 * qs.r, t1 = v1 * qs.r, t2 = v2 * qs.r, t3 = v3 * qs.r;
    const float u0 = t0 + kMagic, u1 = t1 + kMagic, u2 = t2 + kMagic, u3 = t3 + kMagic;
    // safe: each quotient is farther than 2^-14 from a half-integer (the comparisons are false for NaN)
    const bool safe = qs.fast && fabsf(t0 - (u0 - kMagic)) <= 0.49993f && fabsf(t1 - (u1 - kMagic)) <= 0.49993f &&
                      fabsf(t2 - (u2 - kMagic)) <= 0.49993f && fabsf(t3 - (u3 - kMagic)) <= 0.49993f;
    if (safe) {
        const uint32_t lo = __byte_perm(__float_as_uint(u0), __float_as_uint(u1), 0x0040);
        const uint32_t hi = __byte_perm(__float_as_uint(u2), __float_as_uint(u3), 0x0040);
        return __byte_perm(lo, hi, 0x5410);
    }
    return pack_i8x4(quant_exact(v0, qs.s), quant_exact(v1, qs.s), quant_exact(v2, qs.s), quant_exact(v3, qs.s));
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

// 16-byte loads: lane l of a group of LPB = 128 / EPL lanes owns EPL = 16 / sizeof(T) consecutive elements of one
// 128-wide K block, a warp covers 32 / LPB blocks per load, and kQuantUnroll loads are issued before the first is
// used so that enough bytes are in flight to cover the DRAM latency (one block per warp at a time reached a
// quarter of the copy bandwidth; four loads per lane, held as fp32, 0.55 of it on bf16 input).  The loaded 16 bytes
// stay in registers as they came (four registers per load whatever the type) and are unpacked at their use: a byte in
// flight costs a register byte, and bf16 unpacked to fp32 before the wait had cost two.  fp32 input, which is bound by
// the memory system, takes eight loads per lane (0.76-0.78 -> 0.84-0.86 of the copy bandwidth); bf16 input, which is bound
// by instruction issue (about eighteen instructions per element), four (eight measured 3 % slower).
// a [M,K] (K % EPL == 0, rows 16-byte aligned) -> q int8 [M,K], s fp32 [M, ceil(K/128)].
constexpr int kQuantBlocksPerItem = 8;  // 128-wide blocks per warp and iteration, whatever the type (1 x 8 or 2 x 4)

template <typename T>
GI8_DEVICE void unpack16(const uint4& u, float (&v)[16 / sizeof(T)]);

template <>
GI8_DEVICE void unpack16<float>(const uint4& u, float (&v)[4])
{
    v[0] = __uint_as_float(u.x), v[1] = __uint_as_float(u.y), v[2] = __uint_as_float(u.z), v[3] = __uint_as_float(u.w);
}

template <>
GI8_DEVICE void unpack16<__nv_bfloat16>(const uint4& u, float (&v)[8])
{
    v[0] = __uint_as_float(u.x << 16), v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16), v[3] = __uint_as_float(u.y & 0xffff0000u);
    v[4] = __uint_as_float(u.z << 16), v[5] = __uint_as_float(u.z & 0xffff0000u);
    v[6] = __uint_as_float(u.w << 16), v[7] = __uint_as_float(u.w & 0xffff0000u);
}

// Residency: four CTAs per SM for fp32 input (64 registers; five measured 0.84 -> 0.75 of the copy bandwidth), five for
// bf16 input (48 registers with a few spilled bytes; 0.58 -> 0.62: more warps to cover its longer instruction chains).
template <typename T>
__global__ void __launch_bounds__(kQuantThreads, sizeof(T) == 4 ? 4 : 5)
quantize_token_block_kernel(const T* __restrict__ a, int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int K,
                            int KB)
{
    constexpr int EPL = 16 / sizeof(T);   // elements per lane and load
    constexpr int LPB = 128 / EPL;        // lanes per 128-wide block
    constexpr int BPL = 32 / LPB;         // blocks per warp and load
    constexpr int kQuantUnroll = sizeof(T) == 4 ? 8 : 4;  // 16-byte loads per lane in flight
    constexpr int BPI = BPL * kQuantUnroll;  // blocks per warp and iteration
    static_assert(BPI == kQuantBlocksPerItem, "the host sizes the grid by this");
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPB, ll = lane % LPB;
    // Work item = BPI consecutive blocks of one row (one 32-bit division per item instead of one 64-bit division
    // per block: the index arithmetic, not the memory system, bounded the first version of this kernel).
    const uint32_t groups = static_cast<uint32_t>((KB + BPI - 1) / BPI);
    const uint32_t warps_total = gridDim.x * (kQuantThreads / 32);
    const uint32_t items_total = static_cast<uint32_t>(M) * groups;  // the host checks that this fits
    for (uint32_t item = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); item < items_total; item += warps_total) {
        const uint32_t row = item / groups;
        const int kb0 = static_cast<int>(item - row * groups) * BPI + sub;   // this lane's block of load 0
        const int col0 = kb0 * 128 + ll * EPL;                               // load u: BPL blocks further per u
        const int64_t off0 = static_cast<int64_t>(row) * K + col0;
        uint4 raw[kQuantUnroll];
#pragma unroll
        for (int u = 0; u < kQuantUnroll; ++u) {
            const bool ok = col0 + u * (BPL * 128) < K;   // also false for blocks past the end of the row
            raw[u] = ok ? __ldg(reinterpret_cast<const uint4*>(a + (off0 + u * (BPL * 128)))) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < kQuantUnroll; ++u) {
            float v[EPL];
            unpack16<T>(raw[u], v);
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < EPL; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
            for (int o = LPB / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const QuantScale sc = make_quant_scale(amax);
            const int kb = kb0 + u * BPL;
            if (ll == 0 && kb < KB) s[static_cast<int64_t>(row) * KB + kb] = sc.s;
            if (col0 + u * (BPL * 128) < K) {
                uint32_t w[EPL / 4];
#pragma unroll
                for (int j = 0; j < EPL; j += 4) w[j / 4] = quant_pack4(v[j], v[j + 1], v[j + 2], v[j + 3], sc);
                int8_t* dst = q + (off0 + u * (BPL * 128));
                if constexpr (EPL == 8) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
                else *reinterpret_cast<uint32_t*>(dst) = w[0];
            }
        }
    }
}

// One CTA per row: per-token scale over the whole row (decode shapes).  The row is read twice (the second
// read hits L1/L2), keeping register use independent of K.
template <typename T>
__global__ void __launch_bounds__(kQuantThreads)
quantize_token_row_kernel(const T* __restrict__ a, int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int K)
{
    __shared__ float warp_amax[kQuantThreads / 32];
    __shared__ float row_amax;
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
            row_amax = m;
            s[row] = sc;
        }
        __syncthreads();
        const QuantScale sc = make_quant_scale(row_amax);
        for (int col = threadIdx.x * 4; col < K; col += kQuantThreads * 4) {
            float v[4];
            load4<T>(src + col, true, v);
            *reinterpret_cast<uint32_t*>(q + row * K + col) =
                quant_pack4(v[0], v[1], v[2], v[3], sc);
        }
        __syncthreads();
    }
}

// Walsh-Hadamard rotation along K in blocks of H (a power of two, 128 <= H <= 16384, H | K) fused with the
// per-token per-128-block quantiser: out = quantise( FWHT_H(row block) * H^-1/2 ).
// The transform is the textbook in-place butterfly, strides h = 1, 2, 4, ... ascending, (a, b) -> (a + b, a - b):
// every output of a stage is ONE fp32 add or subtract of two outputs of the stage before, so the result does not
// depend on which thread computes it and equals a sequential CPU loop bit for bit.
// One CTA of min(256, H / 4) threads per (row, H block); thread t owns elements [t * E, t * E + E), E = H / threads:
// strides below E run in registers, strides E .. 16 E between the lanes of a warp (shuffles), the remaining ones
// (at most three: eight warps) through shared memory.  HBM traffic is that of the plain quantiser; the arithmetic
// is K * log2(H) adds per row, of the order of the memory time on B200.
template <typename T, int E>
__global__ void __launch_bounds__(kQuantThreads)
hadamard_quantize_token_block_kernel(const T* __restrict__ a, int8_t* __restrict__ q, float* __restrict__ s, int K, int KB,
                                     int H, float norm)
{
    extern __shared__ float had_smem[];  // H floats when the CTA has more than one warp
    const int t = threadIdx.x;
    const int lane = t & 31;
    const int hb_per_row = K / H;
    const int64_t row = blockIdx.x / hb_per_row;
    const int hb = blockIdx.x - static_cast<int>(row) * hb_per_row;
    const int col0 = hb * H + t * E;
    float v[E];
#pragma unroll
    for (int j = 0; j < E; j += 4) {
        float w[4];
        load4<T>(a + row * K + col0 + j, true, w);
        v[j] = w[0], v[j + 1] = w[1], v[j + 2] = w[2], v[j + 3] = w[3];
    }
    // strides 1 .. E/2: both elements of a pair in this thread
#pragma unroll
    for (int h = 1; h < E; h <<= 1) {
#pragma unroll
        for (int j = 0; j < E; ++j) {
            if ((j & h) == 0) {
                const float x0 = v[j], x1 = v[j + h];
                v[j] = x0 + x1;
                v[j + h] = x0 - x1;
            }
        }
    }
    // strides E .. 16 E: partner element in lane ^ m
    const int lanes = blockDim.x < 32 ? blockDim.x : 32;
    for (int m = 1; m < lanes; m <<= 1) {
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], m);
            v[j] = upper ? other - v[j] : v[j] + other;
        }
    }
    // strides 32 E ..: partner element in another warp
    for (int m = 32; m < static_cast<int>(blockDim.x); m <<= 1) {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < E; ++j) had_smem[j * blockDim.x + t] = v[j];  // [j][t]: conflict-free
        __syncthreads();
        const bool upper = (t & m) != 0;
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const float other = had_smem[j * blockDim.x + (t ^ m)];
            v[j] = upper ? other - v[j] : v[j] + other;
        }
    }
    // normalise, then the quantiser's rule on each 128-wide block (128 / E consecutive lanes)
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < E; ++j) {
        v[j] *= norm;
        amax = fmaxf(amax, fabsf(v[j]));
    }
#pragma unroll
    for (int o = 1; o < 128 / E; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const QuantScale sc = make_quant_scale(amax);
    if ((t * E) % 128 == 0) s[row * KB + col0 / 128] = sc.s;
    int8_t* dst = q + row * K + col0;
#pragma unroll
    for (int j = 0; j < E; j += 4)
        *reinterpret_cast<uint32_t*>(dst + j) =
            quant_pack4(v[j], v[j + 1], v[j + 2], v[j + 3], sc);
}

}  // namespace gi8
