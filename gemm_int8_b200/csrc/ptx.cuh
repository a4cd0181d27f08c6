// Inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA tensor copies,
// tensor memory (TMEM) management, tcgen05.mma (kind::i8) and tcgen05.ld.
// Every wait in this file is bounded: it gives up after a wall-clock limit and reports failure
// so that the calling kernel can record an error and drain instead of hanging the GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gi8 {

#define GI8_DEVICE __device__ __forceinline__

// ---------------------------------------------------------------------------------------------
// misc
// ---------------------------------------------------------------------------------------------
GI8_DEVICE uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

GI8_DEVICE uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// One lane of a fully converged warp is elected.
GI8_DEVICE bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may
// start while the previous kernel in the stream is still draining; every thread must pass pdl_wait() before it
// touches global memory that an earlier kernel may have written (or overwrites memory an earlier kernel reads).
// pdl_launch_dependents() tells the runtime that the NEXT kernel's CTAs may be scheduled as SMs free up.
GI8_DEVICE void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
GI8_DEVICE void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
GI8_DEVICE void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}


// Makes mbarrier initialisation visible to the async proxy (TMA, tcgen05.commit).
GI8_DEVICE void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// Orders generic-proxy shared-memory writes before later async-proxy (TMA store) reads.
GI8_DEVICE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

GI8_DEVICE void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One elected lane of the (converged) warp arrives; predicated, so no branch.  `bar_addr` is a shared-memory address.
GI8_DEVICE void mbar_arrive_elected_addr(uint32_t bar_addr)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t"
        "}\n" ::"r"(bar_addr)
        : "memory");
}

GI8_DEVICE void mbar_arrive_expect_tx(uint64_t* bar, uint32_t tx_bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(tx_bytes)
                 : "memory");
}

// `bar_addr` is a shared-memory address.
GI8_DEVICE bool mbar_try_wait_addr(uint32_t bar_addr, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar_addr), "r"(parity)
        : "memory");
    return ok != 0;
}

GI8_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) { return mbar_try_wait_addr(smem_u32(bar), parity); }

// Non-blocking test of the phase with the given parity (try_wait may suspend the thread for a while).
GI8_DEVICE bool mbar_test_wait_addr(uint32_t bar_addr, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar_addr), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wall-clock limit of one wait.  Generous against any legitimate stall (a whole kernel takes
// milliseconds), short enough that a protocol bug ends the kernel instead of hanging the GPU.
#ifndef GI8_WAIT_LIMIT_NS
#define GI8_WAIT_LIMIT_NS 250000000ull
#endif

// Bounded wait for the phase with the given parity to complete.  Returns false on timeout.
GI8_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > GI8_WAIT_LIMIT_NS) return false;
    }
}

// ---------------------------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), 2-D tiles, no multicast
// ---------------------------------------------------------------------------------------------
GI8_DEVICE void prefetch_tensormap(const CUtensorMap* m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// global -> shared tile load; completion is signalled as transaction bytes on `bar`.
// c0 is the innermost (contiguous) coordinate and must keep c0 * elemsize a multiple of 16 bytes.
GI8_DEVICE void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

GI8_DEVICE void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1,
                                 uint64_t cache_policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "l"(cache_policy)
        : "memory");
}

// shared -> global tile store (bulk async-group completion).  Never issued at a negative coordinate.
GI8_DEVICE void tma_store_2d(const CUtensorMap* map, const void* smem_src, int32_t c0, int32_t c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
                 : "memory");
}

GI8_DEVICE void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until at most N of this thread's store groups still READ their shared-memory source.
template <int N>
GI8_DEVICE void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Waits until at most N of this thread's store groups are incomplete (writes performed).
template <int N>
GI8_DEVICE void tma_store_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

GI8_DEVICE uint64_t l2_policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

GI8_DEVICE uint64_t l2_policy_evict_last()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ---------------------------------------------------------------------------------------------
// Tensor memory (TMEM)
// ---------------------------------------------------------------------------------------------
// Whole-warp calls.  ncols is a power of two in [32, 512].  The base address (lane 0, first
// column) is written to *smem_result.
GI8_DEVICE void tmem_alloc(uint32_t* smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}

GI8_DEVICE void tmem_relinquish_alloc_permit()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

GI8_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

GI8_DEVICE void tcgen05_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
GI8_DEVICE void tcgen05_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// tcgen05.mma, kind::i8 (int8 x int8 -> int32 in TMEM), operands from shared memory
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B produces when the box is
// 128 bytes wide).  Fields: start address >> 4 [0,14); leading byte offset >> 4 [16,30) (unused
// for swizzled K-major, set to 1); stride byte offset >> 4 [32,46) = distance between groups of
// eight rows = 1024 bytes; descriptor version 1 [46,48); layout type 2 = SWIZZLE_128B [61,64).
// The tile base must be 1024-byte aligned; stepping along K inside the 128-byte row is done by
// adding the byte offset (>> 4) to the start-address field.
GI8_DEVICE uint64_t make_smem_desc_k128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor for kind::i8: D = int32 (format 2 at bits [4,6)), A and B signed 8-bit
// (1 at bits [7,10) and [10,13)), both K-major (bits 15, 16 clear), N >> 3 at [17,23),
// M >> 4 at [24,29).  Bit 3 selects a saturating accumulator.
__host__ __device__ constexpr uint32_t make_idesc_i8(uint32_t m, uint32_t n, bool saturate)
{
    return (saturate ? (1u << 3) : 0u) | (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T.  Issued by ONE thread.  accumulate == 0 overwrites D.
GI8_DEVICE void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Makes `bar` receive one arrival when every tcgen05.mma issued so far by this thread has
// completed (implies tcgen05.fence::before_thread_sync).  Issued by ONE thread.
GI8_DEVICE void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05.ld: TMEM -> registers.  Shape 32x32b: thread t of the warp reads lane (base_lane + t);
// the warp may only touch the 32-lane quarter (warp_id % 4).  Register j holds column (col + j).
// ---------------------------------------------------------------------------------------------
GI8_DEVICE void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

GI8_DEVICE void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}


GI8_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// small numeric helpers
// ---------------------------------------------------------------------------------------------
// Two fp32 -> packed bf16x2 (lo in bits [0,16)), round to nearest even.
GI8_DEVICE uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}


GI8_DEVICE uint16_t to_bf16_bits(float f)
{
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
}

// ---------------------------------------------------------------------------------------------
// Thread-block clusters and two-CTA (cta_group::2) forms
// ---------------------------------------------------------------------------------------------
// Cluster barrier: a hardware barrier without a time limit -- every thread of every CTA of the cluster must reach
// it unconditionally.
GI8_DEVICE void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

GI8_DEVICE uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Address of `local_smem_addr` in the shared memory of cluster CTA `rank`.
GI8_DEVICE uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}

GI8_DEVICE void st_dsmem_u32(uint32_t cluster_addr, uint32_t v)
{
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}


GI8_DEVICE void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t leader_bar_cluster_addr, int32_t c0,
                                 int32_t c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}

GI8_DEVICE void umma_i8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One arrival on the barrier at cluster address `bar_cluster_addr` once all MMAs issued so far have completed.
GI8_DEVICE void umma_commit_pair(uint32_t bar_cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

// Arrival on a barrier in (possibly) another CTA of the cluster, default semantics (release at CTA scope): what orders
// the tensor-memory accesses around it is the tcgen05 fence the caller issues, and a cluster-scope release costs a
// cluster-wide memory fence per arrival.
GI8_DEVICE void mbar_arrive_cluster(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

GI8_DEVICE void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}

GI8_DEVICE void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }

GI8_DEVICE void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

}  // namespace gi8
