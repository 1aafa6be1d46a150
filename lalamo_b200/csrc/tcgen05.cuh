// What the kernels on the fifth-generation tensor cores share: transaction barriers with bounded
// waits, TMA tile loads and bulk stores, shared-memory and instruction descriptors, tcgen05.mma and
// its commit, tensor-memory loads, and the driver's tensor-map encoder looked up at run time.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace lb {

constexpr unsigned long long kTcWaitNanoseconds = 2000000000ull;   // how long a wait on a barrier lasts before it gives up

__device__ __forceinline__ uint32_t smem_address(const void* pointer) { return static_cast<uint32_t>(__cvta_generic_to_shared(pointer)); }

__device__ __forceinline__ void barrier_init(uint64_t* barrier, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(barrier)), "r"(count) : "memory");
}
__device__ __forceinline__ void barrier_expect(uint64_t* barrier, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(barrier)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool barrier_test(uint64_t* barrier, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_address(barrier)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ unsigned long long nanoseconds_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for the phase with the given parity to complete; false if kTcWaitNanoseconds ran out.  Polls
// (a parked try_wait wakes later than a poll sees the phase: 1 us per product in the decode step),
// with a short sleep between polls once the wait has lasted a while.
__device__ __forceinline__ bool barrier_wait(uint64_t* barrier, uint32_t parity, unsigned long long limit = kTcWaitNanoseconds) {
    for (int spin = 0; spin < 64; ++spin)
        if (barrier_test(barrier, parity)) return true;
    const unsigned long long start = nanoseconds_now();
    for (;;) {
        for (int spin = 0; spin < 64; ++spin) {
            if (barrier_test(barrier, parity)) return true;
            __nanosleep(32);
        }
        if (nanoseconds_now() - start > limit) return false;
    }
}

// The same without sleeping between polls, for waits on the critical path of a short loop (the
// sleep overshoots by a good part of a microsecond).
__device__ __forceinline__ bool barrier_wait_busy(uint64_t* barrier, uint32_t parity) {
    for (int spin = 0; spin < 64; ++spin)
        if (barrier_test(barrier, parity)) return true;
    const unsigned long long start = nanoseconds_now();
    for (;;) {
        for (int spin = 0; spin < 256; ++spin)
            if (barrier_test(barrier, parity)) return true;
        if (nanoseconds_now() - start > kTcWaitNanoseconds) return false;
    }
}

// The same with the thread parked in hardware between looks (mbarrier.try_wait): it wakes a little
// later than a poll would see the phase, but takes no issue slots meanwhile; for a thread that does
// nothing but wait beside warps that compute on the same scheduler.
__device__ __forceinline__ bool barrier_wait_parked(uint64_t* barrier, uint32_t parity) {
    if (barrier_test(barrier, parity)) return true;
    const unsigned long long start = nanoseconds_now();
    for (;;) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_address(barrier)), "r"(parity), "r"(100000u)
            : "memory");
        if (done) return true;
        if (nanoseconds_now() - start > kTcWaitNanoseconds) return false;
    }
}

__device__ __forceinline__ void tma_load_2d(void* destination, const CUtensorMap* map, int x, int y, uint64_t* barrier) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_address(destination)), "l"(map), "r"(smem_address(barrier)), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, groups
// of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t tile_descriptor(const void* tile) {
    const uint64_t address = smem_address(tile);
    return ((address & 0x3FFFFull) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

template <int BN>
__device__ __forceinline__ constexpr uint32_t instruction_descriptor() {
    // D float32, A and B bfloat16, both K-major, N = BN, M = 128.
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* barrier) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_address(barrier)) : "memory");
}

// 32 consecutive columns of this thread's lane of tensor memory.
__device__ __forceinline__ void tmem_load_32(uint32_t address, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
        "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(address)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 16 consecutive columns of this thread's lane of tensor memory.
__device__ __forceinline__ void tmem_load_16(uint32_t address, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(address)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// A box of shared memory (rows of the box contiguous) to the tensor at (x, y); what lies outside the
// tensor is not written.  `add` sums into the tensor instead (float32 there: the residual stream).
__device__ __forceinline__ void bulk_store_2d(const CUtensorMap* map, const void* source, int x, int y, bool add) {
    if (add) {
        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_address(source)),
                     "r"(x), "r"(y)
                     : "memory");
    } else {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_address(source)), "r"(x), "r"(y)
                     : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// The same into a tensor of three dimensions (never added).
__device__ __forceinline__ void bulk_store_3d(const CUtensorMap* map, const void* source, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(smem_address(source)), "r"(x), "r"(y), "r"(z)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ __forceinline__ void named_barrier(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

__device__ __forceinline__ void barrier_arrive(uint64_t* barrier) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(barrier)) : "memory");
}

// ---- two CTAs of a cluster on one tile (cta_group::2): the even CTA of the pair issues the products,
// which read both CTAs' shared memory and write both CTAs' tensor memory.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}
// The address, in the cluster's shared window, of the CTA `rank`'s copy of a shared variable of this CTA.
__device__ __forceinline__ uint32_t cluster_address(const void* local, uint32_t rank) {
    uint32_t address;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(address) : "r"(smem_address(local)), "r"(rank));
    return address;
}
// Every thread of every CTA of the cluster.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void barrier_arrive_cluster(uint32_t cluster_barrier) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_barrier) : "memory");
}
// A tile into this CTA's shared memory whose bytes count on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* destination, const CUtensorMap* map, int x, int y, uint32_t cluster_barrier) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_address(destination)), "l"(map), "r"(cluster_barrier), "r"(x), "r"(y)
        : "memory");
}
// D float32 [256, BN] over the pair (128 rows in each CTA's tensor memory), A [256, 16] and B [BN, 16]
// bfloat16, K-major: each CTA holds its 128 rows of A and its BN / 2 rows of B at the same shared offsets.
template <int BN>
__device__ __forceinline__ constexpr uint32_t instruction_descriptor_pair() {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
}
__device__ __forceinline__ void mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(0u)
        : "memory");
}
// Arrives, once the products issued so far are done, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void mma_commit_pair(uint64_t* barrier) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_address(barrier)),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}

}  // namespace lb

namespace lb {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
    static EncodeTiled function = nullptr;
    if (function == nullptr) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) == cudaSuccess && result == cudaDriverEntryPointSuccess)
            function = reinterpret_cast<EncodeTiled>(entry);
    }
    return function;
}

}  // namespace lb
