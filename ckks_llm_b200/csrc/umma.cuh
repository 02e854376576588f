// Thin wrappers over the sm_100a PTX used by the tensor-core kernels: mbarriers with bounded
// waits, bulk asynchronous copies, tensor-memory management, tcgen05.mma (kind::i8) and its
// shared-memory and instruction descriptors.
#pragma once
#include "common.cuh"

namespace ckb {
namespace umma {

constexpr int TM = 128;            // rows of the M-side operand per instruction (UMMA M)
constexpr long long WAIT_BUDGET = 4000000000ll;   // default clock budget of a device-side wait, about two seconds

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the budget (clock cycles) ran out (flags[1] receives `where` and stays
// set until the host reads and clears it) or when another role of the CTA has given up (abort is the CTA's
// shared flag, looked at from the slow path only).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* flags, int where, const int* abort,
                                          long long budget = WAIT_BUDGET) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63) == 0) {
            if (*(const volatile int*)abort) return false;
            if (clock64() - t0 > budget) {
                atomicCAS(&flags[1], 0, where);      // the first site to give up is the one reported
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
// Shared memory -> global memory bulk copy (16-byte aligned addresses, size a multiple of 16), tracked by the
// issuing thread's bulk groups.  The source must have been made visible to the asynchronous proxy first.
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until the sources of this thread's bulk groups have been read (the shared memory may be rewritten)
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// until this thread's bulk groups are complete (the destinations are written)
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 B,
// 128 B from one K half to the next (leading offset), 256 B from one 8-row group to the
// next (stride offset), descriptor version 1.
// Shared-memory addresses are below 2^18, so the 14-bit address field is addr >> 4 and a byte
// offset inside the stage is added to the low word as offset >> 4 without touching the rest.
constexpr uint32_t DESC_LO = (uint32_t)(128 >> 4) << 16;                    // leading offset
constexpr uint32_t DESC_HI = (uint32_t)(256 >> 4) | (1u << (46 - 32));      // stride offset, version
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr16) {            // addr16 = shared address >> 4
    return ((uint64_t)DESC_HI << 32) | (uint64_t)(DESC_LO + addr16);
}
// Instruction descriptor: s32 accumulate, A signed or unsigned 8-bit, B unsigned 8-bit,
// both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool a_signed) {
    return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
}


}  // namespace umma
}  // namespace ckb
