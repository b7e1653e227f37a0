// PTX helpers of the tcgen05 (5th-generation tensor core) kernels: mbarriers with bounded
// waits, the commit that makes a batch of MMAs arrive on an mbarrier, the shared-memory matrix
// descriptor of a 128-byte-swizzled K-major tile, tensor-memory loads.
#pragma once

#include <cstdint>

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: false if the phase did not complete within the limit, or if another role of
// the CTA has already given up.  The verdict is WARP-UNIFORM: every lane polls until it either
// sees the phase or runs out of polls, then the warp votes, so that no lane can leave a loop
// that the rest of its warp stays in (the instructions that follow a wait - tcgen05.ld,
// __syncwarp, named barriers - need the whole warp).  Call it with all 32 lanes.
__device__ __forceinline__ bool mbar_wait_lane(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                               uint32_t limit) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          uint32_t limit) {
    return __all_sync(0xffffffffu, mbar_wait_lane(bar, parity, abort_flag, limit)) != 0;
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
// UMMA shared-memory descriptor for a K-major, 128-byte-swizzled tile whose rows are 128
// bytes and whose 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: 8 rows
    d |= (uint64_t)1 << 46;                        // descriptor version
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
// 32 consecutive 32-bit columns of this thread's tensor-memory lane (the warp's 32 lanes).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
        "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
          "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
          "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace
