// Bulk asynchronous copies global -> shared (the TMA engine's untiled form, cp.async.bulk) completing on an
// mbarrier.  One thread issues a copy of any multiple of 16 bytes between 16-byte aligned addresses; the threads
// that consume the data wait on the barrier's phase.  Every wait is bounded: a copy that does not land within
// the limit makes the kernel record it in a device-global counter, stop issuing copies, give the copies it still
// has in flight one more bounded wait each (a CTA must not exit with a bulk copy into its shared memory pending)
// and return instead of spinning.  The host reads the counter after the stream has been synchronised and reports
// the call as failed when it moved.
#pragma once

#include <stdint.h>

#include "gguf_common.cuh"

namespace gguf {

GGUF_D uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

GGUF_D void mbarrier_init(uint64_t *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
// Makes barrier initialisations and earlier generic-proxy accesses to shared memory visible to the async proxy.
GGUF_D void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// The issuing thread: announce `bytes` on the barrier (one arrival) and start the copy.
GGUF_D void bulk_load(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

// An arrival that brings no bytes (a thread with nothing to copy, on a barrier that counts every thread).
GGUF_D void mbarrier_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// Waits for the phase with parity `parity` to complete; false when the limit ran out.  A try_wait suspends the
// thread for a hardware-defined time slice, so the limit is many milliseconds, far beyond any copy.
constexpr int kBulkWaitLimit = 1 << 18;
GGUF_D bool mbarrier_wait(uint64_t *bar, uint32_t parity, int limit = kBulkWaitLimit) {
    const uint32_t addr = smem_addr(bar);
    for (int i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

}  // namespace gguf
