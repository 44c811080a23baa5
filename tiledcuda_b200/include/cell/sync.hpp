// Copy-completion fences. The reference's versions are cp.async group fences (include/cell/sync.hpp:7-23);
// the names and meanings are kept. One addition: data that generic-proxy copies (cp.async, st.shared) put
// into shared memory must be made visible to the async proxy before tcgen05.mma reads it, so
// __copy_async() also issues that proxy fence. MmaBarrier is the completion object for tcgen05.mma,
// CopyBarrier the one for tensor-map loads; both wait with a limit the caller may set.
#pragma once

#include <cstdint>

#include "config.hpp"

namespace tiledcuda::cell {

template <int N>
DEVICE void wait_group() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

DEVICE void commit_copy_group() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }

// Orders this thread's generic-proxy writes to shared memory before later async-proxy reads of it.
DEVICE void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// Commit everything issued so far, wait for it, and publish it to the tensor core. Follow with
// __syncthreads() before another thread (or an MMA) uses the data.
DEVICE void __copy_async() {
    commit_copy_group();
    wait_group<0>();
    fence_async_proxy();
}

// Bounded wait on the phase `parity` of the mbarrier at shared-memory address `bar`: polls until the phase
// completes or `limit_ns` nanoseconds have passed (the clock is read every 256 polls, so short limits are
// honoured to within a few microseconds). Returns false when it gave up. Nothing traps or spins forever.
constexpr uint64_t kDefaultWaitLimitNs = 2000000000ull;   // two seconds: far above any legitimate wait

DEVICE bool bounded_barrier_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    uint32_t done = 0;
    uint64_t t0 = 0;
    for (uint32_t it = 0; !done; ++it) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (!done && (it & 0xffu) == 0xffu) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > limit_ns)
                return false;
        }
    }
    return true;
}

// Completion tracking for tcgen05.mma: one mbarrier in shared memory. `init` by one thread before use
// (followed by __syncthreads); `commit` by the thread that issued the MMAs; `wait` by every thread that
// needs the result or wants to overwrite the operands. The wait is bounded: it gives up after `limit_ns`
// (two seconds unless the caller says otherwise) and returns false; the caller then skips its result,
// frees its TMEM and reports through a status word.
class MmaBarrier {
  public:
    DEVICE explicit MmaBarrier(uint64_t* smem_bar) : bar_(static_cast<uint32_t>(__cvta_generic_to_shared(smem_bar))), phase_(0) {}

    DEVICE void init() {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }

    DEVICE void commit() {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_) : "memory");
    }

    DEVICE bool wait(uint64_t limit_ns = kDefaultWaitLimitNs) {
        if (!bounded_barrier_wait(bar_, phase_, limit_ns)) return false;
        phase_ ^= 1u;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        return true;
    }

  private:
    uint32_t bar_;
    uint32_t phase_;
};

// Completion tracking for tensor-map (TMA) loads: the issuing thread arms the barrier with the number of
// bytes that will land (`expect`), the loads complete on it, everyone who reads the tile waits. Same bounded
// wait as MmaBarrier.
class CopyBarrier {
  public:
    DEVICE explicit CopyBarrier(uint64_t* smem_bar) : ptr_(smem_bar), bar_(static_cast<uint32_t>(__cvta_generic_to_shared(smem_bar))), phase_(0) {}

    DEVICE void init() {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }

    DEVICE void expect(uint32_t bytes) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_), "r"(bytes) : "memory");
    }

    DEVICE uint64_t* get() const { return ptr_; }

    DEVICE bool wait(uint64_t limit_ns = kDefaultWaitLimitNs) {
        if (!bounded_barrier_wait(bar_, phase_, limit_ns)) return false;
        phase_ ^= 1u;
        return true;
    }

  private:
    uint64_t* ptr_;
    uint32_t bar_;
    uint32_t phase_;
};

}  // namespace tiledcuda::cell
