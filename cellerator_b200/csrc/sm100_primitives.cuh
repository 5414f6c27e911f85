// Inline PTX of the sm_100a primitives the tensor-core kernels share: mbarriers with bounded waits,
// bulk asynchronous copies into shared memory, tcgen05 MMA issue / commit, and TMEM loads.
// Every wait is bounded: after 2^22 polls the CTA's abort flag is raised and all waits of the CTA
// return at once, so a kernel always runs to its end and frees its TMEM.
#pragma once

#include <cstdint>

namespace cb200 {

__device__ __forceinline__ std::uint32_t smem_addr(const void *p) { return static_cast<std::uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(std::uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(std::uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_arrive_expect_tx(std::uint32_t bar, std::uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(std::uint32_t bar, std::uint32_t parity) {
    std::uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0u;
}
// Bounded wait.  Once any wait of the CTA has timed out (`*abort_flag` set) waits return at once.
// Returns true when the wait was given up (its own bound ran out, or another wait's did): the flag is
// looked at only while the barrier is not ready, so a wait that succeeds at once costs nothing extra.
constexpr int kPollLimit = 1 << 22;
__device__ __forceinline__ bool bar_wait(std::uint32_t bar, std::uint32_t parity, volatile int *abort_flag, int limit = kPollLimit) {
    int spins = 0;
    while (!bar_try_wait(bar, parity)) {
        if (*abort_flag != 0) return true;
        if (++spins > limit) {
            *abort_flag = 1;
            return true;
        }
    }
    return false;
}
// The same for a barrier that is normally microseconds away (a ring with slack, a whole row group of MMAs): the
// warp sleeps `ns` between polls, which leaves the issue slots of its scheduler to the warps that are working.
__device__ __forceinline__ bool bar_wait_sleeping(std::uint32_t bar, std::uint32_t parity, volatile int *abort_flag, unsigned ns) {
    int spins = 0;
    while (!bar_try_wait(bar, parity)) {
        if (*abort_flag != 0) return true;
        if (++spins > kPollLimit / 4) {
            *abort_flag = 1;
            return true;
        }
        __nanosleep(ns);
    }
    return false;
}
// Bounded wait that does not look at the abort flag: what a role uses, after the CTA has aborted, to let the
// copies or MMAs it still has in flight finish before the CTA gives up its shared memory and TMEM.
__device__ __forceinline__ bool bar_wait_drain(std::uint32_t bar, std::uint32_t parity, int limit = kPollLimit) {
    for (int spins = 0; spins <= limit; ++spins)
        if (bar_try_wait(bar, parity)) return true;
    return false;
}
// One contiguous global -> shared copy by the copy engine (this GPU's own memory, no multicast).
__device__ __forceinline__ void bulk_copy_g2s(std::uint32_t dst, const void *src, std::uint32_t bytes, std::uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Values loaded from a shared-memory buffer must be in their registers before a barrier arrival hands the buffer
// back to the copy engine; when they are only used later that is not a given: with the arrival straight after such
// loads a kernel of this library read refilled data (reproducibly).  Here the arrival's address depends on a warp vote
// over a word that depends on every loaded register (pass their OR), so it cannot be issued before those loads have
// returned; `zero` is a value that is 0 at run time without the compiler knowing it (say, the sign bit of a count
// among the kernel's arguments), which keeps the vote in the address.
__device__ __forceinline__ void arrive_when_loaded(std::uint32_t bar, std::uint32_t or_of_loaded_registers, int lane, std::uint32_t zero) {
    const unsigned seen = __ballot_sync(0xffffffffu, or_of_loaded_registers != 0u);
    if (lane == 0) bar_arrive(bar + (seen & zero));
}

// K-major operand with the 128-byte swizzle (the A tile): 8-row atoms of 1,024 bytes follow each
// other (SBO = 1,024 B), the leading offset is not used for this layout (encoded as 1), and a
// K = 16 step inside a 64-gene half moves the start address by 32 bytes.  Atoms are 1,024-byte
// aligned, so the base-offset field stays 0.
__device__ __forceinline__ std::uint64_t smem_desc_sw128(std::uint32_t addr) {
    std::uint64_t d = 0;
    d |= static_cast<std::uint64_t>((addr & 0x3ffffu) >> 4);
    d |= static_cast<std::uint64_t>(1) << 16;
    d |= static_cast<std::uint64_t>(1024u >> 4) << 32;
    d |= static_cast<std::uint64_t>(1) << 46; // descriptor version of this architecture
    d |= static_cast<std::uint64_t>(2) << 61; // 128-byte swizzle
    return d;
}
// kind::f16 instruction descriptor: D fp32, A and B both bf16 (format 1) or both fp16 (format 0), both K-major,
// M = 128.
__host__ __device__ constexpr std::uint32_t instr_desc(int n, bool fp16_operands = false) {
    return (1u << 4) | ((fp16_operands ? 0u : 1u) << 7) | ((fp16_operands ? 0u : 1u) << 10) |
           ((static_cast<std::uint32_t>(n) >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(std::uint32_t tmem_d, std::uint64_t desc_a, std::uint64_t desc_b, std::uint32_t idesc,
                                         bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(std::uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(std::uint32_t taddr, float (&v)[32]) {
    std::uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
          "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
          "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

} // namespace cb200
