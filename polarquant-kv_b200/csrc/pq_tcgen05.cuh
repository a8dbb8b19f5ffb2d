// tcgen05 / TMEM / TMA / mbarrier wrappers shared by the tensor-core kernels (inline PTX, sm_100a).
#pragma once
#include <cuda.h>   // CUtensorMap and its enums only; the encoder is looked up at run time

#include "pq_common.cuh"

namespace pq {

// ------------------------------------------------------------------ tcgen05 / mbarrier wrappers
__device__ __forceinline__ uint32_t sm_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// K-major, no-swizzle shared-memory matrix descriptor (sm_100 format, version field = 1)
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_byte_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbar_addr), "r"(bytes) : "memory");
}
// One box of a 2-D tensor map into shared memory; x (halves) must be a multiple of 8.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y,
                                            uint32_t mbar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
            "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(mbar_addr)
        : "memory");
}
// Contiguous global -> shared copy that reports its bytes to an mbarrier; both addresses and the size
// are multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t mbar_addr) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_dst),
                 "l"(gsrc), "r"(bytes), "r"(mbar_addr)
                 : "memory");
}
// Contiguous shared -> global copy; both addresses and the size are multiples of 16.
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(gdst), "r"(smem_src), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar_addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(mbar_addr) : "memory");
}
// Named barrier over `count` threads that also ORs a flag across them (same result in every thread).
__device__ __forceinline__ bool group_barrier_any(uint32_t id, uint32_t count, bool flag) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "barrier.cta.red.or.pred p, %2, %3, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(r)
        : "r"((uint32_t)flag), "r"(id), "r"(count)
        : "memory");
    return r != 0u;
}
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
// kind::f16 instruction descriptor: D = f32, A = B = f16, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t umma_idesc_f16(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
static_assert((256 >> 3) < 64, "N field of the instruction descriptor is 6 bits");
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
// Same, descriptors given as (low, high) 32-bit halves: the high halves are constants and the low
// halves differ from a base by compile-time offsets, which keeps the issuing lane's work per MMA small.
__device__ __forceinline__ void umma_f16_split(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
        "}\n" ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Warp-uniform form: every lane executes the call with identical operands, only lanes with
// `issue` != 0 (exactly one) issue the MMA.  Keeping the control flow uniform lets the
// descriptor arithmetic stay in uniform registers.
__device__ __forceinline__ void umma_f16_split_pred(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                    uint32_t b_hi, uint32_t idesc, uint32_t accumulate,
                                                    uint32_t issue) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pi;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 pi, %7, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
        "}\n" ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}
// A operand from tensor memory (lane = row, each 32-bit column holds two consecutive float16 along K),
// B from shared memory; warp-uniform form as above.
__device__ __forceinline__ void umma_f16_ts_pred(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc, uint32_t accumulate, uint32_t issue) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pi;\n\t"
        ".reg .b64 db;\n\t"
        "setp.ne.b32 pi, %6, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "@pi tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
        "}\n" ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pred(uint32_t mbar_addr, uint32_t issue) {
    asm volatile(
        "{\n\t.reg .pred pi;\n\t"
        "setp.ne.b32 pi, %1, 0;\n\t"
        "@pi tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(mbar_addr),
        "r"(issue)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar_addr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar_addr)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot_addr, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot_addr), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
// 32 consecutive float32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(float (&v)[32], uint32_t taddr) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld32(float2 (&v)[16], uint32_t taddr) {
    tmem_ld32(*reinterpret_cast<float(*)[32]>(&v[0]), taddr);
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
// Bounded wait on a phase parity: gives up after about a second (2^31 clock ticks) and reports
// failure, so a lost completion can never hang the GPU.  `sleep_ns` > 0 backs off between polls
// (for the issuing lane, whose waits are long and whose polling would steal issue slots from the
// epilogue warps on its scheduler).
__device__ __forceinline__ bool mbar_wait(uint32_t addr, uint32_t parity, const volatile uint32_t* abort = nullptr,
                                          unsigned sleep_ns = 0) {
    long long t0 = 0;
    for (int it = 0; it < (1 << 24); ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((it & 63) == 63) {
            if (abort && *abort) return false;       // another thread of the CTA already gave up
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > (1ll << 31)) return false;
        }
    }
    return false;
}

}  // namespace pq
