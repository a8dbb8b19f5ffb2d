// Shared device helpers for the polarquant_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "polarquant_b200.h"

namespace pq {

constexpr int kBlockElems = 32;  // elements per block_pq4 block

__host__ __device__ constexpr int block_bytes(int n_bits) { return 2 + kBlockElems * n_bits / 8; }

// ---------------------------------------------------------------- warp-level MMA
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col); fragment layout with
// g = lane / 4, t = lane % 4:
//   a0 = A[g][2t, 2t+1]   a1 = A[g+8][2t, 2t+1]   a2 = A[g][2t+8, 2t+9]   a3 = A[g+8][2t+8, 2t+9]
//   b0 = B[2t, 2t+1][g]   b1 = B[2t+8, 2t+9][g]
//   c0, c1 = C[g][2t, 2t+1]   c2, c3 = C[g+8][2t, 2t+1]
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                            const void* smem_row) {
    uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// ---------------------------------------------------------------- async copies
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_8(void* smem_dst, const void* gmem_src) {
    uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ---------------------------------------------------------------- small numerics
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Two-term float16 split of a float: v ~= hi + lo with |lo| <= ulp16(hi)/2.
__device__ __forceinline__ void split_half(float v, __half& hi, __half& lo) {
    hi = __float2half_rn(v);
    lo = __float2half_rn(v - __half2float(hi));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Device error flags of the prefill kernel, read and cleared (defined in pq_prefill_attn.cu).
int prefill_error_flags(unsigned int* flags);
// Device error flags of the decode kernel, read and cleared (defined in pq_decode_attn.cu).
int decode_error_flags(unsigned int* flags);
// pq_dequant.cu: bit 0 a bounded wait gave up
int dequant_error_flags(unsigned int* flags);
// pq_lse_merge.cu: bit 0 a wait for a peer's records gave up
int exchange_error_flags(unsigned int* flags);

}  // namespace pq
