// pq_dequant: stored block_pq4 blocks -> centroid[idx] * float(d) (rotated space) ->
// inverse rotation v @ R -> float32 or float16.
//
// Follows dequantize_with_codebook (src/polarquant_kv_cuda/lloyd_max.py:93-98), the radius
// restore of quantizer.decompress (python/polarquant_kv/quantizer.py:151) and
// inverse_rotate (python/polarquant_kv/rotation.py:61); the float16 output is clamped to
// +-65504 like decompress_gpu (src/polarquant_kv_cuda/decompress_kernel.py:47-51).
//
// The inverse rotation is a [vectors x D] . [D x D] contraction on the 5th-generation tensor cores
// (tcgen05.mma kind::f16, M = 128, accumulators in tensor memory) with both operands as two float16
// terms and three product terms (hi*hi + hi*lo + lo*hi), which keeps float32-level accuracy (2e-6 of
// a vector's largest component against the float64 reference).  A persistent CTA owns 128 vectors at a
// time and runs the compress pipeline backwards:
//   worker warps (4 per 32-dim block)  a thread dequantises one block of one vector - centroid * radius
//       in float32 exactly as the reference, times a power of two per vector (so tiny vectors keep their
//       precision) - and writes its hi and lo float16 terms as four 16-byte chunks each into the K-major
//       A tiles in shared memory (two pairs of tiles: tile i+1 is produced while tile i is contracted);
//       the stored bytes of the next tile are loaded before the epilogue so they are in flight;
//   MMA warp  one lane issues, per tile, D/16 MMAs A_hi x [R_hi ; R_lo] (N = 2D: columns [0, D) receive
//       hi*hi, [D, 2D) hi*lo) and D/16 MMAs A_lo x R_hi on top of the first D columns; tcgen05.commit
//       releases the A tiles and hands the accumulator (one of two) to the epilogue;
//   the same worker warps, one tile behind, read their 32 output columns of both halves from tensor
//       memory (thread = vector), add, rescale and store 64 or 128 contiguous bytes per vector.
// R is split into the two float16 terms of 4096 R and laid out as the B operand once per CTA.
// All waits are bounded (a lost completion sets an error flag instead of hanging).
// Bound: 72 B in + 256 or 512 B out per vector (HBM).
#include "pq_tcgen05.cuh"

namespace pq {

constexpr int kDqVecs = 128;

// bit 0: a bounded wait gave up (read and cleared through pq_poll_device_errors, bit 6 there)
static __device__ unsigned int g_dequant_error = 0;

struct DequantParams {
    const uint8_t* blocks;
    const float* rot;
    void* out;
    int64_t n_vec;
    int out_is_fp16;
    float cb[16];
};

template <int D>
struct DequantCfg {
    static constexpr int NBLK = D / 32;
    static constexpr int kWorkers = 32 * 4 * NBLK;                // one thread per (vector, block)
    static constexpr int kThreads = kWorkers + 32;                // + the MMA warp
    static constexpr int kATile = kDqVecs * D * 2;                // one float16 term of a 128-vector tile
    static constexpr int kBBytes = 2 * D * D * 2;                 // [R_hi ; R_lo] as the stacked B operand
    static constexpr int kAccCols = 2 * D;                        // accumulator columns per buffer
    static constexpr int kWarpSegMax = (32 / NBLK) * NBLK * 18;   // packed bytes of a warp's vectors, 4-bit (576)
    // A tiles (2 buffers x 2 terms) | B | codebook copies | per-vector scales (4 tiles) | the warps' packed
    // bytes | barriers | alignment
    static constexpr size_t smem_bytes() {
        return 4 * (size_t)kATile + kBBytes + 16 * 32 * 4 + 4 * kDqVecs * 4 + (kWorkers / 32) * kWarpSegMax + 128 + 128;
    }
};

// Byte offset of 16-byte chunk `kc` of row `r` in a K-major operand tile with `rows` rows (8-row x 16-byte
// core matrices, 128 bytes each; consecutive 8-row groups 128 bytes apart, consecutive K chunks rows/8 * 128).
__device__ __forceinline__ uint32_t dq_chunk_off(int rows, int r, int kc) {
    return (uint32_t)(kc * (rows / 8) * 128 + (r >> 3) * 128 + (r & 7) * 16);
}

// packed float32x2 arithmetic: two round-to-nearest operations per instruction
__device__ __forceinline__ float2 dq_mul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;\n"
        : "=l"(*reinterpret_cast<unsigned long long*>(&d))
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return d;
}
__device__ __forceinline__ float2 dq_fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n"
        : "=l"(*reinterpret_cast<unsigned long long*>(&d))
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return d;
}

// 32 bytes to global memory at a 32-byte boundary in one instruction
__device__ __forceinline__ void stg_256(void* dst, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}

template <int D, int BITS>
__global__ void __launch_bounds__(DequantCfg<D>::kThreads, 1) pq_dequant_kernel(const DequantParams p) {
    using C = DequantCfg<D>;
    constexpr int NBLK = C::NBLK;
    constexpr int BB = block_bytes(BITS);
    constexpr int VB = NBLK * BB;
    constexpr int WORKERS = C::kWorkers;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* sp = smem_raw + ((128u - (sm_addr(smem_raw) & 127u)) & 127u);
    uint8_t* a_tiles = sp;                      sp += 4 * C::kATile;      // [buffer][term]
    uint8_t* b_tile = sp;                       sp += C::kBBytes;
    float* cbs = reinterpret_cast<float*>(sp);  sp += 16 * 32 * 4;        // a copy of the codebook per lane
    // [tile & 3][vector] power-of-two scale.  A worker may already produce tile i + 1 while another still
    // reads the scales of tile i - 2 in its epilogue (tile i + 2 cannot start before that: its A tiles are
    // free only after the MMAs of tile i, which need every worker's tile i), hence four slots.
    float* vscale = reinterpret_cast<float*>(sp); sp += 4 * kDqVecs * 4;
    uint8_t* segs = sp;                         sp += (C::kWorkers / 32) * C::kWarpSegMax;   // [warp] packed bytes
    uint64_t* mbar = reinterpret_cast<uint64_t*>(sp);
    // [0], [1]: A tiles of buffer b written; [2], [3]: A tiles of buffer b consumed by their MMAs;
    // [4], [5]: accumulator b complete; [6], [7]: accumulator b read out by every worker
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 8);
    volatile uint32_t* abort_s = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---- set-up: B = [R_hi ; R_lo] with B[n][k] = 4096 R[k][n] (out[v][n] = sum_k x[v][k] R[k][n])
    for (int e = tid; e < D * D; e += C::kThreads) {
        const int k = e / D, n = e - k * D;                               // coalesced along n
        const float v = p.rot[e] * 4096.f;
        const __half h = __float2half_rn(v);
        const __half l = __float2half_rn(v - __half2float(h));
        const uint32_t off = dq_chunk_off(2 * D, n, k >> 3) + (k & 7) * 2;
        *reinterpret_cast<__half*>(b_tile + off) = h;
        *reinterpret_cast<__half*>(b_tile + off + dq_chunk_off(2 * D, D, 0)) = l;      // rows D .. 2D-1
    }
    for (int e = tid; e < 16 * 32; e += C::kThreads) cbs[e] = p.cb[e >> 5];
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) mbar_init(sm_addr(mbar + i), WORKERS);
        for (int i = 2; i < 6; ++i) mbar_init(sm_addr(mbar + i), 1);
        for (int i = 6; i < 8; ++i) mbar_init(sm_addr(mbar + i), WORKERS);
        *abort_s = 0u;
    }
    if (warp == 0) tmem_alloc(sm_addr(tmem_slot), 2 * C::kAccCols);
    fence_async_smem();          // B is read by the tensor core through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t n_tiles = (p.n_vec + kDqVecs - 1) / kDqVecs;
    const int64_t n_my = (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;      // tiles of this CTA
    bool ok = true;

    if (warp == WORKERS / 32) {
        // ---- MMA warp: every lane runs the loop (uniform waits and descriptor arithmetic), lane 0 issues
        constexpr uint32_t idesc_full = umma_idesc_f16(2 * D), idesc_half = umma_idesc_f16(D);
        constexpr uint32_t kLboA = (kDqVecs / 8) * 128, kLboB = (2 * D / 8) * 128;   // K-chunk strides
        constexpr uint32_t d_hi = (128u >> 4) | (1u << 14);                         // 8-row groups 128 B apart, no swizzle
        const uint32_t b_lo0 = ((sm_addr(b_tile) >> 4) & 0x3FFFu) | ((kLboB >> 4) << 16);
        const uint32_t issue = lane == 0 ? 1u : 0u;
        for (int64_t i = 0; i < n_my && ok; ++i) {
            const uint32_t b = (uint32_t)(i & 1), use = (uint32_t)(i >> 1);
            ok = mbar_wait(sm_addr(mbar + b), use & 1u, abort_s, 32) && ok;                       // A written
            if (i >= 2) ok = mbar_wait(sm_addr(mbar + 6 + b), (use - 1u) & 1u, abort_s, 32) && ok;   // accumulator free
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + b * C::kAccCols;
            const uint32_t ah0 = ((sm_addr(a_tiles + (2 * b) * C::kATile) >> 4) & 0x3FFFu) | ((kLboA >> 4) << 16);
            const uint32_t al0 = ((sm_addr(a_tiles + (2 * b + 1) * C::kATile) >> 4) & 0x3FFFu) | ((kLboA >> 4) << 16);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)          // a k-step is two 16-byte chunks
                umma_f16_split_pred(acc, ah0 + ks * ((2 * kLboA) >> 4), d_hi, b_lo0 + ks * ((2 * kLboB) >> 4), d_hi,
                                    idesc_full, ks ? 1u : 0u, issue);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)          // lo term of the vectors x hi term of R: the first D rows of B
                umma_f16_split_pred(acc, al0 + ks * ((2 * kLboA) >> 4), d_hi, b_lo0 + ks * ((2 * kLboB) >> 4), d_hi,
                                    idesc_half, 1u, issue);
            umma_commit_pred(sm_addr(mbar + 2 + b), issue);      // the A tiles may be overwritten
            umma_commit_pred(sm_addr(mbar + 4 + b), issue);      // the accumulator is complete
        }
        if (!ok && lane == 0) { *abort_s = 1u; atomicOr(&g_dequant_error, 1u); }
    } else {
        // ---- worker warps
        // produce: this thread's (vector, block).  Eight neighbouring lanes own eight neighbouring vectors
        // of the same block, so that their 16-byte chunk stores into the A tiles fill 128 contiguous bytes
        // (a quarter warp per shared-memory wavefront, no bank conflicts); the blocks of a vector sit
        // 32 / NBLK lanes apart.
        constexpr int VPW = 32 / NBLK;                            // vectors per warp
        const int vec = warp * VPW + (lane % VPW), blk = lane / VPW;
        const int q = warp & 3, cc = warp >> 2;                   // epilogue: TMEM lane quarter, 32-column chunk
        const int row = 32 * q + lane;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(32 * q) << 16);
        // The stored bytes of a warp's VPW vectors are one contiguous segment of VPW * VB bytes (576 or 320):
        // the warp loads it as 16-byte pieces, one or two per lane, a tile ahead, and passes it through a
        // shared-memory slot from which every thread picks its block (18 or 10 bytes at a 2-byte boundary).
        constexpr int kSeg = VPW * VB;                            // a multiple of 16
        constexpr int kPieces = kSeg / 16;                        // 36 or 20
        const int64_t total_bytes = p.n_vec * VB;
        uint4 piece0 = make_uint4(0u, 0u, 0u, 0u), piece1 = make_uint4(0u, 0u, 0u, 0u);
        auto load_piece = [&](int64_t byte0) -> uint4 {           // 16 bytes at a 16-byte boundary, zeros past the end
            uint4 r = make_uint4(0u, 0u, 0u, 0u);
            if (byte0 + 16 <= total_bytes) {
                r = __ldg(reinterpret_cast<const uint4*>(p.blocks + byte0));
            } else if (byte0 < total_bytes) {                     // the last piece of the tensor: 2-byte loads
                uint32_t w[4] = {0u, 0u, 0u, 0u};
                for (int h = 0; h < 8 && byte0 + 2 * h < total_bytes; ++h)
                    w[h >> 1] |= (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p.blocks + byte0) + h) << (16 * (h & 1));
                r = make_uint4(w[0], w[1], w[2], w[3]);
            }
            return r;
        };
        auto fetch = [&](int64_t tile) {
            const int64_t seg0 = (tile * kDqVecs + (int64_t)warp * VPW) * VB;
            piece0 = lane < kPieces ? load_piece(seg0 + 16 * lane) : make_uint4(0u, 0u, 0u, 0u);
            piece1 = 32 + lane < kPieces ? load_piece(seg0 + 16 * (32 + lane)) : make_uint4(0u, 0u, 0u, 0u);
        };
        uint8_t* seg = segs + warp * C::kWarpSegMax;
        uint32_t words[BITS];                                     // 32 packed indices of this thread's block
        float d_cur = 0.f;
        auto unpack_block = [&]() {                               // registers -> slot -> this thread's block
            __syncwarp();
            if (lane < kPieces) *reinterpret_cast<uint4*>(seg + 16 * lane) = piece0;
            if (32 + lane < kPieces) *reinterpret_cast<uint4*>(seg + 16 * (32 + lane)) = piece1;
            __syncwarp();
            const int off = (lane % VPW) * VB + blk * BB;         // 2-byte aligned; 4-byte aligned for even blocks
            const uint32_t* w32 = reinterpret_cast<const uint32_t*>(seg + (off & ~3));
            uint32_t w[BITS + 1];
#pragma unroll
            for (int k = 0; k <= BITS; ++k) w[k] = w32[k];
            if (off & 2) {
                d_cur = __half2float(__ushort_as_half((unsigned short)(w[0] >> 16)));
#pragma unroll
                for (int k = 0; k < BITS; ++k) words[k] = w[k + 1];
            } else {
                d_cur = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu)));
#pragma unroll
                for (int k = 0; k < BITS; ++k) words[k] = __funnelshift_r(w[k], w[k + 1], 16);
            }
        };
        auto epilogue = [&](int64_t i) {                          // tile number i of this CTA
            const uint32_t b = (uint32_t)(i & 1), use = (uint32_t)(i >> 1);
            ok = mbar_wait(sm_addr(mbar + 4 + b), use & 1u, abort_s) && ok;
            if (!ok) return;
            tc_fence_after();
            float hi[32], lo[32];
            tmem_ld32(hi, tmem_lane + b * C::kAccCols + cc * 32);
            tmem_ld32(lo, tmem_lane + b * C::kAccCols + D + cc * 32);
            tc_fence_before();
            mbar_arrive(sm_addr(mbar + 6 + b));                   // this thread's part of the accumulator is in registers
            const int64_t tile = (int64_t)blockIdx.x + i * gridDim.x;
            const int64_t v = tile * kDqVecs + row;
            if (v >= p.n_vec) return;
            const float s = vscale[(i & 3) * kDqVecs + row] * (1.0f / 4096.f);
            const size_t off = (size_t)v * D + cc * 32;
            // 32-byte stores: every store instruction of a thread fills a whole sector
            if (p.out_is_fp16) {
                __half* dst = static_cast<__half*>(p.out) + off;
#pragma unroll
                for (int j = 0; j < 32; j += 16) {
                    uint32_t w[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float a = (hi[j + 2 * u] + lo[j + 2 * u]) * s, c = (hi[j + 2 * u + 1] + lo[j + 2 * u + 1]) * s;
                        w[u] = pack_half2(fminf(fmaxf(a, -65504.f), 65504.f), fminf(fmaxf(c, -65504.f), 65504.f));
                    }
                    stg_256(dst + j, w);
                }
            } else {
                float* dst = static_cast<float*>(p.out) + off;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint32_t w[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) w[u] = __float_as_uint((hi[j + u] + lo[j + u]) * s);
                    stg_256(dst + j, w);
                }
            }
        };
        fetch(blockIdx.x);
        for (int64_t i = 0; i < n_my && ok; ++i) {
            const uint32_t b = (uint32_t)(i & 1), use = (uint32_t)(i >> 1);
            // ---- produce tile i: its A tiles must have been consumed by the MMAs of tile i - 2
            if (i >= 2) ok = mbar_wait(sm_addr(mbar + 2 + b), (use - 1u) & 1u, abort_s) && ok;
            if (!ok) break;
            {
                unpack_block();
                const float d = d_cur;
                // one power of two per vector: largest block radius -> [1, 2)
                float dmax = d;
#pragma unroll
                for (int o = VPW; o < 32; o <<= 1) dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, o));
                const uint32_t be = __float_as_uint(dmax) >> 23;
                const bool normal = be > 0 && be < 255;
                const float sc = normal ? __uint_as_float((254u - be) << 23) : 1.0f;
                if (blk == 0) vscale[(i & 3) * kDqVecs + vec] = normal ? __uint_as_float(be << 23) : 1.0f;
                uint8_t* ah = a_tiles + (2 * b) * C::kATile;
                uint8_t* al = ah + C::kATile;
                const float2 ds2 = make_float2(d * sc, d * sc), neg1 = make_float2(-1.f, -1.f);
#pragma unroll
                for (int c = 0; c < 4; ++c) {                     // four 16-byte chunks of 8 elements
                    uint32_t wh[4], wl[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int j = 8 * c + 2 * u;
                        uint32_t i0, i1;
                        if (BITS == 4) {
                            i0 = (words[j >> 3] >> ((j & 7) * 4)) & 0xFu;
                            i1 = (words[j >> 3] >> ((j & 7) * 4 + 4)) & 0xFu;
                        } else {
                            i0 = (words[j >> 4] >> ((j & 15) * 2)) & 0x3u;
                            i1 = (words[j >> 4] >> ((j & 15) * 2 + 2)) & 0x3u;
                        }
                        // centroid * radius rounded once to float32 as the reference does; the power of two
                        // rides on the radius (it commutes with that rounding)
                        const float2 x = dq_mul2(make_float2(cbs[i0 * 32 + lane], cbs[i1 * 32 + lane]), ds2);
                        const __half2 h = __floats2half2_rn(x.x, x.y);
                        const float2 lo = dq_fma2(__half22float2(h), neg1, x);     // exact: x - float(h)
                        wh[u] = *reinterpret_cast<const uint32_t*>(&h);
                        wl[u] = pack_half2(lo.x, lo.y);
                    }
                    const uint32_t off = dq_chunk_off(kDqVecs, vec, blk * 4 + c);
                    *reinterpret_cast<uint4*>(ah + off) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                    *reinterpret_cast<uint4*>(al + off) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                }
            }
            fence_async_smem();                                   // the tensor core reads the tiles through the async proxy
            mbar_arrive(sm_addr(mbar + b));
            fetch((int64_t)blockIdx.x + (i + 1) * gridDim.x);     // in flight during the epilogue below
            // ---- epilogue of the tile before
            if (i >= 1) epilogue(i - 1);
        }
        if (ok && n_my >= 1) epilogue(n_my - 1);
        if (!ok && lane == 0) { *abort_s = 1u; atomicOr(&g_dequant_error, 1u); }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 2 * C::kAccCols);
}

// Read and clear this file's device error flag (for pq_poll_device_errors).
int dequant_error_flags(unsigned int* flags) {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_dequant_error, sizeof(v)) != cudaSuccess) return PQ_ERR_CUDA;
    if (v && cudaMemcpyToSymbol(g_dequant_error, &zero, sizeof(zero)) != cudaSuccess) return PQ_ERR_CUDA;
    *flags = v;
    return PQ_OK;
}

template <int D, int BITS>
static int launch_dequant(const DequantParams& p, cudaStream_t st) {
    using C = DequantCfg<D>;
    const size_t smem = C::smem_bytes();
    auto kern = pq_dequant_kernel<D, BITS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return PQ_ERR_CUDA;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return PQ_ERR_CUDA;
    const int64_t n_tiles = (p.n_vec + kDqVecs - 1) / kDqVecs;
    const int grid = (int)(n_tiles < sms ? n_tiles : sms);          // persistent: one CTA per SM (tensor memory)
    kern<<<grid, C::kThreads, smem, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
}

}  // namespace pq

extern "C" int pq_dequant(const void* blocks, int64_t n_vec, int head_dim, int n_bits,
                          const float* codebook, const float* rot, void* out, int out_is_fp16,
                          void* stream) {
    using namespace pq;
    if (n_vec < 0) return PQ_ERR_BAD_SHAPE;
    if (head_dim != 64 && head_dim != 128) return PQ_ERR_BAD_HEAD_DIM;
    if (n_bits != 2 && n_bits != 4) return PQ_ERR_BAD_BITS;
    if (n_vec == 0) return PQ_OK;
    if (!blocks || !codebook || !rot || !out) return PQ_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(blocks) & 15) || (reinterpret_cast<uintptr_t>(rot) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 31))
        return PQ_ERR_MISALIGNED;
    DequantParams p{};
    p.blocks = static_cast<const uint8_t*>(blocks);
    p.rot = rot;
    p.out = out;
    p.n_vec = n_vec;
    p.out_is_fp16 = out_is_fp16;
    for (int i = 0; i < 16; ++i) p.cb[i] = i < (1 << n_bits) ? codebook[i] : 0.f;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (head_dim == 64) return n_bits == 4 ? launch_dequant<64, 4>(p, st) : launch_dequant<64, 2>(p, st);
    return n_bits == 4 ? launch_dequant<128, 4>(p, st) : launch_dequant<128, 2>(p, st);
}
