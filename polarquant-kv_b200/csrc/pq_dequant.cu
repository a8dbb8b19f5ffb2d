// pq_dequant: stored block_pq4 blocks -> centroid[idx] * float(d) (rotated space) ->
// inverse rotation v @ R -> float32 or float16.
//
// Follows dequantize_with_codebook (src/polarquant_kv_cuda/lloyd_max.py:93-98), the radius
// restore of quantizer.decompress (python/polarquant_kv/quantizer.py:151) and
// inverse_rotate (python/polarquant_kv/rotation.py:61); the float16 output is clamped to
// +-65504 like decompress_gpu (src/polarquant_kv_cuda/decompress_kernel.py:47-51).
//
// The inverse rotation is a [vectors x D] . [D x D] contraction on the tensor cores
// (mma.sync.m16n8k16, float32 accumulation) with both operands as two float16 terms and three
// product terms (hi*hi + hi*lo + lo*hi), which keeps float32-level accuracy (2e-6 of a vector's largest
// component against the float64 reference).  A CTA of 16 warps owns 128 vectors at a time:
//   1. a thread dequantises one block (32 elements) of one vector: centroid * radius in float32 exactly
//      as the reference, times a power of two per vector (so tiny vectors keep their precision), split
//      into hi/lo float16 rows of a shared-memory tile (rows padded against bank conflicts); the stored
//      bytes of the next tile are already in registers by then (loaded before the previous contraction);
//   2. a warp multiplies 32 vectors by D/4 output columns: A fragments by ldmatrix from the tile,
//      B fragments (R split on the fly at set-up, already in fragment order) from shared memory;
//   3. results leave the accumulators as 8- or 4-byte stores, rescaled per vector.
// Bound: 72 B in + 256 or 512 B out per vector (HBM); the three-term contraction on mma.sync costs
// about as much tensor time as the bytes cost HBM time.
#include "pq_common.cuh"

namespace pq {

constexpr int kDqVecs = 128;
constexpr int kDqThreads = 512;

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
    static constexpr int LD = D + 8;                              // halves per tile row (16-byte skew)
    static constexpr int kTileBytes = kDqVecs * LD * 2;           // one term of the dequantised tile
    static constexpr int kRBytes = D * D * 2;                     // one term of R in fragment order
    static constexpr size_t smem_bytes() { return 2 * (size_t)kTileBytes + 2 * (size_t)kRBytes + 16 * 32 * 4 + kDqVecs * 4; }
};

template <int D, int BITS>
__global__ void __launch_bounds__(kDqThreads, 1) pq_dequant_kernel(const DequantParams p) {
    using C = DequantCfg<D>;
    constexpr int NBLK = D / 32;
    constexpr int BB = block_bytes(BITS);
    constexpr int VB = NBLK * BB;
    constexpr int LD = C::LD;
    constexpr int KS = D / 16;                                    // k-steps
    constexpr int NTW = D / 32;                                   // 8-column n-tiles per warp (a quarter of D)
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __half* xh = reinterpret_cast<__half*>(smem_raw);             // [128][LD] hi term
    __half* xl = xh + kDqVecs * LD;                               // [128][LD] lo term
    uint2* rh = reinterpret_cast<uint2*>(smem_raw + 2 * C::kTileBytes);   // [KS][D/8][32] B fragments, hi term of 4096 R
    uint2* rl = rh + KS * (D / 8) * 32;                                     // lo term
    float* cbs = reinterpret_cast<float*>(rl + KS * (D / 8) * 32);          // [16][32]: a copy of the codebook per lane
    float* vscale = cbs + 16 * 32;                                          // [128] 1 / (power-of-two scale of a vector)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // ---- set-up: R as B fragments.  out[v][n] = sum_k x[v][k] R[k][n]: B[k][n] = R[k][n];
    // fragment (ks, nt), lane (g, t): b0 = (R[16ks+2t][8nt+g], R[16ks+2t+1][8nt+g]), b1 = rows +8, +9.
    for (int e = tid; e < KS * (D / 8) * 32; e += kDqThreads) {
        const int ln = e & 31, nt = (e >> 5) % (D / 8), ks = (e >> 5) / (D / 8);
        const int gg = ln >> 2, tt = ln & 3, n = nt * 8 + gg, k0 = ks * 16 + 2 * tt;
        float v[4] = {p.rot[(size_t)k0 * D + n] * 4096.f, p.rot[(size_t)(k0 + 1) * D + n] * 4096.f,
                      p.rot[(size_t)(k0 + 8) * D + n] * 4096.f, p.rot[(size_t)(k0 + 9) * D + n] * 4096.f};
        const __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        rh[e] = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        rl[e] = make_uint2(pack_half2(v[0] - f0.x, v[1] - f0.y), pack_half2(v[2] - f1.x, v[3] - f1.y));
    }
    for (int e = tid; e < 16 * 32; e += kDqThreads) cbs[e] = p.cb[e >> 5];

    const int64_t n_tiles = (p.n_vec + kDqVecs - 1) / kDqVecs;
    // this thread's (vector, block) of every tile; the NBLK threads of a vector are neighbouring lanes
    const bool has_pair = tid < kDqVecs * NBLK;
    const int vec = tid / NBLK, blk = tid % NBLK;
    uint32_t words[BITS];                                         // 32 packed indices of the next tile's block
    float d_next = 0.f;
    auto fetch = [&](int64_t tile) {
        d_next = 0.f;
#pragma unroll
        for (int w = 0; w < BITS; ++w) words[w] = 0u;
        const int64_t v = tile * kDqVecs + vec;
        if (has_pair && tile < n_tiles && v < p.n_vec) {
            const uint16_t* src = reinterpret_cast<const uint16_t*>(p.blocks + v * VB + blk * BB);
            d_next = __half2float(__ushort_as_half(__ldg(src)));
#pragma unroll
            for (int w = 0; w < BITS; ++w)
                words[w] = (uint32_t)__ldg(src + 1 + 2 * w) | ((uint32_t)__ldg(src + 2 + 2 * w) << 16);
        }
    };
    fetch(blockIdx.x);
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t v0 = tile * kDqVecs;
        const int n_valid = (int)((p.n_vec - v0) < kDqVecs ? (p.n_vec - v0) : kDqVecs);
        __syncthreads();                                          // the previous tile is consumed (and set-up done)
        // ---- 1. dequantise this thread's block into the tile
        if (has_pair) {
            const float d = d_next;
            // one power of two per vector: largest block radius -> [1, 2)
            float dmax = d;
#pragma unroll
            for (int o = 1; o < NBLK; o <<= 1) dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, o));
            const uint32_t be = __float_as_uint(dmax) >> 23;
            const float sc = (be > 0 && be < 255) ? __uint_as_float((254u - be) << 23) : 1.0f;
            if (blk == 0) vscale[vec] = (be > 0 && be < 255) ? __uint_as_float(be << 23) : 1.0f;
            __half* oh = xh + vec * LD + blk * 32;
            __half* ol = xl + vec * LD + blk * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                uint32_t i0, i1;
                if (BITS == 4) {
                    i0 = (words[j >> 3] >> ((j & 7) * 4)) & 0xFu;
                    i1 = (words[j >> 3] >> ((j & 7) * 4 + 4)) & 0xFu;
                } else {
                    i0 = (words[j >> 4] >> ((j & 15) * 2)) & 0x3u;
                    i1 = (words[j >> 4] >> ((j & 15) * 2 + 2)) & 0x3u;
                }
                const float x0 = __fmul_rn(cbs[i0 * 32 + lane], d) * sc, x1 = __fmul_rn(cbs[i1 * 32 + lane], d) * sc;
                const __half2 h = __floats2half2_rn(x0, x1);
                const float2 f = __half22float2(h);
                *reinterpret_cast<__half2*>(oh + j) = h;
                *reinterpret_cast<uint32_t*>(ol + j) = pack_half2(x0 - f.x, x1 - f.y);
            }
        }
        fetch(tile + gridDim.x);                                  // in flight during the contraction
        __syncthreads();
        // ---- 2. contraction: warp -> rows 32*(warp & 3) .. +31, columns (D/4)*(warp >> 2) .. + D/4 - 1
        const int r0 = 32 * (warp & 3), nt0 = (warp >> 2) * NTW;
        float acc[2][NTW][4];
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[m][nt][j] = 0.f;
#pragma unroll 2
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t ah[2][4], al[2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                // ldmatrix x4: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
                const int row = r0 + 16 * m + (lane & 7) + ((lane >> 3) & 1) * 8, col = ks * 16 + (lane >> 4) * 8;
                ldmatrix_x4(ah[m][0], ah[m][1], ah[m][2], ah[m][3], xh + row * LD + col);
                ldmatrix_x4(al[m][0], al[m][1], al[m][2], al[m][3], xl + row * LD + col);
            }
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) {
                const uint2 bh = rh[(ks * (D / 8) + nt0 + nt) * 32 + lane], bl = rl[(ks * (D / 8) + nt0 + nt) * 32 + lane];
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    mma_16816(acc[m][nt], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bh.x, bh.y);
                    mma_16816(acc[m][nt], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bl.x, bl.y);
                    mma_16816(acc[m][nt], al[m][0], al[m][1], al[m][2], al[m][3], bh.x, bh.y);
                }
            }
        }
        // ---- 3. store: C rows g / g+8, columns 2t, 2t+1 of every n-tile
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int row = r0 + 16 * m + g + 8 * hrow;
                if (row >= n_valid) continue;
                const float s = vscale[row] * (1.0f / 4096.f);
#pragma unroll
                for (int nt = 0; nt < NTW; ++nt) {
                    const float a = acc[m][nt][2 * hrow] * s, b = acc[m][nt][2 * hrow + 1] * s;
                    const size_t off = (size_t)(v0 + row) * D + (nt0 + nt) * 8 + 2 * t;
                    if (p.out_is_fp16) {
                        *reinterpret_cast<__half2*>(static_cast<__half*>(p.out) + off) =
                            __floats2half2_rn(fminf(fmaxf(a, -65504.f), 65504.f), fminf(fmaxf(b, -65504.f), 65504.f));
                    } else {
                        *reinterpret_cast<float2*>(static_cast<float*>(p.out) + off) = make_float2(a, b);
                    }
                }
            }
    }
}

template <int D, int BITS>
static int launch_dequant(const DequantParams& p, cudaStream_t st) {
    const size_t smem = DequantCfg<D>::smem_bytes();
    auto kern = pq_dequant_kernel<D, BITS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return PQ_ERR_CUDA;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return PQ_ERR_CUDA;
    const int64_t n_tiles = (p.n_vec + kDqVecs - 1) / kDqVecs;
    const int64_t cap = (int64_t)sms * (D == 128 ? 1 : 2);
    const int grid = (int)(n_tiles < cap ? n_tiles : cap);
    kern<<<grid, kDqThreads, smem, st>>>(p);
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
    if ((reinterpret_cast<uintptr_t>(blocks) & 3) || (reinterpret_cast<uintptr_t>(rot) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 7))
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
