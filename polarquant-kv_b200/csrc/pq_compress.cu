// pq_compress: fused rotate -> per-32 radius -> nearest Lloyd-Max centroid -> pack
// [-> QJL 1-bit residual sketch], for block_pq4 storage.
//
// One CTA (4 x D/32 warps) owns a tile of 128 vectors; a warp owns 32 vectors x one 32-element block.  The rotation  xr = x @ R^T  is a dense
// contraction on tensor cores.  x is float16 (exact); R is pre-split on the host into two
// float16 terms  4096*R = hi + lo  so that, with float32 accumulation, xr carries about
// 22 mantissa bits of R and matches the float64-then-float32 rotation of the numpy
// reference (python/polarquant_kv/rotation.py:48) to a few 1e-8 relative.  Everything
// after the contraction follows the reference's float32 arithmetic exactly:
//   radius  = sqrt(sum of squares), summed in numpy's axis-reduction order
//             (eight strided partial sums, then a balanced tree),
//   guard   = radius < 1e-30 -> radius 0, indices 0      (quantizer.py:107-119),
//   dir     = xr / radius (IEEE division)                 (quantizer.py:121),
//   index   = #thresholds strictly below dir, the thresholds being the exact float32
//             decision points of argmin_i |dir - c_i|     (lloyd_max.py:82-90),
//   d       = float16(min(radius, 65504))                 (compress_kernel.py:178),
//   packing = low nibble first                            (compress_kernel.py:34-50).
// QJL (qjl.py:25-35, compress_kernel.py:168-175): the residual e = xr - d*c[idx] stays in
// rotated space; signs of P e equal signs of (P R^T) e_rot, evaluated as a second
// three-term float16 contraction (e_hi*P_hi + e_hi*P_lo + e_lo*P_hi).
#include <cmath>
#include <cstring>

#include "pq_common.cuh"

namespace pq {

constexpr int kTileVecs = 128;
// warps: 4 along the vectors (32 each) x D/32 along the outputs (one 32-element block each)
__host__ __device__ constexpr int compress_threads(int D) { return 32 * 4 * (D / 32); }

struct CompressParams {
    const __half* x;
    const __half* rot_split;   // [D][2D]
    const __half* jl_split;    // [M][2D] or null
    uint8_t* blocks_out;
    uint8_t* qjl_bits_out;
    __half* qjl_norm_out;
    int64_t n_vec;
    int jl_dim;
    float cb[16];
    // Index search table: a normalised coordinate y falls into bucket k = round(64 y) + 64;
    // index = base[k] + (y > t[k]).  A bucket holds at most one decision threshold.
    float bucket_t[132];
    uint32_t bucket_base[132];
};

template <int D>
struct CompressSmem {
    static constexpr int kRStride = 2 * D + 8;   // halves per row of the split matrices
    static constexpr int kXStride = D + 8;       // halves per row of the vector tile
};

template <int D, int BITS, bool QJL>
__global__ void __launch_bounds__(compress_threads(D), 1) pq_compress_kernel(const CompressParams p) {
    constexpr int kCompressThreads = compress_threads(D);
    constexpr int WN = D / 32;                    // warps along the output dims
    constexpr int NBLK = D / 32;
    constexpr int BB = block_bytes(BITS);
    constexpr int VB = NBLK * BB;                 // bytes per stored vector
    constexpr int RS = CompressSmem<D>::kRStride;
    constexpr int XS = CompressSmem<D>::kXStride;
    constexpr int NT = 4;                         // n-tiles (8 outputs) per warp: one 32-element block
    constexpr int BREP = QJL ? 1 : 16;            // lane copies of the index-search table
    constexpr int NLEV = 1 << BITS;

    extern __shared__ __align__(16) uint8_t smem_raw[];
    __half* Rs = reinterpret_cast<__half*>(smem_raw);                       // [D][RS]
    __half* Xs = Rs + D * RS;                                               // [128][XS]
    uint8_t* outs = reinterpret_cast<uint8_t*>(Xs + kTileVecs * XS);        // [128][VB]
    // QJL-only regions
    __half* Ps = reinterpret_cast<__half*>(outs + kTileVecs * VB);          // [M][RS]
    __half* Elo = Ps + (QJL ? p.jl_dim : 0) * RS;                           // [128][XS]
    float* escale = reinterpret_cast<float*>(Elo + (QJL ? kTileVecs * XS : 0));  // [128]
    float* enorm2 = escale + kTileVecs;                                     // [128][4]
    uint8_t* bits_s = reinterpret_cast<uint8_t*>(enorm2 + 4 * kTileVecs);   // [128][M/8]
    float* cb_s = reinterpret_cast<float*>(bits_s + (QJL ? kTileVecs * (p.jl_dim / 8) : 0));  // [16]
    uint2* bucket_s = reinterpret_cast<uint2*>(cb_s + 16);                  // [256][BREP] {threshold bits, base}
    // second vector tile for prefetching (not with QJL: the residual tiles take the room)
    __half* Xs2 = reinterpret_cast<__half*>(bucket_s + 256 * BREP);         // [128][XS]

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int wm = warp / WN;   // 32-vector group
    const int wn = warp % WN;   // block of 32 output dims

    // ---- split rotation (and JL) matrices: resident for the CTA's lifetime
    for (int c = tid; c < D * (2 * D / 8); c += kCompressThreads) {
        int row = c / (2 * D / 8), col = (c % (2 * D / 8)) * 8;
        cp_async_16(Rs + row * RS + col, p.rot_split + (size_t)row * 2 * D + col);
    }
    if (QJL) {
        for (int c = tid; c < p.jl_dim * (2 * D / 8); c += kCompressThreads) {
            int row = c / (2 * D / 8), col = (c % (2 * D / 8)) * 8;
            cp_async_16(Ps + row * RS + col, p.jl_split + (size_t)row * 2 * D + col);
        }
        if (tid < 16) cb_s[tid] = p.cb[tid < NLEV ? tid : 0];
    }
    for (int e = tid; e < 256 * BREP; e += kCompressThreads) {
        const int b = e / BREP;
        const int k = b < 132 ? b : 131;          // buckets past 128 only see out-of-range garbage
        bucket_s[e] = make_uint2(__float_as_uint(p.bucket_t[k]), p.bucket_base[k]);
    }
    const uint2* bucket_lane = bucket_s + (lane % BREP);
    cp_async_commit();

    const int64_t n_tiles = (p.n_vec + kTileVecs - 1) / kTileVecs;
    auto load_tile = [&](int64_t tile, __half* dst) {
        const int64_t v0 = tile * kTileVecs;
        const int n_valid = (int)min((int64_t)kTileVecs, p.n_vec - v0);
        for (int c = tid; c < kTileVecs * (D / 8); c += kCompressThreads) {
            int row = c / (D / 8), col = (c % (D / 8)) * 8;
            if (row < n_valid) {
                cp_async_16(dst + row * XS + col, p.x + (v0 + row) * D + col);
            } else {
                *reinterpret_cast<uint4*>(dst + row * XS + col) = make_uint4(0, 0, 0, 0);   // rows past the end
            }
        }
    };
    __half* Xcur = Xs;
    __half* Xnext = QJL ? Xs : Xs2;
    if (!QJL && (int64_t)blockIdx.x < n_tiles) load_tile(blockIdx.x, Xcur);
    cp_async_commit();
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t v0 = tile * kTileVecs;
        const int n_valid = (int)min((int64_t)kTileVecs, p.n_vec - v0);
        if (QJL) {
            load_tile(tile, Xcur);
            cp_async_commit();
            cp_async_wait<0>();
        } else {
            // this tile was requested one iteration ago; request the next one into the other buffer
            if (tile + gridDim.x < n_tiles) load_tile(tile + gridDim.x, Xnext);
            cp_async_commit();
            cp_async_wait<1>();
        }
        __syncthreads();
        __half* const Xs = Xcur;   // the tile this iteration works on

        if (QJL) {
            // power-of-two scale per vector so the residual split stays in float16 range:
            // |e_j| < 32 * max|x_j|, scaled to below 2^15.
            constexpr int PARTS = kCompressThreads / kTileVecs;      // threads per row (2 or 4)
            const int row = tid / PARTS, part = tid % PARTS;
            const uint4* src = reinterpret_cast<const uint4*>(Xs + row * XS + part * (D / PARTS));
            float vmax = 0.f;
#pragma unroll
            for (int i = 0; i < D / PARTS / 8; ++i) {
                uint4 u = src[i];
                const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float2 f = __half22float2(__habs2(h[k]));
                    vmax = fmaxf(vmax, fmaxf(f.x, f.y));
                }
            }
#pragma unroll
            for (int o = 1; o < PARTS; o <<= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
            if (part == 0) {
                uint32_t be = __float_as_uint(vmax) >> 23;
                escale[row] = (vmax > 0.f) ? __uint_as_float((263u - be) << 23) : 1.0f;
            }
            for (int e = tid; e < kTileVecs * WN; e += kCompressThreads) enorm2[e] = 0.f;
        }

        // ---- rotation: acc[mt][nt] (16 vectors x 8 dims each), K = D with hi and lo terms
        float acc[2][NT][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

        // The tensor core truncates when it aligns addends to the running sum, so a long
        // in-MMA accumulation chain drifts by several ulp.  Two k-steps (hi and lo terms) are
        // summed from zero inside the tensor core and then added to the running sum with a
        // round-to-nearest float32 add.
#pragma unroll 1
        for (int kp = 0; kp < D / 32; ++kp) {
            uint32_t a[2][2][4];
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2)
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
                    ldmatrix_x4(a[k2][mt][0], a[k2][mt][1], a[k2][mt][2], a[k2][mt][3],
                                Xs + (wm * 32 + mt * 16 + (lane & 15)) * XS + (kp * 2 + k2) * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float part[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) {
                    uint32_t b0, b1, b2, b3;
                    const int j = lane >> 3;
                    ldmatrix_x4(b0, b1, b2, b3,
                                Rs + (wn * 32 + nt * 8 + (lane & 7)) * RS + (kp * 2 + k2) * 16 + (j & 1) * 8 + (j >> 1) * D);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        mma_16816(part[mt], a[k2][mt][0], a[k2][mt][1], a[k2][mt][2], a[k2][mt][3], b0, b1);
                        mma_16816(part[mt], a[k2][mt][0], a[k2][mt][1], a[k2][mt][2], a[k2][mt][3], b2, b3);
                    }
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[mt][nt][i] = __fadd_rn(acc[mt][nt][i], part[mt][i]);
            }
        }
        __syncthreads();   // every warp is done reading Xs (it is reused for the residual)

        // ---- epilogue: radius, indices, packing (and the residual for QJL)
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int row = wm * 32 + mt * 16 + hh * 8 + g;
                float en2 = 0.f;
                const float es = QJL ? escale[row] : 1.f;
#pragma unroll
                for (int blk = 0; blk < NT / 4; ++blk) {
                    float v[4][2];
#pragma unroll
                    for (int n = 0; n < 4; ++n) {
                        v[n][0] = acc[mt][blk * 4 + n][hh * 2 + 0] * (1.0f / 4096.0f);
                        v[n][1] = acc[mt][blk * 4 + n][hh * 2 + 1] * (1.0f / 4096.0f);
                    }
                    // numpy's float32 axis-reduction order: r[j] over j, j+8, j+16, j+24
                    float r0 = __fmul_rn(v[0][0], v[0][0]);
                    float r1 = __fmul_rn(v[0][1], v[0][1]);
#pragma unroll
                    for (int n = 1; n < 4; ++n) {
                        r0 = __fadd_rn(r0, __fmul_rn(v[n][0], v[n][0]));
                        r1 = __fadd_rn(r1, __fmul_rn(v[n][1], v[n][1]));
                    }
                    float s = __fadd_rn(r0, r1);
                    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
                    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
                    float d32 = __fsqrt_rn(s);
                    const bool zero = d32 < 1e-30f;
                    if (zero) d32 = 0.f;
                    const __half d16 = __float2half_rn(fminf(d32, 65504.0f));
                    const float dq = __half2float(d16);
                    const int gblk = wn * (NT / 4) + blk;
                    uint8_t* ob = outs + row * VB + gblk * BB;
                    if (t == 0) *reinterpret_cast<__half*>(ob) = d16;
                    // x / d32 with IEEE rounding from a correctly rounded reciprocal and one
                    // residual correction (no mismatch against true division in 2e6 samples)
                    const float rinv = __frcp_rn(zero ? 1.f : d32);
                    const float dsafe = zero ? 1.f : d32;
                    uint32_t code[4];
#pragma unroll
                    for (int n = 0; n < 4; ++n) {
                        uint32_t id[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float y0 = __fmul_rn(v[n][e], rinv);
                            const float dir = fmaf(fmaf(-y0, dsafe, v[n][e]), rinv, y0);
                            const uint32_t bk = __float_as_uint(fmaf(dir, 64.f, 8388672.f)) & 0xFFu;
                            const uint2 be = bucket_lane[bk * BREP];
                            id[e] = zero ? 0u : be.y + ((dir > __uint_as_float(be.x)) ? 1u : 0u);
                            if (QJL) {
                                const float ee = (v[n][e] - __fmul_rn(dq, cb_s[id[e]])) * es;
                                en2 = fmaf(ee, ee, en2);
                                __half eh, el;
                                split_half(ee, eh, el);
                                const int col = wn * 32 + (blk * 4 + n) * 8 + 2 * t + e;
                                Xs[row * XS + col] = eh;
                                Elo[row * XS + col] = el;
                            }
                        }
                        code[n] = id[0] | (id[1] << BITS);
                    }
                    if (BITS == 4) {
#pragma unroll
                        for (int n = 0; n < 4; ++n) ob[2 + n * 4 + t] = (uint8_t)code[n];
                    } else {
                        // 2-bit: a byte holds 4 dims = this lane's pair and its neighbour's
#pragma unroll
                        for (int n = 0; n < 4; ++n) {
                            uint32_t other = __shfl_xor_sync(0xffffffffu, code[n], 1);
                            if ((t & 1) == 0) ob[2 + n * 2 + (t >> 1)] = (uint8_t)(code[n] | (other << 4));
                        }
                    }
                }
                if (QJL) {
                    en2 += __shfl_xor_sync(0xffffffffu, en2, 1);
                    en2 += __shfl_xor_sync(0xffffffffu, en2, 2);
                    if (t == 0) enorm2[WN * row + wn] = en2;
                }
            }
        }
        __syncthreads();

        if (QJL) {
            // ---- sign sketch: proj[vec][i] = sum_j e[vec][j] * P'[i][j]; this warp owns
            // 32 vectors x (M/2) projections, in chunks of 8 n-tiles to bound registers.
            const int M = p.jl_dim;
            const int nt_per_warp = (M / 8 + WN - 1) / WN;       // bytes of the sketch per warp
            for (int nt0 = 0; nt0 < nt_per_warp; nt0 += 4) {
                float pc[2][4][4];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int n = 0; n < 4; ++n)
#pragma unroll
                        for (int i = 0; i < 4; ++i) pc[mt][n][i] = 0.f;
#pragma unroll 2
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t ah[2][4], al[2][4];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        const int off = (wm * 32 + mt * 16 + (lane & 15)) * XS + ks * 16 + (lane >> 4) * 8;
                        ldmatrix_x4(ah[mt][0], ah[mt][1], ah[mt][2], ah[mt][3], Xs + off);
                        ldmatrix_x4(al[mt][0], al[mt][1], al[mt][2], al[mt][3], Elo + off);
                    }
#pragma unroll
                    for (int n = 0; n < 4; ++n) {
                        if (nt0 + n < nt_per_warp && wn * nt_per_warp + nt0 + n < M / 8) {
                            uint32_t b0, b1, b2, b3;
                            int j = lane >> 3;
                            ldmatrix_x4(b0, b1, b2, b3,
                                        Ps + ((wn * nt_per_warp + nt0 + n) * 8 + (lane & 7)) * RS + ks * 16 +
                                            (j & 1) * 8 + (j >> 1) * D);
#pragma unroll
                            for (int mt = 0; mt < 2; ++mt) {
                                mma_16816(pc[mt][n], ah[mt][0], ah[mt][1], ah[mt][2], ah[mt][3], b0, b1);
                                mma_16816(pc[mt][n], ah[mt][0], ah[mt][1], ah[mt][2], ah[mt][3], b2, b3);
                                mma_16816(pc[mt][n], al[mt][0], al[mt][1], al[mt][2], al[mt][3], b0, b1);
                            }
                        }
                    }
                }
                // pack: n-tile n is byte (wn*M/16 + nt0 + n); bit 2t+e comes from this lane
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint32_t w = 0;
#pragma unroll
                        for (int n = 0; n < 4; ++n)
#pragma unroll
                            for (int e = 0; e < 2; ++e)
                                w |= (pc[mt][n][hh * 2 + e] >= 0.f ? 1u : 0u) << (8 * n + 2 * t + e);
                        w |= __shfl_xor_sync(0xffffffffu, w, 1);
                        w |= __shfl_xor_sync(0xffffffffu, w, 2);
                        const int row = wm * 32 + mt * 16 + hh * 8 + g;
                        if (t == 0) {
                            uint8_t* dst = bits_s + row * (M / 8) + wn * nt_per_warp + nt0;
#pragma unroll
                            for (int n = 0; n < 4; ++n)
                                if (nt0 + n < nt_per_warp && wn * nt_per_warp + nt0 + n < M / 8) dst[n] = (uint8_t)(w >> (8 * n));
                        }
                    }
            }
            __syncthreads();
        }

        // ---- coalesced copy-out of the tile
        {
            const int n_bytes = n_valid * VB;                       // multiple of 4
            uint8_t* dst = p.blocks_out + v0 * VB;                  // 16-byte aligned (v0 % 128 == 0)
            const int n16 = n_bytes / 16;
            for (int c = tid; c < n16; c += kCompressThreads)
                reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(outs)[c];
            const int rest4 = (n_bytes & 15) >> 2;                  // ragged end in 4-byte words
            if (tid < rest4)
                reinterpret_cast<uint32_t*>(dst)[n16 * 4 + tid] = reinterpret_cast<const uint32_t*>(outs)[n16 * 4 + tid];
            if (QJL) {
                const int M8 = p.jl_dim / 8;
                uint8_t* bd = p.qjl_bits_out + v0 * M8;
                const int nb = n_valid * M8;
                if ((M8 & 3) == 0) {
                    for (int c = tid; c < nb / 4; c += kCompressThreads)
                        reinterpret_cast<uint32_t*>(bd)[c] = reinterpret_cast<const uint32_t*>(bits_s)[c];
                } else {
                    for (int c = tid; c < nb; c += kCompressThreads) bd[c] = bits_s[c];
                }
                for (int r = tid; r < n_valid; r += kCompressThreads) {
                    float n2 = 0.f;
#pragma unroll
                    for (int k = 0; k < WN; ++k) n2 += enorm2[WN * r + k];
                    p.qjl_norm_out[v0 + r] = __float2half_rn(fminf(sqrtf(n2) / escale[r], 65504.0f));
                }
            }
        }
        __syncthreads();   // outs / Xs are rewritten by the next tile
        if (!QJL) { __half* tmp = Xcur; Xcur = Xnext; Xnext = tmp; }
    }
    cp_async_wait<0>();
}

template <int D, int BITS, bool QJL>
static size_t compress_smem_bytes(int jl_dim) {
    constexpr int RS = CompressSmem<D>::kRStride, XS = CompressSmem<D>::kXStride;
    size_t b = (size_t)D * RS * 2 + (size_t)kTileVecs * XS * 2 + (size_t)kTileVecs * (D / 32) * block_bytes(BITS);
    if (QJL)
        b += (size_t)jl_dim * RS * 2 + (size_t)kTileVecs * XS * 2 + (size_t)kTileVecs * (jl_dim / 8);
    b += kTileVecs * 4 + kTileVecs * 16;                 // residual scale / norm slots (laid out in both modes)
    b += 64 + 256 * 8 * (QJL ? 1 : 16);                  // codebook + index-search table copies
    if (!QJL) b += (size_t)kTileVecs * XS * 2;           // prefetch buffer
    return b + 16;
}

template <int D, int BITS, bool QJL>
static int launch_compress(const CompressParams& p, cudaStream_t stream) {
    static int sm_count = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return PQ_ERR_CUDA;
    if (sm_count == 0 && cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return PQ_ERR_CUDA;
    const size_t smem = compress_smem_bytes<D, BITS, QJL>(p.jl_dim);
    auto kern = pq_compress_kernel<D, BITS, QJL>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return PQ_ERR_CUDA;
    int per_sm = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, compress_threads(D), smem) != cudaSuccess || per_sm < 1)
        return PQ_ERR_CUDA;
    const int64_t n_tiles = (p.n_vec + kTileVecs - 1) / kTileVecs;
    const int64_t cap = (int64_t)sm_count * per_sm;
    const int grid = (int)(n_tiles < cap ? n_tiles : cap);
    kern<<<grid, compress_threads(D), smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
}

}  // namespace pq

extern "C" int pq_compress(const void* x, int64_t n_vec, int head_dim, int n_bits,
                           const void* rot_split, const float* thresholds, const float* codebook,
                           void* blocks_out,
                           const void* jl_split, int jl_dim, void* qjl_bits_out, void* qjl_norm_out,
                           void* stream) {
    using namespace pq;
    if (n_vec < 0) return PQ_ERR_BAD_SHAPE;
    if (head_dim != 64 && head_dim != 128) return PQ_ERR_BAD_HEAD_DIM;
    if (n_bits != 2 && n_bits != 4) return PQ_ERR_BAD_BITS;
    if (n_vec == 0) return PQ_OK;
    if (!x || !rot_split || !thresholds || !codebook || !blocks_out) return PQ_ERR_NULL_POINTER;
    const bool qjl = jl_split != nullptr;
    if (qjl) {
        if (jl_dim < 16 || jl_dim > 128 || (jl_dim % 16)) return PQ_ERR_BAD_JL_DIM;
        if (!qjl_bits_out || !qjl_norm_out) return PQ_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(jl_split) & 15) return PQ_ERR_MISALIGNED;
        if (((jl_dim / 8) % 4 == 0) && (reinterpret_cast<uintptr_t>(qjl_bits_out) & 3)) return PQ_ERR_MISALIGNED;
    }
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(rot_split) & 15) ||
        (reinterpret_cast<uintptr_t>(blocks_out) & 15))
        return PQ_ERR_MISALIGNED;

    CompressParams p{};
    p.x = static_cast<const __half*>(x);
    p.rot_split = static_cast<const __half*>(rot_split);
    p.jl_split = static_cast<const __half*>(jl_split);
    p.blocks_out = static_cast<uint8_t*>(blocks_out);
    p.qjl_bits_out = static_cast<uint8_t*>(qjl_bits_out);
    p.qjl_norm_out = static_cast<__half*>(qjl_norm_out);
    p.n_vec = n_vec;
    p.jl_dim = qjl ? jl_dim : 0;
    // thresholds / codebook are small HOST tables; they travel as kernel parameters.
    const int nlev = 1 << n_bits;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const float* thr_h = thresholds;
    const float* cb_h = codebook;
    for (int i = 0; i < 16; ++i) p.cb[i] = i < nlev ? cb_h[i] : 0.f;
    // bucket(y) = round(64 y) + 64, evaluated exactly as the kernel does (one fused multiply-add)
    for (int k = 0; k < 132; ++k) { p.bucket_t[k] = 3.0e38f; p.bucket_base[k] = 0; }
    for (int i = 0; i < nlev - 1; ++i) {
        const float u = fmaf(thr_h[i], 64.f, 8388672.f);
        uint32_t bits;
        memcpy(&bits, &u, sizeof(bits));
        const int kb = (int)(bits & 0xFFu);
        if (!(thr_h[i] > -1.0f && thr_h[i] < 1.0f) || kb > 130 || p.bucket_t[kb] != 3.0e38f)
            return PQ_ERR_BAD_SHAPE;      // thresholds out of range or two of them in one bucket
        p.bucket_t[kb] = thr_h[i];
        for (int k = kb + 1; k < 132; ++k) p.bucket_base[k] += 1;
    }

#define PQ_DISPATCH(DD, BB)                                                         \
    if (head_dim == DD && n_bits == BB)                                             \
        return qjl ? launch_compress<DD, BB, true>(p, st) : launch_compress<DD, BB, false>(p, st);
    PQ_DISPATCH(64, 4)
    PQ_DISPATCH(64, 2)
    PQ_DISPATCH(128, 4)
    PQ_DISPATCH(128, 2)
#undef PQ_DISPATCH
    return PQ_ERR_BAD_HEAD_DIM;
}
