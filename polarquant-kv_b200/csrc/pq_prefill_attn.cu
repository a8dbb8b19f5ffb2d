// pq_prefill_attn: seq_q >= 1 query tokens per head against a block_pq4 cache.
//
// Same rotated-space arithmetic as the decode kernel (softmax(q K^T * scale) V evaluated on
// centroid * radius values, python/polarquant_kv/attention.py:111-163), organised for many
// query rows: a CTA owns 128 query rows of one KV head (rows = (query head, position)
// pairs of the GQA group, 16 per warp) and walks the sequence in tiles of 32 tokens.
// Each tile of K and V is dequantised ONCE per CTA into shared memory as two float16 terms
// (value = hi + lo, about 22 bits) and both contractions run on tensor cores
// (mma.sync.m16n8k16, float32 accumulate) as three-term products hi*hi + hi*lo + lo*hi,
// which keeps float32-level accuracy.  Online softmax in registers; the result is
// normalised and rotated back (o @ R) through shared memory.
//
// causal == 0 reproduces the reference (no mask, src/polarquant_kv_cuda/attention_kernel.py:
// 92-113); causal == 1 lets query position i see tokens [0, seq_len - seq_q + i].
#include "pq_common.cuh"

namespace pq {

constexpr int kPfWarps = 8;
constexpr int kPfThreads = kPfWarps * 32;
constexpr int kPfRows = kPfWarps * 16;   // query rows per CTA
constexpr int kPfTok = 32;               // tokens per KV tile

struct PrefillParams {
    const __half* q;       // [B, Hq, Sq, D]
    const uint8_t* kb;
    const uint8_t* vb;
    const float* rot;
    void* out;             // [B, Hq, Sq, D]
    int64_t S, Scap;
    int Hq, Hkv, G, Sq;
    int causal, out_is_fp16;
    float scale_log2;
    float cbk[16], cbv[16];
};

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  const void* smem_row) {
    uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// Expand `ntok` tokens of one operand into hi/lo float16 centroid tiles [kPfTok][LD] and the
// float32 radii [kPfTok][NBLK].  `tab` maps a byte of packed indices to its centroids:
// 4-bit: uint2 {half2 hi, half2 lo}; 2-bit: uint4 {hi01, hi23, lo01, lo23}.
template <int D, int BITS, int LD>
__device__ __forceinline__ void dequant_tile(const uint8_t* __restrict__ src, int ntok, const uint8_t* tab,
                                             __half* hi, __half* lo, float* dd, int tid) {
    constexpr int NBLK = D / 32, BB = block_bytes(BITS), TB = NBLK * BB;
    if (BITS == 4) {
        // work item: 32 bits of indices = 8 elements
        for (int w = tid; w < kPfTok * NBLK * 4; w += kPfThreads) {
            const int tok = w / (NBLK * 4), rem = w % (NBLK * 4), blk = rem >> 2, qw = rem & 3;
            uint4 vh = make_uint4(0, 0, 0, 0), vl = make_uint4(0, 0, 0, 0);
            if (tok < ntok) {
                const uint8_t* b = src + (size_t)tok * TB + blk * BB;
                const uint16_t* p16 = reinterpret_cast<const uint16_t*>(b + 2 + qw * 4);
                const uint32_t bits = (uint32_t)p16[0] | ((uint32_t)p16[1] << 16);
                const uint2 e0 = reinterpret_cast<const uint2*>(tab)[bits & 0xFF];
                const uint2 e1 = reinterpret_cast<const uint2*>(tab)[(bits >> 8) & 0xFF];
                const uint2 e2 = reinterpret_cast<const uint2*>(tab)[(bits >> 16) & 0xFF];
                const uint2 e3 = reinterpret_cast<const uint2*>(tab)[bits >> 24];
                vh = make_uint4(e0.x, e1.x, e2.x, e3.x);
                vl = make_uint4(e0.y, e1.y, e2.y, e3.y);
                if (qw == 0) dd[tok * NBLK + blk] = __half2float(*reinterpret_cast<const __half*>(b));
            } else if (qw == 0) {
                dd[tok * NBLK + blk] = 0.f;
            }
            *reinterpret_cast<uint4*>(hi + tok * LD + blk * 32 + qw * 8) = vh;
            *reinterpret_cast<uint4*>(lo + tok * LD + blk * 32 + qw * 8) = vl;
        }
    } else {
        // work item: 16 bits of indices = 8 elements
        for (int w = tid; w < kPfTok * NBLK * 4; w += kPfThreads) {
            const int tok = w / (NBLK * 4), rem = w % (NBLK * 4), blk = rem >> 2, qw = rem & 3;
            uint4 vh = make_uint4(0, 0, 0, 0), vl = make_uint4(0, 0, 0, 0);
            if (tok < ntok) {
                const uint8_t* b = src + (size_t)tok * TB + blk * BB;
                const uint32_t bits = *reinterpret_cast<const uint16_t*>(b + 2 + qw * 2);
                const uint4 e0 = reinterpret_cast<const uint4*>(tab)[bits & 0xFF];
                const uint4 e1 = reinterpret_cast<const uint4*>(tab)[bits >> 8];
                vh = make_uint4(e0.x, e0.y, e1.x, e1.y);
                vl = make_uint4(e0.z, e0.w, e1.z, e1.w);
                if (qw == 0) dd[tok * NBLK + blk] = __half2float(*reinterpret_cast<const __half*>(b));
            } else if (qw == 0) {
                dd[tok * NBLK + blk] = 0.f;
            }
            *reinterpret_cast<uint4*>(hi + tok * LD + blk * 32 + qw * 8) = vh;
            *reinterpret_cast<uint4*>(lo + tok * LD + blk * 32 + qw * 8) = vl;
        }
    }
}

// Byte -> centroid table (not replicated: the tile expansion is a small part of the work).
template <int BITS>
__device__ __forceinline__ void build_byte_table(uint8_t* tab, const float* cb, int tid) {
    for (int b = tid; b < 256; b += kPfThreads) {
        if (BITS == 4) {
            __half h0, l0, h1, l1;
            split_half(cb[b & 15] * 64.0f, h0, l0);
            split_half(cb[b >> 4] * 64.0f, h1, l1);
            __half2 hi = __halves2half2(h0, h1), lo = __halves2half2(l0, l1);
            reinterpret_cast<uint2*>(tab)[b] =
                make_uint2(*reinterpret_cast<uint32_t*>(&hi), *reinterpret_cast<uint32_t*>(&lo));
        } else {
            __half h[4], l[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) split_half(cb[(b >> (2 * k)) & 3] * 64.0f, h[k], l[k]);
            __half2 h01 = __halves2half2(h[0], h[1]), h23 = __halves2half2(h[2], h[3]);
            __half2 l01 = __halves2half2(l[0], l[1]), l23 = __halves2half2(l[2], l[3]);
            reinterpret_cast<uint4*>(tab)[b] =
                make_uint4(*reinterpret_cast<uint32_t*>(&h01), *reinterpret_cast<uint32_t*>(&h23),
                           *reinterpret_cast<uint32_t*>(&l01), *reinterpret_cast<uint32_t*>(&l23));
        }
    }
}

template <int D, int KBITS, int VBITS>
__global__ void __launch_bounds__(kPfThreads, 1) pq_prefill_attn_kernel(const PrefillParams p) {
    constexpr int NBLK = D / 32;
    constexpr int LD = D + 8;                         // padded row (halves) of the K/V tiles
    constexpr int TBK = NBLK * block_bytes(KBITS), TBV = NBLK * block_bytes(VBITS);
    constexpr int KSTEPS = D / 16;
    constexpr int NT_O = D / 8;

    extern __shared__ __align__(16) uint8_t smem[];
    __half* Khi = reinterpret_cast<__half*>(smem);            // [32][LD]
    __half* Klo = Khi + kPfTok * LD;
    __half* Vhi = Klo + kPfTok * LD;
    __half* Vlo = Vhi + kPfTok * LD;
    __half* Qhi = Vlo + kPfTok * LD;                          // [128][LD]
    __half* Qlo = Qhi + kPfRows * LD;
    float* stage = reinterpret_cast<float*>(Qhi);             // [128][D+4] float, reuses Q tiles at the end
    __shared__ float cbk_s[16], cbv_s[16];
    __shared__ float dK[kPfTok * NBLK], dV[kPfTok * NBLK];
    __shared__ __align__(16) uint8_t tabk[4096], tabv[4096];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row_tile = blockIdx.x, kvrow = blockIdx.y;
    const int b = kvrow / p.Hkv, hkv = kvrow % p.Hkv;
    const int n_rows = p.G * p.Sq;                            // query rows sharing this KV head
    const int row0 = row_tile * kPfRows;

    if (tid < 16) { cbk_s[tid] = p.cbk[tid]; cbv_s[tid] = p.cbv[tid]; }
    __syncthreads();
    build_byte_table<KBITS>(tabk, cbk_s, tid);
    build_byte_table<VBITS>(tabv, cbv_s, tid);

    // ---- rotate the CTA's query rows: q_rot = q @ R^T, scaled by scale*log2(e), split hi/lo
    for (int e = tid; e < kPfRows * D; e += kPfThreads) {
        const int r = e / D, i = e % D;
        const int row = row0 + r;
        float acc = 0.f;
        if (row < n_rows) {
            const int head = hkv * p.G + row / p.Sq, sq = row % p.Sq;
            const __half2* qv = reinterpret_cast<const __half2*>(p.q + (((size_t)b * p.Hq + head) * p.Sq + sq) * D);
            const float2* rv = reinterpret_cast<const float2*>(p.rot + (size_t)i * D);
#pragma unroll 8
            for (int j = 0; j < D / 2; ++j) {
                const float2 qq = __half22float2(qv[j]);
                const float2 rr = __ldg(rv + j);
                acc = fmaf(qq.x, rr.x, acc);
                acc = fmaf(qq.y, rr.y, acc);
            }
            acc *= p.scale_log2;
        }
        __half h, l;
        split_half(acc, h, l);
        Qhi[r * LD + i] = h;
        Qlo[r * LD + i] = l;
    }
    __syncthreads();

    uint32_t qh[KSTEPS][4], ql[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        const int off = (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8;
        ldmatrix_x4(qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], Qhi + off);
        ldmatrix_x4(ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], Qlo + off);
    }

    // per-thread rows: g and g+8 of the warp's 16
    int limit[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int row = row0 + warp * 16 + hh * 8 + g;
        const int sq = row % p.Sq;
        limit[hh] = p.causal ? (int)(p.S - p.Sq + sq + 1) : (int)p.S;      // tokens [0, limit)
        if (row >= n_rows) limit[hh] = 0;
    }
    // the CTA can stop after the largest limit among its rows
    int64_t kv_end = p.S;
    if (p.causal) {
        const int last_row = min(row0 + kPfRows, n_rows) - 1;
        // rows are (head, position) pairs; a tile may span several heads, so take the max
        int max_sq = 0;
        if (row0 / p.Sq != last_row / p.Sq) max_sq = p.Sq - 1;
        else max_sq = last_row % p.Sq;
        kv_end = p.S - p.Sq + max_sq + 1;
        if (kv_end > p.S) kv_end = p.S;
        if (kv_end < 0) kv_end = 0;
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

    const uint8_t* k_row = p.kb + (size_t)kvrow * p.Scap * TBK;
    const uint8_t* v_row = p.vb + (size_t)kvrow * p.Scap * TBV;

    for (int64_t tok0 = 0; tok0 < kv_end; tok0 += kPfTok) {
        const int ntok = (p.S - tok0) < kPfTok ? (int)(p.S - tok0) : kPfTok;
        __syncthreads();   // previous tile fully consumed
        dequant_tile<D, KBITS, LD>(k_row + tok0 * TBK, ntok, tabk, Khi, Klo, dK, tid);
        dequant_tile<D, VBITS, LD>(v_row + tok0 * TBV, ntok, tabv, Vhi, Vlo, dV, tid);
        __syncthreads();

        // ---- S = Q K^T : 16 rows x 32 tokens per warp, one 32-dim block at a time so the
        // block radius can scale the partial sums in float32
        float s[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
        for (int blk = 0; blk < NBLK; ++blk) {
            float c[4][4];
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) c[n][i] = 0.f;
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {
                const int ks = blk * 2 + k2;
#pragma unroll
                for (int n = 0; n < 4; n += 2) {
                    // two token n-tiles per ldmatrix: (tok n*8.., k 0-7), (.., k 8-15), (tok (n+1)*8.., ..)
                    uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
                    const int j = lane >> 3;
                    const int off = ((n + (j >> 1)) * 8 + (lane & 7)) * LD + ks * 16 + (j & 1) * 8;
                    ldmatrix_x4(h0, h1, h2, h3, Khi + off);
                    ldmatrix_x4(l0, l1, l2, l3, Klo + off);
                    mma_16816(c[n], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], h0, h1);
                    mma_16816(c[n], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], l0, l1);
                    mma_16816(c[n], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], h0, h1);
                    mma_16816(c[n + 1], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], h2, h3);
                    mma_16816(c[n + 1], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], l2, l3);
                    mma_16816(c[n + 1], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], h2, h3);
                }
            }
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const float d0 = dK[(n * 8 + 2 * t) * NBLK + blk] * (1.0f / 64.0f);
                const float d1 = dK[(n * 8 + 2 * t + 1) * NBLK + blk] * (1.0f / 64.0f);
                s[n][0] = fmaf(d0, c[n][0], s[n][0]);
                s[n][1] = fmaf(d1, c[n][1], s[n][1]);
                s[n][2] = fmaf(d0, c[n][2], s[n][2]);
                s[n][3] = fmaf(d1, c[n][3], s[n][3]);
            }
        }
        // ---- mask, online softmax (rows g and g+8)
    #pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float mx = -INFINITY;
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int tok = (int)tok0 + n * 8 + 2 * t + e;
                    if (tok >= limit[hh]) s[n][hh * 2 + e] = -INFINITY;
                    mx = fmaxf(mx, s[n][hh * 2 + e]);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[hh], mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = fast_exp2(m_run[hh] - m_use);
            float sum = 0.f;
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pv = fast_exp2(s[n][hh * 2 + e] - m_use);
                    s[n][hh * 2 + e] = pv;
                    sum += pv;
                }
            l_run[hh] = l_run[hh] * alpha + sum;
            m_run[hh] = m_new;
#pragma unroll
            for (int n = 0; n < NT_O; ++n) {
                o[n][hh * 2 + 0] *= alpha;
                o[n][hh * 2 + 1] *= alpha;
            }
        }
        // ---- O += P V, one 32-dim block at a time: the value radius of (token, block) is
        // folded into P before the float16 split.  C fragments of P map onto A fragments:
        // k-step kk covers token n-tiles 2kk and 2kk+1.
#pragma unroll
        for (int blk = 0; blk < NBLK; ++blk) {
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                uint32_t pah[4], pal[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    // r: 0 -> (row g, n-tile 2kk), 1 -> (row g+8, 2kk), 2 -> (row g, 2kk+1), 3 -> (row g+8, 2kk+1)
                    const int n = 2 * kk + (r >> 1), hh = r & 1;
                    const float d0 = dV[(n * 8 + 2 * t) * NBLK + blk];
                    const float d1 = dV[(n * 8 + 2 * t + 1) * NBLK + blk];
                    __half h0, l0, h1, l1;
                    split_half(s[n][hh * 2 + 0] * d0, h0, l0);
                    split_half(s[n][hh * 2 + 1] * d1, h1, l1);
                    __half2 hv = __halves2half2(h0, h1), lv = __halves2half2(l0, l1);
                    pah[r] = *reinterpret_cast<uint32_t*>(&hv);
                    pal[r] = *reinterpret_cast<uint32_t*>(&lv);
                }
#pragma unroll
                for (int nn = 0; nn < 4; nn += 2) {
                    const int n = blk * 4 + nn;
                    uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
                    const int j = lane >> 3;
                    const int off = (kk * 16 + (j & 1) * 8 + (lane & 7)) * LD + (n + (j >> 1)) * 8;
                    ldmatrix_x4_trans(h0, h1, h2, h3, Vhi + off);
                    ldmatrix_x4_trans(l0, l1, l2, l3, Vlo + off);
                    mma_16816(o[n], pah[0], pah[1], pah[2], pah[3], h0, h1);
                    mma_16816(o[n], pah[0], pah[1], pah[2], pah[3], l0, l1);
                    mma_16816(o[n], pal[0], pal[1], pal[2], pal[3], h0, h1);
                    mma_16816(o[n + 1], pah[0], pah[1], pah[2], pah[3], h2, h3);
                    mma_16816(o[n + 1], pah[0], pah[1], pah[2], pah[3], l2, l3);
                    mma_16816(o[n + 1], pal[0], pal[1], pal[2], pal[3], h2, h3);
                }
            }
        }
    }

    // ---- normalise, stage in shared memory, rotate back: out = o_rot @ R
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
    __syncthreads();   // Q tiles are dead (fragments live in registers); reuse them as the stage
    constexpr int SLD = D + 4;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const float inv = l_run[hh] > 0.f ? (1.0f / 64.0f) / l_run[hh] : 0.f;
        float* dst = stage + (warp * 16 + hh * 8 + g) * SLD;
#pragma unroll
        for (int n = 0; n < NT_O; ++n) {
            dst[n * 8 + 2 * t + 0] = o[n][hh * 2 + 0] * inv;
            dst[n * 8 + 2 * t + 1] = o[n][hh * 2 + 1] * inv;
        }
    }
    __syncthreads();
    for (int e = tid; e < kPfRows * D; e += kPfThreads) {
        const int r = e / D, i = e % D;
        const int row = row0 + r;
        if (row >= n_rows) continue;
        const float* src = stage + r * SLD;
        float acc = 0.f;
#pragma unroll 8
        for (int j = 0; j < D; ++j) acc = fmaf(src[j], __ldg(p.rot + (size_t)j * D + i), acc);
        const int head = hkv * p.G + row / p.Sq, sq = row % p.Sq;
        const size_t off = (((size_t)b * p.Hq + head) * p.Sq + sq) * D + i;
        if (p.out_is_fp16) static_cast<__half*>(p.out)[off] = __float2half_rn(fminf(fmaxf(acc, -65504.f), 65504.f));
        else static_cast<float*>(p.out)[off] = acc;
    }
}

template <int D, int KBITS, int VBITS>
static int launch_prefill(const PrefillParams& p, int rows, cudaStream_t st) {
    constexpr int LD = D + 8;
    const size_t tiles = (size_t)4 * kPfTok * LD * 2;
    const size_t qtiles = (size_t)2 * kPfRows * LD * 2;
    const size_t stage = (size_t)kPfRows * (D + 4) * 4;
    const size_t smem = tiles + (qtiles > stage ? qtiles : stage) + 16;
    auto kern = pq_prefill_attn_kernel<D, KBITS, VBITS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return PQ_ERR_CUDA;
    const int n_rows = p.G * p.Sq;
    dim3 grid((n_rows + kPfRows - 1) / kPfRows, rows, 1);
    kern<<<grid, kPfThreads, smem, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
}

}  // namespace pq

extern "C" int pq_prefill_attn(const void* q, const void* k_blocks, const void* v_blocks,
                               int batch, int q_heads, int kv_heads, int seq_q, int64_t seq_len,
                               int64_t seq_capacity, int head_dim, int k_bits, int v_bits,
                               const float* codebook_k, const float* codebook_v, const float* rot,
                               float scale, int causal, void* out, int out_is_fp16, void* stream) {
    using namespace pq;
    if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || seq_q < 0 || seq_len < 0 ||
        seq_capacity < seq_len)
        return PQ_ERR_BAD_SHAPE;
    if (head_dim != 64 && head_dim != 128) return PQ_ERR_BAD_HEAD_DIM;
    if ((k_bits != 2 && k_bits != 4) || (v_bits != 2 && v_bits != 4)) return PQ_ERR_BAD_BITS;
    if (batch == 0 || seq_q == 0) return PQ_OK;
    if (!q || !rot || !codebook_k || !codebook_v || !out) return PQ_ERR_NULL_POINTER;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (seq_len == 0) {
        const size_t n = (size_t)batch * q_heads * seq_q * head_dim * (out_is_fp16 ? 2 : 4);
        return cudaMemsetAsync(out, 0, n, st) == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
    }
    if (!k_blocks || !v_blocks) return PQ_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(k_blocks) & 3) || (reinterpret_cast<uintptr_t>(v_blocks) & 3) ||
        (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(rot) & 15))
        return PQ_ERR_MISALIGNED;
    const int rows = batch * kv_heads;
    if (rows > 65535) return PQ_ERR_TOO_LARGE;
    PrefillParams p{};
    p.q = static_cast<const __half*>(q);
    p.kb = static_cast<const uint8_t*>(k_blocks);
    p.vb = static_cast<const uint8_t*>(v_blocks);
    p.rot = rot;
    p.out = out;
    p.S = seq_len;
    p.Scap = seq_capacity;
    p.Hq = q_heads;
    p.Hkv = kv_heads;
    p.G = q_heads / kv_heads;
    p.Sq = seq_q;
    p.causal = causal;
    p.out_is_fp16 = out_is_fp16;
    p.scale_log2 = scale * 1.4426950408889634f;
    for (int i = 0; i < 16; ++i) {
        p.cbk[i] = i < (1 << k_bits) ? codebook_k[i] : 0.f;
        p.cbv[i] = i < (1 << v_bits) ? codebook_v[i] : 0.f;
    }
#define PQ_PF(DD, KB, VB) \
    if (head_dim == DD && k_bits == KB && v_bits == VB) return launch_prefill<DD, KB, VB>(p, rows, st);
    PQ_PF(64, 4, 4) PQ_PF(64, 4, 2) PQ_PF(64, 2, 4) PQ_PF(64, 2, 2)
    PQ_PF(128, 4, 4) PQ_PF(128, 4, 2) PQ_PF(128, 2, 4) PQ_PF(128, 2, 2)
#undef PQ_PF
    return PQ_ERR_BAD_HEAD_DIM;
}
