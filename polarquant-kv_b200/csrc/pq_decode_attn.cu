// pq_decode_attn: one query token per sequence against a block_pq4 cache, GQA-aware,
// flash-decoding split over the sequence with the (m, l, o) partials merged in-kernel.
//
// Arithmetic model (matches python/polarquant_kv/attention.py:111-163 evaluated on the
// stored blocks): attention is computed in ROTATED space.  q_rot = q @ R^T once per CTA;
// score = scale * sum_blocks d_blk * sum_j q_rot[j] * c[idx_j]; softmax; o_rot = sum_t p_t *
// d_blk * c[idx]; out = o_rot @ R.  Only packed blocks are read from HBM, each byte once per
// KV head: all query heads of a KV head (up to 8 per CTA) share it.
//
// Why tensor cores in a bandwidth-bound kernel: with G query heads per KV head the
// centroid products cost 2*G FMAs per stored nibble, more than the FP32 pipe can issue
// at HBM speed.  Both contractions therefore run as mma.sync.m16n8k16 with two-term
// float16 operands (value = hi + lo, ~22 mantissa bits) and float32 accumulation, which
// keeps the float32-level accuracy the 2e-3 output tolerance needs (a single float16
// rounding of the dequantised K is 15x too coarse on outlier-channel data).  Centroids
// come from a shared-memory table indexed by a whole byte (two nibbles / four crumbs per
// lookup, hi and lo terms in one entry), replicated per lane so lookups never conflict.
//
// Work split: grid = (n_splits, batch*kv_heads, ceil(G/8)); 8 warps per CTA; a warp owns
// 16-token tiles of its CTA's range, streamed through a private 3-stage cp.async ring.
// Each CTA reduces its warps' partials in shared memory and writes one (m, l, o) record
// per query head; the last CTA of a (row, head-group) to arrive (atomic ticket, no
// spinning) merges all records, normalises, rotates back and resets the ticket.
#include "pq_common.cuh"

namespace pq {

constexpr int kDecWarps = 8;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kTileTok = 16;
constexpr int kStages = 3;
constexpr int kHeadsPerCta = 8;
constexpr float kCbScale = 64.0f;   // centroids are stored x64 in the table (keeps lo terms normal)

struct DecodeParams {
    const __half* q;           // [B, Hq, D]
    const uint8_t* kb;         // [rows, Scap, D/32, BBk]
    const uint8_t* vb;         // [rows, Scap, D/32, BBv]
    const float* rot;          // [D, D]
    const float* jl;           // [M, D] or null
    const uint8_t* qjl_bits;   // [rows, Scap, M/8]
    const __half* qjl_norms;   // [rows, Scap]
    void* out;                 // [B, Hq, D]
    float* partial_out;        // [B, Hq, D+2] or null
    float* records;            // scratch: [rows*HG][splits][8][D+2]
    unsigned int* tickets;     // scratch: [rows*HG]
    int64_t S, Scap;
    int Hq, Hkv, G, HG;
    int splits, tiles_per_split;
    int jl_dim;
    int out_is_fp16;
    float scale_log2;          // softmax scale * log2(e)
    float cbk[16], cbv[16];
};

// ------------------------------------------------------------------ centroid tables
// 4-bit: entry(byte) = {half2(c[b&15], c[b>>4]) hi, same lo}, 8 bytes, 16 lane copies.
// 2-bit: entry(byte) = {c[b&3], c[b>>2&3] | c[b>>4&3], c[b>>6] hi ; same lo}, 16 bytes, 8 copies.
template <int BITS>
struct Table {
    static constexpr int kBytes = 32768;
    __device__ static void build(uint8_t* tab, const float* cb, int tid) {
        if (BITS == 4) {
            for (int e = tid; e < 256 * 16; e += kDecThreads) {
                const int b = e >> 4;
                __half h0, l0, h1, l1;
                split_half(cb[b & 15] * kCbScale, h0, l0);
                split_half(cb[b >> 4] * kCbScale, h1, l1);
                __half2 hi = __halves2half2(h0, h1), lo = __halves2half2(l0, l1);
                uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&hi), *reinterpret_cast<uint32_t*>(&lo));
                reinterpret_cast<uint2*>(tab)[e] = v;
            }
        } else {
            for (int e = tid; e < 256 * 8; e += kDecThreads) {
                const int b = e >> 3;
                __half h[4], l[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) split_half(cb[(b >> (2 * k)) & 3] * kCbScale, h[k], l[k]);
                __half2 h01 = __halves2half2(h[0], h[1]), h23 = __halves2half2(h[2], h[3]);
                __half2 l01 = __halves2half2(l[0], l[1]), l23 = __halves2half2(l[2], l[3]);
                uint4 v = make_uint4(*reinterpret_cast<uint32_t*>(&h01), *reinterpret_cast<uint32_t*>(&h23),
                                     *reinterpret_cast<uint32_t*>(&l01), *reinterpret_cast<uint32_t*>(&l23));
                reinterpret_cast<uint4*>(tab)[e] = v;
            }
        }
    }
};

// 4-bit lookup: byte value already multiplied by 128 (entry stride of 16 copies x 8 bytes).
__device__ __forceinline__ uint2 lut4(const uint8_t* tab_lane, uint32_t byte_x128) {
    return *reinterpret_cast<const uint2*>(tab_lane + byte_x128);
}
__device__ __forceinline__ uint4 lut2(const uint8_t* tab_lane, uint32_t byte_x128) {
    return *reinterpret_cast<const uint4*>(tab_lane + byte_x128);
}

// ------------------------------------------------------------------ tile staging
// Copies `n` bytes (multiple of 4) from global `src` (4-byte aligned) to `dst_base +
// (src & 15)`, so source and destination share their 16-byte phase; the middle goes as
// 16-byte cp.async, the ragged ends as 4-byte ones.  Returns nothing; the caller commits.
__device__ __forceinline__ void stage_bytes(uint8_t* dst_base, const uint8_t* src, int n, int lane) {
    const uint32_t phase = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src)) & 15u;
    uint8_t* dst = dst_base + phase;
    int head = phase ? (int)(16u - phase) : 0;
    if (head > n) head = n;
    const int mid = (n - head) & ~15;
    const int tail = n - head - mid;
    if (lane < (head >> 2)) {
        uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst + lane * 4));
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src + lane * 4));
    }
    for (int c = lane; c < (mid >> 4); c += 32) cp_async_16(dst + head + c * 16, src + head + c * 16);
    if (lane < (tail >> 2)) {
        uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst + head + mid + lane * 4));
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src + head + mid + lane * 4));
    }
}

// 32 bits at a 2-byte aligned shared address.
__device__ __forceinline__ uint32_t lds32_align2(const uint8_t* p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    if ((a & 2) == 0) return *reinterpret_cast<const uint32_t*>(p);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(p - 2);
    return __funnelshift_r(w[0], w[1], 16);
}

template <int D, int KBITS, int VBITS, bool QJL>
struct DecodeCfg {
    static constexpr int NBLK = D / 32;
    static constexpr int BBK = block_bytes(KBITS), BBV = block_bytes(VBITS);
    static constexpr int TBK = NBLK * BBK, TBV = NBLK * BBV;     // bytes per token
    static constexpr int kStageK = kTileTok * TBK + 16;
    static constexpr int kStageV = kTileTok * TBV + 16;
    static constexpr int kStageN = 48;                            // 16 float16 norms + slack
    static constexpr int kTabK = Table<KBITS>::kBytes;
    static constexpr int kTabV = (KBITS == VBITS) ? 0 : Table<VBITS>::kBytes;
    static constexpr int kSignTab = QJL ? 16 * 16 * 8 : 0;
    __host__ __device__ static int stage_bits(int jl_dim) { return QJL ? kTileTok * (jl_dim / 8) + 16 : 0; }
    __host__ __device__ static int stage_bytes_total(int jl_dim) {
        return kStageK + kStageV + (QJL ? stage_bits(jl_dim) + kStageN : 0);
    }
    __host__ __device__ static size_t smem_bytes(int jl_dim) {
        size_t ring = (size_t)kDecWarps * kStages * stage_bytes_total(jl_dim);
        size_t work = kTabK + kTabV + kSignTab + ring;
        size_t merge = (size_t)kDecWarps * kHeadsPerCta * (D + 2) * 4;   // aliases tables + ring
        size_t qbuf = (size_t)kHeadsPerCta * (D + (QJL ? jl_dim : 0)) * 4 + 2 * kHeadsPerCta * D * 4;
        return (work > merge ? work : merge) + qbuf + 64;
    }
};

template <int D, int KBITS, int VBITS, bool QJL>
__global__ void __launch_bounds__(kDecThreads, 2) pq_decode_attn_kernel(const DecodeParams p) {
    using C = DecodeCfg<D, KBITS, VBITS, QJL>;
    constexpr int NBLK = C::NBLK;
    extern __shared__ __align__(16) uint8_t smem[];
    // layout: [q buffers][tables][ring]  (merge area aliases tables + ring afterwards)
    float* q_in = reinterpret_cast<float*>(smem);                        // [8][D]   original-space q
    float* q_rot = q_in + kHeadsPerCta * D;                              // [8][D]   rotated, scaled
    float* q_jl = q_rot + kHeadsPerCta * D;                              // [8][M]   (QJL)
    float* o_fin = q_jl + (QJL ? kHeadsPerCta * p.jl_dim : 0);           // [8][D]   final stage
    uint8_t* work = reinterpret_cast<uint8_t*>(o_fin + kHeadsPerCta * D);
    work = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(work) + 15) & ~uintptr_t(15));
    uint8_t* tabk = work;
    uint8_t* tabv = (KBITS == VBITS) ? tabk : tabk + C::kTabK;
    uint8_t* signtab = work + C::kTabK + C::kTabV;
    uint8_t* ring = signtab + C::kSignTab;
    float* merge = reinterpret_cast<float*>(work);                       // [8 warps][8][D+2]
    __shared__ unsigned int s_ticket;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, row = blockIdx.y, hg = blockIdx.z;
    const int b = row / p.Hkv, hkv = row % p.Hkv;
    const int Gp = min(kHeadsPerCta, p.G - hg * kHeadsPerCta);           // query heads of this CTA
    const int head0 = hkv * p.G + hg * kHeadsPerCta;                      // first query head
    const int M = QJL ? p.jl_dim : 0;

    // ---- token range of this CTA and of this warp
    const int64_t tiles_total = (p.S + kTileTok - 1) / kTileTok;
    const int64_t tile_begin = (int64_t)split * p.tiles_per_split;
    const int64_t tile_end = min(tiles_total, tile_begin + p.tiles_per_split);
    const int stage_sz = C::stage_bytes_total(M);
    uint8_t* my_ring = ring + (size_t)warp * kStages * stage_sz;
    const uint8_t* k_row = p.kb + (size_t)row * p.Scap * C::TBK;
    const uint8_t* v_row = p.vb + (size_t)row * p.Scap * C::TBV;
    const uint8_t* bits_row = QJL ? p.qjl_bits + (size_t)row * p.Scap * (M / 8) : nullptr;
    const uint8_t* norm_row = QJL ? reinterpret_cast<const uint8_t*>(p.qjl_norms + (size_t)row * p.Scap) : nullptr;

    auto issue_tile = [&](int64_t tile, int slot) {
        if (tile < tile_end) {
            const int64_t tok0 = tile * kTileTok;
            const int ntok = (int)min((int64_t)kTileTok, p.S - tok0);
            uint8_t* st = my_ring + slot * stage_sz;
            stage_bytes(st, k_row + tok0 * C::TBK, ntok * C::TBK, lane);
            stage_bytes(st + C::kStageK, v_row + tok0 * C::TBV, ntok * C::TBV, lane);
            if (QJL) {
                stage_bytes(st + C::kStageK + C::kStageV, bits_row + tok0 * (M / 8), ntok * (M / 8), lane);
                // norms: 2 bytes per token; copy whole 4-byte words around them (the row is
                // 4-byte aligned at even tokens, tok0 is a multiple of 16)
                stage_bytes(st + C::kStageK + C::kStageV + C::stage_bits(M), norm_row + tok0 * 2,
                            ((ntok * 2 + 3) & ~3), lane);
            }
        }
        cp_async_commit();
    };
    // first tiles in flight before the prologue math
    issue_tile(tile_begin + warp, 0);
    issue_tile(tile_begin + warp + kDecWarps, 1);

    // ---- prologue: tables, query rotation (and JL projection of the query)
    Table<KBITS>::build(tabk, p.cbk, tid);
    if (KBITS != VBITS) Table<VBITS>::build(tabv, p.cbv, tid);
    if (QJL) {
        // sign table: nibble -> 4 halves of +-1; entry 8 bytes, 16 lane copies
        for (int e = tid; e < 16 * 16; e += kDecThreads) {
            const int nib = e >> 4;
            __half2 a = __floats2half2_rn((nib & 1) ? 1.f : -1.f, (nib & 2) ? 1.f : -1.f);
            __half2 c = __floats2half2_rn((nib & 4) ? 1.f : -1.f, (nib & 8) ? 1.f : -1.f);
            reinterpret_cast<uint2*>(signtab)[e] =
                make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&c));
        }
    }
    for (int e = tid; e < kHeadsPerCta * D; e += kDecThreads) {
        const int h = e / D, j = e % D;
        q_in[e] = h < Gp ? __half2float(p.q[((size_t)b * p.Hq + head0 + h) * D + j]) : 0.f;
    }
    __syncthreads();
    // q_rot[h][i] = sum_j q[h][j] * R[i][j]; a warp takes rows i = warp, warp+8, ...
    {
        constexpr int JP = D / 32;
        for (int i = warp; i < D + M; i += kDecWarps) {
            const float* mrow = i < D ? p.rot + (size_t)i * D : p.jl + (size_t)(i - D) * D;
            float r[JP];
#pragma unroll
            for (int k = 0; k < JP; ++k) r[k] = mrow[lane + 32 * k];
#pragma unroll
            for (int h = 0; h < kHeadsPerCta; ++h) {
                float s = 0.f;
#pragma unroll
                for (int k = 0; k < JP; ++k) s = fmaf(r[k], q_in[h * D + lane + 32 * k], s);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) {
                    if (i < D) q_rot[h * D + i] = s * p.scale_log2;
                    else q_jl[h * M + (i - D)] = s * (QJL ? p.scale_log2 / (float)p.jl_dim : 0.f);
                }
            }
        }
    }
    __syncthreads();

    // ---- A fragments of the query: rows 0-7 carry hi(q[head]), rows 8-15 lo(q[head]).
    // k-slot mapping inside a 32-dim block, k-step ks: slots (2t,2t+1) <-> dims 8t+4ks+(0,1),
    // slots (2t+8,2t+9) <-> dims 8t+4ks+(2,3): the 8 nibbles of this lane's 32-bit word.
    uint32_t qa[NBLK][2][4];
#pragma unroll
    for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            const float* src = q_rot + g * D + blk * 32 + 8 * t + 4 * ks;
            __half h[4], l[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) split_half(src[k], h[k], l[k]);
            __half2 v;
            v = __halves2half2(h[0], h[1]); qa[blk][ks][0] = *reinterpret_cast<uint32_t*>(&v);
            v = __halves2half2(l[0], l[1]); qa[blk][ks][1] = *reinterpret_cast<uint32_t*>(&v);
            v = __halves2half2(h[2], h[3]); qa[blk][ks][2] = *reinterpret_cast<uint32_t*>(&v);
            v = __halves2half2(l[2], l[3]); qa[blk][ks][3] = *reinterpret_cast<uint32_t*>(&v);
        }

    // table base for this lane's private copy
    const uint8_t* tabk_lane = tabk + (KBITS == 4 ? (lane & 15) * 8 : (lane & 7) * 16);
    const uint8_t* tabv_lane = tabv + (VBITS == 4 ? (lane & 15) * 8 : (lane & 7) * 16);
    const uint8_t* sign_lane = signtab + (lane & 15) * 8;

    // ---- running softmax state of head g (m shared by the 4 lanes of a row, l per lane)
    float m_run = -INFINITY, l_run = 0.f;
    float o_acc[NBLK][2][4];
#pragma unroll
    for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) o_acc[blk][mt][i] = 0.f;

    int slot = 0;
    for (int64_t tile = tile_begin + warp; tile < tile_end; tile += kDecWarps) {
        issue_tile(tile + 2 * kDecWarps, (slot + 2) % kStages);
        cp_async_wait<2>();
        __syncwarp();
        const uint8_t* st = my_ring + slot * stage_sz;
        const int64_t tok0 = tile * kTileTok;
        const int ntok = (int)min((int64_t)kTileTok, p.S - tok0);
        const uint8_t* ks_base = st + (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(k_row + tok0 * C::TBK)) & 15u);
        const uint8_t* vs_base = st + C::kStageK +
                                 (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(v_row + tok0 * C::TBV)) & 15u);

        // ================= scores: 2 sub-tiles of 8 tokens, token = 8*sub + g as MMA column
        float sc[2][2];
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            const uint8_t* tokp = ks_base + (sub * 8 + g) * C::TBK;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                if (KBITS == 4) {
                    const uint32_t w = lds32_align2(tokp + blk * C::BBK + 2 + 4 * t);
                    const uint2 e0 = lut4(tabk_lane, (w << 7) & 0x7F80u);
                    const uint2 e1 = lut4(tabk_lane, (w >> 1) & 0x7F80u);
                    const uint2 e2 = lut4(tabk_lane, (w >> 9) & 0x7F80u);
                    const uint2 e3 = lut4(tabk_lane, (w >> 17) & 0x7F80u);
                    mma_16816(c, qa[blk][0][0], qa[blk][0][1], qa[blk][0][2], qa[blk][0][3], e0.x, e1.x);
                    mma_16816(c, qa[blk][0][0], qa[blk][0][1], qa[blk][0][2], qa[blk][0][3], e0.y, e1.y);
                    mma_16816(c, qa[blk][1][0], qa[blk][1][1], qa[blk][1][2], qa[blk][1][3], e2.x, e3.x);
                    mma_16816(c, qa[blk][1][0], qa[blk][1][1], qa[blk][1][2], qa[blk][1][3], e2.y, e3.y);
                } else {
                    const uint32_t h = *reinterpret_cast<const uint16_t*>(tokp + blk * C::BBK + 2 + 2 * t);
                    const uint4 e0 = lut2(tabk_lane, (h << 7) & 0x7F80u);
                    const uint4 e1 = lut2(tabk_lane, (h >> 1) & 0x7F80u);
                    mma_16816(c, qa[blk][0][0], qa[blk][0][1], qa[blk][0][2], qa[blk][0][3], e0.x, e0.y);
                    mma_16816(c, qa[blk][0][0], qa[blk][0][1], qa[blk][0][2], qa[blk][0][3], e0.z, e0.w);
                    mma_16816(c, qa[blk][1][0], qa[blk][1][1], qa[blk][1][2], qa[blk][1][3], e1.x, e1.y);
                    mma_16816(c, qa[blk][1][0], qa[blk][1][1], qa[blk][1][2], qa[blk][1][3], e1.z, e1.w);
                }
                // C: rows g (hi of head g) and g+8 (lo), columns = tokens 8*sub + 2t, 2t+1
                const uint8_t* dp = ks_base + (sub * 8 + 2 * t) * C::TBK + blk * C::BBK;
                const float d0 = __half2float(*reinterpret_cast<const __half*>(dp));
                const float d1 = __half2float(*reinterpret_cast<const __half*>(dp + C::TBK));
                s0 = fmaf(d0, c[0] + c[2], s0);
                s1 = fmaf(d1, c[1] + c[3], s1);
            }
            sc[sub][0] = s0 * (1.0f / kCbScale);
            sc[sub][1] = s1 * (1.0f / kCbScale);
        }

        if (QJL) {
            // corr[head][token] = sum_i (+-1) * qp[head][i] (already scaled by scale*log2e/M)
            const uint8_t* bs_base = st + C::kStageK + C::kStageV +
                                     (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(bits_row + tok0 * (M / 8))) & 15u);
            const uint8_t* ns_base = st + C::kStageK + C::kStageV + C::stage_bits(M) +
                                     (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(norm_row + tok0 * 2)) & 15u);
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                const uint8_t* tb = bs_base + (sub * 8 + g) * (M / 8);
                for (int ks = 0; ks < M / 16; ++ks) {
                    const uint32_t h = *reinterpret_cast<const uint16_t*>(tb + 2 * ks);
                    const uint2 e = *reinterpret_cast<const uint2*>(sign_lane + (((h >> (4 * t)) & 0xFu) << 7));
                    const float* src = q_jl + g * M + ks * 16 + 4 * t;
                    __half hh[4], ll[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) split_half(src[k], hh[k], ll[k]);
                    __half2 v0 = __halves2half2(hh[0], hh[1]), v1 = __halves2half2(ll[0], ll[1]);
                    __half2 v2 = __halves2half2(hh[2], hh[3]), v3 = __halves2half2(ll[2], ll[3]);
                    mma_16816(c, *reinterpret_cast<uint32_t*>(&v0), *reinterpret_cast<uint32_t*>(&v1),
                              *reinterpret_cast<uint32_t*>(&v2), *reinterpret_cast<uint32_t*>(&v3), e.x, e.y);
                }
                const __half* np = reinterpret_cast<const __half*>(ns_base) + sub * 8 + 2 * t;
                // a zero residual norm switches the correction off (qjl.py:49-50)
                if (__half2float(np[0]) != 0.f) sc[sub][0] += c[0] + c[2];
                if (__half2float(np[1]) != 0.f) sc[sub][1] += c[1] + c[3];
            }
        }

        // mask tokens past the end of the sequence
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
#pragma unroll
            for (int e = 0; e < 2; ++e)
                if (sub * 8 + 2 * t + e >= ntok) sc[sub][e] = -INFINITY;

        // ================= online softmax for head g over the 16 tokens of the tile
        float tmax = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m_run, tmax);
        const float alpha = fast_exp2(m_run - m_new);      // exp2(-inf) = 0 on the first tile
        float pr[2][2];
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
#pragma unroll
            for (int e = 0; e < 2; ++e) pr[sub][e] = fast_exp2(sc[sub][e] - m_new);
        l_run = l_run * alpha + (pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]);
        m_run = m_new;
        // rescale the accumulators: their columns are heads 2t, 2t+1
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
            const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4);
            const float a1 = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    o_acc[blk][mt][0] *= a0; o_acc[blk][mt][1] *= a1;
                    o_acc[blk][mt][2] *= a0; o_acc[blk][mt][3] *= a1;
                }
        }

        // ================= values: O[dim][head] += V^T[dim][token] * (p*d)[token][head]
        // A rows: g <-> dim 4g+2mt, g+8 <-> dim 4g+2mt+1 of the block; k slots = tokens
        // (2t, 2t+1 | 8+2t, 9+2t); B column g = head g with the same token slots.
#pragma unroll
        for (int blk = 0; blk < NBLK; ++blk) {
            // weights of this lane's 4 tokens for head g, times the block radius
            float w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int tok = (k >> 1) * 8 + 2 * t + (k & 1);
                const float d = __half2float(*reinterpret_cast<const __half*>(vs_base + tok * C::TBV + blk * C::BBV));
                w[k] = tok < ntok ? pr[k >> 1][k & 1] * d : 0.f;
            }
            __half wh[4], wl[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) split_half(w[k], wh[k], wl[k]);
            __half2 t0 = __halves2half2(wh[0], wh[1]), t1 = __halves2half2(wh[2], wh[3]);
            __half2 t2 = __halves2half2(wl[0], wl[1]), t3 = __halves2half2(wl[2], wl[3]);
            const uint32_t bh0 = *reinterpret_cast<uint32_t*>(&t0), bh1 = *reinterpret_cast<uint32_t*>(&t1);
            const uint32_t bl0 = *reinterpret_cast<uint32_t*>(&t2), bl1 = *reinterpret_cast<uint32_t*>(&t3);

            uint32_t ahi[2][4], alo[2][4];   // [m-tile][a0..a3]
#pragma unroll
            for (int pair = 0; pair < 2; ++pair) {
                const uint8_t* pa = vs_base + (pair * 8 + 2 * t) * C::TBV + blk * C::BBV + 2;
                if (VBITS == 4) {
                    const uint32_t ha = *reinterpret_cast<const uint16_t*>(pa + 2 * g);
                    const uint32_t hb = *reinterpret_cast<const uint16_t*>(pa + C::TBV + 2 * g);
                    const uint32_t m1 = (ha & 0x0F0Fu) | ((hb & 0x0F0Fu) << 4);          // dims 0, 2
                    const uint32_t m2 = ((ha >> 4) & 0x0F0Fu) | (hb & 0xF0F0u);           // dims 1, 3
                    const uint2 e0 = lut4(tabv_lane, (m1 << 7) & 0x7F80u);
                    const uint2 e1 = lut4(tabv_lane, (m2 << 7) & 0x7F80u);
                    const uint2 e2 = lut4(tabv_lane, (m1 >> 1) & 0x7F80u);
                    const uint2 e3 = lut4(tabv_lane, (m2 >> 1) & 0x7F80u);
                    ahi[0][pair * 2 + 0] = e0.x; ahi[0][pair * 2 + 1] = e1.x;
                    alo[0][pair * 2 + 0] = e0.y; alo[0][pair * 2 + 1] = e1.y;
                    ahi[1][pair * 2 + 0] = e2.x; ahi[1][pair * 2 + 1] = e3.x;
                    alo[1][pair * 2 + 0] = e2.y; alo[1][pair * 2 + 1] = e3.y;
                } else {
                    const uint32_t ba = pa[g], bb = pa[C::TBV + g];
                    const uint32_t m1 = (ba & 3u) | ((bb & 3u) << 2) | ((ba & 0xCu) << 2) | ((bb & 0xCu) << 4);
                    const uint32_t ua = ba >> 4, ub = bb >> 4;
                    const uint32_t m2 = (ua & 3u) | ((ub & 3u) << 2) | ((ua & 0xCu) << 2) | ((ub & 0xCu) << 4);
                    const uint4 e0 = lut2(tabv_lane, m1 << 7);
                    const uint4 e1 = lut2(tabv_lane, m2 << 7);
                    ahi[0][pair * 2 + 0] = e0.x; ahi[0][pair * 2 + 1] = e0.y;
                    alo[0][pair * 2 + 0] = e0.z; alo[0][pair * 2 + 1] = e0.w;
                    ahi[1][pair * 2 + 0] = e1.x; ahi[1][pair * 2 + 1] = e1.y;
                    alo[1][pair * 2 + 0] = e1.z; alo[1][pair * 2 + 1] = e1.w;
                }
            }
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                mma_16816(o_acc[blk][mt], ahi[mt][0], ahi[mt][1], ahi[mt][2], ahi[mt][3], bh0, bh1);
                mma_16816(o_acc[blk][mt], ahi[mt][0], ahi[mt][1], ahi[mt][2], ahi[mt][3], bl0, bl1);
                mma_16816(o_acc[blk][mt], alo[mt][0], alo[mt][1], alo[mt][2], alo[mt][3], bh0, bh1);
            }
        }
        __syncwarp();
        slot = (slot + 1) % kStages;
    }
    cp_async_wait<0>();

    // ---- reduce the row sum over the 4 lanes of a head
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncthreads();   // tables and rings are dead: the merge area takes their place

    // per-warp record: merge[warp][head][0]=m, [1]=l, [2+dim]=o
    {
        float* rec = merge + (size_t)warp * kHeadsPerCta * (D + 2);
        if (t == 0) {
            rec[g * (D + 2) + 0] = m_run;
            rec[g * (D + 2) + 1] = l_run;
        }
#pragma unroll
        for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int head = 2 * t + (i & 1);
                    const int dim = blk * 32 + 4 * g + 2 * mt + (i >> 1);
                    rec[head * (D + 2) + 2 + dim] = o_acc[blk][mt][i] * (1.0f / kCbScale);
                }
    }
    __syncthreads();

    // ---- CTA record = merge of the 8 warp records
    const size_t group = (size_t)row * p.HG + hg;
    float* cta_rec = p.records + (group * p.splits + split) * kHeadsPerCta * (D + 2);
    for (int e = tid; e < kHeadsPerCta * (D + 2); e += kDecThreads) {
        const int head = e / (D + 2), col = e % (D + 2);
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) mx = fmaxf(mx, merge[(w * kHeadsPerCta + head) * (D + 2)]);
        float val;
        if (col == 0) {
            val = mx;
        } else {
            val = 0.f;
#pragma unroll
            for (int w = 0; w < kDecWarps; ++w) {
                const float mw = merge[(w * kHeadsPerCta + head) * (D + 2)];
                const float s = (mw == -INFINITY) ? 0.f : fast_exp2(mw - mx);
                val = fmaf(s, merge[(w * kHeadsPerCta + head) * (D + 2) + col], val);
            }
        }
        __stcg(cta_rec + e, val);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(p.tickets + group, 1u);
    __syncthreads();
    if (s_ticket != (unsigned)(p.splits - 1)) return;
    __threadfence();

    // ---- last CTA of this (row, head group): merge the split records
    const float* recs = p.records + group * p.splits * kHeadsPerCta * (D + 2);
    for (int e = tid; e < kHeadsPerCta * D; e += kDecThreads) {
        const int head = e / D, dim = e % D;
        float mx = -INFINITY;
        for (int s = 0; s < p.splits; ++s) mx = fmaxf(mx, __ldcg(recs + (s * kHeadsPerCta + head) * (D + 2)));
        float l = 0.f, o = 0.f;
        for (int s = 0; s < p.splits; ++s) {
            const float* r = recs + (s * kHeadsPerCta + head) * (D + 2);
            const float ms = __ldcg(r);
            const float sc = (ms == -INFINITY) ? 0.f : fast_exp2(ms - mx);
            l = fmaf(sc, __ldcg(r + 1), l);
            o = fmaf(sc, __ldcg(r + 2 + dim), o);
        }
        if (p.partial_out) {
            if (head < Gp) {
                float* dst = p.partial_out + ((size_t)b * p.Hq + head0 + head) * (D + 2);
                dst[2 + dim] = o;
                if (dim == 0) { dst[0] = mx; dst[1] = l; }
            }
        } else {
            o_fin[e] = l > 0.f ? o / l : 0.f;
        }
    }
    if (tid == 0) p.tickets[group] = 0;   // ready for the next call on this stream
    if (p.partial_out) return;
    __syncthreads();
    // out[head][i] = sum_j o_fin[head][j] * R[j][i]
    for (int e = tid; e < kHeadsPerCta * D; e += kDecThreads) {
        const int head = e / D, i = e % D;
        if (head >= Gp) continue;
        float acc = 0.f;
#pragma unroll 8
        for (int j = 0; j < D; ++j) acc = fmaf(o_fin[head * D + j], __ldg(p.rot + (size_t)j * D + i), acc);
        const size_t off = ((size_t)b * p.Hq + head0 + head) * D + i;
        if (p.out_is_fp16) static_cast<__half*>(p.out)[off] = __float2half_rn(fminf(fmaxf(acc, -65504.f), 65504.f));
        else static_cast<float*>(p.out)[off] = acc;
    }
}

// ------------------------------------------------------------------ host side
static int device_sms() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}

static int choose_splits(int batch, int q_heads, int kv_heads, int64_t seq_len, int sms) {
    if (sms <= 0) sms = 148;
    const int G = q_heads / kv_heads;
    const int64_t groups = (int64_t)batch * kv_heads * ((G + kHeadsPerCta - 1) / kHeadsPerCta);
    const int64_t tiles = (seq_len + kTileTok - 1) / kTileTok;
    // aim for about 4 CTAs per SM in total (2 resident x 2 waves), at least 2 tiles per warp
    int64_t want = (4LL * sms + groups - 1) / groups;
    const int64_t max_by_work = tiles / (2 * kDecWarps);
    if (want > max_by_work) want = max_by_work;
    if (want < 1) want = 1;
    if (want > 1024) want = 1024;
    return (int)want;
}

template <int D, int KBITS, int VBITS, bool QJL>
static int launch_decode(const DecodeParams& p, int rows, cudaStream_t st) {
    using C = DecodeCfg<D, KBITS, VBITS, QJL>;
    const size_t smem = C::smem_bytes(p.jl_dim);
    auto kern = pq_decode_attn_kernel<D, KBITS, VBITS, QJL>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return PQ_ERR_CUDA;
    dim3 grid(p.splits, rows, p.HG);
    kern<<<grid, kDecThreads, smem, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
}

}  // namespace pq

extern "C" int pq_decode_attn_default_splits(int batch, int q_heads, int kv_heads, int64_t seq_len, int head_dim) {
    (void)head_dim;
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) return 1;
    return pq::choose_splits(batch, q_heads, kv_heads, seq_len, pq::device_sms());
}

extern "C" size_t pq_decode_attn_scratch_bytes(int batch, int q_heads, int kv_heads, int64_t seq_len,
                                               int head_dim, int n_splits) {
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) return 0;
    if (n_splits <= 0) n_splits = pq::choose_splits(batch, q_heads, kv_heads, seq_len, pq::device_sms());
    const int G = q_heads / kv_heads;
    const size_t groups = (size_t)batch * kv_heads * ((G + pq::kHeadsPerCta - 1) / pq::kHeadsPerCta);
    const size_t tickets = (groups * sizeof(unsigned int) + 255) & ~size_t(255);
    return tickets + groups * n_splits * pq::kHeadsPerCta * (head_dim + 2) * sizeof(float);
}

extern "C" int pq_decode_attn(const void* q, const void* k_blocks, const void* v_blocks,
                              int batch, int q_heads, int kv_heads, int64_t seq_len, int64_t seq_capacity,
                              int head_dim, int k_bits, int v_bits,
                              const float* codebook_k, const float* codebook_v, const float* rot, float scale,
                              const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                              void* out, int out_is_fp16, void* partial_out,
                              int n_splits, void* scratch, size_t scratch_bytes, void* stream) {
    using namespace pq;
    if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || seq_len < 0 || seq_capacity < seq_len)
        return PQ_ERR_BAD_SHAPE;
    if (head_dim != 64 && head_dim != 128) return PQ_ERR_BAD_HEAD_DIM;
    if ((k_bits != 2 && k_bits != 4) || (v_bits != 2 && v_bits != 4)) return PQ_ERR_BAD_BITS;
    if (batch == 0) return PQ_OK;
    if (!q || !rot || !codebook_k || !codebook_v || (!out && !partial_out) || !scratch) return PQ_ERR_NULL_POINTER;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool qjl = jl_matrix != nullptr;
    if (qjl) {
        if (jl_dim < 16 || jl_dim > 128 || (jl_dim % 16)) return PQ_ERR_BAD_JL_DIM;
        if (!qjl_bits || !qjl_norms) return PQ_ERR_NULL_POINTER;
        if ((reinterpret_cast<uintptr_t>(qjl_bits) & 15) || (reinterpret_cast<uintptr_t>(qjl_norms) & 15) ||
            (seq_capacity & 1))
            return PQ_ERR_MISALIGNED;
    }
    if (seq_len == 0) {
        // empty sequence -> zeros (attention.py:127-131); partial: m = -inf, l = 0, o = 0
        const size_t n = (size_t)batch * q_heads;
        if (partial_out) {
            if (cudaMemsetAsync(partial_out, 0, n * (head_dim + 2) * 4, st) != cudaSuccess) return PQ_ERR_CUDA;
            return PQ_OK;   // m = 0 with l = 0 carries no weight in pq_lse_merge
        }
        if (cudaMemsetAsync(out, 0, n * head_dim * (out_is_fp16 ? 2 : 4), st) != cudaSuccess) return PQ_ERR_CUDA;
        return PQ_OK;
    }
    if (!k_blocks || !v_blocks) return PQ_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(k_blocks) & 15) || (reinterpret_cast<uintptr_t>(v_blocks) & 15) ||
        (reinterpret_cast<uintptr_t>(scratch) & 255) || (reinterpret_cast<uintptr_t>(rot) & 15))
        return PQ_ERR_MISALIGNED;
    const int64_t tiles = (seq_len + kTileTok - 1) / kTileTok;
    if (n_splits <= 0) n_splits = choose_splits(batch, q_heads, kv_heads, seq_len, device_sms());
    if (n_splits > tiles) n_splits = (int)tiles;
    if (scratch_bytes < pq_decode_attn_scratch_bytes(batch, q_heads, kv_heads, seq_len, head_dim, n_splits))
        return PQ_ERR_SCRATCH_TOO_SMALL;
    const int rows = batch * kv_heads;
    if (rows > 65535) return PQ_ERR_TOO_LARGE;

    DecodeParams p{};
    p.q = static_cast<const __half*>(q);
    p.kb = static_cast<const uint8_t*>(k_blocks);
    p.vb = static_cast<const uint8_t*>(v_blocks);
    p.rot = rot;
    p.jl = jl_matrix;
    p.qjl_bits = static_cast<const uint8_t*>(qjl_bits);
    p.qjl_norms = static_cast<const __half*>(qjl_norms);
    p.out = out;
    p.partial_out = static_cast<float*>(partial_out);
    p.S = seq_len;
    p.Scap = seq_capacity;
    p.Hq = q_heads;
    p.Hkv = kv_heads;
    p.G = q_heads / kv_heads;
    p.HG = (p.G + kHeadsPerCta - 1) / kHeadsPerCta;
    p.splits = n_splits;
    p.tiles_per_split = (int)((tiles + n_splits - 1) / n_splits);
    p.jl_dim = qjl ? jl_dim : 0;
    p.out_is_fp16 = out_is_fp16;
    p.scale_log2 = scale * 1.4426950408889634f;
    for (int i = 0; i < 16; ++i) {
        p.cbk[i] = i < (1 << k_bits) ? codebook_k[i] : 0.f;
        p.cbv[i] = i < (1 << v_bits) ? codebook_v[i] : 0.f;
    }
    const size_t groups = (size_t)rows * p.HG;
    p.tickets = static_cast<unsigned int*>(scratch);
    p.records = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + ((groups * sizeof(unsigned int) + 255) & ~size_t(255)));

#define PQ_DEC(DD, KB, VB)                                                                     \
    if (head_dim == DD && k_bits == KB && v_bits == VB)                                        \
        return qjl ? launch_decode<DD, KB, VB, true>(p, rows, st) : launch_decode<DD, KB, VB, false>(p, rows, st);
    PQ_DEC(64, 4, 4) PQ_DEC(64, 4, 2) PQ_DEC(64, 2, 4) PQ_DEC(64, 2, 2)
    PQ_DEC(128, 4, 4) PQ_DEC(128, 4, 2) PQ_DEC(128, 2, 4) PQ_DEC(128, 2, 2)
#undef PQ_DEC
    return PQ_ERR_BAD_HEAD_DIM;
}
