// pq_prefill_attn: seq_q >= 1 query tokens per head against a block_pq4 cache, on the 5th-gen
// tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Same rotated-space arithmetic as the decode kernel (softmax(q K^T * scale) V evaluated on
// centroid * radius values, python/polarquant_kv/attention.py:111-163), organised for many
// query rows: a CTA owns 128 query rows of one KV head (rows = (query head, position) pairs of
// the GQA group; TMEM lane = row) and walks the sequence in tiles of 64 tokens.  Every operand
// is a pair of float16 terms (value = hi + lo, about 22 bits) and every contraction a
// three-term product hi*hi + hi*lo + lo*hi with float32 accumulation, which keeps float32-level
// accuracy.  Radii: a token's largest block radius dmax is applied in float32 (to the score
// column / to the probability before its split); the tiles hold (d / dmax) * centroid * 1024.
//
// Roles (no CTA-wide barrier inside the loop; all waits are bounded mbarrier waits):
//   dequant warps (16, fused kernel) - expand tile i+1 of K, then of V, into double-buffered shared-memory
//                     tiles in the 128-byte-swizzled layout the tensor core reads; or
//   copy warp (workspace kernel)    - the same tiles, expanded once by pq_prefill_expand_kernel, arrive by
//                     cp.async.bulk from the workspace;
//   MMA warp(s)     - S(i) = Q K(i)^T into one of three TMEM buffers, ahead of the softmax (A = the rotated
//                     query in shared memory; B = the K tile with its hi and lo rows stacked, N = 128), and
//                     O += P(i) V(i) (A = P in tensor memory, B = V as an MN-major operand).  The fused kernel
//                     issues both from one warp, the workspace kernel from two;
//   softmax warps   - two (fused) or four (workspace) threads per query row: read S from TMEM, scale, mask,
//                     exchange partial row maxima, online softmax with a lazy rescale of O (only when a
//                     row's maximum grew by more than 2^8), write P * dmax_v as float16 hi/lo back into the
//                     S columns of the tile (the A operand of the second contraction).
// Tensor memory (512 columns): S0 | S1 | S2 (128 each) | O (128).
// The query rotation q @ R^T and the final o @ R run before and after the loop, on the tensor core too.
//
// causal == 0 reproduces the reference (no mask, src/polarquant_kv_cuda/attention_kernel.py:
// 92-113); causal == 1 lets query position i see tokens [0, seq_len - seq_q + i].
#include "pq_tcgen05.cuh"

namespace pq {

// Bit 2 of the device error flags: a bounded wait in the prefill kernel gave up.
static __device__ unsigned int g_prefill_error = 0;

constexpr int kPfRows = 128;                 // query rows per CTA = TMEM lanes
constexpr int kPfTok = 64;                   // tokens per KV tile
constexpr int kPfRowWarps = 4;               // warps that cover the 128 TMEM lanes once (rotation epilogues)
constexpr int kPfDeqWarps = 16;
constexpr int kPfDeqThreads = kPfDeqWarps * 32;
// Warp roles.  Fused kernel: 8 softmax warps (two threads per query row), 16 dequant warps, 1 MMA warp.
// Workspace kernel: 16 softmax warps (four threads per row, row maxima exchanged through spare
// TMEM columns), 1 copy warp, 1 MMA warp.
__host__ __device__ constexpr int pf_split(bool pre) { return pre ? 4 : 2; }             // softmax threads per row
__host__ __device__ constexpr int pf_soft_warps(bool pre) { return 4 * pf_split(pre); }
__host__ __device__ constexpr int pf_mma_warp(bool pre) { return pre ? pf_soft_warps(pre) + 1 : pf_soft_warps(pre) + kPfDeqWarps; }
// Workspace kernel: two MMA warps, the first issues the score MMAs (and the rotations), the second the value
// MMAs (MMA issue is its critical path).  Fused kernel: one warp issues both, interleaved.
__host__ __device__ constexpr int pf_threads(bool pre) { return (pf_mma_warp(pre) + (pre ? 2 : 1)) * 32; }
constexpr float kPfValScale = 1024.0f;       // tiles hold 1024 * (d / dmax) * centroid
constexpr float kPfRescaleGap = 8.0f;        // log2 units a row maximum may grow before O is rescaled

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
    const uint8_t* ws;     // expanded tiles (see PrefillCfg::kRec) or null
};

// Barriers that two roles wait on come in pairs, one per tile parity: a barrier's next phase can then
// only complete after every waiter has seen the current one (a waiter never lags a whole phase).
// K / V tiles and their radii are double-buffered (index = tile parity); the score buffers in tensor memory are
// triple-buffered (index = tile mod 3), so S(i) does not have to wait for P(i-2) V(i-2).
enum { PF_K_FULL = 0, PF_V_FULL = 2, PF_S_FULL = 4, PF_S_FREE = 7, PF_PV_DONE = 10, PF_P_FULL = 12, PF_AUX = 13,
       PF_P_USED = 14, PF_NBAR = 17 };

// Byte offset of element (row r, column col) of a [rows][64*h columns] float16 tile stored as
// 64-column halves of `rows` 128-byte rows, 16-byte chunks XOR-swizzled with the row (SWIZZLE_128B).
__device__ __forceinline__ uint32_t sw128_off(int rows, int r, int col) {
    return (uint32_t)((col >> 6) * rows * 128 + (r >> 3) * 1024 + (r & 7) * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4) +
                      (col & 7) * 2);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
        "%30,%31,%32};\n" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
        "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
        "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// 16-bit read-only global load that the compiler may not move: the dequant warps issue the next
// tile's loads before they start on the current tile, and the loads must stay there.
__device__ __forceinline__ uint32_t ldg_u16_pinned(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];\n" : "=h"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float4 lds_f4(uint32_t saddr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
    return v;
}

// 8 packed words into consecutive columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n\t"
                 "tcgen05.wait::st.sync.aligned;\n" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}

// 16 packed words into consecutive columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n\t"
                 "tcgen05.wait::st.sync.aligned;\n" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                 : "memory");
}

// One float32 into / four out of this thread's TMEM lane (row-maximum exchange between the warps of a row group).
__device__ __forceinline__ void tmem_st1(uint32_t taddr, float v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};\n\t"
                 "tcgen05.wait::st.sync.aligned;\n" ::"r"(taddr), "r"(__float_as_uint(v))
                 : "memory");
}
__device__ __forceinline__ float4 tmem_ld4(uint32_t taddr) {
    uint32_t a, b, c, d;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n\t"
                 "tcgen05.wait::ld.sync.aligned;\n"
                 : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
                 : "r"(taddr)
                 : "memory");
    return make_float4(__uint_as_float(a), __uint_as_float(b), __uint_as_float(c), __uint_as_float(d));
}

// 16 consecutive float32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(float (&v)[16], uint32_t taddr) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
                 "tcgen05.wait::ld.sync.aligned;\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Two 32-column loads of this thread's TMEM lane with one wait.
__device__ __forceinline__ void tmem_ld32x2(float (&a)[32], float (&b)[32], uint32_t taddr_a, uint32_t taddr_b) {
    uint32_t ra[32], rb[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(ra[0]), "=r"(ra[1]), "=r"(ra[2]), "=r"(ra[3]), "=r"(ra[4]), "=r"(ra[5]), "=r"(ra[6]), "=r"(ra[7]), "=r"(ra[8]), "=r"(ra[9]), "=r"(ra[10]), "=r"(ra[11]), "=r"(ra[12]), "=r"(ra[13]), "=r"(ra[14]), "=r"(ra[15]), "=r"(ra[16]), "=r"(ra[17]), "=r"(ra[18]), "=r"(ra[19]), "=r"(ra[20]), "=r"(ra[21]), "=r"(ra[22]), "=r"(ra[23]), "=r"(ra[24]), "=r"(ra[25]), "=r"(ra[26]), "=r"(ra[27]), "=r"(ra[28]), "=r"(ra[29]), "=r"(ra[30]), "=r"(ra[31]), "=r"(rb[0]), "=r"(rb[1]), "=r"(rb[2]), "=r"(rb[3]), "=r"(rb[4]), "=r"(rb[5]), "=r"(rb[6]), "=r"(rb[7]), "=r"(rb[8]), "=r"(rb[9]), "=r"(rb[10]), "=r"(rb[11]), "=r"(rb[12]), "=r"(rb[13]), "=r"(rb[14]), "=r"(rb[15]), "=r"(rb[16]), "=r"(rb[17]), "=r"(rb[18]), "=r"(rb[19]), "=r"(rb[20]), "=r"(rb[21]), "=r"(rb[22]), "=r"(rb[23]), "=r"(rb[24]), "=r"(rb[25]), "=r"(rb[26]), "=r"(rb[27]), "=r"(rb[28]), "=r"(rb[29]), "=r"(rb[30]), "=r"(rb[31])
        : "r"(taddr_a), "r"(taddr_b)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) { a[i] = __uint_as_float(ra[i]); b[i] = __uint_as_float(rb[i]); }
}

// One thread's share of a 64-token tile of one operand: work item = 8 consecutive elements of one
// (token, block).  A thread's items k = 0..N-1 share block and position and sit 256 / (4 * NBLK) tokens
// apart, so every address is one per-thread base plus compile-time offsets.  load() fetches the raw
// bytes (indices and the token's block radii) into registers, expand() writes the hi / lo tiles
// (1024 * (d / dmax) * centroid) and the per-token largest radius.  Splitting the two lets the next
// tile's loads fly while this tile is expanded.
template <int D, int BITS>
struct RawItems {
    static constexpr int NBLK = D / 32, BB = block_bytes(BITS), TB = NBLK * BB;
    static constexpr int N = kPfTok * NBLK * 4 / kPfDeqThreads;           // items per thread
    static constexpr int TSTEP = kPfDeqThreads / (NBLK * 4);              // tokens between a thread's items
    uint32_t bits[N];
    uint32_t rad[N][NBLK / 2];                                            // the token's radii, two per word

    // Raw 16-bit loads of the next tile.  issue() only starts them (no result is touched, so all of
    // them are in flight together); pack() combines them once they have landed.
    struct Pending {
        uint32_t r[N][NBLK];
        uint32_t b[N][BITS == 4 ? 2 : 1];
    };
    // src = first byte of the tile; tok0 / blk / qw = this thread's first item
    __device__ __forceinline__ static void issue(Pending& pd, const uint8_t* __restrict__ src, int ntok, int tok0,
                                                 int blk, int qw) {
        const uint8_t* tb0 = src + tok0 * TB;
#pragma unroll
        for (int k = 0; k < N; ++k) {
            // rows past the end re-read the tile's first token (always valid) and are zeroed in pack()
            const uint8_t* tb = (tok0 + k * TSTEP < ntok) ? tb0 + k * TSTEP * TB : src;
#pragma unroll
            for (int j = 0; j < NBLK; ++j) pd.r[k][j] = ldg_u16_pinned(tb + j * BB);
            if (BITS == 4) {
                pd.b[k][0] = ldg_u16_pinned(tb + blk * BB + 2 + qw * 4);
                pd.b[k][1] = ldg_u16_pinned(tb + blk * BB + 4 + qw * 4);
            } else {
                pd.b[k][0] = ldg_u16_pinned(tb + blk * BB + 2 + qw * 2);
            }
        }
    }
    __device__ __forceinline__ void pack(const Pending& pd, int ntok, int tok0) {
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const bool valid = tok0 + k * TSTEP < ntok;
#pragma unroll
            for (int j = 0; j < NBLK / 2; ++j) rad[k][j] = valid ? (pd.r[k][2 * j] | (pd.r[k][2 * j + 1] << 16)) : 0u;
            bits[k] = BITS == 4 ? (pd.b[k][0] | (pd.b[k][BITS == 4 ? 1 : 0] << 16)) : pd.b[k][0];
        }
    }
    __device__ __forceinline__ void load(const uint8_t* __restrict__ src, int ntok, int tok0, int blk, int qw) {
        Pending pd;
        issue(pd, src, ntok, tok0, blk, qw);
        pack(pd, ntok, tok0);
    }

    // off0 = sw128 offset of the thread's first item; later items are whole 8-token groups further
    // dmax_scale: factor stored with the per-token radius (the K side folds the tile scale 1/1024 in)
    __device__ __forceinline__ void expand(const float* cb, uint8_t* hi, uint8_t* lo, float* dmax_out, float dmax_scale,
                                           int tok0, int blk, bool first, uint32_t off0) const {
        static_assert(TSTEP % 8 == 0, "items of a thread must keep their row inside the 8-row swizzle group");
#pragma unroll
        for (int k = 0; k < N; ++k) {
            float dmax = 0.f, d = 0.f;
#pragma unroll
            for (int j = 0; j < NBLK; ++j) {
                const float dj = __half2float(__ushort_as_half((unsigned short)(rad[k][j >> 1] >> (16 * (j & 1)))));
                dmax = fmaxf(dmax, dj);
                if (j == blk) d = dj;
            }
            const float r = dmax > 0.f ? __fdividef(d, dmax) : 0.f;        // rows past the end: radii 0 -> zeros
            uint32_t h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float v0 = cb[(bits[k] >> (2 * e * BITS)) & ((1u << BITS) - 1u)] * r;
                const float v1 = cb[(bits[k] >> ((2 * e + 1) * BITS)) & ((1u << BITS) - 1u)] * r;
                const __half2 hh = __floats2half2_rn(v0, v1);
                const float2 hf = __half22float2(hh);
                h[e] = *reinterpret_cast<const uint32_t*>(&hh);
                l[e] = pack_half2(v0 - hf.x, v1 - hf.y);
            }
            const uint32_t off = off0 + (uint32_t)(k * (TSTEP / 8) * 1024);
            *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
            if (first) dmax_out[tok0 + k * TSTEP] = dmax * dmax_scale;
        }
    }
};

template <int D>
struct PrefillCfg {
    static constexpr uint32_t QB = kPfRows * D * 2;            // one term of the query tile
    static constexpr uint32_t KB = kPfTok * D * 2;             // one term of a K or V tile
    static constexpr uint32_t PB = kPfRows * kPfTok * 2;       // one term of the probability tile
    static constexpr uint32_t kTiles = 2 * QB + 8 * KB + 2 * PB;       // K and V tiles are double-buffered
    static constexpr uint32_t kSmall = 4 * kPfTok * 4 + 32 * 4 + PF_NBAR * 8 + 24;
    static constexpr size_t smem_bytes() { return (size_t)kTiles + kSmall + 1024; }
    // Workspace record of one (kv row, 64-token tile): K hi | K lo | V hi | V lo tiles exactly as they
    // sit in shared memory, then the per-token largest radii of K and of V (64 floats each).
    static constexpr uint32_t kRec = 4 * KB + 2 * kPfTok * 4;
    // TMEM columns: S0 | S1 | S2 (128 each: q_hi*k_hi + q_lo*k_hi in the first 64, q_hi*k_lo in the second 64) |
    // O (128).  The rotations before and after the loop use columns [0, 2D).
    static constexpr uint32_t kTmemCols = 512;
    static constexpr uint32_t kSCols = 2 * kPfTok;
    static constexpr uint32_t kOCol = 3 * kSCols;
};

// Expands one 64-token tile of K and of V per CTA into the workspace (grid: tiles x kv rows).
template <int D, int KBITS, int VBITS>
__global__ void __launch_bounds__(kPfDeqThreads) pq_prefill_expand_kernel(const PrefillParams p, uint8_t* ws,
                                                                             int n_tiles) {
    using C = PrefillCfg<D>;
    constexpr int NBLK = D / 32;
    constexpr int TBK = NBLK * block_bytes(KBITS), TBV = NBLK * block_bytes(VBITS);
    __shared__ float cbk_s[16], cbv_s[16];
    const int dt = threadIdx.x, tile = blockIdx.x, kvrow = blockIdx.y;
    if (dt < 16) { cbk_s[dt] = p.cbk[dt] * kPfValScale; cbv_s[dt] = p.cbv[dt] * kPfValScale; }
    __syncthreads();
    const int it_tok = dt / (NBLK * 4), it_blk = (dt % (NBLK * 4)) >> 2, it_qw = dt & 3;
    const bool it_first = (dt % (NBLK * 4)) == 0;
    const uint32_t it_off = sw128_off(kPfTok, it_tok, it_blk * 32 + it_qw * 8);
    const uint32_t it_offk = sw128_off(2 * kPfTok, it_tok, it_blk * 32 + it_qw * 8);   // K: hi and lo rows stacked
    const int64_t tok0 = (int64_t)tile * kPfTok;
    const int ntok = (int)min((int64_t)kPfTok, p.S - tok0);
    uint8_t* rec = ws + ((size_t)kvrow * n_tiles + tile) * C::kRec;
    float* dmax = reinterpret_cast<float*>(rec + 4 * C::KB);
    RawItems<D, KBITS> rk;
    RawItems<D, VBITS> rv;
    rk.load(p.kb + ((size_t)kvrow * p.Scap + tok0) * TBK, ntok, it_tok, it_blk, it_qw);
    rv.load(p.vb + ((size_t)kvrow * p.Scap + tok0) * TBV, ntok, it_tok, it_blk, it_qw);
    rk.expand(cbk_s, rec, rec + kPfTok * 128, dmax, 1.0f / kPfValScale, it_tok, it_blk, it_first, it_offk);
    rv.expand(cbv_s, rec + 2 * C::KB, rec + 3 * C::KB, dmax + kPfTok, 1.0f, it_tok, it_blk, it_first, it_off);
}

// PRE: the tiles come expanded from the workspace (bulk copies by one warp) instead of being
// dequantised by sixteen warps of this CTA.
template <int D, int KBITS, int VBITS, bool PRE>
__global__ void __launch_bounds__(pf_threads(PRE), 1) pq_prefill_attn_kernel(const PrefillParams p) {
    constexpr int kPfSoftWarps = pf_soft_warps(PRE), NSPLIT = pf_split(PRE), kMmaWarp = pf_mma_warp(PRE);
    const int kPfThreads = blockDim.x;
    using C = PrefillCfg<D>;
    constexpr int NBLK = D / 32;
    constexpr int TBK = NBLK * block_bytes(KBITS), TBV = NBLK * block_bytes(VBITS);

    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* Qh = base;
    uint8_t* Ql = Qh + C::QB;
    uint8_t* Kh = Ql + C::QB;                 // buffer b: hi at Kh + b * 2KB, lo one KB further
    uint8_t* Vh = Kh + 4 * C::KB;             // same for V
    uint8_t* Ph = Vh + 4 * C::KB;
    uint8_t* Pl = Ph + C::PB;
    uint8_t* small = base + C::kTiles;
    float* dmaxK = reinterpret_cast<float*>(small);                       // [2][64]
    float* dmaxV = dmaxK + 2 * kPfTok;                                    // [2][64]
    float* cbk_s = dmaxV + 2 * kPfTok;
    float* cbv_s = cbk_s + 16;
    uint64_t* mbar = reinterpret_cast<uint64_t*>(cbv_s + 16);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + PF_NBAR);
    volatile uint32_t* abort_s = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row_tile = blockIdx.x, kvrow = blockIdx.y;
    const int b = kvrow / p.Hkv, hkv = kvrow % p.Hkv;
    const int n_rows = p.G * p.Sq;                            // query rows sharing this KV head
    const int row0 = row_tile * kPfRows;

    if (tid < 16) { cbk_s[tid] = p.cbk[tid] * kPfValScale; cbv_s[tid] = p.cbv[tid] * kPfValScale; }
    if (tid == 0) {
        for (int k = 0; k < 2; ++k) {
            mbar_init(sm_addr(mbar + PF_K_FULL + k), PRE ? 1 : kPfDeqThreads);
            mbar_init(sm_addr(mbar + PF_V_FULL + k), PRE ? 1 : kPfDeqThreads);
            mbar_init(sm_addr(mbar + PF_PV_DONE + k), 1);
        }
        for (int k = 0; k < 3; ++k) {
            mbar_init(sm_addr(mbar + PF_S_FULL + k), 1);
            mbar_init(sm_addr(mbar + PF_S_FREE + k), kPfSoftWarps * 32);
            mbar_init(sm_addr(mbar + PF_P_USED + k), 1);      // P V(i) has consumed the P held in score buffer i mod 3
        }
        mbar_init(sm_addr(mbar + PF_P_FULL), kPfSoftWarps * 32);
        mbar_init(sm_addr(mbar + PF_AUX), 1);                 // the two rotations before and after the loop
        *abort_s = 0u;
    }
    if (warp == 0) tmem_alloc(sm_addr(tmem_slot), C::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- rotate the CTA's query rows on the tensor core: q_rot = q @ R^T with R as two float16
    // terms of 4096*R stacked along N ([R_hi ; R_lo], 2D rows), q exact in float16.  Operands are built
    // in the (still unused) tile buffers: A = q tile in the P buffers, B in the K/V buffers.
    {
        uint8_t* Aq = Ph;                                                  // [128][D] float16, 2 * PB = 128 * D * 2 bytes
        uint8_t* Bq = Kh;                                                  // [2D][D] float16, 4 * KB = 2D * D * 2 bytes
        for (int w = tid; w < kPfRows * (D / 8); w += kPfThreads) {
            const int r = w / (D / 8), c = w % (D / 8);
            const int row = row0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < n_rows) {
                const int head = hkv * p.G + row / p.Sq, sq = row % p.Sq;
                v = __ldg(reinterpret_cast<const uint4*>(p.q + (((size_t)b * p.Hq + head) * p.Sq + sq) * D) + c);
            }
            *reinterpret_cast<uint4*>(Aq + sw128_off(kPfRows, r, c * 8)) = v;
        }
        for (int w = tid; w < D * (D / 8); w += kPfThreads) {
            const int n = w / (D / 8), c = w % (D / 8);
            const float4 a = __ldg(reinterpret_cast<const float4*>(p.rot + (size_t)n * D + c * 8));
            const float4 bq = __ldg(reinterpret_cast<const float4*>(p.rot + (size_t)n * D + c * 8 + 4));
            const float x[8] = {a.x * 4096.f, a.y * 4096.f, a.z * 4096.f, a.w * 4096.f,
                                bq.x * 4096.f, bq.y * 4096.f, bq.z * 4096.f, bq.w * 4096.f};
            uint32_t h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __half2 hh = __floats2half2_rn(x[2 * e], x[2 * e + 1]);
                const float2 hf = __half22float2(hh);
                h[e] = *reinterpret_cast<const uint32_t*>(&hh);
                l[e] = pack_half2(x[2 * e] - hf.x, x[2 * e + 1] - hf.y);
            }
            *reinterpret_cast<uint4*>(Bq + sw128_off(2 * D, n, c * 8)) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4*>(Bq + sw128_off(2 * D, D + n, c * 8)) = make_uint4(l[0], l[1], l[2], l[3]);
        }
        fence_async_smem();          // the tensor core reads shared memory through the async proxy
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        const uint32_t tmem_base0 = *tmem_slot;
        if (warp == kMmaWarp) {
            if (lane == 0) {
                constexpr uint32_t idesc = umma_idesc_f16(2 * D);
                constexpr uint32_t d_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
                const uint32_t a_lo = ((sm_addr(Aq) >> 4) & 0x3FFFu) | (1u << 16);
                const uint32_t b_lo = ((sm_addr(Bq) >> 4) & 0x3FFFu) | (1u << 16);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t ao = (uint32_t)(((ks >> 2) * (kPfRows * 128) + (ks & 3) * 32) >> 4);
                    const uint32_t bo = (uint32_t)(((ks >> 2) * (2 * D * 128) + (ks & 3) * 32) >> 4);
                    umma_f16_split(tmem_base0, a_lo + ao, d_hi, b_lo + bo, d_hi, idesc, ks ? 1u : 0u);
                }
                umma_commit(sm_addr(mbar + PF_AUX));
            }
            __syncwarp();
        }
        if (warp < kPfRowWarps) {
            bool okq = mbar_wait(sm_addr(mbar + PF_AUX), 0u, abort_s);
            tc_fence_after();
            const uint32_t tlane = tmem_base0 + ((uint32_t)(warp * 32) << 16);
            const float sc = p.scale_log2 * (1.0f / 4096.0f);
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                float vh[32], vl[32];
                tmem_ld32(vh, tlane + c * 32);
                tmem_ld32(vl, tlane + D + c * 32);
                uint32_t h[16], l[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float x0 = (vh[2 * e] + vl[2 * e]) * sc, x1 = (vh[2 * e + 1] + vl[2 * e + 1]) * sc;
                    const __half2 hh = __floats2half2_rn(x0, x1);
                    const float2 hf = __half22float2(hh);
                    h[e] = *reinterpret_cast<const uint32_t*>(&hh);
                    l[e] = pack_half2(x0 - hf.x, x1 - hf.y);
                }
                // the query tile goes to shared memory in the swizzled K-major layout (A operand of the scores)
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    const uint32_t off = sw128_off(kPfRows, tid, c * 32 + g8 * 8);
                    *reinterpret_cast<uint4*>(Qh + off) = make_uint4(h[4 * g8], h[4 * g8 + 1], h[4 * g8 + 2], h[4 * g8 + 3]);
                    *reinterpret_cast<uint4*>(Ql + off) = make_uint4(l[4 * g8], l[4 * g8 + 1], l[4 * g8 + 2], l[4 * g8 + 3]);
                }
            }
            if (!okq) { *abort_s = 1u; if (lane == 0) atomicOr(&g_prefill_error, 4u); }
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();          // query tiles complete; operand buffers and TMEM free for the loop
        tc_fence_after();
    }
    const uint32_t tmem_base = *tmem_slot;

    // tokens this CTA has to visit
    int64_t kv_end = p.S;
    if (p.causal) {
        const int last_row = min(row0 + kPfRows, n_rows) - 1;
        // rows are (head, position) pairs; a tile may span several heads, so take the max
        const int max_sq = (row0 / p.Sq != last_row / p.Sq) ? p.Sq - 1 : last_row % p.Sq;
        kv_end = p.S - p.Sq + max_sq + 1;
        if (kv_end > p.S) kv_end = p.S;
        if (kv_end < 0) kv_end = 0;
    }
    const int n_tiles = (int)((kv_end + kPfTok - 1) / kPfTok);
    const uint8_t* k_row = p.kb + (size_t)kvrow * p.Scap * TBK;
    const uint8_t* v_row = p.vb + (size_t)kvrow * p.Scap * TBV;
    bool ok = true;
    float inv_l = 0.f;                                                    // row owners: 1 / (1024 * row sum)

    if (warp < kPfSoftWarps) {
        // =================================================== softmax: NSPLIT threads per query row
        const int q = warp & 3, hf = warp >> 2;                           // TMEM lane quarter, token part of the tile
        const int r = q * 32 + lane;
        const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
        const int row = row0 + r;
        int limit = p.causal ? (int)(p.S - p.Sq + (row % p.Sq) + 1) : (int)p.S;        // tokens [0, limit)
        if (limit > p.S) limit = (int)p.S;
        if (row >= n_rows || limit < 0) limit = 0;
        float m_run = -INFINITY, m_used = -INFINITY, l_run = 0.f;
        const uint32_t prow = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        constexpr int HT = kPfTok / NSPLIT;                               // tokens per thread and tile
        const uint32_t dk_addr = sm_addr(dmaxK), dv_addr = sm_addr(dmaxV);
        int sk = 0;                                                       // score buffer of tile i: i mod 3
        uint32_t sk_par = 0;                                              // phase parity of that buffer's barriers: (i / 3) & 1
        for (int i = 0; i < n_tiles && ok; ++i, sk = (sk == 2 ? 0 : sk + 1), sk_par ^= (sk == 0 ? 1u : 0u)) {
            const int sb = i & 1;                                         // K / V tile buffer and radii slot
            ok = mbar_wait(sm_addr(mbar + PF_S_FULL + sk), sk_par, abort_s) && ok;
            ok = mbar_wait(sm_addr(mbar + PF_K_FULL + sb), (i >> 1) & 1, abort_s) && ok;   // dmaxK[sb] is visible
            tc_fence_after();
            float mx = -INFINITY, tile_dv = 0.f;
            float s[HT];
            {
                float sl[HT];                                            // the q_hi * k_lo part of the same scores
                if (HT == 32) {
                    tmem_ld32x2(*reinterpret_cast<float(*)[32]>(&s[0]), *reinterpret_cast<float(*)[32]>(&sl[0]),
                                tlane + sk * C::kSCols + hf * HT, tlane + sk * C::kSCols + kPfTok + hf * HT);
                } else {
                    tmem_ld16(*reinterpret_cast<float(*)[16]>(&s[0]), tlane + sk * C::kSCols + hf * HT);
                    tmem_ld16(*reinterpret_cast<float(*)[16]>(&sl[0]), tlane + sk * C::kSCols + kPfTok + hf * HT);
                }
#pragma unroll
                for (int t = 0; t < HT; ++t) s[t] += sl[t];
            }
            {
                const uint32_t dk4 = dk_addr + (uint32_t)((sb * kPfTok + hf * HT) * 4);
                const int tok0 = i * kPfTok + hf * HT;
#pragma unroll
                for (int t4 = 0; t4 < HT / 4; ++t4) {
                    const float4 d4 = lds_f4(dk4 + t4 * 16);
                    s[4 * t4 + 0] *= d4.x;
                    s[4 * t4 + 1] *= d4.y;
                    s[4 * t4 + 2] *= d4.z;
                    s[4 * t4 + 3] *= d4.w;
                }
                if (tok0 + HT > limit) {                                  // only tiles that reach past the row's limit
#pragma unroll
                    for (int t = 0; t < HT; ++t)
                        if (tok0 + t >= limit) s[t] = -INFINITY;
                }
            }
            // this thread's scores are in registers and the key radii are read: the S buffer and dmaxK[sb]
            // are free as far as this thread is concerned
            tc_fence_before();
            mbar_arrive(sm_addr(mbar + PF_S_FREE + sk));
            {
                // partial maximum of this thread's tokens; the threads of a row swap partials through shared
                // memory (one set per tile parity) with the row group's named barrier in between
#pragma unroll
                for (int t = 0; t < HT; ++t) mx = fmaxf(mx, s[t]);
                // ... together with the largest value radius of their tokens (the weights are probability
                // times that radius, split into float16 terms: the lazy rescale below must leave room for it)
                ok = mbar_wait(sm_addr(mbar + PF_V_FULL + sb), (i >> 1) & 1, abort_s) && ok;   // dmaxV[sb] is visible
                float dvl = 0.f;
                {
                    const uint32_t dvx = dv_addr + (uint32_t)((sb * kPfTok + hf * HT) * 4);
#pragma unroll
                    for (int t4 = 0; t4 < HT / 4; ++t4) {
                        const float4 d4 = lds_f4(dvx + t4 * 16);
                        dvl = fmaxf(fmaxf(dvl, fmaxf(d4.x, d4.y)), fmaxf(d4.z, d4.w));
                    }
                }
                float* xm = reinterpret_cast<float*>(Ph) + sb * 4 * kPfRows;          // [parity][part][row]
                float* xd = reinterpret_cast<float*>(Ph) + 12 * kPfRows + sb * 4 * kPfRows;
                xm[hf * kPfRows + r] = mx;
                xd[hf * kPfRows + r] = dvl;
                asm volatile("bar.sync %0, %1;\n" ::"r"(1 + q), "r"(32 * NSPLIT) : "memory");
#pragma unroll
                for (int k = 0; k < NSPLIT; ++k) {
                    mx = fmaxf(mx, xm[k * kPfRows + r]);
                    dvl = fmaxf(dvl, xd[k * kPfRows + r]);
                }
                tile_dv = dvl;
            }
            m_run = fmaxf(m_run, mx);
            // Probabilities first (registers only), relative to the maximum this tile will use: that work
            // overlaps the previous tile's P V, which must be complete before P is rewritten or O rescaled.
            // The row maximum may run ahead of the one in use by up to 2^8, less when the tile holds large
            // radii: probability * radius stays below 2^15, inside the float16 range.
            const float gap = fminf(kPfRescaleGap, 15.0f - __log2f(tile_dv));
            const bool grow = m_run > m_used + gap;                     // also true on the first finite maximum
            const bool rescale = __any_sync(0xffffffffu, grow);         // same outcome in every warp of a row group
            const float m_old = m_used;
            if (rescale) m_used = m_run;
            const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
            const uint32_t dv4 = dv_addr + (uint32_t)((sb * kPfTok + hf * HT) * 4);
            float sum = 0.f;
            uint32_t ph[HT / 2], pl[HT / 2];
#pragma unroll
            for (int c = 0; c < HT / 8; ++c) {
                const float4 da = lds_f4(dv4 + c * 32), db = lds_f4(dv4 + c * 32 + 16);
                const float dv[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int t = c * 8 + 2 * e;
                    const float p0 = fast_exp2(s[t] - m_sub), p1 = fast_exp2(s[t + 1] - m_sub);
                    sum += p0 + p1;
                    const float w0 = p0 * dv[2 * e], w1 = p1 * dv[2 * e + 1];
                    const __half2 hh = __floats2half2_rn(w0, w1);
                    const float2 hfl = __half22float2(hh);
                    ph[c * 4 + e] = *reinterpret_cast<const uint32_t*>(&hh);
                    pl[c * 4 + e] = pack_half2(w0 - hfl.x, w1 - hfl.y);
                }
            }
            if (i > 0 && rescale) {
                // O may only be touched once the previous tile's P V has completed
                ok = mbar_wait(sm_addr(mbar + PF_PV_DONE + ((i - 1) & 1)), ((i - 1) >> 1) & 1, abort_s) && ok;
                tc_fence_after();
                const float alpha = (m_used == -INFINITY) ? 1.f : fast_exp2(m_old - m_used);   // exp2(-inf) = 0
                // the row's O columns in 32-column chunks, dealt round-robin to the row's threads
#pragma unroll 1
                for (int c = hf; c < D / 32; c += NSPLIT) {
                    float o[32];
                    const uint32_t col = C::kOCol + c * 32;
                    tmem_ld32(o, tlane + col);
#pragma unroll
                    for (int k = 0; k < 32; ++k) o[k] *= alpha;
                    tmem_st32(tlane + col, o);
                }
                l_run *= alpha;
            }
            // P goes into the (now dead) S columns of this tile as the A operand of the second contraction:
            // hi term in columns [0, 32) of the buffer, lo term in [32, 64), two tokens per column.  The MMA
            // warp issues S(i + 2), which overwrites these columns, after P(i) V(i); the tensor core runs them in order.
            if (HT == 16) {
                tmem_st8(tlane + sk * C::kSCols + hf * (HT / 2), *reinterpret_cast<const uint32_t(*)[8]>(&ph[0]));
                tmem_st8(tlane + sk * C::kSCols + kPfTok / 2 + hf * (HT / 2), *reinterpret_cast<const uint32_t(*)[8]>(&pl[0]));
            } else {
                tmem_st16(tlane + sk * C::kSCols + hf * (HT / 2), *reinterpret_cast<const uint32_t(*)[16]>(&ph[0]));
                tmem_st16(tlane + sk * C::kSCols + kPfTok / 2 + hf * (HT / 2), *reinterpret_cast<const uint32_t(*)[16]>(&pl[0]));
            }
            tc_fence_before();
            l_run += sum;
            mbar_arrive(sm_addr(mbar + PF_P_FULL));
        }
        if (n_tiles > 0) {
            ok = mbar_wait(sm_addr(mbar + PF_PV_DONE + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1, abort_s) && ok;
            tc_fence_after();
        }
        // row sum over the row's threads (all kept relative to the same m_used), through the dead Ph tile
        float* xchg = reinterpret_cast<float*>(Ph) + 8 * kPfRows;             // past the row-maximum slots
        xchg[hf * kPfRows + r] = l_run;
        asm volatile("bar.sync %0, %1;\n" ::"r"(1 + q), "r"(32 * NSPLIT) : "memory");
        l_run = 0.f;
#pragma unroll
        for (int k = 0; k < NSPLIT; ++k) l_run += xchg[k * kPfRows + r];
        inv_l = l_run > 0.f ? (1.0f / kPfValScale) / l_run : 0.f;
    } else if (PRE && warp < kMmaWarp) {
        // =================================================== copy warp: expanded tiles from the workspace
        if (warp == kPfSoftWarps) {
            const uint8_t* rec0 = p.ws + (size_t)kvrow * ((p.S + kPfTok - 1) / kPfTok) * C::kRec;
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int bb = i & 1;
                const uint32_t par2 = (uint32_t)(((i >> 1) - 1) & 1);
                const uint8_t* rec = rec0 + (size_t)i * C::kRec;
                if (i >= 2) {        // tile i - 2 used this K buffer and radii slot; its scores sit in buffer (i - 2) mod 3
                    const int k2 = (i - 2) % 3;
                    const uint32_t p3 = (uint32_t)(((i - 2) / 3) & 1);
                    ok = mbar_wait(sm_addr(mbar + PF_S_FULL + k2), p3, abort_s, 64) && ok;
                    ok = mbar_wait(sm_addr(mbar + PF_S_FREE + k2), p3, abort_s, 64) && ok;
                }
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t bar = sm_addr(mbar + PF_K_FULL + bb);
                    mbar_expect_tx(bar, 2 * C::KB + kPfTok * 4);
                    bulk_load(sm_addr(Kh + bb * 2 * C::KB), rec, 2 * C::KB, bar);
                    bulk_load(sm_addr(dmaxK + bb * kPfTok), rec + 4 * C::KB, kPfTok * 4, bar);
                }
                __syncwarp();
                if (i >= 2) ok = mbar_wait(sm_addr(mbar + PF_PV_DONE + bb), par2, abort_s, 64) && ok;
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t bar = sm_addr(mbar + PF_V_FULL + bb);
                    mbar_expect_tx(bar, 2 * C::KB + kPfTok * 4);
                    bulk_load(sm_addr(Vh + bb * 2 * C::KB), rec + 2 * C::KB, 2 * C::KB, bar);
                    bulk_load(sm_addr(dmaxV + bb * kPfTok), rec + 4 * C::KB + kPfTok * 4, kPfTok * 4, bar);
                }
                __syncwarp();
            }
        }
    } else if (warp < kMmaWarp) {
        // =================================================== dequantisation, one tile ahead of the MMAs
        const int dt = tid - kPfSoftWarps * 32;
        // this thread's first work item: token, block, 8-element position; the same for every tile
        const int it_tok = dt / (NBLK * 4), it_blk = (dt % (NBLK * 4)) >> 2, it_qw = dt & 3;
        const bool it_first = (dt % (NBLK * 4)) == 0;
        const uint32_t it_off = sw128_off(kPfTok, it_tok, it_blk * 32 + it_qw * 8);
        const uint32_t it_offk = sw128_off(2 * kPfTok, it_tok, it_blk * 32 + it_qw * 8);
        RawItems<D, KBITS> rk;
        RawItems<D, VBITS> rv;
        if (n_tiles > 0) {
            rk.load(k_row, (int)min((int64_t)kPfTok, p.S), it_tok, it_blk, it_qw);
            rv.load(v_row, (int)min((int64_t)kPfTok, p.S), it_tok, it_blk, it_qw);
        }
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int bb = i & 1;
            const uint32_t par2 = (uint32_t)(((i >> 1) - 1) & 1);         // phase of tile i - 2 on a per-parity barrier
            // this tile's raw bytes are in registers; start the next tile's loads before the arithmetic
            RawItems<D, KBITS> nk;
            RawItems<D, VBITS> nv;
            typename RawItems<D, KBITS>::Pending pk;
            typename RawItems<D, VBITS>::Pending pv;
            const bool more = i + 1 < n_tiles;
            const int64_t tok1 = more ? (int64_t)(i + 1) * kPfTok : 0;            // (the last tile re-reads tile 0)
            const int ntok1 = (int)min((int64_t)kPfTok, p.S - tok1);
            RawItems<D, KBITS>::issue(pk, k_row + tok1 * TBK, ntok1, it_tok, it_blk, it_qw);
            RawItems<D, VBITS>::issue(pv, v_row + tok1 * TBV, ntok1, it_tok, it_blk, it_qw);
            // K buffer bb: free once S(i-2) is complete; its dmaxK slot once the softmax of tile i-2 has read it
            if (i >= 2) {            // tile i - 2 used this K buffer and radii slot; its scores sit in buffer (i - 2) mod 3
                const int k2 = (i - 2) % 3;
                const uint32_t p3 = (uint32_t)(((i - 2) / 3) & 1);
                ok = mbar_wait(sm_addr(mbar + PF_S_FULL + k2), p3, abort_s) && ok;
                ok = mbar_wait(sm_addr(mbar + PF_S_FREE + k2), p3, abort_s) && ok;
            }
            if (!ok) break;
            rk.expand(cbk_s, Kh + bb * 2 * C::KB, Kh + bb * 2 * C::KB + kPfTok * 128, dmaxK + bb * kPfTok,
                      1.0f / kPfValScale, it_tok, it_blk, it_first, it_offk);
            fence_async_smem();
            mbar_arrive(sm_addr(mbar + PF_K_FULL + bb));
            nk.pack(pk, ntok1, it_tok);           // the loads issued at the top have landed by now
            nv.pack(pv, ntok1, it_tok);
            // V buffer bb (and dmaxV[bb]): free once P(i-2) V(i-2) has completed
            if (i >= 2) ok = mbar_wait(sm_addr(mbar + PF_PV_DONE + bb), par2, abort_s) && ok;
            if (!ok) break;
            rv.expand(cbv_s, Vh + bb * 2 * C::KB, Vh + bb * 2 * C::KB + C::KB, dmaxV + bb * kPfTok, 1.0f, it_tok, it_blk,
                      it_first, it_off);
            fence_async_smem();
            mbar_arrive(sm_addr(mbar + PF_V_FULL + bb));
            rk = nk;
            rv = nv;
        }
    } else {
        // =================================================== MMA issue (all lanes loop, lane 0 issues)
        const uint32_t issue = lane == 0 ? 1u : 0u;
        constexpr uint32_t idesc_s = umma_idesc_f16(kPfTok);                   // M 128, N 64, A and B K-major
        constexpr uint32_t idesc_s2 = umma_idesc_f16(2 * kPfTok);              // N 128: hi and lo rows of K at once
        constexpr uint32_t idesc_pv = umma_idesc_f16(D) | (1u << 16);          // M 128, N D, B MN-major
        constexpr uint32_t d_hi = (1024u >> 4) | (1u << 14) | (2u << 29);      // 8-row groups 1024 B apart, SWIZZLE_128B
        const uint32_t k_h0 = ((sm_addr(Kh) >> 4) & 0x3FFFu) | (1u << 16);
        // V: 64-dim atoms kPfTok*128 B apart (leading offset), 8-token groups 1024 B apart
        constexpr uint32_t v_lbo = ((kPfTok * 128u) >> 4) << 16;
        const uint32_t v_h0 = ((sm_addr(Vh) >> 4) & 0x3FFFu) | v_lbo;
        const uint32_t q_h = ((sm_addr(Qh) >> 4) & 0x3FFFu) | (1u << 16), q_l = ((sm_addr(Ql) >> 4) & 0x3FFFu) | (1u << 16);
        auto issue_s = [&](int i) {
            const int sb = i & 1, sk = i % 3;                    // K tile buffer, score buffer
            if (i >= 3) {
                // score buffer sk: the scores of tile i - 3 have been read, and the P that replaced them has been
                // consumed by P(i-3) V(i-3) (with one issuing warp the tensor core's in-order execution already
                // gives that order; with two it has to be waited for)
                const uint32_t p3 = (uint32_t)(((i - 3) / 3) & 1);
                ok = mbar_wait(sm_addr(mbar + PF_S_FREE + sk), p3, abort_s, 32) && ok;
                if (PRE) ok = mbar_wait(sm_addr(mbar + PF_P_USED + sk), p3, abort_s, 32) && ok;
            }
            ok = mbar_wait(sm_addr(mbar + PF_K_FULL + sb), (i >> 1) & 1, abort_s, 32) && ok;
            if (!ok) return;
            tc_fence_after();
            {
                // K tile: per 64-dim half 128 rows (64 hi tokens, then 64 lo).  q_hi against all 128 rows
                // (one MMA, N = 128: columns [0, 64) hi products, [64, 128) lo products), q_lo against the hi rows.
                const uint32_t acc = tmem_base + sk * C::kSCols;
                const uint32_t k_b = k_h0 + (uint32_t)(sb * 2 * (C::KB >> 4));
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t qo = (uint32_t)(((ks >> 2) * (kPfRows * 128) + (ks & 3) * 32) >> 4);
                    const uint32_t ko = (uint32_t)(((ks >> 2) * (2 * kPfTok * 128) + (ks & 3) * 32) >> 4);
                    umma_f16_split_pred(acc, q_h + qo, d_hi, k_b + ko, d_hi, idesc_s2, ks ? 1u : 0u, issue);
                    umma_f16_split_pred(acc, q_l + qo, d_hi, k_b + ko, d_hi, idesc_s, 1u, issue);
                }
                umma_commit_pred(sm_addr(mbar + PF_S_FULL + sk), issue);
            }
            __syncwarp();
        };
        if (PRE && warp == kMmaWarp) {
            for (int i = 0; i < n_tiles && ok; ++i) issue_s(i);
        } else
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int sb = i & 1;
            if (!PRE) {                       // one warp: S(i+1) goes out before P(i) V(i)
                if (i == 0) issue_s(0);
                if (i + 1 < n_tiles) issue_s(i + 1);
            }
            ok = mbar_wait(sm_addr(mbar + PF_P_FULL), i & 1, abort_s, 32) && ok;
            ok = mbar_wait(sm_addr(mbar + PF_V_FULL + sb), (i >> 1) & 1, abort_s, 32) && ok;
            if (!ok) break;
            tc_fence_after();
            {
                const uint32_t acc = tmem_base + C::kOCol;
                const uint32_t v_h = v_h0 + (uint32_t)(sb * 2 * (C::KB >> 4)), v_l = v_h + (C::KB >> 4);
#pragma unroll
                for (int kt = 0; kt < kPfTok / 16; ++kt) {
                    const uint32_t vo = (uint32_t)((kt * 16 * 128) >> 4);
                    const uint32_t p_h = tmem_base + (i % 3) * C::kSCols + kt * 8, p_l = p_h + kPfTok / 2;
                    umma_f16_ts_pred(acc, p_h, v_h + vo, d_hi, idesc_pv, (i > 0 || kt > 0) ? 1u : 0u, issue);
                    umma_f16_ts_pred(acc, p_h, v_l + vo, d_hi, idesc_pv, 1u, issue);
                    umma_f16_ts_pred(acc, p_l, v_h + vo, d_hi, idesc_pv, 1u, issue);
                }
                umma_commit_pred(sm_addr(mbar + PF_PV_DONE + sb), issue);
                if (PRE) umma_commit_pred(sm_addr(mbar + PF_P_USED + (i % 3)), issue);
            }
            __syncwarp();
        }
    }
    if (!ok) {
        *abort_s = 1u;
        if (lane == 0) atomicOr(&g_prefill_error, 4u);
    }
    tc_fence_before();
    __syncthreads();          // every tile buffer is dead
    tc_fence_after();

    // ---- normalise and rotate back on the tensor core: out = o_rot @ R as o_hi*Rt_hi + o_hi*Rt_lo +
    // o_lo*Rt_hi with Rt = 4096 * R^T.  A = o as two float16 terms in the query buffers, B = [Rt_hi ; Rt_lo]
    // stacked along N in the K/V buffers.
    {
        uint8_t* Bq = Kh;
        if (warp < kPfRowWarps) {
            const uint32_t tlane = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                float o[32];
                if (n_tiles > 0) {
                    tmem_ld32(o, tlane + C::kOCol + c * 32);
                } else {
#pragma unroll
                    for (int k = 0; k < 32; ++k) o[k] = 0.f;
                }
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    uint32_t h[4], l[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int k = g8 * 8 + 2 * e;
                        const float x0 = o[k] * inv_l, x1 = o[k + 1] * inv_l;
                        const __half2 hh = __floats2half2_rn(x0, x1);
                        const float2 hf = __half22float2(hh);
                        h[e] = *reinterpret_cast<const uint32_t*>(&hh);
                        l[e] = pack_half2(x0 - hf.x, x1 - hf.y);
                    }
                    const uint32_t off = sw128_off(kPfRows, tid, c * 32 + g8 * 8);
                    *reinterpret_cast<uint4*>(Qh + off) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4*>(Ql + off) = make_uint4(l[0], l[1], l[2], l[3]);
                }
            }
        }
        // B[n][j] = 4096 * R[j][n]: lanes walk n, so the reads of R are contiguous
        for (int w = tid; w < D * (D / 8); w += kPfThreads) {
            const int c = w / D, n = w % D;
            uint32_t h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x0 = __ldg(p.rot + (size_t)(c * 8 + 2 * e) * D + n) * 4096.f;
                const float x1 = __ldg(p.rot + (size_t)(c * 8 + 2 * e + 1) * D + n) * 4096.f;
                const __half2 hh = __floats2half2_rn(x0, x1);
                const float2 hf = __half22float2(hh);
                h[e] = *reinterpret_cast<const uint32_t*>(&hh);
                l[e] = pack_half2(x0 - hf.x, x1 - hf.y);
            }
            *reinterpret_cast<uint4*>(Bq + sw128_off(2 * D, n, c * 8)) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4*>(Bq + sw128_off(2 * D, D + n, c * 8)) = make_uint4(l[0], l[1], l[2], l[3]);
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();          // operands complete, every thread has read its part of O
        tc_fence_after();
        if (warp == kMmaWarp) {
            if (lane == 0) {
                constexpr uint32_t idesc2 = umma_idesc_f16(2 * D), idesc1 = umma_idesc_f16(D);
                constexpr uint32_t d_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
                const uint32_t ah = ((sm_addr(Qh) >> 4) & 0x3FFFu) | (1u << 16), al = ((sm_addr(Ql) >> 4) & 0x3FFFu) | (1u << 16);
                const uint32_t b_lo = ((sm_addr(Bq) >> 4) & 0x3FFFu) | (1u << 16);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t ao = (uint32_t)(((ks >> 2) * (kPfRows * 128) + (ks & 3) * 32) >> 4);
                    const uint32_t bo = (uint32_t)(((ks >> 2) * (2 * D * 128) + (ks & 3) * 32) >> 4);
                    umma_f16_split(tmem_base, ah + ao, d_hi, b_lo + bo, d_hi, idesc2, ks ? 1u : 0u);
                }
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {       // o_lo against the hi rows only (N = D)
                    const uint32_t ao = (uint32_t)(((ks >> 2) * (kPfRows * 128) + (ks & 3) * 32) >> 4);
                    const uint32_t bo = (uint32_t)(((ks >> 2) * (2 * D * 128) + (ks & 3) * 32) >> 4);
                    umma_f16_split(tmem_base, al + ao, d_hi, b_lo + bo, d_hi, idesc1, 1u);
                }
                umma_commit(sm_addr(mbar + PF_AUX));
            }
            __syncwarp();
        }
        if (warp < kPfRowWarps) {
            const bool oko = mbar_wait(sm_addr(mbar + PF_AUX), 1u, abort_s);
            tc_fence_after();
            const uint32_t tlane = tmem_base + ((uint32_t)(warp * 32) << 16);
            const int row = row0 + tid;
            const int head = hkv * p.G + (row < n_rows ? row / p.Sq : 0), sq = row < n_rows ? row % p.Sq : 0;
            const size_t off = (((size_t)b * p.Hq + head) * p.Sq + sq) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                float va[32], vb[32];
                tmem_ld32(va, tlane + c * 32);
                tmem_ld32(vb, tlane + D + c * 32);
                if (row < n_rows) {
                    if (p.out_is_fp16) {
                        __half* dst = static_cast<__half*>(p.out) + off + c * 32;
#pragma unroll
                        for (int k = 0; k < 32; k += 2) {
                            const float x0 = (va[k] + vb[k]) * (1.0f / 4096.0f), x1 = (va[k + 1] + vb[k + 1]) * (1.0f / 4096.0f);
                            *reinterpret_cast<__half2*>(dst + k) = __floats2half2_rn(fminf(fmaxf(x0, -65504.f), 65504.f),
                                                                                      fminf(fmaxf(x1, -65504.f), 65504.f));
                        }
                    } else {
                        float* dst = static_cast<float*>(p.out) + off + c * 32;
#pragma unroll
                        for (int k = 0; k < 32; k += 4)
                            *reinterpret_cast<float4*>(dst + k) = make_float4((va[k] + vb[k]) * (1.0f / 4096.0f),
                                                                              (va[k + 1] + vb[k + 1]) * (1.0f / 4096.0f),
                                                                              (va[k + 2] + vb[k + 2]) * (1.0f / 4096.0f),
                                                                              (va[k + 3] + vb[k + 3]) * (1.0f / 4096.0f));
                    }
                }
            }
            if (!oko) { *abort_s = 1u; if (lane == 0) atomicOr(&g_prefill_error, 4u); }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, C::kTmemCols);
}

template <int D, int KBITS, int VBITS>
static int launch_prefill(const PrefillParams& p, int rows, uint8_t* ws, cudaStream_t st) {
    const size_t smem = PrefillCfg<D>::smem_bytes();
    const int n_rows = p.G * p.Sq;
    dim3 grid((n_rows + kPfRows - 1) / kPfRows, rows, 1);
    if (ws) {
        // expand every tile once, then run the attention kernel on the expanded tiles
        const int n_tiles = (int)((p.S + kPfTok - 1) / kPfTok);
        pq_prefill_expand_kernel<D, KBITS, VBITS><<<dim3(n_tiles, rows, 1), kPfDeqThreads, 0, st>>>(p, ws, n_tiles);
        if (cudaGetLastError() != cudaSuccess) return PQ_ERR_CUDA;
        auto kern = pq_prefill_attn_kernel<D, 4, 4, true>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return PQ_ERR_CUDA;
        kern<<<grid, pf_threads(true), smem, st>>>(p);
    } else {
        auto kern = pq_prefill_attn_kernel<D, KBITS, VBITS, false>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return PQ_ERR_CUDA;
        kern<<<grid, pf_threads(false), smem, st>>>(p);
    }
    return cudaGetLastError() == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
}

// Read and clear this file's device error flag (for pq_poll_device_errors).
int prefill_error_flags(unsigned int* flags) {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_prefill_error, sizeof(v)) != cudaSuccess) return PQ_ERR_CUDA;
    if (v && cudaMemcpyToSymbol(g_prefill_error, &zero, sizeof(zero)) != cudaSuccess) return PQ_ERR_CUDA;
    *flags = v;
    return PQ_OK;
}

}  // namespace pq

extern "C" size_t pq_prefill_attn_workspace_bytes(int batch, int kv_heads, int64_t seq_len, int head_dim) {
    if (batch <= 0 || kv_heads <= 0 || seq_len <= 0 || (head_dim != 64 && head_dim != 128)) return 0;
    const size_t rec = head_dim == 64 ? pq::PrefillCfg<64>::kRec : pq::PrefillCfg<128>::kRec;
    return (size_t)batch * kv_heads * (size_t)((seq_len + pq::kPfTok - 1) / pq::kPfTok) * rec;
}

extern "C" int pq_prefill_attn(const void* q, const void* k_blocks, const void* v_blocks,
                               int batch, int q_heads, int kv_heads, int seq_q, int64_t seq_len,
                               int64_t seq_capacity, int head_dim, int k_bits, int v_bits,
                               const float* codebook_k, const float* codebook_v, const float* rot,
                               float scale, int causal, void* out, int out_is_fp16, void* workspace,
                               size_t workspace_bytes, void* stream) {
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
        (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(rot) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & (out_is_fp16 ? 3 : 15)))
        return PQ_ERR_MISALIGNED;
    const int rows = batch * kv_heads;
    if (rows > 65535) return PQ_ERR_TOO_LARGE;
    if (workspace) {
        if (reinterpret_cast<uintptr_t>(workspace) & 15) return PQ_ERR_MISALIGNED;
        if (workspace_bytes < pq_prefill_attn_workspace_bytes(batch, kv_heads, seq_len, head_dim))
            return PQ_ERR_SCRATCH_TOO_SMALL;
    }
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
    p.ws = static_cast<const uint8_t*>(workspace);
    for (int i = 0; i < 16; ++i) {
        p.cbk[i] = i < (1 << k_bits) ? codebook_k[i] : 0.f;
        p.cbv[i] = i < (1 << v_bits) ? codebook_v[i] : 0.f;
    }
#define PQ_PF(DD, KB, VB) \
    if (head_dim == DD && k_bits == KB && v_bits == VB) \
        return launch_prefill<DD, KB, VB>(p, rows, static_cast<uint8_t*>(workspace), st);
    PQ_PF(64, 4, 4) PQ_PF(64, 4, 2) PQ_PF(64, 2, 4) PQ_PF(64, 2, 2)
    PQ_PF(128, 4, 4) PQ_PF(128, 4, 2) PQ_PF(128, 2, 4) PQ_PF(128, 2, 2)
#undef PQ_PF
    return PQ_ERR_BAD_HEAD_DIM;
}
