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
// centroid products cost 2*G FMAs per stored nibble, more than the FP32 pipe can issue at
// HBM speed.  Both contractions therefore run as mma.sync.m16n8k16 with two-term float16
// operands (value = hi + lo, ~22 mantissa bits) and float32 accumulation, which keeps the
// float32-level accuracy the 2e-3 output tolerance needs (one float16 rounding of the
// dequantised K is 15x too coarse on outlier-channel data).
//   scores:  A = centroids of 16 tokens x 16 dims, B = the query heads as MMA columns
//            (4 heads x {hi, lo} in one n-tile, or 8 heads as a hi tile and a lo tile);
//            the block radius multiplies the per-block partial sum in float32.
//   values:  A = centroids^T of 16 dims x 16 tokens, B = p * radius per (token, head)
//            with the same column arrangement.
// Centroids come from a shared-memory table indexed by a whole byte of packed indices
// (two nibbles / four crumbs per lookup, hi and lo terms in one entry), one private copy
// per lane so lookups never bank-conflict; a byte is moved into address position with a
// single byte-permute.
//
// Work split: persistent CTAs, one per SM, 16 warps each, in two independent teams of 8 (one team with the
// key sketch).  The 16-token tiles of all (batch, kv head, head group) rows form one sequence that is cut
// into equal contiguous ranges, one per team (n_splits == 0), or every row is cut into n_splits equal
// segments dealt round-robin (n_splits > 0).  A team rotates the queries of up to four consecutive
// segments of its range in one pass.  Inside a segment a warp owns every 8th tile, staged through a private
// 3-stage ring by bulk copies (rows off the 16-byte grid and ragged last tiles by the warp's own loads).
// Per segment the team reduces its warps' partials in shared memory and writes one (m, l, o) record per
// query head; the last segment of a row to finish (atomic ticket, no spinning) merges the row's records,
// normalises, rotates back and resets the ticket.
#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>

#include "pq_tcgen05.cuh"

namespace pq {

constexpr int kTileTok = 16;
constexpr int kRecHeads = 8;        // head slots per record in the scratch buffer
constexpr float kCbScale = 64.0f;   // key centroids are stored x64 in the table (keeps lo terms normal)
constexpr int kTabBytes = 65536;    // 256 byte values x 256 B: K copies at +0, V copies at +128
// float16 terms per VALUE centroid in the table.  1: the value centroids are scaled (host-side search,
// value_table_scale) so that every one of them is a float16 number to about 3e-5 relative, which keeps
// the output error near 5e-4 of the 2e-3 tolerance and halves the value-side lookups and MMAs;
// 2: {hi, lo} pairs like the keys (float32-level accuracy).  One term fails the 2e-3 bar on short,
// peaked sequences with large values (measured 2.9e-3), so two are used.
// Launch shape, overridable on the compiler command line for timing experiments: warps per CTA, teams
// of warps per CTA (see DecodeCfg), tile stages per warp.  Measured on the 32 x 8 x 8192-token workload with
// one query rotation per segment: 16 warps in 2 teams 141.8 us, 20 warps in 2 teams 143.8, 20 warps in one
// team 149.5, 4 teams 142-149.  (With the rotation shared by a team's segments - 137 us - the query buffers of
// four teams or the rings of twenty warps no longer fit shared memory; two stages instead of three: 138.4.)
#ifndef PQ_DEC_TEAMS
#define PQ_DEC_TEAMS 2
#endif
#ifndef PQ_DEC_STAGES
#define PQ_DEC_STAGES 3
#endif
#ifndef PQ_DEC_WARPS
#define PQ_DEC_WARPS 16
#endif
constexpr int kVTerms = 2;

// Device error flags of this file (read and cleared through pq_poll_device_errors):
// bit 0: the shared-memory window started too high for the fixed-address table, nothing was computed;
// bit 1: a bounded wait for a tile copy gave up.
static __device__ unsigned int g_decode_error = 0;

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
    int64_t S, Scap;           // S: the length the work plan is made for
    // When set, the number of tokens attended to is read from device memory at kernel start and
    // clamped to [0, S] (a step of a captured graph whose cache grows on the device).
    const int64_t* seq_len_dev;
    int Hq, Hkv, G, HG, n_rows;
    int splits, tiles_per_split, max_segs;   // splits == 0: balanced contiguous partition
    int n_workers;             // balanced mode: teams that own a range of tiles (<= teams in the grid)
    int jl_dim;
    int out_is_fp16;
    float scale_log2;          // softmax scale * log2(e)
    float v_scale, v_inv;      // value centroids are stored x v_scale; v_inv = 1 / v_scale
    float cbk[16], cbv[16];
};

// ------------------------------------------------------------------ shared-memory access
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint32_t v;
    asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }\n" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_u32(uint32_t a, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ float lds_half_as_float(uint32_t a) {
    float v;
    asm volatile("{ .reg .b16 h; ld.shared.b16 h, [%1]; cvt.f32.f16 %0, h; }\n" : "=f"(v) : "r"(a));
    return v;
}
// The centroid table sits at shared address kTabAddr (a multiple of 64 KB), one 256-byte row
// per byte value.  `lane_const` = kTabAddr | offset of this lane's copy inside a row (< 256),
// so byte J of w dropped into bits 8..15 of lane_const IS the address of the entry.
constexpr uint32_t kTabAddr = 0x10000u;
template <int J>
__device__ __forceinline__ uint32_t entry_addr(uint32_t w, uint32_t lane_const) {
    return __byte_perm(w, lane_const, 0x7604u | (J << 4));
}
// the same with the byte number held in a register: sel = byte_selector(j)
__device__ __forceinline__ uint32_t byte_selector(int j) { return 0x7604u | ((uint32_t)j << 4); }
__device__ __forceinline__ uint32_t entry_addr_sel(uint32_t w, uint32_t lane_const, uint32_t sel) {
    return __byte_perm(w, lane_const, sel);
}
// 32 bits of packed indices at a shared address whose alignment class is known statically
template <bool ALIGNED4>
__device__ __forceinline__ uint32_t lds_word(uint32_t a) {
    if (ALIGNED4) return lds_u32(a);
    return __byte_perm(lds_u16(a), lds_u16(a + 2), 0x5410);
}

// ------------------------------------------------------------------ centroid tables
// Row r (256 B) belongs to byte value r; `half_off` is 0 for the K copies and 128 for the V copies;
// `cs` holds the split centroids as bit patterns: cs[i] = hi16(scale*c[i]) | lo16 << 16.
// TERMS == 2 (two float16 terms per centroid):
//   4-bit: entry = {half2(c[r&15], c[r>>4]) hi, same lo}, 8 bytes, 16 lane copies;
//   2-bit: entry = {hi(c[r&3], c[r>>2&3]), lo(same), hi(c[r>>4&3], c[r>>6]), lo(same)}, 16 bytes, 8 copies.
// TERMS == 1 (hi terms only):
//   4-bit: entry = half2(c[r&15], c[r>>4]), 4 bytes, 32 lane copies;
//   2-bit: entry = {hi(c[r&3], c[r>>2&3]), hi(c[r>>4&3], c[r>>6])}, 8 bytes, 16 copies.
template <int BITS, int TERMS>
__device__ __forceinline__ void build_table(uint8_t* tab, int half_off, const uint32_t* cs, int tid, int nthreads) {
    if (BITS == 4 && TERMS == 2) {
        for (int e = tid; e < 256 * 16; e += nthreads) {
            const int b = e >> 4, copy = e & 15;
            const uint32_t c0 = cs[b & 15], c1 = cs[b >> 4];
            *reinterpret_cast<uint2*>(tab + b * 256 + half_off + copy * 8) =
                make_uint2(__byte_perm(c0, c1, 0x5410), __byte_perm(c0, c1, 0x7632));
        }
    } else if (BITS == 4) {
        for (int e = tid; e < 256 * 32; e += nthreads) {
            const int b = e >> 5, copy = e & 31;
            *reinterpret_cast<uint32_t*>(tab + b * 256 + half_off + copy * 4) =
                __byte_perm(cs[b & 15], cs[b >> 4], 0x5410);
        }
    } else if (TERMS == 2) {
        for (int e = tid; e < 256 * 8; e += nthreads) {
            const int b = e >> 3, copy = e & 7;
            const uint32_t c0 = cs[b & 3], c1 = cs[(b >> 2) & 3], c2 = cs[(b >> 4) & 3], c3 = cs[b >> 6];
            *reinterpret_cast<uint4*>(tab + b * 256 + half_off + copy * 16) =
                make_uint4(__byte_perm(c0, c1, 0x5410), __byte_perm(c0, c1, 0x7632),
                           __byte_perm(c2, c3, 0x5410), __byte_perm(c2, c3, 0x7632));
        }
    } else {
        for (int e = tid; e < 256 * 16; e += nthreads) {
            const int b = e >> 4, copy = e & 15;
            const uint32_t c0 = cs[b & 3], c1 = cs[(b >> 2) & 3], c2 = cs[(b >> 4) & 3], c3 = cs[b >> 6];
            *reinterpret_cast<uint2*>(tab + b * 256 + half_off + copy * 8) =
                make_uint2(__byte_perm(c0, c1, 0x5410), __byte_perm(c2, c3, 0x5410));
        }
    }
}

// ------------------------------------------------------------------ tile staging (slow path)
// Rows whose byte streams are not 16-byte aligned, and the ragged last tile of a sequence, are
// copied by the warp itself: `n` bytes from `src`, the rest of the `cap` bytes cleared (tokens past
// the end must read as finite numbers: radius 0).  K/V tiles go as 4-byte words (block sizes are
// multiples of 2 and tokens of 4 bytes), the sketch side band byte by byte.
__device__ __forceinline__ void copy_words(uint8_t* dst, const uint8_t* src, int n, int cap, int lane) {
    for (int c = lane; c < (cap >> 2); c += 32)
        reinterpret_cast<uint32_t*>(dst)[c] = c < (n >> 2) ? __ldg(reinterpret_cast<const uint32_t*>(src) + c) : 0u;
}
__device__ __forceinline__ void copy_bytes(uint8_t* dst, const uint8_t* src, int n, int cap, int lane) {
    for (int c = lane; c < cap; c += 32) dst[c] = c < n ? __ldg(src + c) : (uint8_t)0;
}

// Asks L2 for `bytes` (a multiple of 16) at a 16-byte aligned global address; nothing waits for it.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(gsrc), "r"(bytes) : "memory");
}

template <int D, int KBITS, int VBITS, int NH, bool QJL>
struct DecodeCfg {
    static constexpr int NBLK = D / 32;
    static constexpr int HPC = 4 * NH;                            // query heads per CTA
    // Warps per CTA and tile stages per warp (16 warps of at most 128 registers; 12, 16 and 20 warps run
    // the tile loop at the same rate).
    static constexpr int NWARPS = PQ_DEC_WARPS;
    static constexpr int NTHREADS = NWARPS * 32;
    // The warps of a CTA form kTeams independent teams, each walking its own range of tiles with its own
    // query buffers and barrier: while one team is between two segments (query rotation, record merge,
    // final rotation) the other keeps the SM's pipes busy.  (A dozen warps already reach the tile rate of
    // twenty, so a team alone nearly fills the SM.)
    static constexpr int kTeams = QJL ? 1 : PQ_DEC_TEAMS;
    static constexpr int kTeamWarps = NWARPS / kTeams;
    static constexpr int kTeamThreads = kTeamWarps * 32;
    static constexpr int kStages = PQ_DEC_STAGES;
    // Query rows rotated in one pass.  The rotation MMA has 16 rows and one segment fills HPC of them, so a
    // team rotates the queries of up to 16 / HPC consecutive segments of its range together: the second
    // and third segment of a team then start without the two memory round trips of a rotation.  (With the
    // key sketch the projected query takes the room, and with eight heads per segment the registers of
    // the second row set spill in the tile loop: there a pass serves one segment.)
    static constexpr int kQRows = (QJL || NH == 2) ? HPC : 16;
    static constexpr int kSegBatch = kQRows / HPC;
    static constexpr int BBK = block_bytes(KBITS), BBV = block_bytes(VBITS);
    static constexpr int TBK = NBLK * BBK, TBV = NBLK * BBV;     // bytes per token
    static constexpr int kStageK = kTileTok * TBK;                // multiples of 64 bytes
    static constexpr int kStageV = kTileTok * TBV;
    static constexpr int kStageN = QJL ? 32 : 0;                  // 16 float16 norms
    static constexpr int kSignTab = QJL ? 16 * 16 * 8 : 0;
    // head of a warp's ring: kStages mbarriers (32 bytes) + the tile's value radii, compacted
    static constexpr int kRingHead = 32 + kTileTok * NBLK * 2;
    __host__ __device__ static int stage_bits(int jl_dim) { return QJL ? kTileTok * (jl_dim / 8) : 0; }
    __host__ __device__ static int stage_bytes_total(int jl_dim) {
        return kStageK + kStageV + stage_bits(jl_dim) + kStageN;
    }
    __host__ __device__ static int qjl_frag_bytes(int jl_dim) { return QJL ? (jl_dim / 16) * 32 * 16 : 0; }
    // Shared-memory plan (byte addresses in the shared window):
    //   [base, 64K)        the teams' query buffers, split codebooks, the rings of the first n_low warps
    //   [64K, 128K)        centroid table (its address is baked into the lookups)
    //   [128K, ...)        sign table, JL query fragments, the rings of the remaining warps
    // A ring = head (see kRingHead) + kStages tile stages; at the end of a work item the warp parks
    // its (m, l, o) record over the stages.
    __host__ __device__ static int ring_bytes(int jl_dim) {
        const int r = kStages * stage_bytes_total(jl_dim), rec = HPC * (D + 2) * 4;
        return kRingHead + (((r > rec ? r : rec) + 15) & ~15);
    }
    __host__ __device__ static int low_fixed(int jl_dim) {
        // per team: rotated queries [kQRows][D], final-stage buffer [HPC][D] (+ the projected query with QJL)
        return ((kTeams * ((kQRows + HPC) * D + (QJL ? HPC * jl_dim : 0)) * 4 + 2 * 16 * 4) + 15) & ~15;
    }
    // rings that fit below the table when the dynamic window starts at or below 8 KB
    __host__ __device__ static int n_low(int jl_dim) {
        int n = (65536 - 8192 - low_fixed(jl_dim)) / ring_bytes(jl_dim);
        return n > NWARPS ? NWARPS : n;
    }
    __host__ __device__ static size_t smem_bytes(int jl_dim) {
        size_t high = kSignTab + qjl_frag_bytes(jl_dim) + (size_t)(NWARPS - n_low(jl_dim)) * ring_bytes(jl_dim);
        return 2 * 65536 + high + 16;
    }
};

// float -> the float16 term this lane contributes: hi, or lo = v - hi
__device__ __forceinline__ float term_of(float v, bool want_lo) {
    const float hi = __half2float(__float2half_rn(v));
    return want_lo ? v - hi : v;
}

__device__ __forceinline__ __half2 as_half2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Two float16 terms of (ph + pl) * d per half: hi = rn(ph*d), lo = rn(pl*d + (ph*d - hi)); the inner
// difference is exact in float16 (error-free product), so hi + lo carries about 22 bits.
__device__ __forceinline__ void weight_terms(uint32_t ph, uint32_t pl, uint32_t dd, uint32_t& bh, uint32_t& bl) {
    const __half2 P = as_half2(ph), L = as_half2(pl), R = as_half2(dd);
    const __half2 hi = __hmul2(P, R);
    const __half2 err = __hfma2(P, R, __hneg2(hi));
    bh = as_u32(hi);
    bl = as_u32(__hfma2(L, R, err));
}

template <int D, int KBITS, int VBITS, int NH, bool QJL>
__global__ void __launch_bounds__(DecodeCfg<D, KBITS, VBITS, NH, QJL>::NTHREADS, 1)
pq_decode_attn_kernel(const DecodeParams p) {
    using C = DecodeCfg<D, KBITS, VBITS, NH, QJL>;
    constexpr int NT = C::NTHREADS;
    constexpr int kStages = C::kStages;
    constexpr int NBLK = C::NBLK;
    constexpr int HPC = C::HPC;
    constexpr int VT = kVTerms;
    constexpr int VENT = (VBITS == 4 ? 4 : 8) * VT;                      // bytes per value-table entry
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kTeams = C::kTeams, TW = C::kTeamWarps, TT = C::kTeamThreads;
    const int team = (threadIdx.x >> 5) / TW;                            // this warp's team
    constexpr int kQRows = C::kQRows, kSegBatch = C::kSegBatch;
    const int team_buf = (kQRows + HPC) * D + (QJL ? HPC * p.jl_dim : 0);   // floats per team
    float* q_rot_all = reinterpret_cast<float*>(smem) + team * team_buf; // [kQRows][D] rotated, scaled
    float* o_fin = q_rot_all + kQRows * D;                               // [HPC][D] final stage
    float* q_jl = o_fin + HPC * D;                                       // [HPC][M] (QJL)
    uint32_t* cs_k = reinterpret_cast<uint32_t*>(reinterpret_cast<float*>(smem) + kTeams * team_buf);   // split centroids
    uint32_t* cs_v = cs_k + 16;
    const uint32_t smem_base = smem_addr(smem);
    uint8_t* low_ring = smem + C::low_fixed(QJL ? p.jl_dim : 0);
    uint8_t* tab = smem + (kTabAddr - smem_base);                        // shared address 64K exactly
    uint8_t* signtab = tab + kTabBytes;
    uint8_t* qjl_frag = signtab + C::kSignTab;
    uint8_t* high_ring = qjl_frag + C::qjl_frag_bytes(QJL ? p.jl_dim : 0);
    __shared__ unsigned int s_ticket_all[kTeams];
    unsigned int& s_ticket = s_ticket_all[team];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tw = warp - team * TW;                                     // warp index inside the team
    const int tid = threadIdx.x - team * TT;                             // thread index inside the team
    const int g = lane >> 2, t = lane & 3;
    // barrier of the team (the whole CTA when there is one team)
    auto team_sync = [&]() {
        if (kTeams == 1) __syncthreads();
        else asm volatile("bar.sync %0, %1;\n" ::"r"(1 + team), "r"(TT) : "memory");
    };
    const int M = QJL ? p.jl_dim : 0;
    const int stage_sz = C::stage_bytes_total(M);
    const int n_low = C::n_low(M);
    if (smem_base + C::low_fixed(M) + n_low * C::ring_bytes(M) > kTabAddr) {   // window starts too high
        if (threadIdx.x == 0) atomicOr(&g_decode_error, 1u);
        return;
    }
    auto ring_of = [&](int w) -> uint8_t* {
        return w < n_low ? low_ring + (size_t)w * C::ring_bytes(M) : high_ring + (size_t)(w - n_low) * C::ring_bytes(M);
    };
    auto rec_of = [&](int w) -> float* { return reinterpret_cast<float*>(ring_of(w) + C::kRingHead); };
    uint8_t* my_ring = ring_of(warp);
    uint8_t* my_stages = my_ring + C::kRingHead;
    const uint32_t ring_addr = smem_addr(my_ring);
    const uint32_t mbar0 = ring_addr;                                    // kStages mbarriers, 8 bytes each
    const uint32_t vrad_addr = ring_addr + 32;                           // [16 tokens][NBLK] float16 radii
    const uint32_t stage_addr0 = ring_addr + C::kRingHead;

    // ---- once per CTA: the lookup tables (the CTA is persistent and walks over work items)
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(mbar0 + 8 * s, 1);
    }
    if (threadIdx.x < 32) {
        const int i = threadIdx.x;
        const float c = i < 16 ? p.cbk[i] * kCbScale : p.cbv[i - 16] * p.v_scale;
        __half h, l;
        split_half(c, h, l);
        cs_k[i] = (uint32_t)__half_as_ushort(h) | ((uint32_t)__half_as_ushort(l) << 16);   // cs_v = cs_k + 16
    }
    if (QJL) {
        // sign table: nibble -> 4 halves of +-1; entry 8 bytes, 16 lane copies
        for (int e = threadIdx.x; e < 16 * 16; e += NT) {
            const int nib = e >> 4;
            __half2 a = __floats2half2_rn((nib & 1) ? 1.f : -1.f, (nib & 2) ? 1.f : -1.f);
            __half2 c = __floats2half2_rn((nib & 4) ? 1.f : -1.f, (nib & 8) ? 1.f : -1.f);
            reinterpret_cast<uint2*>(signtab)[e] =
                make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&c));
        }
    }
    __syncthreads();
    build_table<KBITS, 2>(tab, 0, cs_k, threadIdx.x, NT);
    build_table<VBITS, VT>(tab, 128, cs_v, threadIdx.x, NT);
    __syncthreads();                                  // the last CTA-wide barrier: the teams part here
    // this lane's private table copies (shared-memory byte addresses)
    const uint32_t kconst = kTabAddr | (KBITS == 4 ? (lane & 15) * 8 : (lane & 7) * 16);
    const uint32_t vconst = kTabAddr | (128 + (lane % (128 / VENT)) * VENT);
    const uint32_t sign_lane = smem_addr(signtab) + (lane & 15) * 8;
    const uint32_t qjl_frag_lane = smem_addr(qjl_frag) + lane * 16;
    const int64_t tiles_total = (p.S + kTileTok - 1) / kTileTok;          // of the plan
    int64_t s_len = p.S;                                                  // tokens actually attended to
    if (p.seq_len_dev != nullptr) s_len = max((int64_t)0, min(*p.seq_len_dev, p.S));
    const int valid_tiles = (int)((s_len + kTileTok - 1) / kTileTok);

    // ---- value side: which bytes of a stored block this lane feeds into the MMAs.  Lane group g owns
    // the dims 4g .. 4g+3 of every 32-dim block: two packed bytes (4-bit) or one (2-bit).  The packed
    // bytes of a block start 2 bytes after the block, so they are 4-byte aligned in every second block
    // ("aligned" class) and 2 bytes off in the others ("shifted" class); in both classes the lane's
    // bytes lie inside ONE aligned 32-bit word, at a per-lane offset and byte position.
    uint32_t voff_al, voff_sh, vselA_al, vselA_sh;
    if (VBITS == 4) {
        voff_al = 2 + 4 * (g >> 1);
        voff_sh = 4 * ((g + 1) >> 1);
        vselA_al = byte_selector(2 * (g & 1));
        vselA_sh = byte_selector((g & 1) ? 0 : 2);
    } else {
        voff_al = 2 + 4 * (g >> 2);
        voff_sh = 4 * ((g + 2) >> 2);
        vselA_al = byte_selector(g & 3);
        vselA_sh = byte_selector((g + 2) & 3);
    }
    const uint32_t pshift = (g & 1) ? 16u : 0u;       // odd MMA columns carry the odd dim of a pair
    uint32_t phase = 0;                               // expected parity of each stage's mbarrier
    bool dead = false;                                // a copy wait gave up: finish without waiting again

    // ---- work distribution.  A "virtual row" is one (batch, kv head, head group); its tiles
    // are numbered 0..tiles_total-1.  Balanced mode (p.splits == 0): the tiles of all virtual
    // rows form one sequence that is cut into p.n_workers equal contiguous ranges, one per team (a
    // "worker"); a team walks the segments (pieces of rows) inside its range.  Split mode: every row
    // is cut into p.splits equal segments that are dealt round-robin to the workers.
    const int64_t n_vrows = (int64_t)p.n_rows * p.HG;
    const int64_t all_tiles = n_vrows * tiles_total;
    const uint32_t worker = blockIdx.x * kTeams + team;
    const int64_t n_cta = p.splits ? (int64_t)gridDim.x * kTeams : (int64_t)p.n_workers;   // workers
    // 64-bit divisions cost a few hundred cycles each and a segment needs half a dozen: when every
    // product below fits 32 bits (all but extreme shapes) the same arithmetic runs on 32-bit values.
    const bool small = all_tiles * (n_cta + 1) < (int64_t)0x7FFFFFFF;
    int64_t cur, cur_end;
    if (p.splits) {
        cur = (int64_t)worker;
        cur_end = n_vrows * p.splits;
    } else if ((int64_t)worker >= n_cta) {
        cur = cur_end = 0;                               // fewer tiles than workers: nothing for this team
    } else if (small) {
        cur = (int64_t)(worker * (uint32_t)all_tiles / (uint32_t)n_cta);
        cur_end = (int64_t)((worker + 1u) * (uint32_t)all_tiles / (uint32_t)n_cta);
    } else {
        cur = (int64_t)worker * all_tiles / n_cta;
        cur_end = ((int64_t)worker + 1) * all_tiles / n_cta;
    }
    // q_rot[row][i] = sum_j q[row][j] * R[i][j] (and the JL projection P q) on tensor cores for the query
    // heads of `n_seg` consecutive virtual rows starting at `vrow0`: MMA row r = head r % HPC of virtual
    // row vrow0 + r / HPC (the float16 query is exact), columns = 8 outputs per warp-step, R split into two
    // float16 terms of 4096*R on the fly.  Matrix rows are read as 32-byte pieces by 4 lanes.
    auto rotate_queries = [&](int64_t vrow0, int n_seg) {
        const __half* qrow[2];
        bool have[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {                                    // this lane's MMA rows g and g + 8
            const int mr = g + 8 * r, sg = mr / HPC, hd = mr % HPC;
            have[r] = mr < kQRows && sg < n_seg;
            qrow[r] = p.q;
            if (have[r]) {
                const uint32_t vr = (uint32_t)vrow0 + (uint32_t)sg;      // rows fit 32 bits
                const int rw = (int)(vr / (uint32_t)p.HG), hgx = (int)(vr % (uint32_t)p.HG);
                const int bb = rw / p.Hkv, hk = rw % p.Hkv;
                have[r] = hd < min(HPC, p.G - hgx * HPC);
                qrow[r] = p.q + ((size_t)bb * p.Hq + hk * p.G + hgx * HPC + hd) * D;
            }
        }
        auto rotate_pass = [&](int nt) {                                 // eight output columns
            const int i = nt * 8 + g;                                    // this lane's output column
            const float* mrow = i < D ? p.rot + (size_t)i * D : p.jl + (size_t)(i - D) * D;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const float2 r0 = __ldg(reinterpret_cast<const float2*>(mrow + ks * 16 + 2 * t));
                const float2 r1 = __ldg(reinterpret_cast<const float2*>(mrow + ks * 16 + 8 + 2 * t));
                const uint32_t a0 = have[0] ? *reinterpret_cast<const uint32_t*>(qrow[0] + ks * 16 + 2 * t) : 0u;
                const uint32_t a2 = have[0] ? *reinterpret_cast<const uint32_t*>(qrow[0] + ks * 16 + 8 + 2 * t) : 0u;
                uint32_t a1 = 0u, a3 = 0u;
                if (kQRows > 8) {
                    a1 = have[1] ? *reinterpret_cast<const uint32_t*>(qrow[1] + ks * 16 + 2 * t) : 0u;
                    a3 = have[1] ? *reinterpret_cast<const uint32_t*>(qrow[1] + ks * 16 + 8 + 2 * t) : 0u;
                }
                const float x0 = r0.x * 4096.f, x1 = r0.y * 4096.f, x2 = r1.x * 4096.f, x3 = r1.y * 4096.f;
                const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
                const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
                mma_16816(c, a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                mma_16816(c, a0, a1, a2, a3, pack_half2(x0 - f01.x, x1 - f01.y), pack_half2(x2 - f23.x, x3 - f23.y));
            }
            // C rows g and g + 8, columns 2t, 2t+1 = outputs nt*8 + 2t, +1
            const int o0 = nt * 8 + 2 * t;
            if (o0 < D) {
                if (g < kQRows) {
                    q_rot_all[g * D + o0] = c[0] * (p.scale_log2 / 4096.f);
                    q_rot_all[g * D + o0 + 1] = c[1] * (p.scale_log2 / 4096.f);
                }
                if (kQRows > 8) {
                    q_rot_all[(g + 8) * D + o0] = c[2] * (p.scale_log2 / 4096.f);
                    q_rot_all[(g + 8) * D + o0 + 1] = c[3] * (p.scale_log2 / 4096.f);
                }
            } else if (g < HPC) {                                        // QJL: one segment per pass
                const float sj = QJL ? p.scale_log2 / (4096.f * (float)p.jl_dim) : 0.f;
                q_jl[g * M + o0 - D] = c[0] * sj;
                q_jl[g * M + o0 - D + 1] = c[1] * sj;
            }
        };
        if (QJL) {
            for (int nt = tw; nt < (D + M) / 8; nt += TW) rotate_pass(nt);
        } else {
            // compile-time bounds: the passes of a warp unroll and their matrix loads are in flight together
            constexpr int kRotPasses = (D / 8 + TW - 1) / TW;
#pragma unroll
            for (int it = 0; it < kRotPasses; ++it)
                if (tw + it * TW < D / 8) rotate_pass(tw + it * TW);
        }
    };
    int seg_no = 0;                                                      // segments this team has started
    while (cur < cur_end) {
    int64_t vrow, tile_begin, tile_end;
    int seg_idx, n_segs;
    if (p.splits) {
        vrow = cur / p.splits;
        seg_idx = (int)(cur % p.splits);
        n_segs = p.splits;
        tile_begin = (int64_t)seg_idx * p.tiles_per_split;
        tile_end = min(tiles_total, tile_begin + p.tiles_per_split);
        cur += n_cta;
    } else if (small) {
        const uint32_t tt = (uint32_t)tiles_total, at = (uint32_t)all_tiles, nc = (uint32_t)n_cta;
        const uint32_t c32 = (uint32_t)cur, vr = c32 / tt;
        const uint32_t row_t0 = vr * tt, row_t1 = row_t0 + tt;
        const uint32_t seg_end = min((uint32_t)cur_end, row_t1);
        vrow = vr;
        tile_begin = c32 - row_t0;
        tile_end = seg_end - row_t0;
        // CTA that owns tile x: largest c with floor(c * all_tiles / n_cta) <= x
        const uint32_t c_first = ((row_t0 + 1u) * nc + at - 1u) / at - 1u;
        const uint32_t c_last = (row_t1 * nc + at - 1u) / at - 1u;
        seg_idx = (int)(worker - c_first);
        n_segs = (int)(c_last - c_first + 1u);
        cur = seg_end;
    } else {
        vrow = cur / tiles_total;
        const int64_t row_t0 = vrow * tiles_total, row_t1 = row_t0 + tiles_total;
        const int64_t seg_end = min(cur_end, row_t1);
        tile_begin = cur - row_t0;
        tile_end = seg_end - row_t0;
        // CTA that owns tile x: largest c with floor(c * all_tiles / n_cta) <= x
        const int64_t c_first = ((row_t0 + 1) * n_cta + all_tiles - 1) / all_tiles - 1;
        const int64_t c_last = (row_t1 * n_cta + all_tiles - 1) / all_tiles - 1;
        seg_idx = (int)((int64_t)worker - c_first);
        n_segs = (int)(c_last - c_first + 1);
        cur = seg_end;
    }
    const int row = (int)((uint32_t)vrow / (uint32_t)p.HG), hg = (int)((uint32_t)vrow % (uint32_t)p.HG);   // rows fit 32 bits
    const int b = row / p.Hkv, hkv = row % p.Hkv;
    const int Gp = min(HPC, p.G - hg * HPC);                             // query heads of this segment
    const int head0 = hkv * p.G + hg * HPC;                              // first query head

    const uint8_t* k_row = p.kb + (size_t)row * p.Scap * C::TBK;
    const uint8_t* v_row = p.vb + (size_t)row * p.Scap * C::TBV;
    const uint8_t* bits_row = QJL ? p.qjl_bits + (size_t)row * p.Scap * (M / 8) : nullptr;
    const uint8_t* norm_row = QJL ? reinterpret_cast<const uint8_t*>(p.qjl_norms + (size_t)row * p.Scap) : nullptr;

    // Full tiles of rows whose byte streams start on a 16-byte boundary arrive by bulk copy (one lane
    // issues, the stage's mbarrier counts the bytes); everything else is copied by the warp itself.
    const bool bulk_row = ((reinterpret_cast<uintptr_t>(k_row) | reinterpret_cast<uintptr_t>(v_row) |
                            (QJL ? reinterpret_cast<uintptr_t>(bits_row) | reinterpret_cast<uintptr_t>(norm_row) : 0)) & 15) == 0;
    // Tile numbers inside a row fit 32 bits (the host rejects longer sequences).
    const int t_first = (int)tile_begin + tw, t_end = min((int)tile_end, valid_tiles);
    const int full_tiles = (int)(s_len / kTileTok);                // tiles below this number hold 16 tokens
    auto issue_tile = [&](int tile, int slot) {
        if (tile >= t_end) return;
        const size_t tok0 = (size_t)tile * kTileTok;
        if (bulk_row && tile < full_tiles) {
            if (lane == 0) {
                const uint32_t sa = stage_addr0 + slot * stage_sz, mb = mbar0 + 8 * slot;
                mbar_expect_tx(mb, (uint32_t)stage_sz);
                bulk_load(sa, k_row + tok0 * C::TBK, C::kStageK, mb);
                bulk_load(sa + C::kStageK, v_row + tok0 * C::TBV, C::kStageV, mb);
                if (QJL) {
                    bulk_load(sa + C::kStageK + C::kStageV, bits_row + tok0 * (M / 8), C::stage_bits(M), mb);
                    bulk_load(sa + C::kStageK + C::kStageV + C::stage_bits(M), norm_row + tok0 * 2, C::kStageN, mb);
                }
            }
        } else {
            const int ntok = tile < full_tiles ? kTileTok : (int)(s_len - (int64_t)tok0);
            uint8_t* st = my_stages + slot * stage_sz;
            copy_words(st, k_row + tok0 * C::TBK, ntok * C::TBK, C::kStageK, lane);
            copy_words(st + C::kStageK, v_row + tok0 * C::TBV, ntok * C::TBV, C::kStageV, lane);
            if (QJL) {
                copy_bytes(st + C::kStageK + C::kStageV, bits_row + tok0 * (M / 8), ntok * (M / 8), C::stage_bits(M), lane);
                copy_bytes(st + C::kStageK + C::kStageV + C::stage_bits(M), norm_row + tok0 * 2, ntok * 2, C::kStageN, lane);
            }
        }
    };
    // first tiles in flight before the prologue math
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue_tile(t_first + s * TW, s);
    // The team's next segment starts at tile 0 of the next virtual row: once this warp has issued its last
    // tile here, it asks L2 for the tiles it will start that segment with, so that they arrive from L2
    // rather than from DRAM when nothing else of the team is in flight.
    // (Not with eight heads per segment: the tile loop has no register to spare there.)
    bool prefetch_pending = NH == 1 && !p.splits && cur < cur_end;
    auto prefetch_next_segment = [&]() {
        prefetch_pending = false;
        if (lane != 0) return;
        const uint32_t nv = (uint32_t)vrow + 1u;
        const size_t nrow = nv / (uint32_t)p.HG;
        const uint8_t* kn = p.kb + nrow * p.Scap * C::TBK;
        const uint8_t* vn = p.vb + nrow * p.Scap * C::TBV;
        if (((reinterpret_cast<uintptr_t>(kn) | reinterpret_cast<uintptr_t>(vn)) & 15) != 0) return;
        const int n_next = (int)min(min(cur_end - cur, tiles_total), (int64_t)full_tiles);
#pragma unroll
        for (int s = 0; s < kStages - 1; ++s) {
            const int tile = tw + s * TW;
            if (tile < n_next) {
                bulk_prefetch_l2(kn + (size_t)tile * kTileTok * C::TBK, C::kStageK);
                bulk_prefetch_l2(vn + (size_t)tile * kTileTok * C::TBV, C::kStageV);
            }
        }
    };

    // ---- query rotation (and JL projection of the query), once per pass of up to kSegBatch segments
    int qslot = 0;                                                       // this segment's slot in q_rot_all
    bool rotate_now = true;
    int n_batch = 1;
    if (kSegBatch > 1 && !p.splits) {
        qslot = seg_no % kSegBatch;
        rotate_now = qslot == 0;
        if (rotate_now) {
            // the team's remaining segments are the consecutive virtual rows up to the one of its last tile
            const int64_t last_vrow = small ? (int64_t)((uint32_t)(cur_end - 1) / (uint32_t)tiles_total)
                                            : (cur_end - 1) / tiles_total;
            n_batch = (int)min((int64_t)kSegBatch, last_vrow - vrow + 1);
        }
    }
    ++seg_no;
    if (rotate_now) {
        rotate_queries(vrow, n_batch);
        team_sync();
    }
    const float* q_rot = q_rot_all + qslot * HPC * D;

    // ---- B fragments of the query.  MMA column n = lane group g.
    //   NH == 1: column g is head g>>1, term hi (g even) or lo (g odd);
    //   NH == 2: column g is head (g>>1) + 4*(g&1); a hi tile and a lo tile.  (Accumulator columns
    //            2t, 2t+1 of a lane are then heads t and t+4.)
    // k-slot mapping inside a 32-dim block, k-step ks: slots (2t,2t+1) <-> dims 8t+4ks+(0,1),
    // slots (2t+8,2t+9) <-> dims 8t+4ks+(2,3): the 8 nibbles of the 32-bit word lane t reads.
    uint32_t qb[NBLK][2][2 * NH];
    {
        const int hq = NH == 1 ? (g >> 1) : (g >> 1) + 4 * (g & 1);
        const bool lo1 = (g & 1) != 0;
#pragma unroll
        for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                const float* src = q_rot + hq * D + blk * 32 + 8 * t + 4 * ks;
                if (NH == 1) {
                    qb[blk][ks][0] = pack_half2(term_of(src[0], lo1), term_of(src[1], lo1));
                    qb[blk][ks][1] = pack_half2(term_of(src[2], lo1), term_of(src[3], lo1));
                } else {
                    qb[blk][ks][0] = pack_half2(src[0], src[1]);
                    qb[blk][ks][1] = pack_half2(src[2], src[3]);
                    qb[blk][ks][2] = pack_half2(term_of(src[0], true), term_of(src[1], true));
                    qb[blk][ks][3] = pack_half2(term_of(src[2], true), term_of(src[3], true));
                }
            }
        if (QJL) {
            // fragments of the projected query, one uint4 per (k-step, lane): {b0, b1 | lo b0, lo b1}
            for (int ks = tw; ks < M / 16; ks += TW) {
                const float* src = q_jl + hq * M + ks * 16 + 4 * t;
                uint4 f;
                if (NH == 1) {
                    f.x = pack_half2(term_of(src[0], lo1), term_of(src[1], lo1));
                    f.y = pack_half2(term_of(src[2], lo1), term_of(src[3], lo1));
                    f.z = 0u; f.w = 0u;
                } else {
                    f.x = pack_half2(src[0], src[1]);
                    f.y = pack_half2(src[2], src[3]);
                    f.z = pack_half2(term_of(src[0], true), term_of(src[1], true));
                    f.w = pack_half2(term_of(src[2], true), term_of(src[3], true));
                }
                reinterpret_cast<uint4*>(qjl_frag)[ks * 32 + lane] = f;
            }
        }
    }
    if (QJL) team_sync();                       // the shared fragments of the projected query are complete

    // ---- running softmax state.  A lane holds the scores of its head(s) (NH == 1: head t;
    // NH == 2: heads t and t+4) for tokens 2g and 2g+1 of the tile.
    float m_run[NH], l_run[NH];
#pragma unroll
    for (int h = 0; h < NH; ++h) { m_run[h] = -INFINITY; l_run[h] = 0.f; }
    // output accumulators (MMA C fragments, kept across tiles).  VACC == 1: acc[blk][0][h][j] is dim
    // 32*blk + 4g + j of head t + 4h.  VACC == 2 (two-term value table, four heads): acc[blk][f][h][0..1]
    // are the hi-term sums of dims 32*blk + 4g + 2f + (0, 1) and [2..3] their lo-term sums: rows g / g+8
    // of an MMA are the hi / lo term of one stored byte, so a table entry is an A register pair as loaded.
    // With eight heads that would be 64 accumulators; there the hi terms of the lane's two bytes share
    // one MMA and their lo terms another (a few register moves instead).
    constexpr int VACC = (VT == 2 && NH == 1) ? 2 : 1;
    float acc[NBLK][VACC][NH][4];
#pragma unroll
    for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
        for (int f = 0; f < VACC; ++f)
#pragma unroll
            for (int h = 0; h < NH; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[blk][f][h][j] = 0.f;

    int slot = 0;
    for (int tile = t_first; tile < t_end; tile += TW) {
        issue_tile(tile + (kStages - 1) * TW, slot >= 1 ? slot - 1 : kStages - 1);
        if (NH == 1 && prefetch_pending && tile + (kStages - 1) * TW >= t_end) prefetch_next_segment();
        const bool full = tile < full_tiles;
        if (bulk_row && full) {
            if (!dead && !mbar_wait(mbar0 + 8 * slot, (phase >> slot) & 1u)) {
                dead = true;
                atomicOr(&g_decode_error, 2u);
            }
            phase ^= 1u << slot;
        }
        __syncwarp();
        const uint32_t ks_base = stage_addr0 + slot * stage_sz;
        const uint32_t vs_base = ks_base + C::kStageK;

        // value radii of the tile -> [token][block] float16, so that a lane later fetches the radii of
        // its four tokens with one or two 16-byte loads
        if (NBLK == 4 || lane < 16) {
            const int tok = NBLK == 4 ? (lane >> 1) : lane;
            const int b0 = NBLK == 4 ? 2 * (lane & 1) : 0;
            const uint32_t a = vs_base + tok * C::TBV + b0 * C::BBV;
            sts_u32(vrad_addr + lane * 4, __byte_perm(lds_u16(a), lds_u16(a + C::BBV), 0x5410));
        }

        // ================= scores.  One MMA covers 8 tokens: row g carries the hi term of token
        // 2g+grp and row g+8 its lo term, so one 64-bit table entry {hi, lo} fills the register
        // pair (a0, a1) or (a2, a3) as loaded.  Columns = query heads.  (Even and odd tokens form the
        // two groups because 8 tokens that are two apart start in 8 different bank quads.)
        float sc[NH][2];                                            // [head][token group]
#pragma unroll
        for (int h = 0; h < NH; ++h) { sc[h][0] = 0.f; sc[h][1] = 0.f; }
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
            const uint32_t tok = ks_base + (2 * g + grp) * C::TBK;
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                if (KBITS == 4) {
                    const uint32_t off = blk * C::BBK + 2 + 4 * t;
                    const bool al4 = ((blk * C::BBK + 2) & 3) == 0; // stage base and token stride are 4-aligned
                    const uint32_t w = al4 ? lds_word<true>(tok + off) : lds_word<false>(tok + off);
                    const uint2 e0 = lds_v2(entry_addr<0>(w, kconst)), e1 = lds_v2(entry_addr<1>(w, kconst));
                    const uint2 e2 = lds_v2(entry_addr<2>(w, kconst)), e3 = lds_v2(entry_addr<3>(w, kconst));
                    mma_16816(c, e0.x, e0.y, e1.x, e1.y, qb[blk][0][0], qb[blk][0][1]);
                    mma_16816(c, e2.x, e2.y, e3.x, e3.y, qb[blk][1][0], qb[blk][1][1]);
                    if (NH == 2) {
                        mma_16816(c, e0.x, e0.y, e1.x, e1.y, qb[blk][0][2], qb[blk][0][3]);
                        mma_16816(c, e2.x, e2.y, e3.x, e3.y, qb[blk][1][2], qb[blk][1][3]);
                    }
                } else {
                    const uint32_t h = lds_u16(tok + blk * C::BBK + 2 + 2 * t);
                    const uint4 e0 = lds_v4(entry_addr<0>(h, kconst)), e1 = lds_v4(entry_addr<1>(h, kconst));
                    mma_16816(c, e0.x, e0.y, e0.z, e0.w, qb[blk][0][0], qb[blk][0][1]);
                    mma_16816(c, e1.x, e1.y, e1.z, e1.w, qb[blk][1][0], qb[blk][1][1]);
                    if (NH == 2) {
                        mma_16816(c, e0.x, e0.y, e0.z, e0.w, qb[blk][0][2], qb[blk][0][3]);
                        mma_16816(c, e1.x, e1.y, e1.z, e1.w, qb[blk][1][2], qb[blk][1][3]);
                    }
                }
                // rows g / g+8 = hi / lo term of the token; columns 2t, 2t+1
                const float d = lds_half_as_float(tok + blk * C::BBK);
                if (NH == 1) {      // columns = hi and lo term of head t
                    sc[0][grp] = fmaf(d, (c[0] + c[1]) + (c[2] + c[3]), sc[0][grp]);
                } else {            // columns = heads t, t+4
                    sc[0][grp] = fmaf(d, c[0] + c[2], sc[0][grp]);
                    sc[NH - 1][grp] = fmaf(d, c[1] + c[3], sc[NH - 1][grp]);
                }
            }
        }
#pragma unroll
        for (int h = 0; h < NH; ++h) { sc[h][0] *= (1.0f / kCbScale); sc[h][1] *= (1.0f / kCbScale); }

        if (QJL) {
            // corr[token][head] = sum_i (+-1) * qp[head][i] (qp already scaled by scale*log2e/M);
            // rows g = token 2g, rows g+8 = token 2g+1
            const uint32_t bs_base = vs_base + C::kStageV;
            const uint32_t ns_base = bs_base + C::stage_bits(M);
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t ta = bs_base + (2 * g) * (M / 8), tb = ta + (M / 8);
            for (int ks = 0; ks < M / 16; ++ks) {
                const uint32_t ha = lds_u16(ta + 2 * ks), hb = lds_u16(tb + 2 * ks);
                const uint2 ea = lds_v2(sign_lane + (((ha >> (4 * t)) & 0xFu) << 7));
                const uint2 eb = lds_v2(sign_lane + (((hb >> (4 * t)) & 0xFu) << 7));
                const uint4 f = lds_v4(qjl_frag_lane + ks * 512);
                mma_16816(c, ea.x, eb.x, ea.y, eb.y, f.x, f.y);
                if (NH == 2) mma_16816(c, ea.x, eb.x, ea.y, eb.y, f.z, f.w);
            }
            // a zero residual norm switches the correction off (qjl.py:49-50)
            const bool on0 = lds_u16(ns_base + 2 * (2 * g)) != 0u;
            const bool on1 = lds_u16(ns_base + 2 * (2 * g + 1)) != 0u;
            if (NH == 1) {
                if (on0) sc[0][0] += c[0] + c[1];
                if (on1) sc[0][1] += c[2] + c[3];
            } else {
                if (on0) { sc[0][0] += c[0]; sc[NH - 1][0] += c[1]; }
                if (on1) { sc[0][1] += c[2]; sc[NH - 1][1] += c[3]; }
            }
        }

        // mask tokens past the end of the sequence (only the ragged last tile of a row has any)
        if (!full) {
            const int ntok = (int)(s_len - (int64_t)tile * kTileTok);
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                if (2 * g >= ntok) sc[h][0] = -INFINITY;
                if (2 * g + 1 >= ntok) sc[h][1] = -INFINITY;
            }
        }

        // ================= online softmax over the 16 tokens of the tile (lanes with equal t)
        float pr[NH][2], alpha[NH];
        bool rescale = false;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            float tmax = fmaxf(sc[h][0], sc[h][1]);
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
            const float m_new = fmaxf(m_run[h], tmax);
            alpha[h] = fast_exp2(m_run[h] - m_new);          // exp2(-inf) = 0 on the first tile
            pr[h][0] = fast_exp2(sc[h][0] - m_new);
            pr[h][1] = fast_exp2(sc[h][1] - m_new);
            l_run[h] = l_run[h] * alpha[h] + pr[h][0] + pr[h][1];
            m_run[h] = m_new;
            rescale |= alpha[h] != 1.0f;
        }
        // the accumulators belong to this lane's own head(s)
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
                for (int f = 0; f < VACC; ++f)
#pragma unroll
                    for (int h = 0; h < NH; ++h)
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[blk][f][h][j] *= alpha[h];
        }

        // ================= values: O[dim][head] += sum_tokens centroid[token][dim] * (p * radius)[token][head]
        // One MMA has a dim PAIR per row, k slots (2t, 2t+1) = the even and the odd dim of the pair for
        // token 4t+2u, slots (2t+8, 2t+9) the same for token 4t+2u+1; a table entry, which holds the two
        // dims of a stored byte side by side, is therefore an A register as loaded.  The B column n = g
        // carries head g>>1 and dim parity g&1: the weight sits in the low half (even dim) or the high
        // half (odd dim) and the other half is zero, which splits the pair into two accumulator columns.
        // Weights: p split into two float16 terms once per tile; times the float16 block radius with an
        // error-free product, again two terms, issued as two MMAs.
        __syncwarp();                                               // the compacted radii are in place
        const uint32_t vb_al = vs_base + (4 * t) * C::TBV + voff_al;
        const uint32_t vb_sh = vs_base + (4 * t) * C::TBV + voff_sh;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            // weights of tokens 4t+2u, 4t+2u+1 for head (g>>1) + 4h, two float16 terms each:
            // p[token 4t+k][head] lives in lane (g' = (4t+k)>>1, t' = g>>1), register pr[h][k&1]
            uint32_t PH[NH][2], PL[NH][2];
#pragma unroll
            for (int h = 0; h < NH; ++h)
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const float x = __shfl_sync(0xffffffffu, pr[h][k], ((2 * t + u) << 2) | (g >> 1));
                    const __half hh = __float2half_rn(x);
                    const __half hl = __float2half_rn(x - __half2float(hh));
                    PH[h][k] = (uint32_t)__half_as_ushort(hh) << pshift;
                    PL[h][k] = (uint32_t)__half_as_ushort(hl) << pshift;
                }
            // radii of the two tokens: NBLK/2 words each, two float16 per word
            uint32_t rw[2][NBLK / 2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint32_t a = vrad_addr + (4 * t + 2 * u + k) * (2 * NBLK);
                if (NBLK == 4) {
                    const uint2 v = lds_v2(a);
                    rw[k][0] = v.x; rw[k][NBLK / 2 - 1] = v.y;
                } else {
                    rw[k][0] = lds_u32(a);
                }
            }
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk) {
                const bool shifted = ((blk * C::BBV + 2) & 3) != 0;
                const uint32_t base = (shifted ? vb_sh : vb_al) + blk * C::BBV;
                const uint32_t selA = shifted ? vselA_sh : vselA_al;
                const uint32_t selB = selA + 0x10u;                  // the next byte of the same word
                const uint32_t w0 = lds_u32(base + (2 * u) * C::TBV), w1 = lds_u32(base + (2 * u + 1) * C::TBV);
                // (d, d) of the two tokens for this block
                const uint32_t d0 = __byte_perm(rw[0][blk >> 1], 0u, (blk & 1) ? 0x3232 : 0x1010);
                const uint32_t d1 = __byte_perm(rw[1][blk >> 1], 0u, (blk & 1) ? 0x3232 : 0x1010);
                uint32_t bh0[NH], bh1[NH], bl0[NH], bl1[NH];
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    weight_terms(PH[h][0], PL[h][0], d0, bh0[h], bl0[h]);
                    weight_terms(PH[h][1], PL[h][1], d1, bh1[h], bl1[h]);
                }
                if (VBITS == 4 && VT == 1) {
                    const uint32_t a0 = lds_u32(entry_addr_sel(w0, vconst, selA)), a1 = lds_u32(entry_addr_sel(w0, vconst, selB));
                    const uint32_t a2 = lds_u32(entry_addr_sel(w1, vconst, selA)), a3 = lds_u32(entry_addr_sel(w1, vconst, selB));
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        mma_16816(acc[blk][0][h], a0, a1, a2, a3, bh0[h], bh1[h]);
                        mma_16816(acc[blk][0][h], a0, a1, a2, a3, bl0[h], bl1[h]);
                    }
                } else if (VBITS == 4) {
                    const uint2 e0 = lds_v2(entry_addr_sel(w0, vconst, selA)), e1 = lds_v2(entry_addr_sel(w1, vconst, selA));
                    const uint2 f0 = lds_v2(entry_addr_sel(w0, vconst, selB)), f1 = lds_v2(entry_addr_sel(w1, vconst, selB));
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        if constexpr (VACC == 2) {
                            // {hi, lo} entries fill the register pairs (a0, a1) / (a2, a3) as loaded
                            mma_16816(acc[blk][0][h], e0.x, e0.y, e1.x, e1.y, bh0[h], bh1[h]);
                            mma_16816(acc[blk][0][h], e0.x, e0.y, e1.x, e1.y, bl0[h], bl1[h]);
                            mma_16816(acc[blk][VACC - 1][h], f0.x, f0.y, f1.x, f1.y, bh0[h], bh1[h]);
                            mma_16816(acc[blk][VACC - 1][h], f0.x, f0.y, f1.x, f1.y, bl0[h], bl1[h]);
                        } else {
                            // hi terms of the two bytes in rows g / g+8, then their lo terms; lo x lo is dropped
                            mma_16816(acc[blk][0][h], e0.x, f0.x, e1.x, f1.x, bh0[h], bh1[h]);
                            mma_16816(acc[blk][0][h], e0.x, f0.x, e1.x, f1.x, bl0[h], bl1[h]);
                            mma_16816(acc[blk][0][h], e0.y, f0.y, e1.y, f1.y, bh0[h], bh1[h]);
                        }
                    }
                } else if (VT == 1) {
                    const uint2 e0 = lds_v2(entry_addr_sel(w0, vconst, selA)), e1 = lds_v2(entry_addr_sel(w1, vconst, selA));
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        mma_16816(acc[blk][0][h], e0.x, e0.y, e1.x, e1.y, bh0[h], bh1[h]);
                        mma_16816(acc[blk][0][h], e0.x, e0.y, e1.x, e1.y, bl0[h], bl1[h]);
                    }
                } else {
                    // 2-bit {hi A, lo A, hi B, lo B}: A = dims 4g, 4g+1, B = dims 4g+2, 4g+3
                    const uint4 e0 = lds_v4(entry_addr_sel(w0, vconst, selA)), e1 = lds_v4(entry_addr_sel(w1, vconst, selA));
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        if constexpr (VACC == 2) {
                            mma_16816(acc[blk][0][h], e0.x, e0.y, e1.x, e1.y, bh0[h], bh1[h]);
                            mma_16816(acc[blk][0][h], e0.x, e0.y, e1.x, e1.y, bl0[h], bl1[h]);
                            mma_16816(acc[blk][VACC - 1][h], e0.z, e0.w, e1.z, e1.w, bh0[h], bh1[h]);
                            mma_16816(acc[blk][VACC - 1][h], e0.z, e0.w, e1.z, e1.w, bl0[h], bl1[h]);
                        } else {
                            mma_16816(acc[blk][0][h], e0.x, e0.z, e1.x, e1.z, bh0[h], bh1[h]);
                            mma_16816(acc[blk][0][h], e0.x, e0.z, e1.x, e1.z, bl0[h], bl1[h]);
                            mma_16816(acc[blk][0][h], e0.y, e0.w, e1.y, e1.w, bh0[h], bh1[h]);
                        }
                    }
                }
            }
        }
        __syncwarp();
        slot = slot + 1 == kStages ? 0 : slot + 1;
    }

    if (NH == 1 && prefetch_pending) prefetch_next_segment();            // a warp without tiles in this segment
    // ---- reduce the row sums over the 8 lanes that share a head
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
    }
    __syncwarp();

    // per-warp record over the warp's own (now idle) stages: [head][0] = m, [1] = l, [2 + dim] = o
    {
        float* rec = rec_of(warp);
        if (g == 0) {
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                rec[(t + 4 * h) * (D + 2) + 0] = m_run[h];
                rec[(t + 4 * h) * (D + 2) + 1] = l_run[h];
            }
        }
#pragma unroll
        for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
            for (int h = 0; h < NH; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int dim = blk * 32 + 4 * g + j;
                    float v;
                    if constexpr (VACC == 1) v = acc[blk][0][h][j];
                    else v = acc[blk][j >> 1][h][j & 1] + acc[blk][j >> 1][h][2 + (j & 1)];
                    rec[(t + 4 * h) * (D + 2) + 2 + dim] = v * p.v_inv;
                }
    }
    team_sync();

    // ---- item record = merge of the warp records
    const size_t group = (size_t)vrow;
    float* cta_rec = p.records + (group * p.max_segs + seg_idx) * kRecHeads * (D + 2);
    for (int e = tid; e < HPC * (D + 2); e += TT) {
        const int head = e / (D + 2), col = e % (D + 2);
        float mx = -INFINITY;
        for (int w = team * TW; w < (team + 1) * TW; ++w) mx = fmaxf(mx, rec_of(w)[head * (D + 2)]);
        float val;
        if (col == 0) {
            val = mx;
        } else {
            val = 0.f;
            for (int w = team * TW; w < (team + 1) * TW; ++w) {
                const float* r = rec_of(w) + head * (D + 2);
                const float mw = r[0];
                const float s = (mw == -INFINITY) ? 0.f : fast_exp2(mw - mx);
                val = fmaf(s, r[col], val);
            }
        }
        __stcg(cta_rec + e, val);
    }
    // A row that lies inside this CTA has one record, written and read by this CTA alone: the barrier
    // orders it; no fence, no ticket.
    if (n_segs > 1) __threadfence();
    team_sync();
    if (n_segs > 1) {
        if (tid == 0) s_ticket = atomicAdd(p.tickets + group, 1u);
        team_sync();
    }
    if (n_segs == 1 || s_ticket == (unsigned)(n_segs - 1)) {
        // ---- last segment of this virtual row to finish: merge the segment records
        if (n_segs > 1) __threadfence();
        const float* recs = p.records + group * p.max_segs * kRecHeads * (D + 2);
        // A thread merges its E = HPC * D / TT (head, dim) elements together, four records per round trip to
        // L2: all loads of a round are independent, so a row cut into n segments costs ceil(n / 4) round trips
        // (a long single sequence is cut into a few dozen).
        constexpr int E = (HPC * D + TT - 1) / TT;
        float mx[E], ml[E], mo[E];
#pragma unroll
        for (int j = 0; j < E; ++j) { mx[j] = -INFINITY; ml[j] = 0.f; mo[j] = 0.f; }
        for (int s0 = 0; s0 < n_segs; s0 += 4) {
            float ms[E][4], ls[E][4], os[E][4];
#pragma unroll
            for (int j = 0; j < E; ++j) {
                const int e = min(tid + j * TT, HPC * D - 1);
                const int head = e / D, dim = e % D;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float* r = recs + (min(s0 + u, n_segs - 1) * kRecHeads + head) * (D + 2);
                    ms[j][u] = __ldcg(r);
                    ls[j][u] = __ldcg(r + 1);
                    os[j][u] = __ldcg(r + 2 + dim);
                }
            }
#pragma unroll
            for (int j = 0; j < E; ++j) {
                float m_new = mx[j];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (s0 + u >= n_segs) ms[j][u] = -INFINITY;
                    m_new = fmaxf(m_new, ms[j][u]);
                }
                const float c = (mx[j] == -INFINITY) ? 0.f : fast_exp2(mx[j] - m_new);
                ml[j] *= c;
                mo[j] *= c;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float sc = (ms[j][u] == -INFINITY) ? 0.f : fast_exp2(ms[j][u] - m_new);
                    ml[j] = fmaf(sc, ls[j][u], ml[j]);
                    mo[j] = fmaf(sc, os[j][u], mo[j]);
                }
                mx[j] = m_new;
            }
        }
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const int e = tid + j * TT;
            if (e >= HPC * D) break;
            const int head = e / D, dim = e % D;
            if (p.partial_out) {
                if (head < Gp) {
                    float* dst = p.partial_out + ((size_t)b * p.Hq + head0 + head) * (D + 2);
                    dst[2 + dim] = mo[j];
                    if (dim == 0) { dst[0] = ml[j] > 0.f ? mx[j] : 0.f; dst[1] = ml[j]; }   // empty: m = 0, l = 0 as the host path writes
                }
            } else {
                o_fin[e] = ml[j] > 0.f ? mo[j] / ml[j] : 0.f;
            }
        }
        if (tid == 0) p.tickets[group] = 0;   // ready for the next call on this stream
        if (!p.partial_out) {
            team_sync();
            // out[head][i] = sum_j o_fin[head][j] * R[j][i] on the tensor cores, eight output columns per
            // warp step: rows g = hi term of head g, rows g+8 = its lo term (two float16 terms of the
            // float32 result), B = R split into two float16 terms of 4096*R on the fly; the three product
            // terms hi*hi + lo*hi + hi*lo land in rows g and g+8 of the same lane.  (|o| <= 0.46 * 65504:
            // the hi term cannot overflow.)
            constexpr int kInvPasses = (D / 8 + TW - 1) / TW;
#pragma unroll
            for (int it = 0; it < kInvPasses; ++it) {
                const int nt = tw + it * TW;
                if (nt >= D / 8) break;
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                const int n = nt * 8 + g;                               // B column of this lane
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const int k0 = ks * 16 + 2 * t;
                    const float x0 = __ldg(p.rot + (size_t)k0 * D + n) * 4096.f, x1 = __ldg(p.rot + (size_t)(k0 + 1) * D + n) * 4096.f;
                    const float x2 = __ldg(p.rot + (size_t)(k0 + 8) * D + n) * 4096.f, x3 = __ldg(p.rot + (size_t)(k0 + 9) * D + n) * 4096.f;
                    const __half2 h01 = __floats2half2_rn(x0, x1), h23 = __floats2half2_rn(x2, x3);
                    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
                    // A: row g = head g (hi), row g+8 = head g (lo); k slots 2t, 2t+1 | 2t+8, 2t+9
                    uint32_t a0 = 0u, a1 = 0u, a2 = 0u, a3 = 0u;
                    if (g < HPC) {
                        const float* src = o_fin + g * D + k0;
                        const __half2 p01 = __floats2half2_rn(src[0], src[1]), p23 = __floats2half2_rn(src[8], src[9]);
                        const float2 q01 = __half22float2(p01), q23 = __half22float2(p23);
                        a0 = *reinterpret_cast<const uint32_t*>(&p01);
                        a2 = *reinterpret_cast<const uint32_t*>(&p23);
                        a1 = pack_half2(src[0] - q01.x, src[1] - q01.y);
                        a3 = pack_half2(src[8] - q23.x, src[9] - q23.y);
                    }
                    mma_16816(c, a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                    mma_16816(c, a0, 0u, a2, 0u, pack_half2(x0 - f01.x, x1 - f01.y), pack_half2(x2 - f23.x, x3 - f23.y));
                }
                // C rows g (hi rows) and g+8 (lo rows) of head g; columns 2t, 2t+1 = outputs nt*8 + 2t, +1
                if (g < Gp) {
                    const float r0 = (c[0] + c[2]) * (1.0f / 4096.f), r1 = (c[1] + c[3]) * (1.0f / 4096.f);
                    const size_t off = ((size_t)b * p.Hq + head0 + g) * D + nt * 8 + 2 * t;
                    if (p.out_is_fp16) {
                        static_cast<__half*>(p.out)[off] = __float2half_rn(fminf(fmaxf(r0, -65504.f), 65504.f));
                        static_cast<__half*>(p.out)[off + 1] = __float2half_rn(fminf(fmaxf(r1, -65504.f), 65504.f));
                    } else {
                        static_cast<float*>(p.out)[off] = r0;
                        static_cast<float*>(p.out)[off + 1] = r1;
                    }
                }
            }
        }
    }
    // the next segment reuses the rings (bulk copies land where this segment wrote records and
    // slow-path tiles with ordinary stores) and the query buffers
    fence_async_smem();
    team_sync();
    }   // segments
}

// ------------------------------------------------------------------ host side
static int device_sms() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}

// query heads per CTA: 4 (one MMA n-tile holds 4 heads x {hi, lo}) or 8 (a hi and a lo tile)
static int heads_per_cta(int G) { return G <= 4 ? 4 : 8; }

static int head_groups(int G) { const int h = heads_per_cta(G); return (G + h - 1) / h; }

constexpr int kMaxTeams = PQ_DEC_TEAMS > 2 ? PQ_DEC_TEAMS : 2;

// Balanced mode: number of persistent CTAs and the largest number of segments a row can have.
// A row of T tiles inside a sequence cut into n equal ranges of floor/ceil(all/n) tiles touches at
// most ceil(n / n_vrows) + 1 ranges and never more than T; the bound does not shrink when T grows,
// so scratch sized for a cache's capacity serves every shorter sequence length.
static void balanced_plan(int64_t n_vrows, int64_t tiles_per_row, int sms, int* n_cta, int* max_segs) {
    if (sms <= 0) sms = 148;
    if (n_vrows < 1) n_vrows = 1;
    const int64_t all_tiles = n_vrows * tiles_per_row;
    int64_t n = all_tiles < sms ? all_tiles : sms;
    if (n < 1) n = 1;
    *n_cta = (int)n;
    // ranges are per team of warps, at most kMaxTeams per CTA (the bound also serves kernels with one)
    const int64_t workers = (int64_t)sms * kMaxTeams;
    const int64_t by_cta = (workers + n_vrows - 1) / n_vrows + 1;
    int64_t segs = tiles_per_row < by_cta ? tiles_per_row : by_cta;
    if (segs < 1) segs = 1;
    *max_segs = (int)segs;
}

// Split count offered to callers that want the static scheme: enough segments to fill the
// SMs in whole waves, at least two tiles per warp, at most 64.
static int choose_splits(int batch, int q_heads, int kv_heads, int64_t seq_len, int sms) {
    if (sms <= 0) sms = 148;
    const int G = q_heads / kv_heads;
    const int64_t groups = (int64_t)batch * kv_heads * head_groups(G);
    const int64_t tiles = (seq_len + kTileTok - 1) / kTileTok;
    int64_t max_s = tiles / 32;
    if (max_s > 64) max_s = 64;
    if (max_s < 1) max_s = 1;
    int best = 1;
    double best_eff = -1.0;
    for (int s = 1; s <= max_s; ++s) {
        const double waves = (double)(groups * s) / sms;
        const double full = waves < 1.0 ? 1.0 : (double)(int64_t)(waves + 0.999999);
        const double eff = waves / full;
        if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
    }
    return best;
}

// Scale for the single-term value table: the power-of-two-free factor a in [1, 2) for which
// 64 * a * c[i] is closest to a float16 number for every centroid at once (largest rounding error
// relative to the largest centroid; about 3e-5 for the 16-centroid block codebook against 2.4e-4 for
// an arbitrary scale).  The search runs once per codebook; the last result is cached.
static float value_table_scale(const float* cb, int n) {
    if (kVTerms != 1) return kCbScale;
    static std::mutex mu;
    static float cached_cb[16];
    static int cached_n = 0;
    static float cached_scale = 0.f;
    std::lock_guard<std::mutex> lock(mu);
    if (cached_n == n && std::memcmp(cached_cb, cb, n * sizeof(float)) == 0) return cached_scale;
    float cmax = 0.f;
    for (int i = 0; i < n; ++i) cmax = std::fmax(cmax, std::fabs(cb[i]));
    float best_a = 1.f;
    double best_err = 1e30;
    constexpr int kSteps = 1 << 14;
    for (int s = 0; s < kSteps && cmax > 0.f; ++s) {
        const float a = 1.f + (float)s / kSteps;
        double worst = 0.0;
        for (int i = 0; i < n; ++i) {
            const float x = kCbScale * a * cb[i];
            const double e = std::fabs((double)__half2float(__float2half_rn(x)) - (double)x);
            if (e > worst) worst = e;
        }
        worst /= (double)(kCbScale * a * cmax);
        if (worst < best_err) { best_err = worst; best_a = a; }
    }
    std::memcpy(cached_cb, cb, n * sizeof(float));
    cached_n = n;
    cached_scale = kCbScale * best_a;
    return cached_scale;
}

// Read and clear this file's device error flags (for pq_poll_device_errors).
int decode_error_flags(unsigned int* flags) {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_decode_error, sizeof(v)) != cudaSuccess) return PQ_ERR_CUDA;
    if (v && cudaMemcpyToSymbol(g_decode_error, &zero, sizeof(zero)) != cudaSuccess) return PQ_ERR_CUDA;
    *flags = v;
    return PQ_OK;
}

template <int D, int KBITS, int VBITS, int NH, bool QJL>
static int launch_decode(const DecodeParams& p, int rows, cudaStream_t st) {
    using C = DecodeCfg<D, KBITS, VBITS, NH, QJL>;
    const size_t smem = C::smem_bytes(p.jl_dim);
    auto kern = pq_decode_attn_kernel<D, KBITS, VBITS, NH, QJL>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return PQ_ERR_CUDA;
    int sms = device_sms();
    if (sms <= 0) sms = 148;
    static_assert(C::kTeams <= kMaxTeams, "balanced_plan bounds the segments of a row with kMaxTeams");
    DecodeParams pp = p;
    int64_t workers;                                             // teams that get work
    if (p.splits) {
        workers = (int64_t)p.splits * rows * p.HG;               // items, dealt round-robin
    } else {
        workers = (int64_t)rows * p.HG * ((p.S + kTileTok - 1) / kTileTok);
    }
    if (workers > (int64_t)sms * C::kTeams) workers = (int64_t)sms * C::kTeams;
    if (workers < 1) workers = 1;
    pp.n_workers = (int)workers;
    const int grid = (int)((workers + C::kTeams - 1) / C::kTeams);   // persistent: at most one CTA per SM
    kern<<<grid, C::NTHREADS, smem, st>>>(pp);
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
    const int G = q_heads / kv_heads;
    const size_t groups = (size_t)batch * kv_heads * pq::head_groups(G);
    int segs = n_splits;
    if (n_splits <= 0) {
        int n_cta = 0;
        pq::balanced_plan((int64_t)groups, (seq_len + pq::kTileTok - 1) / pq::kTileTok, pq::device_sms(), &n_cta, &segs);
    }
    const size_t tickets = (groups * sizeof(unsigned int) + 255) & ~size_t(255);
    return tickets + groups * segs * pq::kRecHeads * (head_dim + 2) * sizeof(float);
}

// Argument checks shared by pq_decode_attn and pq_decode_attn_static.  Returns PQ_OK when a launch (or
// the empty-input shortcut) may proceed; *n_splits_io is clamped to [0, tiles].
static int check_decode_args(const void* q, const void* k_blocks, const void* v_blocks, int batch, int q_heads,
                             int kv_heads, int64_t seq_len, int64_t seq_capacity, int head_dim, int k_bits,
                             int v_bits, const float* codebook_k, const float* codebook_v, const float* rot,
                             const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                             const void* out, const void* partial_out, int* n_splits_io) {
    if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || seq_len < 0 || seq_capacity < seq_len)
        return PQ_ERR_BAD_SHAPE;
    if (head_dim != 64 && head_dim != 128) return PQ_ERR_BAD_HEAD_DIM;
    if ((k_bits != 2 && k_bits != 4) || (v_bits != 2 && v_bits != 4)) return PQ_ERR_BAD_BITS;
    const int64_t tiles = (seq_len + pq::kTileTok - 1) / pq::kTileTok;
    if (tiles > 0x7FFFFFF0) return PQ_ERR_TOO_LARGE;
    if (*n_splits_io < 0) *n_splits_io = 0;
    if (*n_splits_io > tiles) *n_splits_io = (int)tiles;
    if (batch == 0) return PQ_OK;
    if (!q || !rot || !codebook_k || !codebook_v || (!out && !partial_out)) return PQ_ERR_NULL_POINTER;
    if (jl_matrix != nullptr) {
        if (jl_dim < 16 || jl_dim > 128 || (jl_dim % 16)) return PQ_ERR_BAD_JL_DIM;
        if (!qjl_bits || !qjl_norms) return PQ_ERR_NULL_POINTER;
        // (rows of the side band that do not start on a 16-byte boundary - any capacity that is not a
        // multiple of 8 has some - are staged by the warps' own byte loads instead of bulk copies)
        if ((reinterpret_cast<uintptr_t>(qjl_bits) & 15) || (reinterpret_cast<uintptr_t>(qjl_norms) & 15))
            return PQ_ERR_MISALIGNED;
    }
    if (seq_len == 0) return PQ_OK;
    if (!k_blocks || !v_blocks) return PQ_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(k_blocks) & 15) || (reinterpret_cast<uintptr_t>(v_blocks) & 15) ||
        (reinterpret_cast<uintptr_t>(rot) & 15))
        return PQ_ERR_MISALIGNED;
    return PQ_OK;
}

// Shared body of pq_decode_attn (length on the host) and pq_decode_attn_dynamic (seq_len is the
// upper bound the plan and the scratch are made for; the kernel reads the length from device memory).
static int decode_attn_impl(const void* q, const void* k_blocks, const void* v_blocks,
                            int batch, int q_heads, int kv_heads, int64_t seq_len, const int64_t* seq_len_dev,
                            int64_t seq_capacity, int head_dim, int k_bits, int v_bits,
                            const float* codebook_k, const float* codebook_v, const float* rot, float scale,
                            const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                            void* out, int out_is_fp16, void* partial_out,
                            int n_splits, void* scratch, size_t scratch_bytes, void* stream) {
    using namespace pq;
    if (seq_len_dev != nullptr && (reinterpret_cast<uintptr_t>(seq_len_dev) & 7)) return PQ_ERR_MISALIGNED;
    const int chk = check_decode_args(q, k_blocks, v_blocks, batch, q_heads, kv_heads, seq_len, seq_capacity, head_dim,
                                      k_bits, v_bits, codebook_k, codebook_v, rot, jl_matrix, jl_dim, qjl_bits,
                                      qjl_norms, out, partial_out, &n_splits);
    if (chk != PQ_OK) return chk;
    if (batch == 0) return PQ_OK;
    if (!scratch) return PQ_ERR_NULL_POINTER;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool qjl = jl_matrix != nullptr;
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
    if (reinterpret_cast<uintptr_t>(scratch) & 255) return PQ_ERR_MISALIGNED;
    const int64_t tiles = (seq_len + kTileTok - 1) / kTileTok;
    if (scratch_bytes < pq_decode_attn_scratch_bytes(batch, q_heads, kv_heads, seq_len, head_dim, n_splits))
        return PQ_ERR_SCRATCH_TOO_SMALL;
    const int rows = batch * kv_heads;

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
    p.seq_len_dev = seq_len_dev;
    p.Scap = seq_capacity;
    p.Hq = q_heads;
    p.Hkv = kv_heads;
    p.n_rows = rows;
    p.G = q_heads / kv_heads;
    p.HG = head_groups(p.G);
    p.splits = n_splits;
    p.tiles_per_split = n_splits ? (int)((tiles + n_splits - 1) / n_splits) : 0;
    if (n_splits) {
        p.max_segs = n_splits;
    } else {
        int n_cta = 0;
        balanced_plan((int64_t)rows * p.HG, tiles, device_sms(), &n_cta, &p.max_segs);
    }
    p.jl_dim = qjl ? jl_dim : 0;
    p.out_is_fp16 = out_is_fp16;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.v_scale = value_table_scale(codebook_v, 1 << v_bits);
    p.v_inv = 1.0f / p.v_scale;
    for (int i = 0; i < 16; ++i) {
        p.cbk[i] = i < (1 << k_bits) ? codebook_k[i] : 0.f;
        p.cbv[i] = i < (1 << v_bits) ? codebook_v[i] : 0.f;
    }
    const size_t groups = (size_t)rows * p.HG;
    p.tickets = static_cast<unsigned int*>(scratch);
    p.records = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + ((groups * sizeof(unsigned int) + 255) & ~size_t(255)));

    const bool wide = heads_per_cta(p.G) == 8;
#define PQ_DEC(DD, KB, VB)                                                                            \
    if (head_dim == DD && k_bits == KB && v_bits == VB) {                                             \
        if (wide) return qjl ? launch_decode<DD, KB, VB, 2, true>(p, rows, st)                        \
                             : launch_decode<DD, KB, VB, 2, false>(p, rows, st);                      \
        return qjl ? launch_decode<DD, KB, VB, 1, true>(p, rows, st)                                  \
                   : launch_decode<DD, KB, VB, 1, false>(p, rows, st);                                \
    }
    PQ_DEC(64, 4, 4) PQ_DEC(64, 4, 2) PQ_DEC(64, 2, 4) PQ_DEC(64, 2, 2)
    PQ_DEC(128, 4, 4) PQ_DEC(128, 4, 2) PQ_DEC(128, 2, 4) PQ_DEC(128, 2, 2)
#undef PQ_DEC
    return PQ_ERR_BAD_HEAD_DIM;
}

extern "C" int pq_decode_attn(const void* q, const void* k_blocks, const void* v_blocks,
                              int batch, int q_heads, int kv_heads, int64_t seq_len, int64_t seq_capacity,
                              int head_dim, int k_bits, int v_bits,
                              const float* codebook_k, const float* codebook_v, const float* rot, float scale,
                              const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                              void* out, int out_is_fp16, void* partial_out,
                              int n_splits, void* scratch, size_t scratch_bytes, void* stream) {
    return decode_attn_impl(q, k_blocks, v_blocks, batch, q_heads, kv_heads, seq_len, nullptr, seq_capacity, head_dim,
                            k_bits, v_bits, codebook_k, codebook_v, rot, scale, jl_matrix, jl_dim, qjl_bits, qjl_norms,
                            out, out_is_fp16, partial_out, n_splits, scratch, scratch_bytes, stream);
}

extern "C" int pq_decode_attn_dynamic(const void* q, const void* k_blocks, const void* v_blocks,
                                      int batch, int q_heads, int kv_heads, int64_t max_seq_len,
                                      const int64_t* seq_len_dev, int64_t seq_capacity,
                                      int head_dim, int k_bits, int v_bits,
                                      const float* codebook_k, const float* codebook_v, const float* rot, float scale,
                                      const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                                      void* out, int out_is_fp16, void* partial_out,
                                      int n_splits, void* scratch, size_t scratch_bytes, void* stream) {
    if (seq_len_dev == nullptr) return PQ_ERR_NULL_POINTER;
    if (max_seq_len <= 0) return PQ_ERR_BAD_SHAPE;       // the plan needs at least one tile
    return decode_attn_impl(q, k_blocks, v_blocks, batch, q_heads, kv_heads, max_seq_len, seq_len_dev, seq_capacity,
                            head_dim, k_bits, v_bits, codebook_k, codebook_v, rot, scale, jl_matrix, jl_dim, qjl_bits,
                            qjl_norms, out, out_is_fp16, partial_out, n_splits, scratch, scratch_bytes, stream);
}

// ------------------------------------------------------------------ no-allocation variant
// pq_decode_attn_static: the same decode attention, for hosts that are not allowed to
// allocate device memory around the call.  Examples: an operator callback of an inference
// runtime that owns every device buffer and hands the operator only its input and output
// tensors; code running while a memory pool is frozen; latency-critical serving loops where
// a cudaMalloc would stall every stream of the device.  Such callers have nowhere to get
// the split-merge scratch from, so this entry point keeps it inside the library: a
// file-scope device array of kStaticScratchBytes that every GPU which loads the library
// carries until the process exits.
//
// The array's name is only a host-side handle; its device address is fetched once per
// device with cudaGetSymbolAddress (with that device current) and that pointer is what the
// kernel receives.
namespace pq {

constexpr size_t kStaticScratchBytes = size_t(8) << 20;   // 8 MiB per GPU
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
// Published once per device; racing first calls from several host threads all store the same
// address, and the release/acquire pair orders the store against later readers.
static std::atomic<void*> g_static_scratch_ptr[kMaxDevices];

// Device address of the static scratch on the current device, or nullptr on failure.
static void* static_scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    void* ptr = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return nullptr;
        g_static_scratch_ptr[dev].store(ptr, std::memory_order_release);
    }
    return ptr;
}

}  // namespace pq

extern "C" size_t pq_decode_attn_static_scratch_capacity(void) { return pq::kStaticScratchBytes; }

extern "C" int pq_decode_attn_static(const void* q, const void* k_blocks, const void* v_blocks,
                                     int batch, int q_heads, int kv_heads, int64_t seq_len, int64_t seq_capacity,
                                     int head_dim, int k_bits, int v_bits,
                                     const float* codebook_k, const float* codebook_v, const float* rot, float scale,
                                     const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                                     void* out, int out_is_fp16, void* partial_out,
                                     int n_splits, void* stream) {
    using namespace pq;
    // Every argument is checked before anything touches the shared array, so a rejected call cannot
    // disturb another call that is still using it.  The split count is fixed here as well, so the
    // size check below and the launch agree.
    const int chk = check_decode_args(q, k_blocks, v_blocks, batch, q_heads, kv_heads, seq_len, seq_capacity, head_dim,
                                      k_bits, v_bits, codebook_k, codebook_v, rot, jl_matrix, jl_dim, qjl_bits,
                                      qjl_norms, out, partial_out, &n_splits);
    if (chk != PQ_OK) return chk;
    if (batch == 0) return PQ_OK;
    const size_t need = pq_decode_attn_scratch_bytes(batch, q_heads, kv_heads, seq_len, head_dim, n_splits);
    if (need > kStaticScratchBytes) return PQ_ERR_STATIC_SCRATCH_EXCEEDED;
    void* scratch = static_scratch_for_current_device();
    if (!scratch) return PQ_ERR_CUDA;
    // The array is shared by all calls and keeps whatever the previous call left.  The
    // only part that must read zero at launch is the ticket counters: clear them on the
    // caller's stream (an aborted earlier launch could have left a count behind).
    const size_t groups = (size_t)batch * kv_heads * head_groups(q_heads / kv_heads);
    const size_t ticket_bytes = (groups * sizeof(unsigned int) + 255) & ~size_t(255);
    if (seq_len > 0 &&
        cudaMemsetAsync(scratch, 0, ticket_bytes, static_cast<cudaStream_t>(stream)) != cudaSuccess)
        return PQ_ERR_CUDA;
    return pq_decode_attn(q, k_blocks, v_blocks, batch, q_heads, kv_heads, seq_len, seq_capacity, head_dim,
                          k_bits, v_bits, codebook_k, codebook_v, rot, scale, jl_matrix, jl_dim, qjl_bits,
                          qjl_norms, out, out_is_fp16, partial_out, n_splits, scratch, kStaticScratchBytes, stream);
}
