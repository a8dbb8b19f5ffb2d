// The llama.cpp bridge's entry points (integration/polarquant-kv.patch of the reference,
// decoded lines 695-763) for sm_100a: the per-vector-radius codec with nibble-packed
// indices, as kernels laid out for a 148-SM part instead of one CTA per vector / per head.
//
//   compress   one warp owns four vectors at a time; Rᵀ sits in shared memory once per CTA
//              (head dims 64 and 128), every R word read feeds four FMAs; the sum of squares
//              is combined in the order of the reference's shared-memory tree (element t with
//              t + 64, then + 32, ... , + 1), so the radius sees the same additions.
//   attention  CTAs own (kv head, query group, slice of S); a warp takes 32 tokens at a time,
//              each lane holds D/32 (rounded up) dims, the 32 partial dot products are
//              transposed and summed with 31 shuffles so that lane t ends with token t's
//              score; online softmax; the slices are merged by the last CTA to finish.
//   rotate / inverse rotate: one CTA per row (a few dozen rows per call).
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "polarquant_llama_abi.h"

namespace {

thread_local int t_last_error = 0;

enum { kErrNull = 1, kErrDim = 2, kErrLevels = 3, kErrHeads = 4, kErrCuda = 5 };

constexpr int kMaxDim = 1024;
constexpr unsigned kFull = 0xffffffffu;

bool fail(int code, const char* what) {
    t_last_error = code;
    fprintf(stderr, "PolarQuant: %s\n", what);
    return false;
}

bool dim_ok(int D) { return D > 0 && D <= kMaxDim && (D & 1) == 0; }

bool launched() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        t_last_error = kErrCuda;
        fprintf(stderr, "PolarQuant: %s\n", cudaGetErrorString(e));
        return false;
    }
    return true;
}

// ---------------------------------------------------------------------------------------------
// rows · Rᵀ and rows · R
// ---------------------------------------------------------------------------------------------

// out[n][j] = sum_k in[n][k] * R[j][k]: a warp per output element, lanes along k (coalesced).
__global__ void __launch_bounds__(256) rotate_rows_kernel(const float* __restrict__ in, const float* __restrict__ R,
                                                          float* __restrict__ out, int D) {
    __shared__ float xs[kMaxDim];
    const int n = blockIdx.x;
    for (int k = threadIdx.x; k < D; k += blockDim.x) xs[k] = in[(size_t)n * D + k];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int j = warp; j < D; j += blockDim.x >> 5) {
        const float* row = R + (size_t)j * D;
        float s = 0.0f;
        for (int k = lane; k < D; k += 32) s = fmaf(xs[k], row[k], s);
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
        if (lane == 0) out[(size_t)n * D + j] = s;
    }
}

// out[n][j] = sum_k in[n][k] * R[k][j]: a thread per output element, k ascending.
__global__ void __launch_bounds__(256) inverse_rotate_rows_kernel(const float* __restrict__ in,
                                                                  const float* __restrict__ R,
                                                                  float* __restrict__ out, int D) {
    __shared__ float xs[kMaxDim];
    const int n = blockIdx.x;
    for (int k = threadIdx.x; k < D; k += blockDim.x) xs[k] = in[(size_t)n * D + k];
    __syncthreads();
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        float s = 0.0f;
        for (int k = 0; k < D; ++k) s = fmaf(xs[k], R[(size_t)k * D + j], s);
        out[(size_t)n * D + j] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// compress
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ int nearest_level(float v, const float* cb, int n_levels) {
    int best = 0;
    float dist = 1e30f;
    for (int i = 0; i < n_levels; ++i) {
        const float d = fabsf(v - cb[i]);
        if (d < dist) { dist = d; best = i; }
    }
    return best;
}

constexpr int kCmpWarps = 8;
constexpr int kCmpVecs = 4;      // vectors a warp carries through the rotation together
constexpr int kCmpSmallN = 4096;

// Head dims 64 and 128.  Lane l owns rotated elements l + 32 i.
template <int D>
__global__ void __launch_bounds__(kCmpWarps * 32) compress_kernel(const float* __restrict__ input,
                                                                   const float* __restrict__ R,
                                                                   const float* __restrict__ codebook,
                                                                   float* __restrict__ radius_out,
                                                                   uint8_t* __restrict__ packed_out,
                                                                   int N, int n_levels) {
    constexpr int DPL = D / 32;
    constexpr int kPitch = D + 1;                       // transposed fill and row reads both conflict-free
    extern __shared__ __align__(16) float smem[];
    float* Rt = smem;                                   // Rt[k][j] = R[j][k]
    float* xs = smem + D * kPitch;                      // [warp][k][kCmpVecs]
    __shared__ float cb[16];
    if (threadIdx.x < n_levels) cb[threadIdx.x] = codebook[threadIdx.x];
    for (int e = threadIdx.x; e < D * D; e += blockDim.x) {
        const int j = e / D, k = e - j * D;
        Rt[k * kPitch + j] = R[e];
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float4* xw = reinterpret_cast<float4*>(xs + warp * D * kCmpVecs);
    const int n_groups = (N + kCmpVecs - 1) / kCmpVecs;
    for (int grp = blockIdx.x * kCmpWarps + warp; grp < n_groups; grp += gridDim.x * kCmpWarps) {
        const int v0 = grp * kCmpVecs;
        // stage the four inputs interleaved: xw[k] = {x0[k], x1[k], x2[k], x3[k]}
        for (int k = lane; k < D; k += 32) {
            float4 x;
            x.x = input[(size_t)v0 * D + k];
            x.y = v0 + 1 < N ? input[(size_t)(v0 + 1) * D + k] : 0.0f;
            x.z = v0 + 2 < N ? input[(size_t)(v0 + 2) * D + k] : 0.0f;
            x.w = v0 + 3 < N ? input[(size_t)(v0 + 3) * D + k] : 0.0f;
            xw[k] = x;
        }
        __syncwarp();
        float acc[kCmpVecs][DPL];
#pragma unroll
        for (int v = 0; v < kCmpVecs; ++v)
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[v][i] = 0.0f;
#pragma unroll 4
        for (int k = 0; k < D; ++k) {
            const float4 x = xw[k];
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const float r = Rt[k * kPitch + lane + 32 * i];
                acc[0][i] = fmaf(x.x, r, acc[0][i]);
                acc[1][i] = fmaf(x.y, r, acc[1][i]);
                acc[2][i] = fmaf(x.z, r, acc[2][i]);
                acc[3][i] = fmaf(x.w, r, acc[3][i]);
            }
        }
        __syncwarp();
#pragma unroll
        for (int v = 0; v < kCmpVecs; ++v) {
            // sum of squares: element t pairs with t + D/2, then + D/4, ... down to + 1
            float sq[DPL];
#pragma unroll
            for (int i = 0; i < DPL; ++i) sq[i] = __fmul_rn(acc[v][i], acc[v][i]);   // no contraction into the adds
#pragma unroll
            for (int h = DPL / 2; h; h >>= 1)
#pragma unroll
                for (int i = 0; i < h; ++i) sq[i] = __fadd_rn(sq[i], sq[i + h]);
            float s = sq[0];
#pragma unroll
            for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
            const float radius = sqrtf(s);
            const bool live = v0 + v < N;
            if (live && lane == 0) radius_out[v0 + v] = radius;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const float dir = radius > 1e-30f ? acc[v][i] / radius : 0.0f;
                const int idx = nearest_level(dir, cb, n_levels);
                const int up = __shfl_down_sync(kFull, idx, 1);
                if (live && !(lane & 1))
                    packed_out[(size_t)(v0 + v) * (D / 2) + (lane >> 1) + 16 * i] = (uint8_t)(idx | (up << 4));
            }
        }
    }
}

// Any even head dim up to 1024: one CTA per vector.
__global__ void __launch_bounds__(256) compress_any_dim_kernel(const float* __restrict__ input,
                                                               const float* __restrict__ R,
                                                               const float* __restrict__ codebook,
                                                               float* __restrict__ radius_out,
                                                               uint8_t* __restrict__ packed_out,
                                                               int D, int n_levels) {
    __shared__ float xs[kMaxDim];
    __shared__ float rot[kMaxDim];
    __shared__ float cb[16];
    __shared__ float part[8];
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x < n_levels) cb[threadIdx.x] = codebook[threadIdx.x];
    for (int k = threadIdx.x; k < D; k += blockDim.x) xs[k] = input[(size_t)n * D + k];
    __syncthreads();
    float sq = 0.0f;
    for (int j = warp; j < D; j += 8) {
        const float* row = R + (size_t)j * D;
        float s = 0.0f;
        for (int k = lane; k < D; k += 32) s = fmaf(xs[k], row[k], s);
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
        if (lane == 0) rot[j] = s;
        sq = fmaf(s, s, sq);
    }
    if (lane == 0) part[warp] = sq;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += part[w];
    const float radius = sqrtf(total);
    if (threadIdx.x == 0) radius_out[n] = radius;
    for (int b = threadIdx.x; b < D / 2; b += blockDim.x) {
        const float d0 = radius > 1e-30f ? rot[2 * b] / radius : 0.0f;
        const float d1 = radius > 1e-30f ? rot[2 * b + 1] / radius : 0.0f;
        packed_out[(size_t)n * (D / 2) + b] =
            (uint8_t)(nearest_level(d0, cb, n_levels) | (nearest_level(d1, cb, n_levels) << 4));
    }
}

// ---------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------

constexpr int kAttWarps = 4;
constexpr int kTile = 32;                     // tokens a warp takes at a time (lane t <-> token t)
constexpr float kLowest = -1e30f;

struct AttnParams {
    const float* q;
    const uint8_t* pk;
    const float* kr;
    const uint8_t* pv;
    const float* vr;
    const float* codebook;
    float* out;
    float* partials;          // [total_q_heads][n_split][2 + 32*DPL], used when n_split > 1
    unsigned* tickets;        // [total_kv_heads * groups], zero between launches
    int gqa, S, D, n_levels, n_split, tiles_per_split;
    float scale;
    int vector_loads;         // rows start on a multiple of the lane's byte count
};

// DPL/2 packed bytes of one row for this lane, zero beyond the row.
template <int DPL>
__device__ __forceinline__ void load_row_bytes(const uint8_t* row, int row_bytes, int lane, bool vec,
                                               uint32_t (&w)[(DPL + 7) / 8]) {
    constexpr int BPL = DPL / 2;
    constexpr int W = (DPL + 7) / 8;
    const int b0 = lane * BPL;
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = 0;
    if (vec && b0 + BPL <= row_bytes) {
        if constexpr (BPL == 1) w[0] = row[b0];
        else if constexpr (BPL == 2) w[0] = *reinterpret_cast<const uint16_t*>(row + b0);
        else if constexpr (BPL == 4) w[0] = *reinterpret_cast<const uint32_t*>(row + b0);
        else if constexpr (BPL == 8) {
            const uint2 t = *reinterpret_cast<const uint2*>(row + b0);
            w[0] = t.x; w[1] = t.y;
        } else {
            const uint4 t = *reinterpret_cast<const uint4*>(row + b0);
            w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
        }
    } else {
#pragma unroll
        for (int b = 0; b < BPL; ++b)
            if (b0 + b < row_bytes) w[b >> 2] |= (uint32_t)row[b0 + b] << (8 * (b & 3));
    }
}

// Centroid pairs of a stored byte: entry (byte, copy) = {codebook[byte & mask], codebook[(byte >> 4) & mask]},
// kPairCopies copies side by side (a lane uses copy lane % kPairCopies, which thins out bank conflicts).
constexpr int kPairCopies = 4;

template <int DPL>
__device__ __forceinline__ void decode_row(const uint32_t (&w)[(DPL + 7) / 8], uint32_t pair_lane, float (&v)[DPL]) {
#pragma unroll
    for (int i = 0; i < DPL / 2; ++i) {
        const uint32_t byte = (w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
        float2 c;
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];\n" : "=f"(c.x), "=f"(c.y) : "r"(pair_lane + byte * (kPairCopies * 8)));
        v[2 * i] = c.x;
        v[2 * i + 1] = c.y;
    }
}

// A warp fetches the packed words of `kChunk` consecutive tokens before it touches any of them, so
// that the loads are in flight together: 32 tokens when a lane's share of a row is one word,
// fewer for the wide head dims.
template <int DPL>
struct Chunk {
    static constexpr int W = (DPL + 7) / 8;
    static constexpr int kTokens = 32 / W;
    static constexpr int kLevel = W == 1 ? 5 : (W == 2 ? 4 : 3);
};

// Rows past `valid` repeat the last valid row: their scores and weights are masked by the caller.
template <int DPL>
__device__ __forceinline__ void load_chunk(const uint8_t* rows, int row_bytes, int first, int valid, int lane, bool vec,
                                           uint32_t (&w)[Chunk<DPL>::kTokens][Chunk<DPL>::W]) {
#pragma unroll
    for (int t = 0; t < Chunk<DPL>::kTokens; ++t)
        load_row_bytes<DPL>(rows + (uint32_t)(min(first + t, valid - 1) * row_bytes), row_bytes, lane, vec, w[t]);
}

template <int DPL, int G>
struct TileScores {
    using C = Chunk<DPL>;
    const uint8_t* rows;      // first row of the tile
    int row_bytes, valid, lane;
    bool vec;
    uint32_t pair_lane;       // shared address of this lane's copy of the pair table
    const float (*q)[DPL];

    // Sums over the 32 lanes of `1 << L` fetched tokens starting at chunk position t; afterwards
    // lane l holds the token t + (l mod 2^L) in out[].
    template <int L>
    __device__ __forceinline__ void reduce(const uint32_t (&w)[C::kTokens][C::W], int t, float (&out)[G]) const {
        if constexpr (L == 0) {
            float kv[DPL];
            decode_row<DPL>(w[t], pair_lane, kv);
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < DPL; ++i) s = fmaf(q[h][i], kv[i], s);
                out[h] = s;
            }
        } else {
            float a[G], b[G];
            reduce<L - 1>(w, t, a);
            reduce<L - 1>(w, t + (1 << (L - 1)), b);
            combine<L>(a, b, out);
        }
    }

    template <int L>
    __device__ __forceinline__ void combine(const float (&a)[G], const float (&b)[G], float (&out)[G]) const {
        const bool upper = lane & (1 << (L - 1));
#pragma unroll
        for (int h = 0; h < G; ++h) {
            const float send = upper ? a[h] : b[h];
            const float keep = upper ? b[h] : a[h];
            out[h] = keep + __shfl_xor_sync(kFull, send, 1 << (L - 1));
        }
    }

    // The same over `1 << L` tokens of the tile starting at token t, chunk by chunk.
    template <int L>
    __device__ __forceinline__ void run(int t, float (&out)[G]) const {
        if constexpr (L == C::kLevel) {
            uint32_t w[C::kTokens][C::W];
            load_chunk<DPL>(rows, row_bytes, t, valid, lane, vec, w);
            reduce<L>(w, 0, out);
        } else {
            float a[G], b[G];
            run<L - 1>(t, a);
            run<L - 1>(t + (1 << (L - 1)), b);
            combine<L>(a, b, out);
        }
    }
};

// Workspace of the sliced launches: records of the slices and one arrival counter per (kv head,
// query group).  Part of the module, so nothing is allocated per call; the last slice to arrive
// puts its counter back to zero.  Launches on one device therefore have to be ordered with
// respect to each other, which the bridge's single compute stream gives.
constexpr size_t kWsFloats = size_t(1) << 20;
constexpr int kWsTickets = 4096;
__device__ float g_partials[kWsFloats];
__device__ unsigned g_tickets[kWsTickets];

template <int DPL, int G>
__global__ void __launch_bounds__(kAttWarps * 32, 3) attention_kernel(const AttnParams p) {
    constexpr int DP = 32 * DPL;                      // padded head dim
    constexpr int REC = DP + 2;                       // partial record: m, l, acc[DP]
    __shared__ __align__(16) float2 pair_tab[256 * kPairCopies];
    __shared__ float sm_m[kAttWarps][G], sm_l[kAttWarps][G];
    __shared__ float sm_acc[kAttWarps][G][DP];
    __shared__ unsigned sm_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, group = blockIdx.y, hkv = blockIdx.z;
    const int hq0 = hkv * p.gqa + group * G;
    const int row_bytes = p.D >> 1;
    const uint32_t mask = (uint32_t)(p.n_levels - 1);
    for (int e = threadIdx.x; e < 256 * kPairCopies; e += blockDim.x) {
        const uint32_t byte = (uint32_t)e / kPairCopies;
        pair_tab[e] = make_float2(p.codebook[byte & mask], p.codebook[(byte >> 4) & mask]);
    }
    __syncthreads();
    const uint32_t pair_lane = (uint32_t)__cvta_generic_to_shared(pair_tab) + (lane % kPairCopies) * 8;

    float q[G][DPL];
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane * DPL + i;
            q[h][i] = d < p.D ? p.q[(size_t)(hq0 + h) * p.D + d] : 0.0f;
        }

    float m[G], l[G], acc[G][DPL];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        m[h] = kLowest;
        l[h] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[h][i] = 0.0f;
    }

    const int n_tiles = (p.S + kTile - 1) / kTile;
    const int tile_lo = split * p.tiles_per_split;
    const int tile_hi = min(n_tiles, tile_lo + p.tiles_per_split);
    const size_t kv_row0 = (size_t)hkv * p.S;
    for (int tile = tile_lo + warp; tile < tile_hi; tile += kAttWarps) {
        const int s0 = tile * kTile;
        const int valid = min(kTile, p.S - s0);
        const float kr = lane < valid ? p.kr[kv_row0 + s0 + lane] : 0.0f;
        const float vr = lane < valid ? p.vr[kv_row0 + s0 + lane] : 0.0f;

        TileScores<DPL, G> ts{p.pk + (kv_row0 + s0) * row_bytes, row_bytes, valid, lane, p.vector_loads != 0,
                              pair_lane, q};
        float sc[G];
        ts.template run<5>(0, sc);

        float w[G];
#pragma unroll
        for (int h = 0; h < G; ++h) {
            const float s = lane < valid ? sc[h] * kr * p.scale : kLowest;
            float tmax = s;
#pragma unroll
            for (int o = 16; o; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(kFull, tmax, o));
            const float m_new = fmaxf(m[h], tmax);
            const float corr = __expf(m[h] - m_new);
            const float pr = lane < valid ? __expf(s - m_new) : 0.0f;
            m[h] = m_new;
            l[h] = l[h] * corr + pr;                   // lane-private share of the denominator
            w[h] = pr * vr;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[h][i] *= corr;
        }

        const uint8_t* vrows = p.pv + (kv_row0 + s0) * row_bytes;
        using C = Chunk<DPL>;
#pragma unroll 1
        for (int c0 = 0; c0 < valid; c0 += C::kTokens) {
            uint32_t vw[C::kTokens][C::W];
            load_chunk<DPL>(vrows, row_bytes, c0, valid, lane, p.vector_loads != 0, vw);
#pragma unroll
            for (int t = 0; t < C::kTokens; ++t) {
                float vv[DPL];
                decode_row<DPL>(vw[t], pair_lane, vv);
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    const float wt = __shfl_sync(kFull, w[h], c0 + t);     // 0 for tokens past `valid`
#pragma unroll
                    for (int i = 0; i < DPL; ++i) acc[h][i] = fmaf(wt, vv[i], acc[h][i]);
                }
            }
        }
    }

    // the CTA's four warps -> one (m, l, acc) per head
#pragma unroll
    for (int h = 0; h < G; ++h) {
        float lt = l[h];
#pragma unroll
        for (int o = 16; o; o >>= 1) lt += __shfl_xor_sync(kFull, lt, o);
        if (lane == 0) { sm_m[warp][h] = m[h]; sm_l[warp][h] = lt; }
#pragma unroll
        for (int i = 0; i < DPL; ++i) sm_acc[warp][h][lane * DPL + i] = acc[h][i];
    }
    __syncthreads();

    const bool single = p.n_split == 1;
    for (int e = threadIdx.x; e < G * DP; e += blockDim.x) {
        const int h = e / DP, d = e - h * DP;
        float mm = sm_m[0][h];
#pragma unroll
        for (int wv = 1; wv < kAttWarps; ++wv) mm = fmaxf(mm, sm_m[wv][h]);
        float ll = 0.0f, aa = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kAttWarps; ++wv) {
            const float c = __expf(sm_m[wv][h] - mm);
            ll = fmaf(sm_l[wv][h], c, ll);
            aa = fmaf(sm_acc[wv][h][d], c, aa);
        }
        if (single) {
            if (d < p.D) p.out[(size_t)(hq0 + h) * p.D + d] = ll > 0.0f ? aa / ll : 0.0f;
        } else {
            float* rec = p.partials + ((size_t)(hq0 + h) * p.n_split + split) * REC;
            if (d == 0) { rec[0] = mm; rec[1] = ll; }
            rec[2 + d] = aa;
        }
    }
    if (single) return;

    // the last slice to finish merges the records of its heads
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(p.tickets + hkv * gridDim.y + group, 1u);
        sm_last = done == (unsigned)p.n_split - 1;
        if (sm_last) p.tickets[hkv * gridDim.y + group] = 0;
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    for (int e = threadIdx.x; e < G * DP; e += blockDim.x) {
        const int h = e / DP, d = e - h * DP;
        if (d >= p.D) continue;
        const float* rec = p.partials + (size_t)(hq0 + h) * p.n_split * REC;
        // eight records per round trip to L2: the loads of a round do not depend on each other
        float mm = kLowest, ll = 0.0f, aa = 0.0f;
        for (int s0 = 0; s0 < p.n_split; s0 += 8) {
            float ms[8], ls[8], as[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float* r = rec + (size_t)min(s0 + u, p.n_split - 1) * REC;
                ms[u] = __ldcg(r);
                ls[u] = __ldcg(r + 1);
                as[u] = __ldcg(r + 2 + d);
            }
            float m_new = mm;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (s0 + u >= p.n_split) { ms[u] = kLowest; ls[u] = 0.0f; as[u] = 0.0f; }
                m_new = fmaxf(m_new, ms[u]);
            }
            const float c = __expf(mm - m_new);
            ll *= c;
            aa *= c;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float cu = __expf(ms[u] - m_new);
                ll = fmaf(ls[u], cu, ll);
                aa = fmaf(as[u], cu, aa);
            }
            mm = m_new;
        }
        p.out[(size_t)(hq0 + h) * p.D + d] = ll > 0.0f ? aa / ll : 0.0f;
    }
}

template <int DPL, int G>
bool launch_attention(const AttnParams& p, dim3 grid, cudaStream_t stream) {
    attention_kernel<DPL, G><<<grid, kAttWarps * 32, 0, stream>>>(p);
    return launched();
}

template <int DPL>
bool dispatch_group(int G, const AttnParams& p, dim3 grid, cudaStream_t stream) {
    if constexpr (DPL * 8 <= 32) if (G == 8) return launch_attention<DPL, 8>(p, grid, stream);
    if constexpr (DPL * 4 <= 32) if (G == 4) return launch_attention<DPL, 4>(p, grid, stream);
    if constexpr (DPL * 2 <= 32) if (G == 2) return launch_attention<DPL, 2>(p, grid, stream);
    return launch_attention<DPL, 1>(p, grid, stream);
}

// Built-in tables of the bridge (patch 985-1003): centroids for head dim 128.
const float kCodebook4[16] = {-0.1547f, -0.1175f, -0.0928f, -0.0722f, -0.0537f, -0.0363f, -0.0193f, -0.0024f,
                              0.0145f,  0.0318f,  0.0498f,  0.0692f,  0.0907f,  0.1157f,  0.1467f,  0.1947f};
const float kCodebook3[8] = {-0.1350f, -0.0820f, -0.0440f, -0.0110f, 0.0220f, 0.0560f, 0.0950f, 0.1500f};
const float kCodebook2[4] = {-0.1050f, -0.0280f, 0.0400f, 0.1200f};

// Uniform(-1, 1) entries from the C library generator, rows orthonormalised in order
// (patch 556-579).
void seeded_rotation(float* R, int D, int seed) {
    srand(seed);
    for (int i = 0; i < D * D; ++i) R[i] = ((float)rand() / RAND_MAX) * 2.0f - 1.0f;
    for (int i = 0; i < D; ++i) {
        float* ri = R + (size_t)i * D;
        for (int j = 0; j < i; ++j) {
            const float* rj = R + (size_t)j * D;
            float dot = 0.0f;
            for (int k = 0; k < D; ++k) dot += ri[k] * rj[k];
            for (int k = 0; k < D; ++k) ri[k] -= dot * rj[k];
        }
        float nn = 0.0f;
        for (int k = 0; k < D; ++k) nn += ri[k] * ri[k];
        nn = sqrtf(nn);
        if (nn > 1e-10f)
            for (int k = 0; k < D; ++k) ri[k] /= nn;
    }
}

}  // namespace

extern "C" {

int polarquant_last_error_c(void) {
    const int e = t_last_error;
    t_last_error = 0;
    return e;
}

void polarquant_rotate_query_cuda_c(const float* q_input, const float* rotation, float* q_rotated,
                                    int total_q_heads, int D, void* stream) {
    if (total_q_heads <= 0 || D <= 0) return;
    if (!q_input || !rotation || !q_rotated) { fail(kErrNull, "rotate_query: NULL pointer"); return; }
    if (D > kMaxDim) { fail(kErrDim, "rotate_query: head dim above 1024"); return; }
    rotate_rows_kernel<<<total_q_heads, 256, 0, (cudaStream_t)stream>>>(q_input, rotation, q_rotated, D);
    launched();
}

void polarquant_inverse_rotate_cuda_c(const float* input, const float* rotation, float* output,
                                      int total_q_heads, int D, void* stream) {
    if (total_q_heads <= 0 || D <= 0) return;
    if (!input || !rotation || !output) { fail(kErrNull, "inverse_rotate: NULL pointer"); return; }
    if (D > kMaxDim) { fail(kErrDim, "inverse_rotate: head dim above 1024"); return; }
    inverse_rotate_rows_kernel<<<total_q_heads, 256, 0, (cudaStream_t)stream>>>(input, rotation, output, D);
    launched();
}

void polarquant_compress_cuda_c(const float* input, const float* rotation, const float* codebook,
                                float* radius_out, uint8_t* packed_out,
                                int N, int D, int n_levels, void* stream) {
    if (N <= 0 || D <= 0) return;
    if (!input || !rotation || !codebook || !radius_out || !packed_out) { fail(kErrNull, "compress: NULL pointer"); return; }
    if (!dim_ok(D)) { fail(kErrDim, "compress: head dim must be even and at most 1024"); return; }
    if (n_levels < 1 || n_levels > 16) { fail(kErrLevels, "compress: n_levels outside [1, 16]"); return; }
    cudaStream_t st = (cudaStream_t)stream;
    // The shared-memory transpose of R costs a fixed 20-odd microseconds per launch; below a few
    // thousand vectors the CTA-per-vector kernel, which streams R from L2, finishes first.
    if ((D == 64 || D == 128) && N >= kCmpSmallN) {
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int n_groups = (N + kCmpVecs - 1) / kCmpVecs;
        const int ctas = std::min((n_groups + kCmpWarps - 1) / kCmpWarps, (D == 64 ? 4 : 2) * sms);
        const size_t smem = ((size_t)D * (D + 1) + (size_t)kCmpWarps * D * kCmpVecs) * sizeof(float);
        cudaError_t e;
        if (D == 64) {
            e = cudaFuncSetAttribute(compress_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess)
                compress_kernel<64><<<ctas, kCmpWarps * 32, smem, st>>>(input, rotation, codebook, radius_out,
                                                                         packed_out, N, n_levels);
        } else {
            e = cudaFuncSetAttribute(compress_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess)
                compress_kernel<128><<<ctas, kCmpWarps * 32, smem, st>>>(input, rotation, codebook, radius_out,
                                                                          packed_out, N, n_levels);
        }
        if (e != cudaSuccess) { fail(kErrCuda, cudaGetErrorString(e)); return; }
    } else {
        compress_any_dim_kernel<<<N, 256, 0, st>>>(input, rotation, codebook, radius_out, packed_out, D, n_levels);
    }
    launched();
}

void polarquant_fused_attention_cuda_c(const float* q_rotated, const uint8_t* packed_k,
                                       const float* k_radius, const uint8_t* packed_v,
                                       const float* v_radius, const float* codebook, float* output,
                                       int total_q_heads, int total_kv_heads,
                                       int S, int D, int n_levels, float scale, void* stream) {
    if (total_q_heads <= 0 || S <= 0 || D <= 0) return;
    if (!q_rotated || !packed_k || !k_radius || !packed_v || !v_radius || !codebook || !output) {
        fail(kErrNull, "attention: NULL pointer");
        return;
    }
    if (!dim_ok(D)) { fail(kErrDim, "attention: head dim must be even and at most 1024"); return; }
    if (n_levels < 1 || n_levels > 16) { fail(kErrLevels, "attention: n_levels outside [1, 16]"); return; }
    if (total_kv_heads <= 0 || total_q_heads % total_kv_heads) {
        fail(kErrHeads, "attention: total_q_heads is not a multiple of total_kv_heads");
        return;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int gqa = total_q_heads / total_kv_heads;
    int DPL = 2;
    while (32 * DPL < D) DPL *= 2;
    int G = 8;
    while (G > 1 && (gqa % G || G * DPL > 32)) G >>= 1;
    const int groups = gqa / G;

    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int n_tiles = (S + kTile - 1) / kTile;
    const int base = total_kv_heads * groups;
    // two CTAs per SM with at least two tiles per warp (three CTAs per SM measured slower:
    // 192 against 150 microseconds at 8 kv heads x 65536 tokens)
    int n_split = std::max(1, std::min((2 * sms + base - 1) / base, n_tiles / (2 * kAttWarps)));
    int tiles_per_split = (n_tiles + n_split - 1) / n_split;
    n_split = (n_tiles + tiles_per_split - 1) / tiles_per_split;

    AttnParams p{};
    p.q = q_rotated; p.pk = packed_k; p.kr = k_radius; p.pv = packed_v; p.vr = v_radius;
    p.codebook = codebook; p.out = output;
    p.gqa = gqa; p.S = S; p.D = D; p.n_levels = n_levels; p.scale = scale;
    const int bpl = DPL / 2;
    p.vector_loads = ((D / 2) % bpl == 0) && (reinterpret_cast<uintptr_t>(packed_k) % bpl == 0) &&
                     (reinterpret_cast<uintptr_t>(packed_v) % bpl == 0);

    if (n_split > 1) {
        const size_t per_split = (size_t)total_q_heads * (32 * DPL + 2);
        if (base > kWsTickets || per_split * 2 > kWsFloats) {
            n_split = 1;
        } else {
            n_split = (int)std::min<size_t>(n_split, kWsFloats / per_split);
        }
        tiles_per_split = (n_tiles + n_split - 1) / n_split;
        n_split = (n_tiles + tiles_per_split - 1) / tiles_per_split;
        if (n_split > 1 &&
            (cudaGetSymbolAddress((void**)&p.partials, g_partials) != cudaSuccess ||
             cudaGetSymbolAddress((void**)&p.tickets, g_tickets) != cudaSuccess)) {
            fail(kErrCuda, "attention: workspace symbol lookup failed");
            cudaGetLastError();
            return;
        }
    }
    p.n_split = n_split;
    p.tiles_per_split = tiles_per_split;
    const dim3 grid(n_split, groups, total_kv_heads);
    switch (DPL) {
        case 2:  dispatch_group<2>(G, p, grid, st); break;
        case 4:  dispatch_group<4>(G, p, grid, st); break;
        case 8:  dispatch_group<8>(G, p, grid, st); break;
        case 16: dispatch_group<16>(G, p, grid, st); break;
        default: dispatch_group<32>(G, p, grid, st); break;
    }
}

struct polarquant_state* polarquant_init_c(int head_dim, int n_kv_heads, int n_q_heads,
                                           int n_layers, int n_kv_max, int n_bits) {
    if (head_dim <= 0 || (head_dim & 1) || head_dim > kMaxDim || n_kv_heads <= 0 || n_layers < 0 || n_kv_max <= 0) {
        fail(kErrDim, "init: bad shape");
        return nullptr;
    }
    const float* cb_host = kCodebook4;
    if (n_bits == 3) cb_host = kCodebook3;
    else if (n_bits == 2) cb_host = kCodebook2;
    else if (n_bits != 4) {
        fprintf(stderr, "PolarQuant: unsupported n_bits=%d, using 4\n", n_bits);
        n_bits = 4;
    }
    polarquant_state* st = new polarquant_state();
    st->enabled = true;
    st->n_bits = n_bits;
    st->n_levels = 1 << n_bits;
    st->head_dim = head_dim;
    st->n_kv_heads = n_kv_heads;
    st->n_q_heads = n_q_heads;
    st->n_layers = n_layers;
    st->n_kv_max = n_kv_max;
    st->codebook = nullptr;
    st->rotation = nullptr;
    st->layers = new polarquant_kv_layer[n_layers > 0 ? n_layers : 1]();

    bool ok = cudaMalloc(&st->codebook, st->n_levels * sizeof(float)) == cudaSuccess &&
              cudaMemcpy(st->codebook, cb_host, st->n_levels * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess;
    if (ok) {
        float* R = new float[(size_t)head_dim * head_dim];
        seeded_rotation(R, head_dim, 42);
        const size_t bytes = (size_t)head_dim * head_dim * sizeof(float);
        ok = cudaMalloc(&st->rotation, bytes) == cudaSuccess &&
             cudaMemcpy(st->rotation, R, bytes, cudaMemcpyHostToDevice) == cudaSuccess;
        delete[] R;
    }
    const size_t packed_bytes = (size_t)n_kv_heads * n_kv_max * (head_dim / 2);
    const size_t radius_bytes = (size_t)n_kv_heads * n_kv_max * sizeof(float);
    for (int l = 0; ok && l < n_layers; ++l) {
        polarquant_kv_layer& L = st->layers[l];
        ok = cudaMalloc(&L.k_packed, packed_bytes) == cudaSuccess && cudaMalloc(&L.k_radius, radius_bytes) == cudaSuccess &&
             cudaMalloc(&L.v_packed, packed_bytes) == cudaSuccess && cudaMalloc(&L.v_radius, radius_bytes) == cudaSuccess &&
             cudaMemset(L.k_packed, 0, packed_bytes) == cudaSuccess && cudaMemset(L.k_radius, 0, radius_bytes) == cudaSuccess &&
             cudaMemset(L.v_packed, 0, packed_bytes) == cudaSuccess && cudaMemset(L.v_radius, 0, radius_bytes) == cudaSuccess;
    }
    if (!ok) {
        cudaGetLastError();
        fail(kErrCuda, "init: device allocation failed");
        polarquant_free_c(st);
        return nullptr;
    }
    const double compressed = 2.0 * n_layers * (double)n_kv_heads * n_kv_max * (head_dim / 2 + sizeof(float));
    const double original = 2.0 * n_layers * (double)n_kv_heads * n_kv_max * head_dim * sizeof(float);
    fprintf(stderr, "PolarQuant-KV initialized: head_dim=%d n_kv_heads=%d n_q_heads=%d n_layers=%d n_bits=%d n_kv_max=%d; "
                    "compressed cache %.2f MB (fp32 %.2f MB, %.1fx)\n",
            head_dim, n_kv_heads, n_q_heads, n_layers, n_bits, n_kv_max, compressed / 1048576.0, original / 1048576.0,
            compressed > 0 ? original / compressed : 0.0);
    return st;
}

void polarquant_free_c(struct polarquant_state* state) {
    if (!state) return;
    if (state->codebook) cudaFree(state->codebook);
    if (state->rotation) cudaFree(state->rotation);
    if (state->layers) {
        for (int l = 0; l < state->n_layers; ++l) {
            polarquant_kv_layer& L = state->layers[l];
            if (L.k_packed) cudaFree(L.k_packed);
            if (L.k_radius) cudaFree(L.k_radius);
            if (L.v_packed) cudaFree(L.v_packed);
            if (L.v_radius) cudaFree(L.v_radius);
        }
        delete[] state->layers;
    }
    delete state;
}

}  // extern "C"
