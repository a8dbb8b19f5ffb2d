// pq_compress: fused rotate -> per-32 radius -> nearest Lloyd-Max centroid -> pack
// [-> QJL 1-bit residual sketch], for block_pq4 storage.
//
// One CTA (4 x D/32 epilogue warps) owns a tile of 128 vectors at a time (persistent over tiles).
// The rotation  xr = x @ R^T  runs on the 5th-gen tensor cores: tcgen05.mma (kind::f16, M = 128,
// K = 16) on shared-memory operands, float32 accumulators in tensor memory (TMEM), read back
// with tcgen05.ld for the epilogue.  x is float16 (exact); R is pre-split on the host into two
// float16 terms  4096*R = hi + lo, so xr carries about 22 mantissa bits of R and matches the
// float64-then-float32 rotation of the numpy reference (python/polarquant_kv/rotation.py:48) to a
// few 1e-8 relative.  Tensor-core accumulation truncates when it aligns addends, so the hi and
// lo products go to separate accumulators that are summed with a round-to-nearest float32 add.
//
// Without the QJL sketch the kernel is a three-role pipeline with no CTA-wide barrier per tile:
//   copy warp   - keeps three vector tiles in flight or in use (TMA, cp.async.bulk.tensor, into the
//                 128-byte-swizzled K-major layout; an mbarrier counts the bytes);
//   MMA warp    - one MMA per k-step with N = 2D ([R_hi ; R_lo] stacked along N) into one of two
//                 TMEM accumulator buffers, as soon as the tile has landed and the buffer has been
//                 read out; tcgen05.commit signals the epilogue and frees the vector buffer;
//   epilogue    - a thread owns one vector x one 32-element block (TMEM lane = vector).  The warps
//                 that share 32 vectors meet at a named barrier and one lane sends those vectors'
//                 packed bytes off with a bulk store.
// With the sketch the same three roles run; the residual goes back into tensor memory as the A operand
// of a second contraction (with P R^T, three float16 product terms) that the MMA warp issues behind the
// next tile's rotation, and the epilogue picks up a tile's sign bits one tile later.
// Everything after the contraction follows the reference's float32 arithmetic exactly:
//   radius  = sqrt(sum of squares), summed in numpy's axis-reduction order
//             (eight strided partial sums, then a balanced tree),
//   guard   = radius < 1e-30 -> radius 0, indices 0      (quantizer.py:107-119),
//   dir     = xr / radius with IEEE rounding              (quantizer.py:121),
//   index   = #thresholds strictly below dir, the thresholds being the exact float32
//             decision points of argmin_i |dir - c_i|     (lloyd_max.py:82-90),
//   d       = float16(min(radius, 65504))                 (compress_kernel.py:178),
//   packing = low nibble first                            (compress_kernel.py:34-50).
// In the epilogue a thread owns one vector x one 32-element block (TMEM lane = vector), so
// the block sums, the division and the packing are thread-local.
// QJL (qjl.py:25-35, compress_kernel.py:168-175): the residual e = xr - d*c[idx] stays in
// rotated space; signs of P e equal signs of (P R^T) e_rot, evaluated as a second
// three-term float16 contraction (e_hi*P_hi + e_hi*P_lo + e_lo*P_hi) on the same path.
//
// Shared-memory operand layout of the constant matrices (K-major, no swizzle): 16-byte chunks of 8
// halves; chunk kc of row r sits at  kc * (rows/8 * 128) + (r / 8) * 128 + (r % 8) * 16  — 8x16-byte
// core matrices, stride 128 B between 8-row groups (SBO), rows/8*128 B between K chunks (LBO).
// The vector tiles arrive by TMA (cp.async.bulk.tensor, one thread issues, an mbarrier counts the
// bytes) in the 128-byte-swizzled K-major layout: boxes of 128 vectors x 64 halves, rows 128 B apart,
// 8-row groups 1024 B apart; the packed tile leaves by bulk stores of 32 vectors.
#include <cmath>
#include <cstring>

#include "pq_tcgen05.cuh"

namespace pq {

// Bit 0: a bounded wait on a completion barrier gave up; bit 1: the dynamic shared-memory window
// started too high for the fixed-address layout.  Read and cleared by pq_poll_device_errors().
// A set bit means the results of that launch are not valid.
static __device__ unsigned int g_compress_error = 0;

constexpr int kTileVecs = 128;
// warps: 4 per warpgroup (TMEM lanes 0..127 = vectors) x D/32 warpgroups (one block each)
__host__ __device__ constexpr int compress_threads(int D) { return 32 * 4 * (D / 32); }
// Two more warps run beside them: one issues the MMAs, one the tile copies.
__host__ __device__ constexpr int compress_launch_threads(int D) { return compress_threads(D) + 64; }

struct CompressParams {
    const __half* x;
    const __half* rot_split;   // [D][2D]
    const __half* jl_split;    // [M][2D] or null
    uint8_t* blocks_out;
    uint8_t* qjl_bits_out;
    __half* qjl_norm_out;
    int64_t n_vec;
    // Output addressing: input vector v = row * tokens_per_row + t lands in token slot
    // row * row_capacity + position + t of the output tensors (one row with capacity n_vec at position 0
    // is the plain contiguous case).
    int64_t tokens_per_row, row_capacity, position;
    // When set, the position is read from device memory at kernel start (a step of a captured graph
    // whose position advances on the device); out of range -> error flag, nothing written.
    const int64_t* position_dev;
    int jl_dim;
    float cb[16];
    // Index search table: a normalised coordinate y falls into bucket k = floor(64 y + 64);
    // index = base[k] + (y > t[k]).  A bucket holds at most one decision threshold.
    float bucket_t[132];
    uint32_t bucket_base[132];
};

// Packed float32x2 arithmetic (sm_100): two IEEE round-to-nearest operations per instruction.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;\n"
        : "=l"(*reinterpret_cast<unsigned long long*>(&d))
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;\n"
        : "=l"(*reinterpret_cast<unsigned long long*>(&d))
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n"
        : "=l"(*reinterpret_cast<unsigned long long*>(&d))
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return d;
}
// 16 packed words into consecutive columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_store16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                 "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// Named barrier over `count` threads.
__device__ __forceinline__ void group_barrier(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory");
}

// Byte offset of 16-byte chunk `kc` of row `r` in a K-major operand tile with `rows` rows.
__device__ __forceinline__ uint32_t chunk_off(int rows, int r, int kc) {
    return (uint32_t)(kc * (rows / 8) * 128 + (r >> 3) * 128 + (r & 7) * 16);
}

// Packed vectors g0 .. g0+rows-1 of a tile (staged at `src`) to their token slots when the output has
// several rows: one bulk store when the group stays inside a row and is aligned, word copies otherwise.
template <int VB, int WG>
__device__ __noinline__ void store_rows_impl(uint8_t* blocks_out, int64_t tokens_per_row, int64_t row_capacity,
                                             int64_t position, int64_t g0, int rows, const uint8_t* src,
                                             int lane, int wg, bool leader) {
    auto slot_of = [&](int64_t v) -> int64_t {
        const int64_t r = v / tokens_per_row;
        return r * row_capacity + position + (v - r * tokens_per_row);
    };
    const int64_t s0 = slot_of(g0);
    const bool contig = slot_of(g0 + rows - 1) == s0 + rows - 1;         // the group stays inside one row
    uint8_t* dst = blocks_out + s0 * VB;
    if (rows == 32 && contig && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        if (leader) bulk_store(dst, sm_addr(src), 32u * VB);
    } else if (contig) {
        for (int c = wg * 32 + lane; c < rows * VB / 4; c += 32 * WG)
            reinterpret_cast<uint32_t*>(dst)[c] = reinterpret_cast<const uint32_t*>(src)[c];
    } else if (lane < rows) {                                            // vectors of several rows: one lane each
        uint32_t* d32p = reinterpret_cast<uint32_t*>(blocks_out + slot_of(g0 + lane) * VB);
        for (int c = wg; c < VB / 4; c += WG) d32p[c] = reinterpret_cast<const uint32_t*>(src + lane * VB)[c];
    }
}

template <int D, int BITS, bool QJL>
struct CompressCfg {
    static constexpr int THREADS = compress_threads(D);
    static constexpr int WG = D / 32;                         // warpgroups = blocks per vector
    static constexpr int VB = (D / 32) * block_bytes(BITS);   // bytes per stored vector
    static constexpr int kRBytes = 4 * D * D;                 // [2D/8 chunks][D rows][16 B]
    static constexpr int kXBytes = (D / 8) * 2048;            // [D/8 chunks][128 rows][16 B]
    // One MMA per k-step with N = 2D ([R_hi ; R_lo] stacked), i.e. two accumulators (hi and lo products)
    // per tile.
    static constexpr int KG = 2;
    // Index table: 129 buckets x 128 bytes at a fixed shared address.  Without the sketch an entry is
    // {threshold, replicated count} (8 bytes, 16 lane copies); with it {threshold, replicated count,
    // centroid below, centroid above} (16 bytes, 8 lane copies), which also yields the dequantised value
    // the residual needs.
    static constexpr int kEntry = QJL ? 16 : 8;
    static constexpr int BREP = 128 / kEntry;
    // Tensor memory.  Without the sketch two rotation accumulators (2D columns each) alternate.  With it:
    // one rotation accumulator (the epilogue reads it out right away, which frees it for the next tile's
    // rotation long before that tile's epilogue starts), the sketch accumulator, and the residual as
    // the A operand of the sketch contraction: hi and lo float16 terms, two dims per 32-bit column.
    static constexpr int kRotCols = KG * D;
    static constexpr int kAccCol = kRotCols;
    static constexpr int kEhiCol = kRotCols + 128;
    static constexpr int kEloCol = kEhiCol + D / 2;
    static constexpr int kTmemCols = QJL ? 512 : 2 * kRotCols;
    static constexpr int kOutBufs = QJL ? 1 : 2;              // packed-tile staging buffers
    static constexpr int kXBufs = QJL ? 2 : 3;                // vector tiles in flight or in use
    // The layout is pinned to absolute shared-memory addresses so that a bucket's address is a single
    // AND-OR of the fused-multiply-add result: the index table sits on a 32 KB boundary, small buffers
    // below it, the operand tiles above.
    //   no sketch:  [low: packed tiles, codebook, barriers][0x8000 table][0x10000 R][X x 3]
    //   sketch:     [low: packed tile, codebook, barriers, exchange, first chunks of P'][0x8000 table]
    //               [rest of P'][R][X x 2]          (P' = the split of P R^T, K-chunk by K-chunk)
    static constexpr uint32_t kTabAddr = 0x8000u;
    static constexpr uint32_t kTabBytes = 129 * 128;
    static constexpr uint32_t kExchBytes = QJL ? 2 * kTileVecs * WG * 4 : 0;      // radii and residual norms
    static constexpr uint32_t kPLowBytes = QJL ? 16384 : 0;
    static constexpr uint32_t kLowBytes = kOutBufs * kTileVecs * VB + 64 + 128 + kExchBytes + kPLowBytes;
    static constexpr uint32_t kPHiAddr = 0xC100u;
    static constexpr uint32_t kPHiMax = (2 * D / 8 > 8 ? 2 * D / 8 - 8 : 0) * 2048;   // at jl_dim 128
    static constexpr uint32_t kRAddr = QJL ? kPHiAddr + kPHiMax : 0x10000u;
    static constexpr uint32_t kXAddr = (kRAddr + kRBytes + 1023u) & ~1023u;
    __host__ __device__ static size_t smem_bytes() { return (size_t)kXAddr + kXBufs * (size_t)kXBytes; }
    // K chunks of P' that live in the low region (an even number: a k-step reads two neighbours)
    __host__ __device__ static int p_low_chunks(int jl_dim) {
        if (!QJL) return 0;
        const int lbo = (jl_dim / 8) * 128, total = 2 * D / 8;
        int n = (int)(kPLowBytes / lbo) & ~1;
        return n < total ? n : total;
    }
};

template <int D, int BITS, bool QJL>
__global__ void __launch_bounds__(compress_launch_threads(D), 1)
pq_compress_kernel(const CompressParams p, const __grid_constant__ CUtensorMap x_map) {
    using C = CompressCfg<D, BITS, QJL>;
    constexpr int THREADS = C::THREADS;
    constexpr int WG = C::WG;
    constexpr int BB = block_bytes(BITS);
    constexpr int VB = C::VB;
    constexpr int BREP = C::BREP;
    constexpr int NLEV = 1 << BITS;
    const int M = QJL ? p.jl_dim : 0;

    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = sm_addr(smem_raw);
    uint8_t* sp = smem_raw + ((128u - (base & 127u)) & 127u);
    // the dynamic window must start low enough for the small buffers to end below the table
    if (sm_addr(sp) + C::kLowBytes > C::kTabAddr) {
        if (threadIdx.x == 0) atomicOr(&g_compress_error, 2u);
        return;
    }
    int64_t position = p.position;
    if (p.position_dev != nullptr) {
        position = *p.position_dev;
        if (position < 0 || position + p.tokens_per_row > p.row_capacity) {
            if (threadIdx.x == 0) atomicOr(&g_compress_error, 32u);
            return;
        }
    }
    uint8_t* outs0 = sp;                        sp += C::kOutBufs * kTileVecs * VB;
    float* cb_s = reinterpret_cast<float*>(sp); sp += 64;
    uint64_t* mbar = reinterpret_cast<uint64_t*>(sp);  sp += 128;
    float* exch_d = reinterpret_cast<float*>(sp);       // [128][WG] radii x 4096 of the tile's blocks
    float* exch_n = exch_d + kTileVecs * WG;            // [128][WG] squared residual norms
    sp += C::kExchBytes;
    uint8_t* p_low = sp;                                // first K chunks of P'
    uint8_t* zero = smem_raw - base;                    // generic address of shared address 0
    uint8_t* bucket_s = zero + C::kTabAddr;
    uint8_t* p_high = zero + C::kPHiAddr;
    uint8_t* Rb = zero + C::kRAddr;
    uint8_t* Xa = zero + C::kXAddr;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(mbar) + 96);
    volatile uint32_t* abort_s = reinterpret_cast<volatile uint32_t*>(reinterpret_cast<uint8_t*>(mbar) + 100);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wg = warp >> 2;                                   // block (32 output dims) this thread owns
    const int row = (warp & 3) * 32 + lane;                     // vector of the tile = TMEM lane
    const int n_plow = C::p_low_chunks(M);
    const uint32_t lbo_p = (uint32_t)(M / 8) * 128;             // bytes between K chunks of P'
    auto p_chunk = [&](int c) -> uint8_t* {
        return c < n_plow ? p_low + (size_t)c * lbo_p : p_high + (size_t)(c - n_plow) * lbo_p;
    };

    // ---- one-time set-up: split matrices, tables, barriers, tensor memory
    for (int id = tid; id < D * (2 * D / 8); id += blockDim.x) {
        const int n = ((id >> 5) % (D / 8)) * 8 + (id & 7), kc = ((id >> 5) / (D / 8)) * 4 + ((id >> 3) & 3);
        // B tile [2D rows][K = D]: the lo term's rows follow the hi term's (N = 2D)
        const int half = kc / (D / 8), kk = kc % (D / 8);
        cp_async_16(Rb + chunk_off(2 * D, half * D + n, kk), p.rot_split + (size_t)n * 2 * D + kc * 8);
    }
    if (QJL) {
        // P' [M rows][K = 2D]: chunk kc holds halves 8kc .. 8kc+7 of every row (hi term first, then lo)
        for (int id = tid; id < M * (2 * D / 8); id += blockDim.x) {
            const int n = id % M, kc = id / M;
            cp_async_16(p_chunk(kc) + (n >> 3) * 128 + (n & 7) * 16, p.jl_split + (size_t)n * 2 * D + kc * 8);
        }
    }
    if (tid < 16) cb_s[tid] = p.cb[tid < NLEV ? tid : 0];
    for (int e = tid; e < 129 * BREP; e += blockDim.x) {
        const int b = e / BREP;
        const int k = b < 132 ? b : 131;          // buckets past 128 only see out-of-range garbage
        // the count is replicated into every index field of the word, so packing a coordinate is one
        // AND-OR with that field's mask
        const uint32_t rep = BITS == 4 ? 0x11111111u : 0x55555555u;
        const uint32_t cnt = p.bucket_base[k];
        if (QJL) {
            const float below = p.cb[cnt < NLEV ? cnt : NLEV - 1], above = p.cb[cnt + 1 < NLEV ? cnt + 1 : NLEV - 1];
            reinterpret_cast<uint4*>(bucket_s)[e] =
                make_uint4(__float_as_uint(p.bucket_t[k]), cnt * rep, __float_as_uint(below), __float_as_uint(above));
        } else {
            reinterpret_cast<uint2*>(bucket_s)[e] = make_uint2(__float_as_uint(p.bucket_t[k]), cnt * rep);
        }
    }
    const uint32_t tab_lane = C::kTabAddr | ((uint32_t)(lane & (BREP - 1)) * C::kEntry);     // this lane's copy
    // Barriers.  [0], [1]: MMAs of rotation accumulator 0 / 1 done; [2..4]: vector buffer landed;
    // [5], [6]: rotation accumulator 0 / 1 read out by every epilogue thread; [7..9]: vector buffer
    // consumed by its MMAs.  With the sketch there is one rotation accumulator ([0], [5]) and
    // [1]: sketch MMAs done, [6]: residual written (and the previous tile's signs read) by every thread.
    if (tid == 0) {
        for (int i = 0; i < 5; ++i) mbar_init(sm_addr(mbar + i), 1);
        for (int i = 5; i < 7; ++i) mbar_init(sm_addr(mbar + i), THREADS);
        for (int i = 7; i < 10; ++i) mbar_init(sm_addr(mbar + i), 1);
        *abort_s = 0u;
    }
    if (warp == 0) tmem_alloc(sm_addr(tmem_slot), C::kTmemCols);
    cp_async_commit();
    cp_async_wait<0>();          // the split matrices are in place ...
    fence_async_smem();          // ... and visible to the tensor core's (async proxy) reads
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    bool ok = true;

    const int64_t n_tiles = (p.n_vec + kTileVecs - 1) / kTileVecs;
    // TMA fetch of one tile into vector buffer `buf` (rows past the end of x arrive as zeros)
    auto fetch_tile = [&](int64_t tile, int buf) {
        const uint32_t bar = sm_addr(mbar + 2 + buf), dst = sm_addr(Xa) + (uint32_t)buf * C::kXBytes;
        mbar_expect_tx(bar, (uint32_t)C::kXBytes);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) tma_load_2d(dst + h * 16384, &x_map, h * 64, (int)(tile * kTileVecs), bar);
    };
    const int64_t n_my = (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;      // tiles of this CTA
    if (warp == THREADS / 32) {
        // ---- MMA warp.  A tile's rotation goes out as soon as its vectors have landed and the
        // accumulator it writes has been read out: one MMA per k-step, N = 2D, columns [0, D) receive the
        // products with R's hi term, [D, 2D) those with its lo term.  With the sketch, the contraction of
        // tile i-1's residual (A operand in tensor memory) with P' follows the rotation of tile i.
        // Every lane runs the loop (so the waits and the descriptor arithmetic stay warp-uniform); lane 0
        // issues.
        constexpr uint32_t idesc = umma_idesc_f16(2 * D);
        constexpr uint32_t kLboB = (2 * D / 8) * 128;                     // K-chunk stride of the stacked R tile
        constexpr uint32_t a_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // 8-row groups 1024 B apart, 128-B swizzle
        constexpr uint32_t b_hi = (128u >> 4) | (1u << 14);                // 8-row groups 128 B apart, no swizzle
        const uint32_t a_lo0 = ((sm_addr(Xa) >> 4) & 0x3FFFu) | (1u << 16);
        const uint32_t b_lo0 = ((sm_addr(Rb) >> 4) & 0x3FFFu) | ((kLboB >> 4) << 16);
        const uint32_t issue = lane == 0 ? 1u : 0u;
        auto issue_sketch = [&]() {
            const uint32_t idesc_p = umma_idesc_f16(M);
            const uint32_t acc = tmem_base + C::kAccCol;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const uint32_t ah = tmem_base + C::kEhiCol + ks * 8, al = tmem_base + C::kEloCol + ks * 8;
                const uint32_t bh = ((sm_addr(p_chunk(2 * ks)) >> 4) & 0x3FFFu) | ((lbo_p >> 4) << 16);
                const uint32_t bl = ((sm_addr(p_chunk(D / 8 + 2 * ks)) >> 4) & 0x3FFFu) | ((lbo_p >> 4) << 16);
                umma_f16_ts_pred(acc, ah, bh, b_hi, idesc_p, ks ? 1u : 0u, issue);
                umma_f16_ts_pred(acc, ah, bl, b_hi, idesc_p, 1u, issue);
                umma_f16_ts_pred(acc, al, bh, b_hi, idesc_p, 1u, issue);
            }
            umma_commit_pred(sm_addr(mbar + 1), issue);
        };
        uint32_t xb = 0, xuse = 0;                          // vector buffer of tile i and how often it was used
        for (int64_t i = 0; i < n_my && ok; ++i) {
            const uint32_t b = QJL ? 0u : ((uint32_t)i & 1u);
            ok = mbar_wait(sm_addr(mbar + 2 + xb), xuse & 1u, abort_s, 32) && ok;
            if (QJL) {
                if (i >= 1) ok = mbar_wait(sm_addr(mbar + 5), (uint32_t)(i - 1) & 1u, abort_s, 32) && ok;
            } else {
                if (i >= 2) ok = mbar_wait(sm_addr(mbar + 5 + b), ((uint32_t)(i >> 1) - 1u) & 1u, abort_s, 32) && ok;
            }
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a_lo = a_lo0 + xb * (uint32_t)(C::kXBytes >> 4);
                const uint32_t acc = tmem_base + b * C::kRotCols;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    // a k-step is 32 B further inside the swizzled 128-byte row, 64 halves fill a 16 KB box
                    umma_f16_split(acc, a_lo + (uint32_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), a_hi,
                                   b_lo0 + (uint32_t)((2 * ks * kLboB) >> 4), b_hi, idesc, ks ? 1u : 0u);
                }
                umma_commit(sm_addr(mbar + b));             // accumulators ready for the epilogue
                umma_commit(sm_addr(mbar + 7 + xb));        // vector buffer free for the next copy
            }
            __syncwarp();
            if (QJL && i >= 1) {
                ok = mbar_wait(sm_addr(mbar + 6), (uint32_t)(i - 1) & 1u, abort_s, 32) && ok;
                if (!ok) break;
                tc_fence_after();
                issue_sketch();
                __syncwarp();
            }
            if (++xb == C::kXBufs) { xb = 0; ++xuse; }
        }
        if (QJL && ok && n_my > 0) {                        // the last tile's sketch
            ok = mbar_wait(sm_addr(mbar + 6), (uint32_t)(n_my - 1) & 1u, abort_s, 32) && ok;
            if (ok) {
                tc_fence_after();
                issue_sketch();
                __syncwarp();
            }
        }
        if (!ok && lane == 0) { *abort_s = 1u; atomicOr(&g_compress_error, 1u); }
    } else if (warp == THREADS / 32 + 1) {
        // ---- copy warp: keeps kXBufs tiles in flight or in use; a buffer is refilled as soon as the
        // MMAs that read it have completed
        uint32_t xb = 0, xuse = 0;
        for (int64_t i = 0; i < n_my && ok; ++i) {
            if (i >= C::kXBufs) ok = mbar_wait(sm_addr(mbar + 7 + xb), (xuse - 1u) & 1u, abort_s, 64) && ok;
            if (!ok) break;
            if (lane == 0) fetch_tile((int64_t)blockIdx.x + i * gridDim.x, (int)xb);
            __syncwarp();
            if (++xb == C::kXBufs) { xb = 0; ++xuse; }
        }
        if (!ok && lane == 0) { *abort_s = 1u; atomicOr(&g_compress_error, 1u); }
    } else {

    // ---- epilogue warps
    // token slot of input vector v in the output tensors
    const bool one_row = p.tokens_per_row >= p.n_vec;            // no 64-bit division on the common path
    auto slot_of = [&](int64_t v) -> int64_t {
        if (one_row) return position + v;
        const int64_t r = v / p.tokens_per_row;
        return r * p.row_capacity + position + (v - r * p.tokens_per_row);
    };
    // signs of the sketch of the tile whose vector `row` sits in token slot `slot`: every thread reads 32
    // projections of its vector from the sketch accumulator and stores their sign bits
    auto store_signs = [&](int64_t slot, bool valid) {
        const int M8 = M / 8;
        for (int cg = wg; cg * 32 < M; cg += WG) {
            float pr[32];
            tmem_ld32(pr, tmem_lane + C::kAccCol + cg * 32);
            // bit j = (projection j >= 0).  One funnel shift per projection moves its sign bit into the
            // word, last projection first; the complement turns "negative" into the stored convention.
            // (A sum of products on a +0 accumulator is never -0, so the sign bit alone decides.)
            uint32_t w = 0;
#pragma unroll
            for (int j = 31; j >= 0; --j) w = __funnelshift_l(__float_as_uint(pr[j]), w, 1);
            w = ~w;
            if (!valid) continue;
            uint8_t* dst = p.qjl_bits_out + slot * M8 + cg * 4;
            if (cg * 32 + 32 <= M && (reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
                *reinterpret_cast<uint32_t*>(dst) = w;
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (cg * 32 + k * 8 < M) dst[k] = (uint8_t)(w >> (8 * k));
            }
        }
    };
    auto store_rows = [&](int64_t g0, int rows, const uint8_t* src, int ln, int w, bool lead) {
        store_rows_impl<VB, WG>(p.blocks_out, p.tokens_per_row, p.row_capacity, position, g0, rows, src, ln, w, lead);
    };
    uint32_t it = 0;
    int64_t slot_prev = 0;
    bool valid_prev = false;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
        const int64_t v0 = tile * kTileVecs;
        const int n_valid = (int)min((int64_t)kTileVecs, p.n_vec - v0);
        const uint32_t rb = QJL ? 0u : (it & 1u);                         // this tile's rotation accumulator
        // The issuing warp runs ahead; without the sketch the accumulators alternate, so their barriers
        // flip parity every second tile.
        ok = mbar_wait(sm_addr(mbar + rb), (QJL ? it : (it >> 1)) & 1u, abort_s) && ok;
        tc_fence_after();
        uint8_t* outs = outs0 + (QJL ? 0u : (it & 1u) * (uint32_t)(kTileVecs * VB));
        const uint32_t tmem_tile = tmem_lane + rb * C::kRotCols;

        // ---- this thread owns vector `row`, block `wg`
        float2 v2[16];                  // 4096 * rotated coordinates, pairs (2k, 2k+1); the scale is a
        tmem_ld32(v2, tmem_tile + wg * 32);  // power of two: every rounding below commutes with it
#pragma unroll
        for (int grp = 1; grp < C::KG; ++grp) {
            float2 part[16];
            tmem_ld32(part, tmem_tile + grp * D + wg * 32);
#pragma unroll
            for (int k = 0; k < 16; ++k) v2[k] = add2(v2[k], part[k]);
        }
        // this thread's part of the accumulator is in registers
        tc_fence_before();
        mbar_arrive(sm_addr(mbar + 5 + rb));
        // numpy's float32 axis-reduction order: r[j] over j, j+8, j+16, j+24 (products rounded
        // separately), then a balanced tree
        float2 r2[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 a = mul2(v2[q], v2[q]);
            a = add2(a, mul2(v2[4 + q], v2[4 + q]));
            a = add2(a, mul2(v2[8 + q], v2[8 + q]));
            r2[q] = add2(a, mul2(v2[12 + q], v2[12 + q]));
        }
        const float ss = __fadd_rn(__fadd_rn(__fadd_rn(r2[0].x, r2[0].y), __fadd_rn(r2[1].x, r2[1].y)),
                                   __fadd_rn(__fadd_rn(r2[2].x, r2[2].y), __fadd_rn(r2[3].x, r2[3].y)));
        const float d_raw = __fsqrt_rn(ss);                          // 4096 * radius
        const bool zero = d_raw < 4096.0f * 1e-30f;
        const float d32 = zero ? 0.f : d_raw * (1.0f / 4096.0f);
        const __half d16 = __float2half_rn(fminf(d32, 65504.0f));
        const float dq = __half2float(d16) * 4096.0f;
        // x / d with IEEE rounding from a correctly rounded reciprocal and one residual
        // correction (no mismatch against true division in 2e6 samples)
        const float dsafe = zero ? 1.f : d_raw;
        const float rinv = __frcp_rn(dsafe);
        const float2 rinv2 = make_float2(rinv, rinv), negd2 = make_float2(-dsafe, -dsafe);
        // bucket key in the mantissa bits of 64 y + 98368: the unit in the last place is 2^-7 and bits
        // 7..14 hold  floor(64 y + 64)
        const float2 c64 = make_float2(64.f, 64.f), cmagic = make_float2(98368.f, 98368.f);
        float en2 = 0.f;
        uint32_t packed[BITS];                                        // 32 indices, low index first
#pragma unroll
        for (int w = 0; w < BITS; ++w) packed[w] = 0u;
        float* v = reinterpret_cast<float*>(&v2[0]);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float2 y0 = mul2(v2[k], rinv2);
            const float2 dir = fma2(fma2(y0, negd2, v2[k]), rinv2, y0);
            const float2 u = fma2(dir, c64, cmagic);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = 2 * k + e;
                const float dj = e ? dir.y : dir.x;
                const uint32_t a = (__float_as_uint(e ? u.y : u.x) & 0x7F80u) | tab_lane;
                // field = count of thresholds in lower buckets, plus one if y is above this bucket's
                const uint32_t sh = (j * BITS) & 31;
                uint32_t& pw = packed[(j * BITS) >> 5];
                if (QJL) {
                    uint4 be;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(be.x), "=r"(be.y), "=r"(be.z), "=r"(be.w) : "r"(a));
                    const bool up = dj > __uint_as_float(be.x);
                    pw |= be.y & (((1u << BITS) - 1u) << sh);
                    if (up) pw += 1u << sh;
                    // residual in rotated space (scaled by 4096): coordinate minus radius * centroid
                    const float ee = fmaf(-dq, __uint_as_float(up ? be.w : be.z), v[j]);
                    en2 = fmaf(ee, ee, en2);
                    v[j] = ee;
                } else {
                    uint2 be;
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];\n" : "=r"(be.x), "=r"(be.y) : "r"(a));
                    pw |= be.y & (((1u << BITS) - 1u) << sh);
                    asm("{\n\t.reg .pred p;\n\t"
                        "setp.gt.f32 p, %1, %2;\n\t"
                        "@p add.u32 %0, %0, %3;\n\t}\n"
                        : "+r"(pw)
                        : "f"(dj), "f"(__uint_as_float(be.x)), "r"(1u << sh));
                }
            }
        }
        if (zero) {                                                   // all-zero block: indices 0
#pragma unroll
            for (int w = 0; w < BITS; ++w) packed[w] = 0u;
        }
        const int q = warp & 3;                                  // row group = TMEM lane quarter
        const bool leader = wg == 0 && lane == 0;
        if (QJL) {
            // the four blocks of a vector live in four warps: exchange radii (for one power-of-two scale
            // per vector) and squared residual norms through shared memory.  The row group meets at a
            // barrier, before which its leader makes sure the bulk store that last read the packed-tile
            // buffer is done.
            exch_d[row * WG + wg] = d_raw;
            exch_n[row * WG + wg] = en2;
            if (leader) bulk_wait_read();
            group_barrier(5u + q, 32u * WG);
        }
        {
            // 2 + 4*BITS bytes at a 2-byte aligned offset: whole words where the alignment allows
            uint8_t* ob = outs + row * VB + wg * BB;
            const uint32_t dbits = __half_as_ushort(d16);
            if ((wg * BB) & 2) {                    // warp-uniform
                *reinterpret_cast<uint16_t*>(ob) = (uint16_t)dbits;
#pragma unroll
                for (int w = 0; w < BITS; ++w) *reinterpret_cast<uint32_t*>(ob + 2 + 4 * w) = packed[w];
            } else {
                *reinterpret_cast<uint32_t*>(ob) = dbits | (packed[0] << 16);
#pragma unroll
                for (int w = 1; w < BITS; ++w)
                    *reinterpret_cast<uint32_t*>(ob + 4 * w) = __funnelshift_r(packed[w - 1], packed[w], 16);
                *reinterpret_cast<uint16_t*>(ob + 4 * BITS) = (uint16_t)(packed[BITS - 1] >> 16);
            }
        }
        int64_t slot = 0;                  // token slot of this thread's vector (padding rows: the last vector's)
        if (QJL) slot = slot_of(v0 + row < p.n_vec ? v0 + row : p.n_vec - 1);
        if (QJL) {
            // One power-of-two scale per vector keeps both residual terms inside the float16 range:
            // |e_j| < 2 * (largest block radius), scaled to below 2^15.
            float dmax = 0.f, n2 = 0.f;
#pragma unroll
            for (int k = 0; k < WG; ++k) {
                dmax = fmaxf(dmax, exch_d[row * WG + k]);
                n2 += exch_n[row * WG + k];
            }
            const uint32_t be = __float_as_uint(dmax) >> 23;
            const float es = be ? __uint_as_float((267u - be) << 23) : 1.0f;
            if (wg == 0 && row < n_valid)
                p.qjl_norm_out[slot] = __float2half_rn(fminf(sqrtf(n2) * (1.0f / 4096.0f), 65504.0f));
            uint32_t ehi[16], elo[16];
#pragma unroll
            const float2 es2 = make_float2(es, es), neg1 = make_float2(-1.f, -1.f);
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                const float2 a = mul2(v2[j >> 1], es2);
                const __half2 h = __floats2half2_rn(a.x, a.y);
                const float2 lo = fma2(__half22float2(h), neg1, a);          // exact: a - float(h)
                ehi[j >> 1] = *reinterpret_cast<const uint32_t*>(&h);
                elo[j >> 1] = pack_half2(lo.x, lo.y);
            }
            // the residual columns and the sketch accumulator are in use until the previous tile's
            // sketch MMAs have completed
            if (it >= 1) {
                ok = mbar_wait(sm_addr(mbar + 1), (it - 1u) & 1u, abort_s) && ok;
                tc_fence_after();
            }
            tmem_store16(tmem_lane + C::kEhiCol + wg * 16, ehi);
            tmem_store16(tmem_lane + C::kEloCol + wg * 16, elo);
            tmem_store_wait();
            if (it >= 1) store_signs(slot_prev, valid_prev);
            tc_fence_before();
            mbar_arrive(sm_addr(mbar + 6));
            slot_prev = slot;
            valid_prev = row < n_valid;
        }
        // ---- the warps that share 32 vectors (one per block) meet at their own barrier; its first
        // lane then sends the 32 packed vectors off with one bulk store.  No CTA-wide barrier.
        fence_async_smem();                  // the bulk store reads `outs` through the async proxy
        if (!QJL && leader) bulk_wait_read();        // the store that last read the other staging buffer is done
        // the barrier also votes: a wait that gave up anywhere in the CTA stops every group
        if (group_barrier_any(1u + q, 32u * WG, !ok || *abort_s != 0u)) {
            *abort_s = 1u;
            break;
        }
        const int rows = min(32, n_valid - 32 * q);
        if (rows > 0) {
            const int64_t g0 = v0 + 32 * q;
            const uint8_t* src = outs + 32 * q * VB;
            if (one_row) {
                uint8_t* dst = p.blocks_out + (position + g0) * VB;
                if (rows == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                    if (leader) bulk_store(dst, sm_addr(src), 32u * VB);
                } else {                                             // ragged end or odd token offset
                    for (int c = wg * 32 + lane; c < rows * VB / 4; c += 32 * WG)
                        reinterpret_cast<uint32_t*>(dst)[c] = reinterpret_cast<const uint32_t*>(src)[c];
                }
            } else {
                store_rows(g0, rows, src, lane, wg, leader);
            }
        }
    }
    if (QJL && ok && it >= 1 && !*abort_s) {             // the last tile's signs
        ok = mbar_wait(sm_addr(mbar + 1), (it - 1u) & 1u, abort_s) && ok;
        tc_fence_after();
        if (ok) store_signs(slot_prev, valid_prev);
    }
    if (wg == 0 && lane == 0) bulk_wait_all();
    if (!ok && lane == 0) atomicOr(&g_compress_error, 1u);
    }   // epilogue warps
    if (*abort_s && tid == 0) {          // give tile copies still in flight time to land
        const long long t0 = clock64();
        while (clock64() - t0 < (1ll << 20)) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, C::kTmemCols);
}

// Tensor map of x as a [n_vec][D] float16 matrix, boxes of 128 vectors x 64 halves, 128-byte swizzle.
// The encoder is a driver entry point, fetched through the runtime so the library links to cudart only.
static int make_x_map(const CompressParams& p, int D, CUtensorMap* map) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || !fn)
            return PQ_ERR_CUDA;
        encode = reinterpret_cast<encode_fn>(fn);
    }
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)p.n_vec};
    const cuuint64_t strides[1] = {(cuuint64_t)D * sizeof(__half)};
    const cuuint32_t box[2] = {64u, (cuuint32_t)kTileVecs};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(p.x), dims, strides, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? PQ_OK : PQ_ERR_CUDA;
}

template <int D, int BITS, bool QJL>
static int launch_compress(const CompressParams& p, cudaStream_t stream) {
    using C = CompressCfg<D, BITS, QJL>;
    static int sm_count = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return PQ_ERR_CUDA;
    if (sm_count == 0 && cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return PQ_ERR_CUDA;
    const size_t smem = C::smem_bytes();
    auto kern = pq_compress_kernel<D, BITS, QJL>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return PQ_ERR_CUDA;
    const int64_t n_tiles = (p.n_vec + kTileVecs - 1) / kTileVecs;
    // one CTA per SM: a CTA holds up to all 512 tensor-memory columns of its SM
    const int grid = (int)(n_tiles < sm_count ? n_tiles : sm_count);
    CUtensorMap x_map;
    memset(&x_map, 0, sizeof(x_map));
    const int st = make_x_map(p, D, &x_map);
    if (st != PQ_OK) return st;
    kern<<<grid, compress_launch_threads(D), smem, stream>>>(p, x_map);
    return cudaGetLastError() == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
}

}  // namespace pq


extern "C" int pq_poll_device_errors(unsigned int* flags_out) {
    if (!flags_out) return PQ_ERR_NULL_POINTER;
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, pq::g_compress_error, sizeof(v)) != cudaSuccess) return PQ_ERR_CUDA;
    if (v && cudaMemcpyToSymbol(pq::g_compress_error, &zero, sizeof(zero)) != cudaSuccess) return PQ_ERR_CUDA;
    unsigned int pf = 0;
    const int st = pq::prefill_error_flags(&pf);
    if (st != PQ_OK) return st;
    unsigned int df = 0;
    const int sd = pq::decode_error_flags(&df);
    if (sd != PQ_OK) return sd;
    unsigned int qf = 0;
    const int sq = pq::dequant_error_flags(&qf);
    if (sq != PQ_OK) return sq;
    unsigned int xf = 0;
    const int sx = pq::exchange_error_flags(&xf);
    if (sx != PQ_OK) return sx;
    *flags_out = v | pf | (df << 3) | (qf << 6) | (xf << 7);
    return PQ_OK;
}

// Shared body of pq_compress_rows (position on the host) and pq_compress_rows_dynamic (position in
// device memory, checked by the kernel).
static int compress_rows_impl(const void* x, int64_t n_rows, int64_t tokens_per_row, int64_t row_capacity,
                              int64_t position, const int64_t* position_dev, int head_dim, int n_bits,
                              const void* rot_split, const float* thresholds, const float* codebook,
                              void* blocks_out,
                              const void* jl_split, int jl_dim, void* qjl_bits_out, void* qjl_norm_out,
                              void* stream) {
    using namespace pq;
    if (n_rows < 0 || tokens_per_row < 0 || position < 0 || row_capacity < position + tokens_per_row)
        return PQ_ERR_BAD_SHAPE;
    if (position_dev != nullptr && (reinterpret_cast<uintptr_t>(position_dev) & 7)) return PQ_ERR_MISALIGNED;
    const int64_t n_vec = n_rows * tokens_per_row;
    if (n_vec > (int64_t)0x7FFFFF00) return PQ_ERR_TOO_LARGE;   // tile coordinates are 32-bit
    if (head_dim != 64 && head_dim != 128) return PQ_ERR_BAD_HEAD_DIM;
    if (n_bits != 2 && n_bits != 4) return PQ_ERR_BAD_BITS;
    if (n_vec == 0) return PQ_OK;
    if (!x || !rot_split || !thresholds || !codebook || !blocks_out) return PQ_ERR_NULL_POINTER;
    const bool qjl = jl_split != nullptr;
    if (qjl) {
        if (jl_dim < 16 || jl_dim > 128 || (jl_dim % 16)) return PQ_ERR_BAD_JL_DIM;
        if (!qjl_bits_out || !qjl_norm_out) return PQ_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(jl_split) & 15) return PQ_ERR_MISALIGNED;
        if (reinterpret_cast<uintptr_t>(qjl_norm_out) & 1) return PQ_ERR_MISALIGNED;
    }
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(rot_split) & 15) ||
        (reinterpret_cast<uintptr_t>(blocks_out) & 3))
        return PQ_ERR_MISALIGNED;

    CompressParams p{};
    p.x = static_cast<const __half*>(x);
    p.rot_split = static_cast<const __half*>(rot_split);
    p.jl_split = static_cast<const __half*>(jl_split);
    p.blocks_out = static_cast<uint8_t*>(blocks_out);
    p.qjl_bits_out = static_cast<uint8_t*>(qjl_bits_out);
    p.qjl_norm_out = static_cast<__half*>(qjl_norm_out);
    p.n_vec = n_vec;
    p.tokens_per_row = tokens_per_row;
    p.row_capacity = row_capacity;
    p.position = position;
    p.position_dev = position_dev;
    p.jl_dim = qjl ? jl_dim : 0;
    // thresholds / codebook are small HOST tables; they travel as kernel parameters.
    const int nlev = 1 << n_bits;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < 16; ++i) p.cb[i] = i < nlev ? codebook[i] : 0.f;
    // bucket(y), evaluated exactly as the kernel does (one fused multiply-add, then mantissa bits):
    // floor(64 y + 64) after rounding to 1/128
    for (int k = 0; k < 132; ++k) { p.bucket_t[k] = 3.0e38f; p.bucket_base[k] = 0; }
    for (int i = 0; i < nlev - 1; ++i) {
        const float u = fmaf(thresholds[i], 64.f, 98368.f);
        uint32_t bits;
        memcpy(&bits, &u, sizeof(bits));
        const int kb = (int)((bits >> 7) & 0xFFu);
        if (!(thresholds[i] > -1.0f && thresholds[i] < 1.0f) || kb > 130 || p.bucket_t[kb] != 3.0e38f)
            return PQ_ERR_BAD_SHAPE;      // thresholds out of range or two of them in one bucket
        p.bucket_t[kb] = thresholds[i];
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

extern "C" int pq_compress_rows(const void* x, int64_t n_rows, int64_t tokens_per_row, int64_t row_capacity,
                                int64_t position, int head_dim, int n_bits,
                                const void* rot_split, const float* thresholds, const float* codebook,
                                void* blocks_out,
                                const void* jl_split, int jl_dim, void* qjl_bits_out, void* qjl_norm_out,
                                void* stream) {
    return compress_rows_impl(x, n_rows, tokens_per_row, row_capacity, position, nullptr, head_dim, n_bits, rot_split,
                              thresholds, codebook, blocks_out, jl_split, jl_dim, qjl_bits_out, qjl_norm_out, stream);
}

extern "C" int pq_compress_rows_dynamic(const void* x, int64_t n_rows, int64_t tokens_per_row, int64_t row_capacity,
                                        const int64_t* position_dev, int head_dim, int n_bits,
                                        const void* rot_split, const float* thresholds, const float* codebook,
                                        void* blocks_out,
                                        const void* jl_split, int jl_dim, void* qjl_bits_out, void* qjl_norm_out,
                                        void* stream) {
    if (position_dev == nullptr) return PQ_ERR_NULL_POINTER;
    return compress_rows_impl(x, n_rows, tokens_per_row, row_capacity, 0, position_dev, head_dim, n_bits, rot_split,
                              thresholds, codebook, blocks_out, jl_split, jl_dim, qjl_bits_out, qjl_norm_out, stream);
}

extern "C" int pq_compress(const void* x, int64_t n_vec, int head_dim, int n_bits,
                           const void* rot_split, const float* thresholds, const float* codebook,
                           void* blocks_out,
                           const void* jl_split, int jl_dim, void* qjl_bits_out, void* qjl_norm_out,
                           void* stream) {
    if (n_vec < 0) return PQ_ERR_BAD_SHAPE;
    return pq_compress_rows(x, 1, n_vec, n_vec, 0, head_dim, n_bits, rot_split, thresholds, codebook, blocks_out,
                            jl_split, jl_dim, qjl_bits_out, qjl_norm_out, stream);
}
