/*
 * polarquant_b200 — C ABI of the B200 (sm_100a) implementation of the PolarQuant-KV
 * block_pq4 hot path: compress, dequantise, decode attention, prefill attention and the
 * cross-GPU partial merge.
 *
 * Conventions (all entry points):
 *   - every pointer is a DEVICE pointer owned by the caller unless it says HOST
 *     (the small tables: thresholds and codebooks, at most 16 floats each, are read on
 *     the host during the call and travel to the kernel as launch parameters);
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call
 *     returns without synchronising; nothing is allocated or freed;
 *   - the return value is a pq_status; 0 is success; pq_strerror() names the others;
 *   - the device the pointers live on must be the current device.
 *
 * Storage layout ("block_pq4", README.md:73-78 of hilllief/polarquant-kv):
 *   a vector of head_dim elements is head_dim/32 consecutive blocks; one block is
 *       struct { __half d; uint8_t qs[32*n_bits/8]; }        18 bytes (4-bit), 10 (2-bit)
 *   d is the float16 Euclidean norm of the 32 rotated elements, qs holds the Lloyd-Max
 *   centroid indices: 4-bit  byte k = idx[2k] | idx[2k+1] << 4,
 *                     2-bit  byte k = idx[4k] | idx[4k+1] << 2 | idx[4k+2] << 4 | idx[4k+3] << 6
 *   (src/polarquant_kv_cuda/compress_kernel.py:34-50 of the reference).
 *   A cache tensor is uint8 [rows, seq, head_dim/32, block_bytes], rows = batch*kv_heads.
 *   QJL side band per key vector: jl_dim/8 sign bytes (bit k of byte j = sign[8j+k],
 *   src/polarquant_kv_cuda/qjl_kernel.py:87-92) and one float16 residual norm.
 *
 * The precedent for a C ABI on this path is the reference's llama.cpp bridge
 * (integration/polarquant-kv.patch, `polarquant_*_cuda_c`, lines 695-763 of the decoded
 * patch): raw device pointers, caller-owned buffers, stream as void*.
 */
#ifndef POLARQUANT_B200_H
#define POLARQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pq_status {
    PQ_OK = 0,
    PQ_ERR_NULL_POINTER = 1,     /* a required pointer is NULL                         */
    PQ_ERR_BAD_HEAD_DIM = 2,     /* head_dim is not 64 or 128                          */
    PQ_ERR_BAD_BITS = 3,         /* n_bits is not 2 or 4                               */
    PQ_ERR_BAD_SHAPE = 4,        /* negative size, q_heads not a multiple of kv_heads… */
    PQ_ERR_BAD_JL_DIM = 5,       /* jl_dim is not a multiple of 16 in [16, 128]        */
    PQ_ERR_MISALIGNED = 6,       /* a buffer does not have the required alignment      */
    PQ_ERR_SCRATCH_TOO_SMALL = 7,/* scratch_bytes is below pq_decode_attn_scratch_bytes */
    PQ_ERR_CUDA = 8,             /* a CUDA runtime call failed (launch error, …)       */
    PQ_ERR_TOO_LARGE = 9,        /* a size exceeds what the entry point supports       */
    PQ_ERR_STATIC_SCRATCH_EXCEEDED = 10 /* pq_decode_attn_static: the shape needs more scratch
                                           than the library's built-in array holds           */
} pq_status;

/* Library version: major*10000 + minor*100 + patch. */
int pq_version(void);

/* Static string for a pq_status value (never NULL). */
const char* pq_strerror(int status);

/* ---------------------------------------------------------------------------------
 * pq_compress — fused rotate + per-32 radius + nearest-centroid + pack [+ QJL sketch].
 *
 * Replaces, on the block_pq4 layout: polarquant_kv.quantizer.compress / compress_batch
 * (python/polarquant_kv/quantizer.py:88-134, 161-195), compress_gpu
 * (src/polarquant_kv_cuda/compress_kernel.py:100-189), turboquant_compress_kernel
 * (csrc/flash_turboquant.cu:111-175) and polarquant_compress_cuda_c (patch:695-763);
 * with jl_split != NULL also compute_signatures_gpu (src/polarquant_kv_cuda/qjl_kernel.py:6-37).
 *
 *   x           float16 [n_vec, head_dim], 16-byte aligned
 *   rot_split   float16 [head_dim, 2*head_dim]: row i = [hi(4096*R[i,:]) | lo(4096*R[i,:])],
 *               the two-term float16 split of the rotation (R as used by v @ R^T);
 *               built by the host helper polarquant_kv.rotation.split_for_device
 *   thresholds  HOST float32 [2^n_bits - 1]: index = number of thresholds strictly below the
 *               normalised coordinate; exact decision points of argmin|v - c_i| in float32
 *   codebook    HOST float32 [2^n_bits] centroids (used for the QJL residual only)
 *   blocks_out  uint8 [n_vec, head_dim/32, block_bytes], 4-byte aligned (16-byte aligned is faster)
 *   jl_split    float16 [jl_dim, 2*head_dim] split of 1024*(P @ R^T), or NULL for no sketch;
 *               jl_dim a multiple of 16 in [16, 128]
 *   qjl_bits_out  uint8 [n_vec, jl_dim/8]      (required when jl_split != NULL)
 *   qjl_norm_out  float16 [n_vec]              (required when jl_split != NULL)
 */
int pq_compress(const void* x, int64_t n_vec, int head_dim, int n_bits,
                const void* rot_split, const float* thresholds, const float* codebook,
                void* blocks_out,
                const void* jl_split, int jl_dim, void* qjl_bits_out, void* qjl_norm_out,
                void* stream);

/* ---------------------------------------------------------------------------------
 * pq_compress_rows — pq_compress that writes into preallocated cache tensors in ONE launch:
 * the input holds n_rows x tokens_per_row vectors ([batch*heads, new tokens, head_dim]); vector
 * (r, t) lands in token slot r * row_capacity + position + t of blocks_out (and of the sketch
 * outputs), i.e. at sequence offset `position` of row r of a cache whose rows hold row_capacity
 * tokens.  This is the append-on-write step of a decode loop (one new token for every
 * (batch, head) row in one launch) and of a prefill (all prompt tokens of all rows at once).
 *
 * Replaces KVCacheManager.append's compress-then-concatenate
 * (src/polarquant_kv_cuda/inference/kv_cache.py:68-116) and the per-(head, token) compress calls
 * of the ggml dispatch (integration/polarquant-kv.patch, decoded lines 802-835).
 * Other arguments as pq_compress.  Requires position + tokens_per_row <= row_capacity.
 */
int pq_compress_rows(const void* x, int64_t n_rows, int64_t tokens_per_row, int64_t row_capacity,
                     int64_t position, int head_dim, int n_bits,
                     const void* rot_split, const float* thresholds, const float* codebook,
                     void* blocks_out,
                     const void* jl_split, int jl_dim, void* qjl_bits_out, void* qjl_norm_out,
                     void* stream);

/* pq_compress_rows_dynamic — pq_compress_rows with the sequence offset read from DEVICE memory when
 * the kernel starts (*position_dev, int64, 8-byte aligned), for a decode step recorded once as a CUDA
 * graph and replayed while the position advances on the device.  The host cannot check the offset:
 * when position + tokens_per_row exceeds row_capacity (or position < 0) the kernel writes nothing and
 * sets bit 5 of pq_poll_device_errors.  No counterpart in the reference (its append concatenates on
 * the host, src/polarquant_kv_cuda/inference/kv_cache.py:93-116). */
int pq_compress_rows_dynamic(const void* x, int64_t n_rows, int64_t tokens_per_row, int64_t row_capacity,
                             const int64_t* position_dev, int head_dim, int n_bits,
                             const void* rot_split, const float* thresholds, const float* codebook,
                             void* blocks_out,
                             const void* jl_split, int jl_dim, void* qjl_bits_out, void* qjl_norm_out,
                             void* stream);

/* pq_poll_device_errors — HOST-synchronising check for device-side failures of earlier launches on
 * the current device.  The tensor-core kernels wait for copies and MMAs through barriers with a time
 * limit (so that a lost completion can never hang the GPU); if a wait ever gives up a bit of
 * *flags_out is set and the output of that launch must be discarded: bit 0 compress (a wait gave
 * up), bit 1 compress (shared-memory window unusable), bit 2 prefill attention (a wait gave up),
 * bit 3 decode attention (shared-memory window unusable, nothing computed), bit 4 decode attention (a
 * wait for a tile copy gave up), bit 5 compress (pq_compress_rows_dynamic found its device-side
 * position out of range; nothing was written), bit 6 dequantise (a wait gave up), bit 7
 * pq_lse_exchange_merge (a peer's records did not arrive within about two seconds; the output rows of the
 * waiting CTAs are left unwritten).
 * The flags are cleared by the call.  No counterpart in the reference (its kernels report nothing). */
int pq_poll_device_errors(unsigned int* flags_out);

/* ---------------------------------------------------------------------------------
 * pq_qjl_sketch — sign sketch of caller-provided residual vectors: bits = (P e >= 0), norms = ||e||,
 * evaluated in float64.  Replaces qjl.compute_signatures (python/polarquant_kv/qjl.py:25-35) and
 * compute_signatures_gpu (src/polarquant_kv_cuda/qjl_kernel.py:6-37) for residuals that do not come from
 * pq_compress (which sketches its own residual in-kernel).
 *
 *   residual   float32 [n_vec, dim]
 *   jl_matrix  float64 [jl_dim, dim] row-major P (device memory)
 *   bits_out   uint8 [n_vec, ceil(jl_dim/8)], bit k of byte j = sign[8j + k]
 *   norms_out  float32 [n_vec]
 */
int pq_qjl_sketch(const float* residual, const double* jl_matrix, int64_t n_vec, int dim, int jl_dim,
                  void* bits_out, float* norms_out, void* stream);

/* ---------------------------------------------------------------------------------
 * pq_dequant — blocks -> centroid * d -> inverse rotation (v @ R).
 *
 * Replaces quantizer.decompress / decompress_batch (python/polarquant_kv/quantizer.py:137-158,
 * 198-219), decompress_gpu (src/polarquant_kv_cuda/decompress_kernel.py:10-51),
 * batch_dequant_4bit (src/polarquant_kv_cuda/fused_cuda_kernels.py:405-435).
 *
 *   blocks     uint8 [n_vec, head_dim/32, block_bytes]
 *   codebook   HOST float32 [2^n_bits]
 *   rot        float32 [head_dim, head_dim] row-major R
 *   out        [n_vec, head_dim], float32 (out_is_fp16 == 0) or float16 clamped to +-65504; 32-byte aligned (blocks: 16-byte aligned)
 */
int pq_dequant(const void* blocks, int64_t n_vec, int head_dim, int n_bits,
               const float* codebook, const float* rot, void* out, int out_is_fp16,
               void* stream);

/* ---------------------------------------------------------------------------------
 * pq_decode_attn — one query token per sequence against the compressed cache (GQA).
 *
 * Replaces attention.compressed_attention for seq_q == 1
 * (python/polarquant_kv/attention.py:83-191), compressed_attention_gpu
 * (src/polarquant_kv_cuda/attention_kernel.py:11-113), turboquant_attention_kernel
 * (csrc/flash_turboquant.cu:27-105), rotate_query/inverse_rotate kernels
 * (csrc/polarquant_full.cu:25-40, 125-140) and polarquant_fused_attention_cuda_c.
 * Non-causal, as the reference.  The query is rotated once inside the kernel, only
 * packed blocks are read, the work is cut into segments whose (m, l, o) partials are
 * merged by the last CTA to finish a row, and the result is rotated back.
 *
 *   q          float16 [batch, q_heads, head_dim]
 *   k_blocks   uint8 [batch*kv_heads, seq_capacity, head_dim/32, block_bytes(k_bits)]
 *   v_blocks   uint8 [batch*kv_heads, seq_capacity, head_dim/32, block_bytes(v_bits)]
 *   seq_len    tokens to attend to (<= seq_capacity); 0 gives an all-zero output
 *   codebook_k/codebook_v  HOST float32 [2^bits]
 *   rot        float32 [head_dim, head_dim] row-major R
 *   scale      softmax scale (1/sqrt(head_dim) in the reference)
 *   jl_matrix  NULL, or the JL matrix for the QJL score correction: float32
 *              [jl_dim, head_dim] row-major P (scores += corr * scale,
 *              attention.py:150-155); then qjl_bits [rows, seq_capacity, jl_dim/8] and
 *              qjl_norms float16 [rows, seq_capacity] are required, both 16-byte aligned
 *              (PQ_ERR_MISALIGNED otherwise), jl_dim a multiple of 16 in [16, 128]
 *   out        [batch, q_heads, head_dim] float32 (out_is_fp16 == 0) or float16
 *   partial_out NULL, or float32 [batch, q_heads, head_dim + 2]: when given, the kernel
 *              skips the final normalisation and inverse rotation and writes
 *              (m, l, o_rotated[head_dim]) per query head instead of `out`
 *              (m in log2 units) — the per-GPU partial of a sequence-sharded decode
 *   n_splits   0 (recommended): all 16-token tiles of all rows form one sequence that is
 *              cut into one equal contiguous range per SM; >= 1: that many equal
 *              sequence ranges per (batch, kv head, head group), dealt to the SMs
 *   scratch    device buffer of at least pq_decode_attn_scratch_bytes(...) bytes,
 *              256-byte aligned, ZERO-FILLED before its first use.  It starts with one
 *              32-bit counter per (batch, kv head, head group), at most batch * q_heads of
 *              them, followed (on the next 256-byte boundary) by the segment records.  The
 *              kernel leaves its counters at zero again, so later calls with the SAME batch,
 *              q_heads and kv_heads on the same stream reuse the buffer as it is; before a
 *              call with another batch or other head counts clear the first
 *              4 * batch * q_heads bytes (rounded up to 256) again, because the records of
 *              a call with fewer counters lie where a larger call keeps its counters
 *              (concurrent calls need separate scratch buffers)
 */
int pq_decode_attn(const void* q, const void* k_blocks, const void* v_blocks,
                   int batch, int q_heads, int kv_heads, int64_t seq_len, int64_t seq_capacity,
                   int head_dim, int k_bits, int v_bits,
                   const float* codebook_k, const float* codebook_v, const float* rot, float scale,
                   const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                   void* out, int out_is_fp16, void* partial_out,
                   int n_splits, void* scratch, size_t scratch_bytes, void* stream);

/* Bytes of scratch pq_decode_attn needs for this shape (n_splits == 0: library default). */
size_t pq_decode_attn_scratch_bytes(int batch, int q_heads, int kv_heads, int64_t seq_len,
                                    int head_dim, int n_splits);

/* The number of splits the library would choose for n_splits == 0 on the current device. */
int pq_decode_attn_default_splits(int batch, int q_heads, int kv_heads, int64_t seq_len, int head_dim);

/* ---------------------------------------------------------------------------------
 * pq_decode_attn_static — pq_decode_attn for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference.  It exists for hosts that have
 * no way to provide the `scratch` buffer of pq_decode_attn: an operator callback inside an
 * inference runtime that owns all device memory and passes the operator nothing but its
 * input and output tensors, code that runs while the device allocator is frozen, or a
 * serving loop that must not risk the device-wide stall of a cudaMalloc.  The split-merge
 * scratch lives in an array built into the library instead (8 MiB of device memory on
 * every GPU that loads the library, held until the process exits; its size is returned by
 * pq_decode_attn_static_scratch_capacity()).
 *
 * Arguments and results are those of pq_decode_attn without `scratch`/`scratch_bytes`.
 * It calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - A shape whose scratch need (pq_decode_attn_scratch_bytes) exceeds the capacity is
 *     rejected with PQ_ERR_STATIC_SCRATCH_EXCEEDED; nothing is launched.  Fewer splits
 *     (`n_splits`) need less scratch.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current).  Make that first call outside any
 *     stream capture.
 *   - All calls on a device share the one array, and it keeps the previous call's
 *     contents; the entry point re-zeroes the part that must start at zero (the ticket
 *     counters) on `stream` before each launch.  Two calls that overlap on the GPU (other
 *     streams, other host threads) would race on the array: serialise them, or use
 *     pq_decode_attn with separate scratch buffers.
 */
int pq_decode_attn_static(const void* q, const void* k_blocks, const void* v_blocks,
                          int batch, int q_heads, int kv_heads, int64_t seq_len, int64_t seq_capacity,
                          int head_dim, int k_bits, int v_bits,
                          const float* codebook_k, const float* codebook_v, const float* rot, float scale,
                          const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                          void* out, int out_is_fp16, void* partial_out,
                          int n_splits, void* stream);

/* pq_decode_attn_dynamic — pq_decode_attn with the sequence length read from DEVICE memory when the
 * kernel starts (*seq_len_dev, int64, 8-byte aligned), clamped to [0, max_seq_len]; max_seq_len (>= 1,
 * <= seq_capacity) is the length the work partition and the scratch are made for
 * (pq_decode_attn_scratch_bytes with max_seq_len).  One recorded launch serves every length up to
 * max_seq_len.  No counterpart in the reference. */
int pq_decode_attn_dynamic(const void* q, const void* k_blocks, const void* v_blocks,
                           int batch, int q_heads, int kv_heads, int64_t max_seq_len,
                           const int64_t* seq_len_dev, int64_t seq_capacity,
                           int head_dim, int k_bits, int v_bits,
                           const float* codebook_k, const float* codebook_v, const float* rot, float scale,
                           const float* jl_matrix, int jl_dim, const void* qjl_bits, const void* qjl_norms,
                           void* out, int out_is_fp16, void* partial_out,
                           int n_splits, void* scratch, size_t scratch_bytes, void* stream);

/* Bytes of the built-in scratch array pq_decode_attn_static can use. */
size_t pq_decode_attn_static_scratch_capacity(void);

/* ---------------------------------------------------------------------------------
 * pq_lse_merge — merge per-GPU (m, l, o_rotated) partials of a sequence-sharded decode
 * (after an all-gather) and rotate back.  No counterpart in the reference, which has no
 * multi-GPU path; it completes pq_decode_attn(partial_out=...) for the long-context case.
 *
 *   partials   float32 [n_parts, n_rows, head_dim + 2] as written through partial_out
 *   out        [n_rows, head_dim] float32 or float16
 */
int pq_lse_merge(const float* partials, int n_parts, int64_t n_rows, int head_dim,
                 const float* rot, void* out, int out_is_fp16, void* stream);

/* ---------------------------------------------------------------------------------
 * pq_lse_exchange_merge — the all-gather of the partial records and pq_lse_merge as ONE kernel over
 * peer memory (GPUs of one node that can address each other: NVLink / NVSwitch peer mappings).  No
 * counterpart in the reference.
 *
 *   peer_buffers  HOST array of `world` device pointers: entry s is rank s's exchange buffer as THIS
 *                 process addresses it (its own entry is a local allocation); every buffer has
 *                 pq_lse_exchange_bytes(world, n_rows, head_dim) bytes, is 128-byte aligned and was
 *                 zeroed once before the first call (all ranks, then a host barrier)
 *   epoch         1 for the first call on these buffers, then 2, 3, ... on every rank alike
 *   local_partial this rank's records [n_rows, head_dim + 2] as written through partial_out
 *
 * Every rank enqueues the call once per step; a rank's kernel stores its records into the peers'
 * buffers, counts itself in, waits (bounded, about two seconds -> bit 7 of pq_poll_device_errors) for
 * the peers' records and merges.  At most `world` = 8 ranks.  Plain peer stores and system-scope
 * atomics; no multicast. */
size_t pq_lse_exchange_bytes(int world, int64_t n_rows, int head_dim);
int pq_lse_exchange_merge(const float* local_partial, int world, int rank, void* const* peer_buffers,
                          uint64_t epoch, int64_t n_rows, int head_dim, const float* rot,
                          void* out, int out_is_fp16, void* stream);

/* ---------------------------------------------------------------------------------
 * pq_prefill_attn — seq_q >= 1 query tokens per head against the compressed cache:
 * K/V tiles are dequantised into shared memory and contracted on the tensor cores
 * (tcgen05.mma, accumulators in tensor memory).  Its bounded waits report through bit 2
 * of pq_poll_device_errors.
 *
 * Replaces attention.compressed_attention for seq_q > 1 and compressed_attention_gpu's
 * dequantise-everything path (src/polarquant_kv_cuda/attention_kernel.py:70-113).
 *
 *   q          float16 [batch, q_heads, seq_q, head_dim], 16-byte aligned
 *   causal     0: every query sees all seq_len tokens (the reference's behaviour);
 *              1: query i sees tokens [0, seq_len - seq_q + i]
 *   out        [batch, q_heads, seq_q, head_dim] float32 (16-byte aligned) or float16
 *   workspace  NULL, or a 16-byte aligned device buffer of at least
 *              pq_prefill_attn_workspace_bytes(...) bytes (1 KB per token and KV head at
 *              head_dim 128).  With a workspace every K/V tile is expanded once by a first
 *              kernel and the attention kernel streams the expanded tiles (faster when
 *              several 128-row query tiles share a KV head: seq_q * q_heads/kv_heads > 128);
 *              without it the attention kernel dequantises the tiles itself.  Contents need
 *              no initialisation and mean nothing after the call.
 */
int pq_prefill_attn(const void* q, const void* k_blocks, const void* v_blocks,
                    int batch, int q_heads, int kv_heads, int seq_q, int64_t seq_len,
                    int64_t seq_capacity, int head_dim, int k_bits, int v_bits,
                    const float* codebook_k, const float* codebook_v, const float* rot,
                    float scale, int causal, void* out, int out_is_fp16,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of workspace pq_prefill_attn can use for this shape (0 for an empty shape). */
size_t pq_prefill_attn_workspace_bytes(int batch, int kv_heads, int64_t seq_len, int head_dim);

#ifdef __cplusplus
}
#endif
#endif /* POLARQUANT_B200_H */
