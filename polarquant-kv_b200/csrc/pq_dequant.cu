// pq_dequant: stored block_pq4 blocks -> centroid[idx] * float(d) (rotated space) ->
// inverse rotation v @ R -> float32 or float16.
//
// Follows dequantize_with_codebook (src/polarquant_kv_cuda/lloyd_max.py:93-98), the radius
// restore of quantizer.decompress (python/polarquant_kv/quantizer.py:151) and
// inverse_rotate (python/polarquant_kv/rotation.py:61); the float16 output is clamped to
// +-65504 like decompress_gpu (src/polarquant_kv_cuda/decompress_kernel.py:47-51).
//
// One CTA of D threads owns 16 vectors at a time; thread i produces output dim i of all 16.
// R (float32, D x D) stays in shared memory, the 16 dequantised vectors are staged
// transposed so a step of the contraction is one conflict-free R read plus broadcasts.
#include "pq_common.cuh"

namespace pq {

constexpr int kDqVecs = 16;

struct DequantParams {
    const uint8_t* blocks;
    const float* rot;
    void* out;
    int64_t n_vec;
    int out_is_fp16;
    float cb[16];
};

template <int D, int BITS>
__global__ void __launch_bounds__(D) pq_dequant_kernel(const DequantParams p) {
    constexpr int NBLK = D / 32;
    constexpr int BB = block_bytes(BITS);
    constexpr int VB = NBLK * BB;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* Rs = reinterpret_cast<float*>(smem_raw);            // [D][D]
    float* dq = Rs + D * D;                                    // [D][16]  (transposed)
    uint8_t* raw = reinterpret_cast<uint8_t*>(dq + D * kDqVecs);  // [16][VB]
    __shared__ float cb_s[16];

    const int tid = threadIdx.x;
    for (int c = tid; c < D * D / 4; c += D)
        reinterpret_cast<float4*>(Rs)[c] = reinterpret_cast<const float4*>(p.rot)[c];
    if (tid < 16) cb_s[tid] = p.cb[tid];

    const int64_t n_tiles = (p.n_vec + kDqVecs - 1) / kDqVecs;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t v0 = tile * kDqVecs;
        const int n_valid = (int)((p.n_vec - v0) < kDqVecs ? (p.n_vec - v0) : kDqVecs);
        __syncthreads();
        // stored bytes of the tile (4-byte granules: VB is a multiple of 4)
        {
            const uint32_t* src = reinterpret_cast<const uint32_t*>(p.blocks + v0 * VB);
            const int n4 = n_valid * VB / 4;
            for (int c = tid; c < kDqVecs * VB / 4; c += D)
                reinterpret_cast<uint32_t*>(raw)[c] = c < n4 ? src[c] : 0u;
        }
        __syncthreads();
        // dequantise: thread j handles element j of every vector
        {
            const int j = tid, blk = j / 32, e = j % 32;
#pragma unroll
            for (int v = 0; v < kDqVecs; ++v) {
                const uint8_t* b = raw + v * VB + blk * BB;
                const float d = __half2float(*reinterpret_cast<const __half*>(b));
                uint32_t idx;
                if (BITS == 4) idx = (b[2 + e / 2] >> ((e & 1) * 4)) & 0xF;
                else           idx = (b[2 + e / 4] >> ((e & 3) * 2)) & 0x3;
                dq[j * kDqVecs + v] = __fmul_rn(cb_s[idx], d);
            }
        }
        __syncthreads();
        float acc[kDqVecs];
#pragma unroll
        for (int v = 0; v < kDqVecs; ++v) acc[v] = 0.f;
        for (int j = 0; j < D; ++j) {
            const float r = Rs[j * D + tid];
            const float4* row = reinterpret_cast<const float4*>(dq + j * kDqVecs);
#pragma unroll
            for (int q4 = 0; q4 < kDqVecs / 4; ++q4) {
                const float4 x = row[q4];
                acc[q4 * 4 + 0] = fmaf(x.x, r, acc[q4 * 4 + 0]);
                acc[q4 * 4 + 1] = fmaf(x.y, r, acc[q4 * 4 + 1]);
                acc[q4 * 4 + 2] = fmaf(x.z, r, acc[q4 * 4 + 2]);
                acc[q4 * 4 + 3] = fmaf(x.w, r, acc[q4 * 4 + 3]);
            }
        }
#pragma unroll
        for (int v = 0; v < kDqVecs; ++v) {
            if (v < n_valid) {
                if (p.out_is_fp16) {
                    float c = fminf(fmaxf(acc[v], -65504.0f), 65504.0f);
                    static_cast<__half*>(p.out)[(v0 + v) * D + tid] = __float2half_rn(c);
                } else {
                    static_cast<float*>(p.out)[(v0 + v) * D + tid] = acc[v];
                }
            }
        }
    }
}

template <int D, int BITS>
static int launch_dequant(const DequantParams& p, cudaStream_t st) {
    const size_t smem = (size_t)D * D * 4 + (size_t)D * kDqVecs * 4 + (size_t)kDqVecs * (D / 32) * block_bytes(BITS);
    auto kern = pq_dequant_kernel<D, BITS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return PQ_ERR_CUDA;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return PQ_ERR_CUDA;
    const int64_t n_tiles = (p.n_vec + kDqVecs - 1) / kDqVecs;
    const int64_t cap = (int64_t)sms * (D == 128 ? 2 : 8);
    const int grid = (int)(n_tiles < cap ? n_tiles : cap);
    kern<<<grid, D, smem, st>>>(p);
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
    if ((reinterpret_cast<uintptr_t>(blocks) & 3) || (reinterpret_cast<uintptr_t>(rot) & 15))
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
