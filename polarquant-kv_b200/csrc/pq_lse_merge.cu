// pq_lse_merge, pq_version, pq_strerror.
//
// pq_lse_merge combines the per-GPU partials of a sequence-sharded decode: every rank ran
// pq_decode_attn(partial_out=...) on its slice of the sequence and the ranks all-gathered
// the [rows, D+2] records (m in log2 units, l, o in rotated space).  The merge is the usual
// log-sum-exp combination followed by the inverse rotation o @ R.  Parts with l == 0 (an
// empty slice) carry no weight and are ignored when the running maximum is taken.
#include "pq_common.cuh"

namespace pq {

// One CTA per output row, D threads (thread i = output dim i).  The records of the parts are fetched eight
// at a time with independent loads (one round trip to L2 for up to eight GPUs), and the inverse rotation
// keeps 32 matrix loads in flight over four accumulators: the kernel is all latency, so what matters is how
// few dependent round trips a row makes.
template <int D>
__global__ void __launch_bounds__(D) pq_lse_merge_kernel(const float* __restrict__ parts, int n_parts,
                                                         int64_t n_rows, const float* __restrict__ rot,
                                                         void* out, int out_is_fp16) {
    __shared__ float o_s[D];
    const int i = threadIdx.x;
    for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
        float mx = -INFINITY, l = 0.f, o = 0.f;
        for (int s0 = 0; s0 < n_parts; s0 += 8) {
            float ms[8], ls[8], os[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int s = min(s0 + u, n_parts - 1);
                const float* r = parts + ((size_t)s * n_rows + row) * (D + 2);
                ms[u] = __ldg(r);
                ls[u] = __ldg(r + 1);
                os[u] = __ldg(r + 2 + i);
            }
            float m_new = mx;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (s0 + u >= n_parts || !(ls[u] > 0.f)) { ls[u] = 0.f; ms[u] = -INFINITY; }   // empty slices carry no weight
                m_new = fmaxf(m_new, ms[u]);
            }
            const float c = (mx == -INFINITY) ? 0.f : fast_exp2(mx - m_new);
            l *= c;
            o *= c;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float sc = (ms[u] == -INFINITY) ? 0.f : fast_exp2(ms[u] - m_new);
                l = fmaf(sc, ls[u], l);
                o = fmaf(sc, os[u], o);
            }
            mx = m_new;
        }
        __syncthreads();
        o_s[i] = l > 0.f ? o / l : 0.f;
        __syncthreads();
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j0 = 0; j0 < D; j0 += 32) {
            float r[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) r[u] = __ldg(rot + (size_t)(j0 + u) * D + i);
#pragma unroll
            for (int u = 0; u < 32; ++u) acc[u & 3] = fmaf(o_s[j0 + u], r[u], acc[u & 3]);
        }
        const float res = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        if (out_is_fp16)
            static_cast<__half*>(out)[row * D + i] = __float2half_rn(fminf(fmaxf(res, -65504.f), 65504.f));
        else
            static_cast<float*>(out)[row * D + i] = res;
    }
}

}  // namespace pq

extern "C" int pq_lse_merge(const float* partials, int n_parts, int64_t n_rows, int head_dim,
                            const float* rot, void* out, int out_is_fp16, void* stream) {
    if (n_parts <= 0 || n_rows < 0) return PQ_ERR_BAD_SHAPE;
    if (head_dim != 64 && head_dim != 128) return PQ_ERR_BAD_HEAD_DIM;
    if (n_rows == 0) return PQ_OK;
    if (!partials || !rot || !out) return PQ_ERR_NULL_POINTER;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = (int)(n_rows < 4096 ? n_rows : 4096);
    if (head_dim == 64)
        pq::pq_lse_merge_kernel<64><<<grid, 64, 0, st>>>(partials, n_parts, n_rows, rot, out, out_is_fp16);
    else
        pq::pq_lse_merge_kernel<128><<<grid, 128, 0, st>>>(partials, n_parts, n_rows, rot, out, out_is_fp16);
    return cudaGetLastError() == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
}

extern "C" int pq_version(void) { return 100; }   // 0.1.0

extern "C" const char* pq_strerror(int status) {
    switch (status) {
        case PQ_OK: return "ok";
        case PQ_ERR_NULL_POINTER: return "a required pointer is NULL";
        case PQ_ERR_BAD_HEAD_DIM: return "head_dim must be 64 or 128";
        case PQ_ERR_BAD_BITS: return "n_bits must be 2 or 4";
        case PQ_ERR_BAD_SHAPE: return "invalid shape argument";
        case PQ_ERR_BAD_JL_DIM: return "jl_dim must be a multiple of 16 in [16, 128]";
        case PQ_ERR_MISALIGNED: return "a buffer is not aligned as required";
        case PQ_ERR_SCRATCH_TOO_SMALL: return "scratch buffer is smaller than pq_decode_attn_scratch_bytes()";
        case PQ_ERR_CUDA: return "a CUDA runtime call failed";
        case PQ_ERR_TOO_LARGE: return "a size exceeds what this entry point supports";
        case PQ_ERR_STATIC_SCRATCH_EXCEEDED:
            return "this shape needs more scratch than the library's built-in array holds (8 MiB); "
                   "use fewer splits or pq_decode_attn with a caller-provided buffer";
        default: return "unknown pq_status";
    }
}
