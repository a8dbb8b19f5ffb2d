// pq_qjl_sketch: sign sketch of arbitrary residual vectors, signs = (P e >= 0) and ||e||, evaluated in
// float64 like the reference (python/polarquant_kv/qjl.py:25-35; bit order of
// src/polarquant_kv_cuda/qjl_kernel.py:87-92: bit k of byte j = sign[8j + k]).
//
// A checking utility beside the hot path: pq_compress produces the sketch of its own residual in-kernel
// on the tensor cores; this entry point serves callers that hold a residual of their own.  One thread
// per output byte (eight projections), float64 fused multiply-adds in the reference's summation order.
#include "pq_common.cuh"

namespace pq {

__global__ void pq_qjl_sketch_kernel(const float* __restrict__ e, const double* __restrict__ P, int64_t n, int d, int m,
                                     uint8_t* __restrict__ bits, float* __restrict__ norms) {
    const int m8 = (m + 7) / 8;
    const int64_t total = n * (int64_t)m8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = idx / m8;
        const int j = (int)(idx - v * m8);
        const float* ev = e + v * d;
        uint32_t byte = 0;
        for (int k = 0; k < 8 && 8 * j + k < m; ++k) {
            const double* row = P + (size_t)(8 * j + k) * d;
            double acc = 0.0;
            for (int i = 0; i < d; ++i) acc = fma(row[i], (double)ev[i], acc);
            byte |= (acc >= 0.0 ? 1u : 0u) << k;
        }
        bits[idx] = (uint8_t)byte;
        if (j == 0) {
            double s = 0.0;
            for (int i = 0; i < d; ++i) s = fma((double)ev[i], (double)ev[i], s);
            norms[v] = (float)sqrt(s);
        }
    }
}

}  // namespace pq

extern "C" int pq_qjl_sketch(const float* residual, const double* jl_matrix, int64_t n_vec, int dim, int jl_dim,
                             void* bits_out, float* norms_out, void* stream) {
    if (n_vec < 0 || dim <= 0 || jl_dim <= 0) return PQ_ERR_BAD_SHAPE;
    if (n_vec == 0) return PQ_OK;
    if (!residual || !jl_matrix || !bits_out || !norms_out) return PQ_ERR_NULL_POINTER;
    const int64_t total = n_vec * (int64_t)((jl_dim + 7) / 8);
    const int grid = (int)(total / 128 + 1 < 65535 ? total / 128 + 1 : 65535);
    pq::pq_qjl_sketch_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        residual, jl_matrix, n_vec, dim, jl_dim, static_cast<uint8_t*>(bits_out), norms_out);
    return cudaGetLastError() == cudaSuccess ? PQ_OK : PQ_ERR_CUDA;
}
