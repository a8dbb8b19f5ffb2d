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

// ---------------------------------------------------------------------------------------------
// pq_lse_exchange_merge: the all-gather of the partial records and their merge as ONE kernel over
// peer memory.  Every rank owns a receive buffer [2][world][rows][D + 2] and `world` arrival counters
// that its peers can address (NVLink peer mapping).  A CTA (one output row at a time)
//   1. stores its row of the local partial record into every peer's receive buffer (slot of this
//      rank, half `epoch & 1`), makes the stores visible system-wide and adds one to the peer's
//      counter for this rank;
//   2. waits until every peer's counter on THIS rank has reached rows * epoch (all rows of that peer
//      for this call have landed; counters only grow, the two halves alternate, and a peer cannot be
//      two calls ahead because each call needs this rank's records of the call before) - with a time
//      limit, after which an error flag is set and the row is left unwritten;
//   3. merges the world records of the row (its own from local memory, the others from the receive
//      buffer, read past L1) and applies the inverse rotation, as pq_lse_merge does.
// Plain peer stores and system-scope atomics only: no multicast, no collective library call.
constexpr int kMaxPeers = 8;

static __device__ unsigned int g_exchange_error = 0;      // bit 0: a wait for a peer's records gave up

struct ExchangeParams {
    const float* local;                         // [rows][D + 2]
    float* recv[kMaxPeers];                     // every rank's receive buffer (own entry = local address)
    unsigned long long* arrived[kMaxPeers];     // every rank's counters [world]
    int world, rank;
    unsigned long long epoch;                   // 1, 2, 3, ... (the same on every rank)
    long long n_rows;
    const float* rot;
    void* out;
    int out_is_fp16;
};

template <int D>
__global__ void __launch_bounds__(D) pq_lse_exchange_merge_kernel(const ExchangeParams p) {
    __shared__ float o_s[D];
    __shared__ int s_ok;
    const int i = threadIdx.x;
    const size_t half = (size_t)(p.epoch & 1ull) * p.world * p.n_rows * (D + 2);
    // ---- 1. this CTA's rows to every peer
    for (long long row = blockIdx.x; row < p.n_rows; row += gridDim.x) {
        const float* src = p.local + row * (D + 2);
        const float a = src[i], b = i < 2 ? src[D + i] : 0.f;
        for (int s = 0; s < p.world; ++s) {
            if (s == p.rank) continue;
            float* dst = p.recv[s] + half + ((size_t)p.rank * p.n_rows + row) * (D + 2);
            dst[i] = a;
            if (i < 2) dst[D + i] = b;
        }
        __threadfence_system();
        __syncthreads();
        if (i == 0)
            for (int s = 0; s < p.world; ++s)
                if (s != p.rank) atomicAdd_system(p.arrived[s] + p.rank, 1ull);
    }
    // ---- 2. every peer's rows of this call have arrived here
    if (i == 0) {
        const unsigned long long target = (unsigned long long)p.n_rows * p.epoch;
        int ok = 1;
        const long long t0 = clock64();
        for (int s = 0; s < p.world && ok; ++s) {
            if (s == p.rank) continue;
            const unsigned long long* flag = p.arrived[p.rank] + s;
            for (;;) {
                unsigned long long v;
                asm volatile("ld.acquire.sys.global.u64 %0, [%1];\n" : "=l"(v) : "l"(flag) : "memory");
                if (v >= target) break;
                if (clock64() - t0 > (1ll << 32)) {          // about two seconds
                    ok = 0;
                    atomicOr(&g_exchange_error, 1u);
                    break;
                }
                __nanosleep(100);
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    // ---- 3. merge and rotate back
    const float* mine = p.recv[p.rank] + half;
    for (long long row = blockIdx.x; row < p.n_rows; row += gridDim.x) {
        float ms[kMaxPeers], ls[kMaxPeers], os[kMaxPeers];
#pragma unroll
        for (int s = 0; s < kMaxPeers; ++s) {
            const int ss = min(s, p.world - 1);
            const float* r = ss == p.rank ? p.local + row * (D + 2) : mine + ((size_t)ss * p.n_rows + row) * (D + 2);
            ms[s] = __ldcg(r);
            ls[s] = __ldcg(r + 1);
            os[s] = __ldcg(r + 2 + i);
        }
        float mx = -INFINITY;
#pragma unroll
        for (int s = 0; s < kMaxPeers; ++s) {
            if (s >= p.world || !(ls[s] > 0.f)) { ls[s] = 0.f; ms[s] = -INFINITY; }      // empty slices carry no weight
            mx = fmaxf(mx, ms[s]);
        }
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int s = 0; s < kMaxPeers; ++s) {
            const float sc = (ms[s] == -INFINITY) ? 0.f : fast_exp2(ms[s] - mx);
            l = fmaf(sc, ls[s], l);
            o = fmaf(sc, os[s], o);
        }
        __syncthreads();
        o_s[i] = l > 0.f ? o / l : 0.f;
        __syncthreads();
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j0 = 0; j0 < D; j0 += 32) {
            float r[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) r[u] = __ldg(p.rot + (size_t)(j0 + u) * D + i);
#pragma unroll
            for (int u = 0; u < 32; ++u) acc[u & 3] = fmaf(o_s[j0 + u], r[u], acc[u & 3]);
        }
        const float res = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        if (p.out_is_fp16)
            static_cast<__half*>(p.out)[row * D + i] = __float2half_rn(fminf(fmaxf(res, -65504.f), 65504.f));
        else
            static_cast<float*>(p.out)[row * D + i] = res;
    }
}

// Read and clear this file's device error flag (for pq_poll_device_errors).
int exchange_error_flags(unsigned int* flags) {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_exchange_error, sizeof(v)) != cudaSuccess) return PQ_ERR_CUDA;
    if (v && cudaMemcpyToSymbol(g_exchange_error, &zero, sizeof(zero)) != cudaSuccess) return PQ_ERR_CUDA;
    *flags = v;
    return PQ_OK;
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

extern "C" size_t pq_lse_exchange_bytes(int world, int64_t n_rows, int head_dim) {
    if (world <= 0 || n_rows < 0 || head_dim <= 0) return 0;
    const size_t recs = 2 * (size_t)world * (size_t)n_rows * (head_dim + 2) * sizeof(float);
    return ((recs + 127) & ~size_t(127)) + 128;              // records, then the arrival counters
}

extern "C" int pq_lse_exchange_merge(const float* local_partial, int world, int rank, void* const* peer_buffers,
                                     uint64_t epoch, int64_t n_rows, int head_dim, const float* rot,
                                     void* out, int out_is_fp16, void* stream) {
    using namespace pq;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || n_rows < 0 || epoch == 0) return PQ_ERR_BAD_SHAPE;
    if (head_dim != 64 && head_dim != 128) return PQ_ERR_BAD_HEAD_DIM;
    if (n_rows == 0) return PQ_OK;
    if (!local_partial || !peer_buffers || !rot || !out) return PQ_ERR_NULL_POINTER;
    ExchangeParams p{};
    const size_t recs = 2 * (size_t)world * (size_t)n_rows * (head_dim + 2) * sizeof(float);
    const size_t counter_off = (recs + 127) & ~size_t(127);
    for (int s = 0; s < world; ++s) {
        if (!peer_buffers[s]) return PQ_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(peer_buffers[s]) & 127) return PQ_ERR_MISALIGNED;
        p.recv[s] = static_cast<float*>(peer_buffers[s]);
        p.arrived[s] = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(peer_buffers[s]) + counter_off);
    }
    p.local = local_partial;
    p.world = world;
    p.rank = rank;
    p.epoch = epoch;
    p.n_rows = n_rows;
    p.rot = rot;
    p.out = out;
    p.out_is_fp16 = out_is_fp16;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // at most one CTA per SM: every CTA must be resident while it waits for the peers
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        return PQ_ERR_CUDA;
    const int grid = (int)(n_rows < sms ? n_rows : sms);
    if (head_dim == 64) pq::pq_lse_exchange_merge_kernel<64><<<grid, 64, 0, st>>>(p);
    else pq::pq_lse_exchange_merge_kernel<128><<<grid, 128, 0, st>>>(p);
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
