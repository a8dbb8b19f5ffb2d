/*
 * polarquant_llama_abi — the entry points the reference's llama.cpp bridge looks up with
 * dlsym/GetProcAddress (integration/polarquant-kv.patch of hilllief/polarquant-kv, decoded:
 * `extern "C"` wrappers at lines 695-763, typedefs of the loader at 1536-1537), exported
 * by libpolarquant_b200.so under the same names with the same argument lists, so that a
 * llama.cpp built with that patch can load this library in place of the patch's own
 * polarquant.cu build.
 *
 * This is a DIFFERENT codec from block_pq4 (polarquant_b200.h): one float32 radius per
 * vector and a codebook for directions of the full head dimension; packed indices are
 * always one nibble per element (byte k = idx[2k] | idx[2k+1] << 4) whatever n_levels is.
 *
 *   layouts (all DEVICE pointers, float32 unless noted, row-major):
 *     input / q_input / q_rotated / output   [N or total_q_heads, D]
 *     rotation                               [D, D]; rotate is x · Rᵀ, inverse is y · R
 *     codebook                               [n_levels], n_levels <= 16
 *     packed_k / packed_v      uint8         [total_kv_heads, S, D/2]
 *     k_radius / v_radius                    [total_kv_heads, S]
 *   q head h reads kv head h / (total_q_heads / total_kv_heads).
 *
 * The functions return void like the ones they replace; where those printed to stderr and
 * returned (or silently read out of bounds) on a shape they could not handle, these record
 * a code that polarquant_last_error_c() returns and clears, and enqueue nothing.
 * D must be even and at most 1024.  There is no limit on S (the patch's attention kernel
 * gave up above 12288 tokens: lines 487-496 of the decoded patch).
 */
#ifndef POLARQUANT_LLAMA_ABI_H
#define POLARQUANT_LLAMA_ABI_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Per-layer device buffers of the state (patch lines 947-956: polarquant_kv_layer). */
struct polarquant_kv_layer {
    uint8_t* k_packed;   /* [n_kv_heads * n_kv_max, head_dim/2] */
    float*   k_radius;   /* [n_kv_heads * n_kv_max]             */
    uint8_t* v_packed;
    float*   v_radius;
};

/* State object the bridge keeps and reads (patch lines 958-972: polarquant_state); the field
 * order and types are the interface, llama.cpp dereferences them. */
struct polarquant_state {
    bool   enabled;
    int    n_bits;
    int    n_levels;
    int    head_dim;
    int    n_kv_heads;
    int    n_q_heads;
    int    n_layers;
    int    n_kv_max;
    float* codebook;                      /* device, [n_levels]            */
    float* rotation;                      /* device, [head_dim, head_dim]  */
    struct polarquant_kv_layer* layers;   /* host array of n_layers        */
};

/* Replaces polarquant_init_c (patch 700-708 → polarquant_init, 581-669): allocates the
 * state, uploads the built-in codebook for n_bits in {2, 3, 4} (anything else falls back
 * to 4 with a message, as there) and the seed-42 Gram-Schmidt rotation, allocates and
 * zeroes the per-layer buffers.  Returns NULL when an allocation fails. */
struct polarquant_state* polarquant_init_c(int head_dim, int n_kv_heads, int n_q_heads,
                                           int n_layers, int n_kv_max, int n_bits);

/* Replaces polarquant_free_c (patch 710-712 → polarquant_free, 671-689).  NULL is fine. */
void polarquant_free_c(struct polarquant_state* state);

/* Replaces polarquant_compress_cuda_c (patch 717-724 → kernel 193-270): rotate, take the
 * Euclidean norm as radius, divide (0 when radius <= 1e-30), nearest centroid by a linear
 * scan that keeps the first of equals, pack two indices per byte. */
void polarquant_compress_cuda_c(const float* input, const float* rotation, const float* codebook,
                                float* radius_out, uint8_t* packed_out,
                                int N, int D, int n_levels, void* stream);

/* Replaces polarquant_rotate_query_cuda_c (patch 729-735 → kernel 395-411). */
void polarquant_rotate_query_cuda_c(const float* q_input, const float* rotation, float* q_rotated,
                                    int total_q_heads, int D, void* stream);

/* Replaces polarquant_fused_attention_cuda_c (patch 740-751 → kernel 276-390):
 * score = dot(q_rotated, codebook[k idx]) * k_radius * scale, softmax over S,
 * output = sum_s w_s * codebook[v idx] * v_radius (still in rotated space).
 * Long sequences are sliced over CTAs through a workspace inside the library (no allocation);
 * calls on one device must be ordered with respect to each other (one stream, as in the bridge). */
void polarquant_fused_attention_cuda_c(const float* q_rotated, const uint8_t* packed_k,
                                       const float* k_radius, const uint8_t* packed_v,
                                       const float* v_radius, const float* codebook, float* output,
                                       int total_q_heads, int total_kv_heads,
                                       int S, int D, int n_levels, float scale, void* stream);

/* Replaces polarquant_inverse_rotate_cuda_c (patch 756-762 → kernel 418-435). */
void polarquant_inverse_rotate_cuda_c(const float* input, const float* rotation, float* output,
                                      int total_q_heads, int D, void* stream);

/* No counterpart in the reference: the status of the calling thread's most recent call
 * above that could not run (0 none, 1 NULL pointer, 2 D odd / non-positive / above 1024,
 * 3 n_levels outside [1, 16], 4 total_q_heads not a multiple of total_kv_heads,
 * 5 a CUDA call failed); reading it resets it to 0. */
int polarquant_last_error_c(void);

#ifdef __cplusplus
}
#endif
#endif /* POLARQUANT_LLAMA_ABI_H */
