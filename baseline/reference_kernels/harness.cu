// C entry points around the leaf kernels of vjsingh1984/inferflux, so that Python
// can call them through ctypes.  This file holds no arithmetic of its own: each
// function forwards its arguments to the reference's own host wrapper, which is
// compiled unmodified from the reference's source tree next to this file
// (runtime/backends/cuda/native/cuda_kernels.cu and
// runtime/backends/cuda/kernels/flash_attention.cu).  All tensors are bfloat16
// unless a name says float; pointers are device pointers; every call is
// asynchronous on the given stream and returns the cudaError_t as an int.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "runtime/backends/cuda/kernels/flash_attention.cuh"
#include "runtime/backends/cuda/native/cuda_kernels.cuh"

namespace ck = inferflux::cuda_kernel;
using bf16 = __nv_bfloat16;

extern "C" {

// cuda_kernels.cu:117-131, rope_type 2 = split-half pairs (what model_type "qwen2" selects)
int ref_rope_neox(void* q, void* k, int seq_len, int n_heads, int n_kv_heads, int head_dim, int n_past,
                  float theta, void* stream) {
  return (int)ck::RoPE<bf16>((bf16*)q, (bf16*)k, seq_len, n_heads, n_kv_heads, head_dim, n_past, theta,
                             (cudaStream_t)stream, 2);
}

// cuda_kernels.cu:468-517
int ref_rms_norm_mixed(const float* input, const void* weight, void* output, int rows, int hidden, float eps,
                       void* stream) {
  return (int)ck::RmsNormMixed<bf16>(input, (const bf16*)weight, (bf16*)output, rows, hidden, eps,
                                     (cudaStream_t)stream);
}

// cuda_kernels.cu:541-596
int ref_residual_add_rms_norm_mixed(float* residual, const void* input, const void* weight, void* output, int rows,
                                    int hidden, float eps, void* stream) {
  return (int)ck::ResidualAddRmsNormMixed<bf16>(residual, (const bf16*)input, (const bf16*)weight, (bf16*)output,
                                                rows, hidden, eps, (cudaStream_t)stream);
}

// cuda_kernels.cu:137-158
int ref_silu_mul(const void* gate, const void* up, void* output, int count, void* stream) {
  return (int)ck::SiluMul<bf16>((const bf16*)gate, (const bf16*)up, (bf16*)output, count, (cudaStream_t)stream);
}

// cuda_kernels.cu:694-735
int ref_bias_add_triple(void* q, void* k, void* v, const void* bq, const void* bk, const void* bv, int rows,
                        int q_dim, int k_dim, int v_dim, void* stream) {
  return (int)ck::BiasAddTriple<bf16>((bf16*)q, (bf16*)k, (bf16*)v, (const bf16*)bq, (const bf16*)bk,
                                      (const bf16*)bv, rows, q_dim, k_dim, v_dim, (cudaStream_t)stream);
}

// cuda_kernels.cu:599-626
int ref_embedding_lookup_f32(const void* table, const int* ids, float* output, int seq_len, int hidden,
                             void* stream) {
  return (int)ck::EmbeddingLookupF32<bf16>((const bf16*)table, ids, output, seq_len, hidden, (cudaStream_t)stream);
}

// flash_attention.cu:405-447; Q [batch, q_len, heads*hd], K and V [batch, kv_len, kv_heads*hd]
int ref_flash_attention2(const void* q, const void* k, const void* v, void* o, int batch, int q_len, int kv_len,
                         int n_heads, int n_kv_heads, int head_dim, float scale, int causal, void* stream) {
  return (int)ck::FlashAttention2Typed<bf16>((const bf16*)q, (const bf16*)k, (const bf16*)v, (bf16*)o, batch, q_len,
                                             kv_len, n_heads, n_kv_heads, head_dim, scale, causal != 0,
                                             (cudaStream_t)stream);
}

// flash_attention.cu:573-601; k_ptrs and v_ptrs are device arrays of device pointers, one per sequence
int ref_flash_decode_multi_seq(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* o,
                               const int* kv_lens, int batch, int n_heads, int n_kv_heads, int head_dim, float scale,
                               void* stream) {
  return (int)ck::FlashDecodeMultiSeq<bf16>((const bf16*)q, (const bf16* const*)k_ptrs, (const bf16* const*)v_ptrs,
                                            (bf16*)o, kv_lens, batch, n_heads, n_kv_heads, head_dim, scale,
                                            (cudaStream_t)stream);
}

}  // extern "C"
