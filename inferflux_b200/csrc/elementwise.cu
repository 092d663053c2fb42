// Embedding gather, fused residual-add + RMSNorm, SwiGLU, type conversion.
//
// Formulas follow the reference's native path:
//   embedding  out[t,:] = float(E[id_t,:])            runtime/backends/cuda/native/cuda_kernels.cu:599-614
//   RMSNorm    y = x * rsqrt(mean(x^2) + eps) * w     cuda_kernels.cu:469-501 (float32 math)
//   add+norm   r += d; y = RMSNorm(r)                 cuda_kernels.cu:541-579
//   SwiGLU     a = g / (1 + exp(-g)) * u              cuda_kernels.cu:137-149
// The reference runs one thread per element with a power-of-two block and a
// shared-memory tree; here a row stays in shared memory between the two
// passes, loads are 16 bytes wide where the row length allows, and any row
// length is taken.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int hidden, int vocab) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {   // never read outside the table
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = Num<T>::to_f(row[i]);
}

IFX_API int ifx_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                             int n_tokens, int hidden, int vocab, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
  if (table_dtype == IFX_F32)
    embed_gather_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)table, ids, out, hidden, vocab);
  else if (table_dtype == IFX_BF16)
    embed_gather_kernel<bf16><<<n_tokens, threads, 0, stream>>>((const bf16*)table, ids, out, hidden, vocab);
  else
    return IFX_ERR_UNSUPPORTED;
  return IFX_LAUNCH_CHECK();
}

// ------------------------------------------------------ residual add + RMSNorm
// One block per output row.  Source row = rows ? rows[blockIdx.x] : blockIdx.x.
// r = residual[src] + (delta ? delta[src] : 0); when write_residual the sum is
// stored back (never in gather mode, where a row may be listed twice).
// n_partials > 1: delta holds that many float32 partial sums of the same
// shape, `partial_stride` elements apart, added in index order.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   int n_partials, long long partial_stride,
                                   const float* __restrict__ weight, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows,
                                   int hidden, int write_residual) {
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const int src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = residual + (size_t)src * hidden;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = r[i];
    if (delta) {
      const TD* d = delta + (size_t)src * hidden + i;
      for (int p = 0; p < n_partials; ++p) v += Num<TD>::to_f(d[(size_t)p * partial_stride]);
    }
    row_buf[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  TO* o = out ? out + (size_t)blockIdx.x * hidden : nullptr;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = row_buf[i];
    if (write_residual) r[i] = v;
    if (o) o[i] = Num<TO>::from_f(v * rstd * weight[i]);
  }
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* residual, const void* delta, int n_partials, long long partial_stride,
                              const float* weight, float eps, void* out, const int* rows, int n_rows,
                              int hidden, int write_residual, cudaStream_t stream) {
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return IFX_ERR_UNSUPPORTED;
  auto kern = add_rmsnorm_kernel<TD, TO>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = 128;
  while (threads < 1024 && threads * 4 < hidden) threads <<= 1;
  kern<<<n_rows, threads, smem, stream>>>(residual, (const TD*)delta, n_partials, partial_stride, weight, eps,
                                          (TO*)out, rows, hidden, write_residual);
  return IFX_LAUNCH_CHECK();
}

// delta_dtype / out_dtype: IFX_F32 or IFX_BF16.  delta and out may be null.
IFX_API int ifx_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int n_partials,
                            long long partial_stride, const float* weight, float eps, void* out,
                            int out_dtype, const int* rows, int n_rows, int hidden,
                            int write_residual, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (rows && write_residual) return IFX_ERR_UNSUPPORTED;
  if (n_partials < 1) n_partials = 1;
  if (delta_dtype == IFX_F32 && out_dtype == IFX_F32)
    return launch_add_rmsnorm<float, float>(residual, delta, n_partials, partial_stride, weight, eps, out, rows, n_rows, hidden, write_residual, stream);
  if (delta_dtype == IFX_BF16 && out_dtype == IFX_BF16)
    return launch_add_rmsnorm<bf16, bf16>(residual, delta, n_partials, partial_stride, weight, eps, out, rows, n_rows, hidden, write_residual, stream);
  if (delta_dtype == IFX_F32 && out_dtype == IFX_BF16)
    return launch_add_rmsnorm<float, bf16>(residual, delta, n_partials, partial_stride, weight, eps, out, rows, n_rows, hidden, write_residual, stream);
  if (delta_dtype == IFX_BF16 && out_dtype == IFX_F32)
    return launch_add_rmsnorm<bf16, float>(residual, delta, n_partials, partial_stride, weight, eps, out, rows, n_rows, hidden, write_residual, stream);
  return IFX_ERR_UNSUPPORTED;
}

// -------------------------------------------------------------------- SwiGLU
// gate_up [M, 2*I] (gate columns first) -> out [M, I]
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int inter) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const long long m = idx / inter;
    const int i = (int)(idx - m * inter);
    const float g = Num<T>::to_f(gate_up[m * 2 * inter + i]);
    const float u = Num<T>::to_f(gate_up[m * 2 * inter + inter + i]);
    out[idx] = Num<T>::from_f(g / (1.0f + expf(-g)) * u);
  }
}

IFX_API int ifx_swiglu(const void* gate_up, void* out, int dtype, int m, int inter, cudaStream_t stream) {
  const long long total = (long long)m * inter;
  if (total <= 0) return 0;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == IFX_F32)
    swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, total, inter);
  else if (dtype == IFX_BF16)
    swiglu_kernel<bf16><<<(int)blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, total, inter);
  else
    return IFX_ERR_UNSUPPORTED;
  return IFX_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- conversion
template <typename TS, typename TD>
__global__ void convert_kernel(const TS* __restrict__ src, TD* __restrict__ dst, long long n) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < n; idx += stride) dst[idx] = Num<TD>::from_f(Num<TS>::to_f(src[idx]));
}

IFX_API int ifx_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (src_dtype == IFX_BF16 && dst_dtype == IFX_F32)
    convert_kernel<bf16, float><<<(int)blocks, threads, 0, stream>>>((const bf16*)src, (float*)dst, n);
  else if (src_dtype == IFX_F32 && dst_dtype == IFX_BF16)
    convert_kernel<float, bf16><<<(int)blocks, threads, 0, stream>>>((const float*)src, (bf16*)dst, n);
  else
    return IFX_ERR_UNSUPPORTED;
  return IFX_LAUNCH_CHECK();
}
