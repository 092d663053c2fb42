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
  pdl_enter();
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

// 8 bfloat16 (16 bytes) per thread per step; hidden a multiple of 8
__global__ void embed_gather_bf16x8_kernel(const bf16* __restrict__ table, const int* __restrict__ ids,
                                           float* __restrict__ out, int hidden, int vocab) {
  pdl_enter();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * hidden);
  float4* o = reinterpret_cast<float4*>(out + (size_t)t * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    uint4 v = ok ? row[i] : make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    const float2 c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
    o[2 * i] = make_float4(a.x, a.y, b.x, b.y);
    o[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
  }
}

IFX_API int ifx_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                             int n_tokens, int hidden, int vocab, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  int ifx_rc = 0;
  const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
  if (table_dtype == IFX_F32)
    ifx_rc = launch_pdl(embed_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, ids, out, hidden, vocab);
  else if (table_dtype == IFX_BF16 && hidden % 8 == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)out & 15) == 0)
    ifx_rc = launch_pdl(embed_gather_bf16x8_kernel, dim3(n_tokens), dim3(threads), 0, stream, (const bf16*)table, ids, out, hidden, vocab);
  else if (table_dtype == IFX_BF16)
    ifx_rc = launch_pdl(embed_gather_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, (const bf16*)table, ids, out, hidden, vocab);
  else
    return IFX_ERR_UNSUPPORTED;
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
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
  pdl_enter();
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

// Vector path: hidden a multiple of 4 and at most 4 * VT * blockDim.  Each thread keeps its
// (up to VT) groups of 4 consecutive values in registers between the sum of squares and the
// scaling, so a row is read once and written once.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&a);
    u.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

// Residual add + RMSNorm, rows whose length is a multiple of 4, 16-byte accesses.  Two shapes of one computation:
//   narrow: 256 threads a row, thread t takes the groups of four elements t, t + 256, ... (J of them) - many rows;
//   wide:   one thread per group (up to 1,024 threads, two groups each beyond that), so that all loads of a row are
//           in flight at once - a step of a few rows, which is all latency.
// Both add a row's squares in the same order, so a row's result does not depend on which shape ran it (that is,
// on how many rows the step has): per thread-of-the-narrow-shape the groups t, t + 256, ... one after the other,
// then the warp tree, then the tree over the 8 warps.  The wide shape passes its groups' sums through shared
// memory to get there.
__device__ __forceinline__ float group_squares(const float4& x) {
  return __fmaf_rn(x.w, x.w, __fmaf_rn(x.z, x.z, __fmaf_rn(x.y, x.y, __fmul_rn(x.x, x.x))));
}
template <typename TD>
__device__ __forceinline__ float4 row_group(const float* r, const TD* delta, int n_partials, long long partial_stride,
                                            size_t at) {
  float4 x = Vec4<float>::load(r + at);
  if (delta && n_partials == 1) {
    const float4 y = Vec4<TD>::load(delta + at);
    x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
  } else if (delta) {
    const TD* d = delta + at;
    // the slices are asked for together (up to 8 at a time) and added in index order: one wait for memory
    // instead of one per slice
    for (int p0 = 0; p0 < n_partials; p0 += 8) {
      float4 y[8];
#pragma unroll
      for (int p = 0; p < 8; ++p)
        y[p] = p0 + p < n_partials ? Vec4<TD>::load(d + (size_t)(p0 + p) * partial_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if (p0 + p < n_partials) { x.x += y[p].x; x.y += y[p].y; x.z += y[p].z; x.w += y[p].w; }
    }
  }
  return x;
}
template <typename TO>
__device__ __forceinline__ void store_normed(TO* o, const float4& v, float rstd, const float4& w) {
  Vec4<TO>::store(o, make_float4(v.x * rstd * w.x, v.y * rstd * w.y, v.z * rstd * w.z, v.w * rstd * w.w));
}

template <typename TD, typename TO, int J>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials,
                       long long partial_stride, const float* __restrict__ weight, float eps,
                       TO* __restrict__ out, const int* __restrict__ rows, int hidden, int write_residual) {
  // the norm's weights are parameters: they are loaded before this kernel waits for the one before it
  pdl_launch_dependents();
  __shared__ float red[32];
  const int groups = hidden >> 2;
  float4 wv[J];
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int gidx = threadIdx.x + j * 256;
    wv[j] = (out && gidx < groups) ? Vec4<float>::load(weight + 4 * gidx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const int src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = residual + (size_t)src * hidden;
  const TD* d = delta ? delta + (size_t)src * hidden : nullptr;
  float4 v[J];
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int gidx = threadIdx.x + j * 256;
    if (gidx < groups) {
      v[j] = row_group<TD>(r, d, n_partials, partial_stride, (size_t)4 * gidx);
      ss = __fadd_rn(ss, group_squares(v[j]));
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  TO* o = out ? out + (size_t)blockIdx.x * hidden : nullptr;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int gidx = threadIdx.x + j * 256;
    if (gidx < groups) {
      if (write_residual) Vec4<float>::store(r + 4 * gidx, v[j]);
      if (o) store_normed<TO>(o + 4 * gidx, v[j], rstd, wv[j]);
    }
  }
}

// The wide shape: JT * 256 threads (JT = min(J, 4)), thread (jt, t) with t its index among 256 takes the groups
// (jt + v * JT) * 256 + t for v < VT, which are the narrow shape's j = jt + v * JT of its thread t.
template <typename TD, typename TO, int J>
__global__ void __launch_bounds__((J < 4 ? J : 4) * 256)
add_rmsnorm_wide_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials,
                        long long partial_stride, const float* __restrict__ weight, float eps,
                        TO* __restrict__ out, const int* __restrict__ rows, int hidden, int write_residual) {
  constexpr int JT = J < 4 ? J : 4, VT = (J + JT - 1) / JT;
  pdl_launch_dependents();
  __shared__ float sq[J][256];
  __shared__ float red[8];
  const int groups = hidden >> 2;
  const int t = threadIdx.x & 255, jt = threadIdx.x >> 8, lane = threadIdx.x & 31;
  float4 wv[VT];
#pragma unroll
  for (int vv = 0; vv < VT; ++vv) {
    const int gidx = (jt + vv * JT) * 256 + t;
    wv[vv] = (out && jt + vv * JT < J && gidx < groups) ? Vec4<float>::load(weight + 4 * gidx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const int src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = residual + (size_t)src * hidden;
  const TD* d = delta ? delta + (size_t)src * hidden : nullptr;
  float4 v[VT];
#pragma unroll
  for (int vv = 0; vv < VT; ++vv) {
    const int j = jt + vv * JT, gidx = j * 256 + t;
    if (j < J) {
      float e = 0.0f;
      if (gidx < groups) {
        v[vv] = row_group<TD>(r, d, n_partials, partial_stride, (size_t)4 * gidx);
        e = group_squares(v[vv]);
      }
      sq[j][t] = e;
    }
  }
  __syncthreads();
  if (threadIdx.x < 256) {                                     // the narrow shape's thread t: its groups one after the other
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < J; ++j)
      if (j * 256 + t < groups) ss = __fadd_rn(ss, sq[j][t]);
    ss = warp_sum(ss);
    if (lane == 0) red[t >> 5] = ss;
  }
  __syncthreads();
  const float total = warp_sum(lane < 8 ? red[lane] : 0.0f);   // as block_sum does for 8 warps
  const float rstd = rsqrtf(total / (float)hidden + eps);
  TO* o = out ? out + (size_t)blockIdx.x * hidden : nullptr;
#pragma unroll
  for (int vv = 0; vv < VT; ++vv) {
    const int j = jt + vv * JT, gidx = j * 256 + t;
    if (j < J && gidx < groups) {
      if (write_residual) Vec4<float>::store(r + 4 * gidx, v[vv]);
      if (o) store_normed<TO>(o + 4 * gidx, v[vv], rstd, wv[vv]);
    }
  }
}

constexpr int NORM_WIDE_MAX_ROWS = 64;   // up to this many rows a step is latency, not bandwidth

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* residual, const void* delta, int n_partials, long long partial_stride,
                              const float* weight, float eps, void* out, const int* rows, int n_rows,
                              int hidden, int write_residual, cudaStream_t stream) {
  int ifx_rc = 0;
  const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) == 0
                       && (partial_stride & 3) == 0;
  if (hidden % 4 == 0 && aligned && hidden <= 4 * 8 * 256) {
    const int j = (hidden / 4 + 255) / 256;                     // groups per thread of the narrow shape
    const bool wide = n_rows <= NORM_WIDE_MAX_ROWS;
#define IFX_NORM_CASE(J)                                                                                              \
    case J:                                                                                                           \
      ifx_rc = wide ? launch_pdl(add_rmsnorm_wide_kernel<TD, TO, J>, dim3(n_rows), dim3((J < 4 ? J : 4) * 256), 0, stream,    \
                                 residual, (const TD*)delta, n_partials, partial_stride, weight, eps, (TO*)out, rows, hidden, \
                                 write_residual)                                                                      \
                    : launch_pdl(add_rmsnorm_vec_kernel<TD, TO, J>, dim3(n_rows), dim3(256), 0, stream, residual,     \
                                 (const TD*)delta, n_partials, partial_stride, weight, eps, (TO*)out, rows, hidden,   \
                                 write_residual);                                                                     \
      break;
    switch (j) {
      IFX_NORM_CASE(1) IFX_NORM_CASE(2) IFX_NORM_CASE(3) IFX_NORM_CASE(4)
      IFX_NORM_CASE(5) IFX_NORM_CASE(6) IFX_NORM_CASE(7) IFX_NORM_CASE(8)
      default: return IFX_ERR_UNSUPPORTED;
    }
#undef IFX_NORM_CASE
    return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return IFX_ERR_UNSUPPORTED;
  auto kern = add_rmsnorm_kernel<TD, TO>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = 128;
  while (threads < 1024 && threads * 4 < hidden) threads <<= 1;
  ifx_rc = launch_pdl(kern, dim3(n_rows), dim3(threads), smem, stream, residual, (const TD*)delta, n_partials, partial_stride, weight, eps,
                                          (TO*)out, rows, hidden, write_residual);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
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
  pdl_enter();
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

// 8 outputs per thread per step: 16-byte loads of gate and up, one 16-byte store; inter a multiple of 8
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, long long total8, int inter8) {
  pdl_enter();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total8; idx += stride) {
    const long long m = idx / inter8;
    const int i = (int)(idx - m * inter8);
    const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + (m * 2 * inter8 + i) * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(gate_up + (m * 2 * inter8 + inter8 + i) * 8);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = ov;
  }
}

IFX_API int ifx_swiglu(const void* gate_up, void* out, int dtype, int m, int inter, cudaStream_t stream) {
  const long long total = (long long)m * inter;
  if (total <= 0) return 0;
  int ifx_rc = 0;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == IFX_BF16 && inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
    const long long total8 = total / 8;
    long long b8 = (total8 + threads - 1) / threads;
    if (b8 > 148 * 16) b8 = 148 * 16;
    ifx_rc = launch_pdl(swiglu_bf16x8_kernel, dim3((int)b8), dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, total8, inter / 8);
    return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
  }
  if (dtype == IFX_F32)
    ifx_rc = launch_pdl(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, total, inter);
  else if (dtype == IFX_BF16)
    ifx_rc = launch_pdl(swiglu_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, total, inter);
  else
    return IFX_ERR_UNSUPPORTED;
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- conversion
template <typename TS, typename TD>
__global__ void convert_kernel(const TS* __restrict__ src, TD* __restrict__ dst, long long n) {
  pdl_enter();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < n; idx += stride) dst[idx] = Num<TD>::from_f(Num<TS>::to_f(src[idx]));
}

IFX_API int ifx_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  int ifx_rc = 0;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (src_dtype == IFX_BF16 && dst_dtype == IFX_F32)
    ifx_rc = launch_pdl(convert_kernel<bf16, float>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)src, (float*)dst, n);
  else if (src_dtype == IFX_F32 && dst_dtype == IFX_BF16)
    ifx_rc = launch_pdl(convert_kernel<float, bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)src, (bf16*)dst, n);
  else
    return IFX_ERR_UNSUPPORTED;
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

IFX_STAMP_READER(ifx_stamps_elementwise)
