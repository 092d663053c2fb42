// Rotary position encoding (rotate-half) fused with the q/k/v bias add and
// the write of keys and values into the paged cache.
//
// Reference formulas (runtime/backends/cuda/native/cuda_kernels.cu:70-115,
// rope_type 2 = split-half pairs): for i in [0, d/2):
//   f = 1 / pow(theta, 2 i / d),  a = pos * f,
//   (x_i, x_{i+d/2}) <- (x_i cos a - x_{i+d/2} sin a,  x_i sin a + x_{i+d/2} cos a)
// applied to q and k; biases are added first (cuda_kernels.cu:694-723), then
// the rotated k and the v row go to the cache
// (runtime/backends/cuda/native/kernels/fused_rope_kv_append.cuh:26-166 does
// this for decode only, with powf/cosf/sinf per element and a dense cache).
//
// Here the angles are computed once per step for all layers (cos/sin tables
// per token, in double precision rounded to float32), and one kernel per layer
// does bias + rotation + paged write for prompts and decoded tokens alike.
#include "common.cuh"
#include "rope_math.cuh"

// cos/sin tables [n_tokens, half] from positions and inverse frequencies.
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                  float* __restrict__ cos_t, float* __restrict__ sin_t, int n_tokens, int half) {
  pdl_enter();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_tokens * half) return;
  const int t = idx / half, i = idx - t * half;
  const double a = (double)positions[t] * inv_freq[i];
  double s, c;
  sincos(a, &s, &c);
  cos_t[idx] = (float)c;
  sin_t[idx] = (float)s;
}

IFX_API int ifx_rope_table(const int* positions, const double* inv_freq, float* cos_t, float* sin_t,
                           int n_tokens, int half, cudaStream_t stream) {
  const int total = n_tokens * half;
  if (total <= 0) return 0;
  int ifx_rc = launch_pdl(rope_table_kernel, dim3((total + 127) / 128), dim3(128), 0, stream, positions, inv_freq, cos_t, sin_t, n_tokens, half);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

// qkv: [n_tokens, (n_heads + 2 n_kv) * head_dim], q heads first, then k, then v.
// q is rotated in place; k (rotated) and v go to the cache at slot_map[t]
// (= page * page_size + offset; negative = do not store).  n_kv may be 0 (a
// layer that reads another layer's cache has only q).
template <typename T>
__global__ void qkv_rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ bias,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         int rot_half, const int* __restrict__ slot_map, PagedKV kv,
                                         int n_heads, int n_kv, int head_dim) {
  pdl_enter();
  const int t = blockIdx.x;
  const int width = (n_heads + 2 * n_kv) * head_dim;
  T* row = qkv + (size_t)t * width;
  const float* ct = cos_t + (size_t)t * rot_half;
  const float* st = sin_t + (size_t)t * rot_half;
  const int slot = n_kv ? slot_map[t] : -1;
  const long long page = slot >= 0 ? (slot >> kv.page_shift) : 0;
  const int off = slot & (kv.page_size - 1);
  T* kc = (T*)kv.k;
  T* vc = (T*)kv.v;
  const int half_dim = head_dim / 2;
  // q and k heads: one work item per (head, i < head_dim/2): elements i and i + rot_half
  // when i < rot_half (rotated), and the tail beyond 2*rot_half unrotated.
  const int rot_heads = n_heads + n_kv;
  for (int w = threadIdx.x; w < rot_heads * half_dim; w += blockDim.x) {
    const int h = w / half_dim, i = w - h * half_dim;
    const int base = h * head_dim;
    int i0, i1;
    float c = 1.0f, s = 0.0f;
    if (i < rot_half) {
      i0 = i; i1 = i + rot_half; c = ct[i]; s = st[i];
    } else {             // unrotated tail: pair up the remaining dims two by two
      i0 = 2 * rot_half + 2 * (i - rot_half); i1 = i0 + 1;
    }
    float x0 = Num<T>::to_f(row[base + i0]);
    float x1 = Num<T>::to_f(row[base + i1]);
    if (bias) { x0 += bias[base + i0]; x1 += bias[base + i1]; }
    const T y0 = Num<T>::from_f(x0 * c - x1 * s);
    const T y1 = Num<T>::from_f(x0 * s + x1 * c);
    if (h < n_heads) {
      row[base + i0] = y0; row[base + i1] = y1;
    } else if (slot >= 0) {
      T* dst = kc + page * kv.page_stride + (size_t)(h - n_heads) * kv.head_stride + (size_t)off * head_dim;
      dst[i0] = y0; dst[i1] = y1;
    }
  }
  if (slot >= 0) {
    const int vbase = (n_heads + n_kv) * head_dim;
    for (int w = threadIdx.x; w < n_kv * head_dim; w += blockDim.x) {
      const int h = w / head_dim, d = w - h * head_dim;
      float x = Num<T>::to_f(row[vbase + w]);
      if (bias) x += bias[vbase + w];
      vc[page * kv.page_stride + (size_t)h * kv.head_stride + (size_t)off * head_dim + d] = Num<T>::from_f(x);
    }
  }
}

// Vector path (bfloat16, whole head rotated, head_dim a multiple of 16): a work item is 8
// consecutive pairs (i .. i+7, i+half .. i+half+7) of one head: two 16-byte loads, two 16-byte stores
// (rope_math.cuh).
template <bool PART, int NB = 4>
__global__ void __launch_bounds__(PART && NB > 1 ? 256 : 512) qkv_rope_kv_write_bf16x8_kernel(bf16* __restrict__ qkv, const float* __restrict__ bias,
                                                const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                const int* __restrict__ slot_map, PagedKV kv,
                                                int n_heads, int n_kv, int head_dim,
                                                const float* __restrict__ partials, int n_partials, long long part_stride) {
  pdl_enter();
  const int t = blockIdx.x;
  const int half = head_dim / 2, hv = half / 8;               // 8-wide groups per half head
  const int width = (n_heads + 2 * n_kv) * head_dim;
  bf16* row = qkv + (size_t)t * width;
  const float* part = PART ? partials + (size_t)t * width : nullptr;
  const float* ct = cos_t + (size_t)t * half;
  const float* st = sin_t + (size_t)t * half;
  const int slot = n_kv ? slot_map[t] : -1;
  const long long page = slot >= 0 ? (slot >> kv.page_shift) : 0;
  const int off = slot & (kv.page_size - 1);
  bf16* kc = (bf16*)kv.k + page * kv.page_stride + (size_t)off * head_dim;
  bf16* vc = (bf16*)kv.v + page * kv.page_stride + (size_t)off * head_dim;
  const int rot_heads = n_heads + n_kv;
  const int rot_items = rot_heads * hv, v_items = slot >= 0 ? n_kv * head_dim / 8 : 0;
  const int vbase = (n_heads + n_kv) * head_dim;
  // one list of 8-wide items, rotated pairs first and values after them, so that a thread's loads of both
  // kinds are in flight together
  for (int w = threadIdx.x; w < rot_items + v_items; w += blockDim.x) {
    if (w < rot_items) {
      const int h = w / hv, i = (w - h * hv) * 8;
      const int base = h * head_dim;
      uint4 p0, p1;
      rope_pairs8<PART, NB>(row, part, n_partials, part_stride, bias, ct, st, base + i, half, i, p0, p1);
      if (h < n_heads) {
        *reinterpret_cast<uint4*>(row + base + i) = p0;
        *reinterpret_cast<uint4*>(row + base + half + i) = p1;
      } else if (slot >= 0) {
        bf16* dst = kc + (size_t)(h - n_heads) * kv.head_stride;
        *reinterpret_cast<uint4*>(dst + i) = p0;
        *reinterpret_cast<uint4*>(dst + half + i) = p1;
      }
    } else {
      const int e0 = (w - rot_items) * 8, h = e0 / head_dim, d = e0 - h * head_dim;
      *reinterpret_cast<uint4*>(vc + (size_t)h * kv.head_stride + d) =
          biased8<PART, NB>(row, part, n_partials, part_stride, bias, vbase + e0);
    }
  }
}

// The same for steps of many tokens: a block takes TOK consecutive tokens and a thread the same 8-wide item of
// each of them, so that its loads of all TOK tokens are in flight together and it reads the bias once.  The
// arithmetic per item is rope_pairs8 / biased8 as above.  F32: the rows come as the product's float32 sums
// (one slice, `sums`), and qkv only receives the rotated q.
template <int TOK, bool F32>
__global__ void __launch_bounds__(512) qkv_rope_kv_write_bf16x8_many_kernel(bf16* __restrict__ qkv, const float* __restrict__ bias,
                                                const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                const int* __restrict__ slot_map, PagedKV kv, int n_tokens,
                                                int n_heads, int n_kv, int head_dim, const float* __restrict__ sums) {
  pdl_enter();
  const int t0 = blockIdx.x * TOK;
  const int half = head_dim / 2, hv = half / 8;
  const int width = (n_heads + 2 * n_kv) * head_dim;
  const int rot_items = (n_heads + n_kv) * hv, v_items = n_kv * head_dim / 8;
  const int vbase = (n_heads + n_kv) * head_dim;
  for (int w = threadIdx.x; w < rot_items + v_items; w += blockDim.x) {
    if (w < rot_items) {
      const int h = w / hv, i = (w - h * hv) * 8;
      const int base = h * head_dim;
      uint4 p0[TOK], p1[TOK];
#pragma unroll
      for (int k = 0; k < TOK; ++k) {
        const int t = min(t0 + k, n_tokens - 1);
        rope_pairs8<F32, 1>(qkv + (size_t)t * width, F32 ? sums + (size_t)t * width : nullptr, 1, 0, bias,
                            cos_t + (size_t)t * half, sin_t + (size_t)t * half, base + i, half, i, p0[k], p1[k]);
      }
#pragma unroll
      for (int k = 0; k < TOK; ++k) {
        const int t = t0 + k;
        if (t >= n_tokens) break;
        if (h < n_heads) {
          bf16* row = qkv + (size_t)t * width;
          *reinterpret_cast<uint4*>(row + base + i) = p0[k];
          *reinterpret_cast<uint4*>(row + base + half + i) = p1[k];
        } else {
          const int slot = slot_map[t];
          if (slot >= 0) {
            bf16* dst = (bf16*)kv.k + (size_t)(slot >> kv.page_shift) * kv.page_stride + (size_t)(h - n_heads) * kv.head_stride +
                        (size_t)(slot & (kv.page_size - 1)) * head_dim;
            *reinterpret_cast<uint4*>(dst + i) = p0[k];
            *reinterpret_cast<uint4*>(dst + half + i) = p1[k];
          }
        }
      }
    } else {
      const int e0 = (w - rot_items) * 8, h = e0 / head_dim, d = e0 - h * head_dim;
      uint4 v[TOK];
#pragma unroll
      for (int k = 0; k < TOK; ++k) {
        const int t = min(t0 + k, n_tokens - 1);
        v[k] = biased8<F32, 1>(qkv + (size_t)t * width, F32 ? sums + (size_t)t * width : nullptr, 1, 0, bias, vbase + e0);
      }
#pragma unroll
      for (int k = 0; k < TOK; ++k) {
        const int t = t0 + k;
        if (t >= n_tokens) break;
        const int slot = slot_map[t];
        if (slot >= 0)
          *reinterpret_cast<uint4*>((bf16*)kv.v + (size_t)(slot >> kv.page_shift) * kv.page_stride + (size_t)h * kv.head_stride +
                                    (size_t)(slot & (kv.page_size - 1)) * head_dim + d) = v[k];
      }
    }
  }
}

IFX_API int ifx_qkv_rope_kv_write(void* qkv, int dtype, const float* bias, const float* cos_t, const float* sin_t,
                                  int rot_dim, const int* slot_map, void* k_layer, void* v_layer,
                                  long long page_stride, int page_size, int n_tokens, int n_heads, int n_kv,
                                  int head_dim, const float* partials, int n_partials, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  int ifx_rc = 0;
  if (head_dim % 2 || rot_dim % 2 || rot_dim > head_dim || rot_dim < 0) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  PagedKV kv;
  kv.k = k_layer; kv.v = v_layer; kv.page_stride = page_stride;
  kv.head_stride = page_size * head_dim; kv.page_size = page_size;
  kv.page_shift = 0;
  while ((1 << kv.page_shift) < page_size) ++kv.page_shift;
  const int work = (n_heads + 2 * n_kv) * head_dim / 2;
  int threads = 64;
  while (threads < 512 && threads * 4 < work) threads <<= 1;
  const bool aligned = (((uintptr_t)qkv | (uintptr_t)k_layer | (uintptr_t)v_layer | (uintptr_t)cos_t | (uintptr_t)sin_t |
                         (uintptr_t)bias) & 15) == 0
                       && (page_stride & 7) == 0;
  if (dtype == IFX_BF16 && rot_dim == head_dim && head_dim % 16 == 0 && aligned) {
    const int work8 = (n_heads + n_kv) * head_dim / 16 + n_kv * head_dim / 8;
    if (partials && (((uintptr_t)partials & 15) || n_partials < 1)) return IFX_ERR_ALIGNMENT;
    const int th_max = partials && n_partials > 1 ? 256 : 512;  // the kernels' launch bounds
    int th = 32;
    while (th < th_max && th < work8) th <<= 1;
    const long long part_stride = (long long)n_tokens * (n_heads + 2 * n_kv) * head_dim;
    constexpr int MANY_TOK = 4;
    if (!partials && n_kv > 0 && n_tokens >= 64 * MANY_TOK)
      ifx_rc = launch_pdl(qkv_rope_kv_write_bf16x8_many_kernel<MANY_TOK, false>, dim3((n_tokens + MANY_TOK - 1) / MANY_TOK), dim3(th), 0,
                          stream, (bf16*)qkv, bias, cos_t, sin_t, slot_map, kv, n_tokens, n_heads, n_kv, head_dim,
                          (const float*)nullptr);
    else if (partials && n_partials == 1 && n_kv > 0 && n_tokens >= 64 * MANY_TOK)
      ifx_rc = launch_pdl(qkv_rope_kv_write_bf16x8_many_kernel<MANY_TOK, true>, dim3((n_tokens + MANY_TOK - 1) / MANY_TOK), dim3(th), 0,
                          stream, (bf16*)qkv, bias, cos_t, sin_t, slot_map, kv, n_tokens, n_heads, n_kv, head_dim, partials);
    else if (partials && n_partials == 1)                         // one slice: no sums to batch, the wider block fits
      ifx_rc = launch_pdl(qkv_rope_kv_write_bf16x8_kernel<true, 1>, dim3(n_tokens), dim3(th), 0, stream, (bf16*)qkv, bias, cos_t,
                          sin_t, slot_map, kv, n_heads, n_kv, head_dim, partials, n_partials, part_stride);
    else if (partials)
      ifx_rc = launch_pdl(qkv_rope_kv_write_bf16x8_kernel<true>, dim3(n_tokens), dim3(th), 0, stream, (bf16*)qkv, bias, cos_t, sin_t,
                          slot_map, kv, n_heads, n_kv, head_dim, partials, n_partials, part_stride);
    else
      ifx_rc = launch_pdl(qkv_rope_kv_write_bf16x8_kernel<false>, dim3(n_tokens), dim3(th), 0, stream, (bf16*)qkv, bias, cos_t, sin_t,
                          slot_map, kv, n_heads, n_kv, head_dim, partials, n_partials, part_stride);
    return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
  }
  if (partials) return IFX_ERR_UNSUPPORTED;                      // partial sums only on the bfloat16 vector path
  if (dtype == IFX_F32)
    ifx_rc = launch_pdl(qkv_rope_kv_write_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (float*)qkv, bias, cos_t, sin_t, rot_dim / 2, slot_map, kv, n_heads, n_kv, head_dim);
  else if (dtype == IFX_BF16)
    ifx_rc = launch_pdl(qkv_rope_kv_write_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, (bf16*)qkv, bias, cos_t, sin_t, rot_dim / 2, slot_map, kv, n_heads, n_kv, head_dim);
  else
    return IFX_ERR_UNSUPPORTED;
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

IFX_STAMP_READER(ifx_stamps_rope)
