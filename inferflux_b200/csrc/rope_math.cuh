// Bias add and rotate-half rotation on groups of 8 values, shared by the kernel that prepares q, k and v of
// a whole step (rope_kv.cu) and by the decode attention kernel that does the same for its own heads
// (attention_bf16.cu).  Both use exactly these operations, in this order and with explicit roundings, so a
// token's q, k and v come out the same bit for bit whichever kernel made them.
#pragma once
#include "common.cuh"

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) { const float2 t = __bfloat1622float2(h[k]); f[2 * k] = t.x; f[2 * k + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  return v;
}
__device__ __forceinline__ void load8f(const float* p, float (&f)[8]) {
  *reinterpret_cast<float4*>(f) = *reinterpret_cast<const float4*>(p);
  *reinterpret_cast<float4*>(f + 4) = *reinterpret_cast<const float4*>(p + 4);
}

// NE groups of 8 values of a row, at elements e[0..NE): from the bfloat16 row itself, or the sum (in slice
// order) of float32 partial sums [n_partials][n_tokens][width] of the product that made it (part points at
// the row in slice 0).  The loads of NB slices are issued before the first sum, so that a thread waits for
// memory once per NB slices and not once per slice.  PART says at compile time which of the two it is.
template <int NE, bool PART, int NB>
__device__ __forceinline__ void load8(const bf16* row, const float* part, int n_partials, long long part_stride,
                                      const int (&e)[NE], float (&f)[NE][8]) {
  if constexpr (!PART) {
#pragma unroll
    for (int j = 0; j < NE; ++j) unpack8(*reinterpret_cast<const uint4*>(row + e[j]), f[j]);
  } else {
#pragma unroll
    for (int j = 0; j < NE; ++j)
#pragma unroll
      for (int k = 0; k < 8; ++k) f[j][k] = 0.0f;
    for (int p0 = 0; p0 < n_partials; p0 += NB) {
      float4 v[NB][NE][2];
#pragma unroll
      for (int q = 0; q < NB; ++q)
        if (p0 + q < n_partials) {
#pragma unroll
          for (int j = 0; j < NE; ++j) {
            v[q][j][0] = *reinterpret_cast<const float4*>(part + (p0 + q) * part_stride + e[j]);
            v[q][j][1] = *reinterpret_cast<const float4*>(part + (p0 + q) * part_stride + e[j] + 4);
          }
        }
#pragma unroll
      for (int q = 0; q < NB; ++q)
        if (p0 + q < n_partials) {
#pragma unroll
          for (int j = 0; j < NE; ++j) {
            const float4 a = v[q][j][0], b = v[q][j][1];
            f[j][0] = __fadd_rn(f[j][0], a.x); f[j][1] = __fadd_rn(f[j][1], a.y);
            f[j][2] = __fadd_rn(f[j][2], a.z); f[j][3] = __fadd_rn(f[j][3], a.w);
            f[j][4] = __fadd_rn(f[j][4], b.x); f[j][5] = __fadd_rn(f[j][5], b.y);
            f[j][6] = __fadd_rn(f[j][6], b.z); f[j][7] = __fadd_rn(f[j][7], b.w);
          }
        }
    }
  }
}

// Elements e0 .. e0+7 and e0+half .. e0+half+7 of one head (e0 counted from the row's start, i = e0's place
// within the head's first half): bias, rotation by the angles whose cosines and sines are ct[i..], st[i..],
// rounded to bfloat16.
template <bool PART, int NB = 4>
__device__ __forceinline__ void rope_pairs8(const bf16* row, const float* part, int n_partials, long long part_stride,
                                            const float* bias, const float* ct, const float* st, int e0, int half, int i,
                                            uint4& lo, uint4& hi) {
  float c[8], s[8], b0[8], b1[8], x[2][8];
  load8f(ct + i, c);                                            // everything this item reads is asked for before the sums
  load8f(st + i, s);
  if (bias) {                                                   // 16-byte aligned: head_dim is a multiple of 16
    load8f(bias + e0, b0);
    load8f(bias + e0 + half, b1);
  }
  const int e[2] = {e0, e0 + half};
  load8<2, PART, NB>(row, part, n_partials, part_stride, e, x);
  float (&x0)[8] = x[0];
  float (&x1)[8] = x[1];
  if (bias) {
#pragma unroll
    for (int k = 0; k < 8; ++k) { x0[k] = __fadd_rn(x0[k], b0[k]); x1[k] = __fadd_rn(x1[k], b1[k]); }
  }
  float y0[8], y1[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    y0[k] = __fmaf_rn(x0[k], c[k], -__fmul_rn(x1[k], s[k]));
    y1[k] = __fmaf_rn(x0[k], s[k], __fmul_rn(x1[k], c[k]));
  }
  lo = pack8(y0);
  hi = pack8(y1);
}

// 8 unrotated values (the value heads): bias, rounded to bfloat16
template <bool PART, int NB = 4>
__device__ __forceinline__ uint4 biased8(const bf16* row, const float* part, int n_partials, long long part_stride,
                                         const float* bias, int e0) {
  float b[8], x[1][8];
  if (bias) load8f(bias + e0, b);
  const int e[1] = {e0};
  load8<1, PART, NB>(row, part, n_partials, part_stride, e, x);
  if (bias) {
#pragma unroll
    for (int k = 0; k < 8; ++k) x[0][k] = __fadd_rn(x[0][k], b[k]);
  }
  return pack8(x[0]);
}
