// Weight-streaming matrix product for a few rows of activations (decode):
// out[M, N] = X[M, K] * W[N, K]^T, bfloat16 in, float32 accumulation, M <= 32.
//
// The reference sends every dense projection to cuBLAS whatever M is
// (runtime/backends/cuda/native/cublas_gemm.cpp:84-102; its hand-written GEMV
// kernels are for quantized weights only).  At M of 1 to 32 the product is bound
// by reading W once, so this kernel is laid out around that read: the weights
// are the 16-row "A" operand of an m16n8k16 MMA and the tokens the 8-column "B"
// operand.  Each lane reads 16 contiguous bytes of two weight rows and 16 bytes
// of one token's activations per 32-wide K chunk; because a dot product does
// not care about the order of K, those 8 consecutive values feed two MMAs
// directly from registers, without shared memory or shuffles.  When there are
// many row tiles each warp owns one over the whole of K; when there are few, the
// warps of a block take interleaved K chunks of one tile and add their partial
// sums in shared memory in a fixed order, and K may also be cut between blocks,
// whose float32 partial results the consumer adds (the fused residual-add +
// norm kernel does).
//
// SwiGLU mode: rows 0-7 of the tile come from the gate half of a stacked
// [gate; up] weight and rows 8-15 from the up half at the same index, so each
// lane holds gate and up of the same output and writes silu(gate) * up
// (runtime/backends/cuda/native/cuda_kernels.cu:137-149) without the
// intermediate [M, 2I] tensor.
#include "common.cuh"

namespace {

// Loads are plain (always from a valid, clamped address) and masked afterwards, so that the
// compiler can issue the loads of an unrolled group together and keep them all in flight.
__device__ __forceinline__ uint4 mask16(uint4 v, bool keep) {
  return keep ? v : make_uint4(0u, 0u, 0u, 0u);
}
__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ T to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 to_out<bf16>(float v) { return __float2bfloat16_rn(v); }

constexpr int KCHUNK = 32, UNROLL = 8;

// A block has RW x KW warps: warp (rw, kw) owns row tile `blockIdx.x * RW + rw` (16 weight
// rows, or 8 gate + 8 up rows in SwiGLU mode) and the K chunks kw, kw + KW, ... of the
// block's K range; the KW partial sums of a row tile are added in shared memory in warp
// order.  gridDim.y > 1 cuts K between blocks: block y writes float32 partial sums to
// out + y * M * ldo... (partial_stride elements apart), to be added by the consumer.
// NT: token tiles of 8 (M <= 8 * NT).
template <int NT, bool SWIGLU, typename TOut, int RW, int KW>
__global__ void __launch_bounds__(RW * KW * 32)
gemv_bf16_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, const float* __restrict__ bias,
                 TOut* __restrict__ out, int M, int n_out, int K, long long ldx, long long ldo,
                 long long partial_stride) {
  __shared__ float red[KW > 1 ? RW * KW : 1][NT][32][4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  const int rw = warp / KW, kw = warp - rw * KW;
  const int tile = blockIdx.x * RW + rw;
  const int n_rows = SWIGLU ? 2 * n_out : n_out;                // rows of W
  int row_a, row_b;
  if (SWIGLU) { row_a = tile * 8 + g; row_b = n_out + row_a; if (row_a >= n_out) row_a = row_b = n_rows; }
  else { row_a = tile * 16 + g; row_b = row_a + 8; }
  const bool ok_a = row_a < n_rows, ok_b = row_b < n_rows;
  const bf16* wa = W + (size_t)(ok_a ? row_a : 0) * K;
  const bf16* wb = W + (size_t)(ok_b ? row_b : 0) * K;
  const bf16* xr[NT];
  bool ok_x[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    ok_x[t] = t * 8 + g < M;
    xr[t] = X + (size_t)(ok_x[t] ? t * 8 + g : 0) * ldx;
  }
  float acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f; }

  const int n_chunks = (K + KCHUNK - 1) / KCHUNK;
  const int per_split = (n_chunks + gridDim.y - 1) / gridDim.y;
  const int c_begin = blockIdx.y * per_split, c_end = min(n_chunks, c_begin + per_split);
  const int k_last = K - 8;                                      // the last 16-byte piece of a row
  for (int c0 = c_begin + kw; c0 < c_end; c0 += KW * UNROLL) {
    uint4 a[UNROLL], b[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {                           // all weight loads first: many bytes in flight
      const int kk = min((c0 + u * KW) * KCHUNK + t4 * 8, k_last);
      a[u] = __ldcs(reinterpret_cast<const uint4*>(wa + kk));
      b[u] = __ldcs(reinterpret_cast<const uint4*>(wb + kk));
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = c0 + u * KW;
      const int kraw = c * KCHUNK + t4 * 8;
      const bool in = c < c_end && kraw < K;
      const int kk = min(kraw, k_last);
      const uint4 av = mask16(a[u], in && ok_a), bv = mask16(b[u], in && ok_b);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint4 x = mask16(__ldg(reinterpret_cast<const uint4*>(xr[t] + kk)), ok_x[t]);
        mma16816(acc[t], av.x, bv.x, av.y, bv.y, x.x, x.y);
        mma16816(acc[t], av.z, bv.z, av.w, bv.w, x.z, x.w);
      }
    }
  }
  if (KW > 1) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
#pragma unroll
      for (int c = 0; c < 4; ++c) red[warp][t][lane][c] = acc[t][c];
    }
    __syncthreads();
    if (kw != 0) return;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < KW; ++w) v += red[rw * KW + w][t][lane][c];
        acc[t][c] = v;
      }
    }
  }
  // this lane holds, per token tile: rows g (c = 0, 1) and g + 8 (c = 2, 3) of tokens t4*2, t4*2 + 1
  TOut* dst = out + (size_t)blockIdx.y * partial_stride;
  const bool add_bias = bias && blockIdx.y == 0;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int token = t * 8 + t4 * 2 + cc;
      if (token >= M) continue;
      const float lo = acc[t][cc], hi = acc[t][cc + 2];
      if (SWIGLU) {
        const int o = tile * 8 + g;
        if (o < n_out) dst[(size_t)token * ldo + o] = to_out<TOut>(lo / (1.0f + expf(-lo)) * hi);
      } else {
        const int ra = tile * 16 + g, rb = ra + 8;
        if (ra < n_out) dst[(size_t)token * ldo + ra] = to_out<TOut>(lo + (add_bias ? bias[ra] : 0.0f));
        if (rb < n_out) dst[(size_t)token * ldo + rb] = to_out<TOut>(hi + (add_bias ? bias[rb] : 0.0f));
      }
    }
  }
}

template <int NT, bool SWIGLU, typename TOut, int RW, int KW>
int launch(const void* X, const void* W, const float* bias, void* out, int M, int n_out, int K, long long ldx,
           long long ldo, int k_splits, long long partial_stride, cudaStream_t stream) {
  const int tiles = SWIGLU ? (n_out + 7) / 8 : (n_out + 15) / 16;
  dim3 grid((tiles + RW - 1) / RW, k_splits);
  gemv_bf16_kernel<NT, SWIGLU, TOut, RW, KW><<<grid, RW * KW * 32, 0, stream>>>(
      (const bf16*)X, (const bf16*)W, bias, (TOut*)out, M, n_out, K, ldx, ldo, partial_stride);
  return IFX_LAUNCH_CHECK();
}

// Block shape by the amount of work: many row tiles -> each warp owns its rows over the whole K
// (no shared-memory sum); few row tiles -> the warps of a block share one row tile and cut K.
template <int NT, bool SWIGLU, typename TOut>
int by_shape(const void* X, const void* W, const float* bias, void* out, int M, int n_out, int K, long long ldx,
             long long ldo, int k_splits, long long partial_stride, cudaStream_t stream) {
  const int tiles = SWIGLU ? (n_out + 7) / 8 : (n_out + 15) / 16;
  const int chunks = (K + KCHUNK - 1) / KCHUNK / k_splits;
  if (tiles >= 1184) return launch<NT, SWIGLU, TOut, 4, 1>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
  if (chunks >= 128) return launch<NT, SWIGLU, TOut, 1, 8>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
  return launch<NT, SWIGLU, TOut, 1, 4>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
}

template <bool SWIGLU, typename TOut>
int by_tiles(const void* X, const void* W, const float* bias, void* out, int M, int n_out, int K, long long ldx,
             long long ldo, int k_splits, long long partial_stride, cudaStream_t stream) {
  if (M <= 8) return by_shape<1, SWIGLU, TOut>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
  if (M <= 16) return by_shape<2, SWIGLU, TOut>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
  return by_shape<4, SWIGLU, TOut>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
}
}  // namespace

// out[M, n_out] = X[M, K] * W^T (+ bias), W [n_out, K]; or, with swiglu != 0, W [2 * n_out, K] = [gate; up]
// and out = silu(X gate^T) * (X up^T).  M <= 32; K a multiple of 8; X rows and W 16-byte aligned.
// k_splits > 1 (float32 output, no swiglu): out is [k_splits, M, n_out], slice s holding the sum over
// the s-th part of K; the caller adds the slices (the fused residual-add + norm kernel does).
IFX_API int ifx_gemv_bf16(const void* X, const void* W, const float* bias, void* out, int out_dtype, int M,
                          int n_out, int K, long long ldx, long long ldo, int swiglu, int k_splits,
                          cudaStream_t stream) {
  if (M <= 0 || n_out <= 0) return 0;
  if (M > 32 || K <= 0 || (K & 7)) return IFX_ERR_UNSUPPORTED;
  if (((uintptr_t)X & 15) || ((uintptr_t)W & 15) || (ldx & 7)) return IFX_ERR_ALIGNMENT;
  if (swiglu && bias) return IFX_ERR_UNSUPPORTED;
  if (k_splits < 1 || k_splits > 64) return IFX_ERR_UNSUPPORTED;
  if (k_splits > 1 && (swiglu || out_dtype != IFX_F32)) return IFX_ERR_UNSUPPORTED;
  const long long ps = (long long)M * ldo;
  if (out_dtype == IFX_BF16)
    return swiglu ? by_tiles<true, bf16>(X, W, bias, out, M, n_out, K, ldx, ldo, 1, 0, stream)
                  : by_tiles<false, bf16>(X, W, bias, out, M, n_out, K, ldx, ldo, 1, 0, stream);
  if (out_dtype == IFX_F32)
    return swiglu ? by_tiles<true, float>(X, W, bias, out, M, n_out, K, ldx, ldo, 1, 0, stream)
                  : by_tiles<false, float>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, ps, stream);
  return IFX_ERR_UNSUPPORTED;
}
