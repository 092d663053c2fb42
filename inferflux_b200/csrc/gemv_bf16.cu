// Weight-streaming matrix product for a few rows of activations (decode):
// out[M, N] = X[M, K] * W[N, K]^T, bfloat16 in, float32 accumulation, M <= 16.
//
// The reference sends every dense projection to cuBLAS whatever M is
// (runtime/backends/cuda/native/cublas_gemm.cpp:84-102; its hand-written GEMV
// kernels are for quantized weights only).  At M of 1 to 16 the product is bound
// by reading W once, so this kernel is laid out around that read: the weights
// are the 16-row "A" operand of an m16n8k16 MMA and the tokens the 8-column "B"
// operand.  Each lane reads 16 contiguous bytes of two weight rows and 16 bytes
// of one token's activations per 32-wide K chunk; because a dot product does
// not care about the order of K, those 8 consecutive values feed two MMAs
// as they are, without shuffles.  To keep the read of W in flight each thread
// copies its 16-byte pieces with cp.async into a shared-memory ring of its own,
// six chunks deep (it reads back only what it copied, so no barrier is needed).
// The warps of a block take interleaved K chunks of the same row tiles and add
// their partial sums in shared memory in warp order; K may also be cut between
// blocks, whose float32 partial results the consumer adds (the fused
// residual-add + norm kernel does).
//
// SwiGLU mode: rows 0-7 of the tile come from the gate half of a stacked
// [gate; up] weight and rows 8-15 from the up half at the same index, so each
// lane holds gate and up of the same output and writes silu(gate) * up
// (runtime/backends/cuda/native/cuda_kernels.cu:137-149) without the
// intermediate [M, 2I] tensor.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint4 mask16(uint4 v, bool keep) {
  return keep ? v : make_uint4(0u, 0u, 0u, 0u);
}

// Weights go from global to shared memory with 16-byte cp.async, each thread into a ring of
// its own (it reads back only what it copied, so no barrier is needed): the copies of the next
// NST - 1 chunks stay in flight while a chunk is multiplied.  A copy whose source is out of range
// has source size 0 and fills zeros.
__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ T to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 to_out<bf16>(float v) { return __float2bfloat16_rn(v); }

constexpr int KCHUNK = 32, NST = 6;

// A block has KW warps that share a group of RT row tiles at a time (a tile is 16 weight rows, or 8 gate
// + 8 up rows in SwiGLU mode) and goes on to the group gridDim.x further until none is left: the grid is
// only as large as the GPU holds at once, and a warp's ring of copies runs on from one group into the
// next, so the read of W never drains between groups.  Warp kw takes the K chunks kw, kw + KW, ... of the
// block's K range for all RT tiles, so one 16-byte read of a token's activations feeds 2 * RT MMAs; the KW
// partial sums are added in shared memory in warp order.  gridDim.y > 1 cuts K between blocks: block y
// writes float32 partial sums partial_stride elements apart, to be added by the consumer.
// NT: token tiles of 8 (M <= 8 * NT).
template <int NT, bool SWIGLU, typename TOut, int RT, int KW>
__global__ void __launch_bounds__(KW * 32)
gemv_bf16_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, const float* __restrict__ bias,
                 TOut* __restrict__ out, int M, int n_out, int K, long long ldx, long long ldo,
                 long long partial_stride, int n_groups) {
  constexpr int THREADS = KW * 32;
  pdl_launch_dependents();
  extern __shared__ __align__(16) uint4 ring[];                 // [NST][2 * RT][threads]: a thread's slots are [..][..][tid]
  constexpr int NBUF = RT * NT >= 4 ? 1 : 2;                    // two buffers (if they fit): a group's sums are read while the next runs
  __shared__ float red[NBUF][KW][RT][NT][32][4];
  const int tid = threadIdx.x, lane = tid & 31, kw = tid >> 5, g = lane >> 2, t4 = lane & 3;
  const int n_rows = SWIGLU ? 2 * n_out : n_out;                // rows of W
  const int n_chunks = (K + KCHUNK - 1) / KCHUNK;
  const int per_split = (n_chunks + gridDim.y - 1) / gridDim.y;
  const int c_begin = blockIdx.y * per_split, c_end = min(n_chunks, c_begin + per_split);
  // this warp's chunks: c_begin + kw, + KW, ...
  const int n_my = c_begin + kw < c_end ? (c_end - c_begin - kw + KW - 1) / KW : 0;
  const int k_last = K - 8;                                      // the last 16-byte piece of a row
  const int my_groups = (int)blockIdx.x < n_groups ? (n_groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

  // the copying side: which group and chunk the next copy belongs to, and that group's rows
  const bf16* wrow[2 * RT];
  bool ok_row[2 * RT];
  auto set_rows = [&](int gi) {
    const int group = blockIdx.x + gi * gridDim.x;
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      const int tile = group * RT + r;
      int row_a, row_b;
      if (SWIGLU) { row_a = tile * 8 + g; row_b = n_out + row_a; if (row_a >= n_out) row_a = row_b = n_rows; }
      else { row_a = tile * 16 + g; row_b = row_a + 8; }
      ok_row[2 * r] = row_a < n_rows;
      ok_row[2 * r + 1] = row_b < n_rows;
      wrow[2 * r] = W + (size_t)(ok_row[2 * r] ? row_a : 0) * K;
      wrow[2 * r + 1] = W + (size_t)(ok_row[2 * r + 1] ? row_b : 0) * K;
    }
  };
  int is_g = n_my > 0 ? 0 : my_groups, is_j = 0, is_slot = 0;
  if (is_g < my_groups) set_rows(0);
  auto issue = [&]() {
    if (is_g < my_groups) {
      const int kraw = (c_begin + kw + is_j * KW) * KCHUNK + t4 * 8;
      const bool in = kraw < K;
      const int kk = min(kraw, k_last);
      uint4* slot = ring + (size_t)(is_slot * 2 * RT) * THREADS + tid;
#pragma unroll
      for (int r = 0; r < 2 * RT; ++r) cp_async16_zfill(slot + r * THREADS, wrow[r] + kk, in && ok_row[r]);
      if (++is_j == n_my) {
        is_j = 0;
        if (++is_g < my_groups) set_rows(is_g);
      }
    }
    cp_async_commit_group();
    is_slot = is_slot + 1 == NST ? 0 : is_slot + 1;
  };
#pragma unroll
  for (int j = 0; j < NST - 1; ++j) issue();
  // The weights are parameters, which no kernel of a step writes, so their first copies are issued before
  // this kernel waits for the one before it: the ring fills while that kernel drains.
  pdl_wait();

  const bf16* xr[NT];
  bool ok_x[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    ok_x[t] = t * 8 + g < M;
    xr[t] = X + (size_t)(ok_x[t] ? t * 8 + g : 0) * ldx;
  }
  // activations come from L1/L2 with plain loads, one chunk ahead of their use
  uint4 xn[NT];
  {
    const int kk = min((c_begin + kw) * KCHUNK + t4 * 8, k_last);
#pragma unroll
    for (int t = 0; t < NT; ++t) xn[t] = __ldg(reinterpret_cast<const uint4*>(xr[t] + kk));
  }
  TOut* dst = out + (size_t)blockIdx.y * partial_stride;
  const bool add_bias = bias && blockIdx.y == 0;
  int c_slot = 0;
  for (int gi = 0; gi < my_groups; ++gi) {
    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int t = 0; t < NT; ++t) { acc[r][t][0] = acc[r][t][1] = acc[r][t][2] = acc[r][t][3] = 0.0f; }
    for (int j = 0; j < n_my; ++j) {
      uint4 x[NT];
#pragma unroll
      for (int t = 0; t < NT; ++t) x[t] = mask16(xn[t], ok_x[t]);
      {
        const int jn = j + 1 < n_my ? j + 1 : 0;                   // the next group starts over at the first chunk
        const int kk = min((c_begin + kw + jn * KW) * KCHUNK + t4 * 8, k_last);
#pragma unroll
        for (int t = 0; t < NT; ++t) xn[t] = __ldg(reinterpret_cast<const uint4*>(xr[t] + kk));
      }
      cp_async_wait_group<NST - 2>();                              // this chunk has landed
      const uint4* slot = ring + (size_t)(c_slot * 2 * RT) * THREADS + tid;
      uint4 w[2 * RT];
#pragma unroll
      for (int r = 0; r < 2 * RT; ++r) w[r] = slot[r * THREADS];
      c_slot = c_slot + 1 == NST ? 0 : c_slot + 1;
      issue();                                                     // reuses the slot of the chunk before this one
#pragma unroll
      for (int r = 0; r < RT; ++r) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma16816(acc[r][t], w[2 * r].x, w[2 * r + 1].x, w[2 * r].y, w[2 * r + 1].y, x[t].x, x[t].y);
          mma16816(acc[r][t], w[2 * r].z, w[2 * r + 1].z, w[2 * r].w, w[2 * r + 1].w, x[t].z, x[t].w);
        }
      }
    }
    float (*rb)[RT][NT][32][4] = red[gi & (NBUF - 1)];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) rb[kw][r][t][lane][c] = acc[r][t][c];
    // With two buffers, one barrier per group: the buffer written now is read below by the warps that
    // finish a tile and is written again two groups on, after the next group's barrier, which those warps
    // reach only when done.
    __syncthreads();
    // warp r (< RT) finishes row tile r: this lane holds, per token tile, rows g (c = 0, 1) and
    // g + 8 (c = 2, 3) of tokens t4*2, t4*2 + 1
    const int r = kw < RT ? kw : 0;
    const int tile = ((int)blockIdx.x + gi * (int)gridDim.x) * RT + r;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (kw >= RT) break;
      float v[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < KW; ++w) sum += rb[w][r][t][lane][c];
        v[c] = sum;
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int token = t * 8 + t4 * 2 + cc;
        if (token >= M) continue;
        const float lo = v[cc], hi = v[cc + 2];
        if (SWIGLU) {
          const int o = tile * 8 + g;
          if (o < n_out) dst[(size_t)token * ldo + o] = to_out<TOut>(lo / (1.0f + expf(-lo)) * hi);
        } else {
          const int ra = tile * 16 + g, rb2 = ra + 8;
          if (ra < n_out) dst[(size_t)token * ldo + ra] = to_out<TOut>(lo + (add_bias ? bias[ra] : 0.0f));
          if (rb2 < n_out) dst[(size_t)token * ldo + rb2] = to_out<TOut>(hi + (add_bias ? bias[rb2] : 0.0f));
        }
      }
    }
    if (NBUF == 1) __syncthreads();
  }
  cp_async_wait_group<0>();
}

// Blocks of one shape that the GPU holds at once (asked once per shape); negative: a CUDA error.
template <int NT, bool SWIGLU, typename TOut, int RT, int KW>
int resident_blocks() {
  static int resident = 0;
  if (!resident) {
    auto kern = gemv_bf16_kernel<NT, SWIGLU, TOut, RT, KW>;
    const size_t smem = (size_t)NST * 2 * RT * KW * 32 * sizeof(uint4);
    // dynamic plus static shared memory passes 48 KB
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return -(int)e;
    int per_sm = 0, dev = 0, sms = 0;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, KW * 32, smem)) != cudaSuccess) return -(int)e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return -(int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return -(int)e;
    resident = per_sm * sms > 0 ? per_sm * sms : 1;
  }
  return resident;
}

// As many blocks as run at once, evened out so that each takes the same number of groups.
inline int grid_width(int resident, int n_groups, int k_splits) {
  int gx = resident / k_splits > 0 ? resident / k_splits : 1;
  if (gx > n_groups) gx = n_groups;
  const int rounds = (n_groups + gx - 1) / gx;
  return (n_groups + rounds - 1) / rounds;
}

template <int NT, bool SWIGLU, typename TOut, int RT, int KW>
int launch(const void* X, const void* W, const float* bias, void* out, int M, int n_out, int K, long long ldx,
           long long ldo, int k_splits, long long partial_stride, cudaStream_t stream) {
  const int tiles = SWIGLU ? (n_out + 7) / 8 : (n_out + 15) / 16;
  const int n_groups = (tiles + RT - 1) / RT;
  const size_t smem = (size_t)NST * 2 * RT * KW * 32 * sizeof(uint4);
  const int resident = resident_blocks<NT, SWIGLU, TOut, RT, KW>();
  if (resident < 0) return -resident;
  dim3 grid(grid_width(resident, n_groups, k_splits), k_splits);
  int ifx_rc = launch_pdl(gemv_bf16_kernel<NT, SWIGLU, TOut, RT, KW>, grid, dim3(KW * 32), smem, stream, (const bf16*)X,
                          (const bf16*)W, bias, (TOut*)out, M, n_out, K, ldx, ldo, partial_stride, n_groups);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

// Block shape by the amount of work: with plenty of row tiles a block takes two (the activations
// are read half as often); short K ranges get 4 warps instead of 8.
struct BlockShape { int rt, kw; };
inline BlockShape block_shape(int tiles, int K, int k_splits) {
  const int chunks = (K + KCHUNK - 1) / KCHUNK / k_splits;
  if (tiles * k_splits >= 1184 && chunks >= 64) return {2, 8};
  if (chunks >= 64) return {1, 8};
  return {1, 4};
}

template <int NT, bool SWIGLU, typename TOut>
int by_shape(const void* X, const void* W, const float* bias, void* out, int M, int n_out, int K, long long ldx,
             long long ldo, int k_splits, long long partial_stride, cudaStream_t stream) {
  const BlockShape bs = block_shape(SWIGLU ? (n_out + 7) / 8 : (n_out + 15) / 16, K, k_splits);
  if (bs.rt == 2) return launch<NT, SWIGLU, TOut, 2, 8>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
  if (bs.kw == 8) return launch<NT, SWIGLU, TOut, 1, 8>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
  return launch<NT, SWIGLU, TOut, 1, 4>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
}

template <bool SWIGLU, typename TOut>
int by_tiles(const void* X, const void* W, const float* bias, void* out, int M, int n_out, int K, long long ldx,
             long long ldo, int k_splits, long long partial_stride, cudaStream_t stream) {
  if (M <= 8) return by_shape<1, SWIGLU, TOut>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
  return by_shape<2, SWIGLU, TOut>(X, W, bias, out, M, n_out, K, ldx, ldo, k_splits, partial_stride, stream);
}
}  // namespace

// out[M, n_out] = X[M, K] * W^T (+ bias), W [n_out, K]; or, with swiglu != 0, W [2 * n_out, K] = [gate; up]
// and out = silu(X gate^T) * (X up^T).  M <= 16; K a multiple of 8; X rows and W 16-byte aligned.
// k_splits > 1 (float32 output, no swiglu): out is [k_splits, M, n_out], slice s holding the sum over
// the s-th part of K; the caller adds the slices (the fused residual-add + norm kernel does).
// W is read before the kernel has waited for the kernel launched before it in the stream, so W must
// not be the output of a kernel of this library launched directly before (weights are parameters).
IFX_API int ifx_gemv_bf16(const void* X, const void* W, const float* bias, void* out, int out_dtype, int M,
                          int n_out, int K, long long ldx, long long ldo, int swiglu, int k_splits,
                          cudaStream_t stream) {
  if (M <= 0 || n_out <= 0) return 0;
  if (M > 16 || K <= 0 || (K & 7)) return IFX_ERR_UNSUPPORTED;
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

// Into how many parts of K a product with float32 partial sums is best cut (1 to max_splits): the
// number that keeps the most warps at work at once, counted with the kernel's own block shapes and
// grid rule, the smallest such number within 15 percent.  It depends on n_out and K only, so the
// way a row is summed does not depend on the batch.  Negative: a CUDA error.
IFX_API int ifx_gemv_bf16_plan(int n_out, int K, int max_splits) {
  if (n_out <= 0 || K <= 0) return 1;
  const int tiles = (n_out + 15) / 16;
  const int n_chunks = (K + KCHUNK - 1) / KCHUNK;
  int warps[65];
  int best = 0;
  if (max_splits > 64) max_splits = 64;
  for (int s = 1; s <= max_splits; ++s) {
    warps[s] = 0;
    if (s > 1 && n_chunks / s < 16) break;
    const BlockShape bs = block_shape(tiles, K, s);
    const int resident = bs.rt == 2 ? resident_blocks<1, false, float, 2, 8>()
                       : bs.kw == 8 ? resident_blocks<1, false, float, 1, 8>()
                                    : resident_blocks<1, false, float, 1, 4>();
    if (resident < 0) return resident;
    const int n_groups = (tiles + bs.rt - 1) / bs.rt;
    warps[s] = grid_width(resident, n_groups, s) * s * bs.kw;
    if (warps[s] > best) best = warps[s];
  }
  for (int s = 1; s <= max_splits; ++s)
    if (warps[s] * 100 >= best * 85) return s;
  return 1;
}

IFX_STAMP_READER(ifx_stamps_gemv)
