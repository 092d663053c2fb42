// Paged grouped-query attention over the cache, any element type: the kernel
// of the float32 path, and the plain counterpart of the bfloat16 kernels.
//
// Reference formulas (runtime/backends/cuda/kernels/flash_attention.cu:52-173):
//   kv_head = head / (n_heads / n_kv);  s_j = (q . k_j) * scale  (scale after the dot, :127-141)
//   causal: key j visible to the query at position p iff j <= p (:70-71,85)
//   online softmax in float32 with expf, running max and sum (:143-171);  o = sum p_j v_j / sum p_j
// The reference runs one block per (query, head) over a dense per-sequence
// buffer.  Here one block takes 16 consecutive new tokens of one request and
// one head, reads keys and values through the request's block table in tiles
// of 32 keys, and serves prompt portions (any number of cached tokens before
// them) and single decoded tokens alike.  A window w > 0 hides keys j <= p - w.
//
// Tiles start at multiples of 32 keys and keys are added in index order, so in
// float32 the result for a token does not depend on how the prompt was cut.
#include "common.cuh"

namespace {
constexpr int BQ = 16;        // query rows per block (2 per warp, 8 warps)
constexpr int BKEYS = 32;     // keys per tile (one per lane)

struct AttnBatch {
  const int* block_tables;    // [n_entries, bt_stride] page of each logical block, -1 = given back
  int bt_stride;
  const int* tile_entry;      // [n_tiles] request entry of each query tile
  const int* tile_q0;         // [n_tiles] first new token (within the entry) of the tile
  const int* entry_q_start;   // [n_entries] row of the entry's first new token in q/out
  const int* entry_q_len;     // [n_entries] new tokens
  const int* entry_ctx_start; // [n_entries] tokens cached before them = position of the first new token
};

template <typename T, int NACC>
__global__ void __launch_bounds__(256)
attn_paged_generic_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                          PagedKV kv, AttnBatch b, int n_heads, int n_kv, int head_dim, float scale, int window) {
  pdl_enter();
  extern __shared__ float smem[];
  float* qs = smem;                               // [BQ][head_dim]
  float* ks = qs + BQ * head_dim;                 // [BKEYS][head_dim + 1]
  float* vs = ks + BKEYS * (head_dim + 1);        // [BKEYS][head_dim]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.x, head = blockIdx.y;
  const int e = b.tile_entry[tile];
  const int q0 = b.tile_q0[tile];
  const int rows = min(BQ, b.entry_q_len[e] - q0);
  if (rows <= 0) return;
  const int tok0 = b.entry_q_start[e] + q0;
  const int pos0 = b.entry_ctx_start[e] + q0;
  const int kvh = head / (n_heads / n_kv);
  const int* bt = b.block_tables + (size_t)e * b.bt_stride;
  const T* kc = (const T*)kv.k + (size_t)kvh * kv.head_stride;
  const T* vc = (const T*)kv.v + (size_t)kvh * kv.head_stride;

  for (int idx = tid; idx < BQ * head_dim; idx += blockDim.x) {
    const int r = idx / head_dim, d = idx - r * head_dim;
    qs[idx] = r < rows ? Num<T>::to_f(q[(size_t)(tok0 + r) * q_stride + (size_t)head * head_dim + d]) : 0.0f;
  }

  const int r0 = warp * 2, r1 = r0 + 1;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[2][NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) { o[0][a] = 0.0f; o[1][a] = 0.0f; }

  const int kend = pos0 + rows - 1;               // last key any row of the tile may see
  int kstart = 0;
  if (window > 0) kstart = max(0, pos0 - window + 1) & ~(BKEYS - 1);

  for (int k0 = kstart; k0 <= kend; k0 += BKEYS) {
    __syncthreads();
    for (int idx = tid; idx < BKEYS * head_dim; idx += blockDim.x) {
      const int j = idx / head_dim, d = idx - j * head_dim;
      const int key = k0 + j;
      float kval = 0.0f, vval = 0.0f;
      if (key <= kend) {
        const int page = bt[key >> kv.page_shift];
        if (page >= 0) {
          const size_t off = (size_t)page * kv.page_stride + (size_t)(key & (kv.page_size - 1)) * head_dim + d;
          kval = Num<T>::to_f(kc[off]);
          vval = Num<T>::to_f(vc[off]);
        }
      }
      ks[j * (head_dim + 1) + d] = kval;
      vs[j * head_dim + d] = vval;
    }
    __syncthreads();
    if (r0 < rows) {                               // warp-uniform
      const bool two = r1 < rows;
      const float* kr = ks + lane * (head_dim + 1);
      const float* qa = qs + r0 * head_dim;
      const float* qb = qs + r1 * head_dim;
      float s0 = 0.0f, s1 = 0.0f;
      for (int d = 0; d < head_dim; ++d) {
        const float kd = kr[d];
        s0 = fmaf(qa[d], kd, s0);
        s1 = fmaf(qb[d], kd, s1);
      }
      const int key = k0 + lane;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        if (rr == 1 && !two) break;
        const int p = pos0 + r0 + rr;
        const bool visible = key <= p && (window <= 0 || key > p - window);
        const float s = visible ? (rr ? s1 : s0) * scale : -INFINITY;
        const float m_new = fmaxf(m[rr], warp_max(s));
        if (m_new == -INFINITY) continue;          // nothing visible to this row yet (warp-uniform)
        const float alpha = expf(m[rr] - m_new);   // exp(-inf) = 0 on the first visible tile
        const float pj = visible ? expf(s - m_new) : 0.0f;
        l[rr] = l[rr] * alpha + warp_sum(pj);
        m[rr] = m_new;
#pragma unroll
        for (int a = 0; a < NACC; ++a) o[rr][a] *= alpha;
        for (int j = 0; j < BKEYS; ++j) {
          const float pjj = __shfl_sync(0xffffffffu, pj, j);
          if (pjj == 0.0f) continue;               // warp-uniform; also keeps stale values out
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
            const int d = lane + 32 * a;
            if (d < head_dim) o[rr][a] = fmaf(pjj, vs[j * head_dim + d], o[rr][a]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = r0 + rr;
    if (r >= rows) continue;
    const float inv = l[rr] > 0.0f ? 1.0f / l[rr] : 0.0f;
    T* orow = out + (size_t)(tok0 + r) * out_stride + (size_t)head * head_dim;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int d = lane + 32 * a;
      if (d < head_dim) orow[d] = Num<T>::from_f(o[rr][a] * inv);
    }
  }
}

template <typename T, int NACC>
int launch_generic(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnBatch b,
                   int n_tiles, int n_heads, int n_kv, int head_dim, float scale, int window, cudaStream_t stream) {
  const size_t smem = ((size_t)BQ * head_dim + (size_t)BKEYS * (head_dim + 1) + (size_t)BKEYS * head_dim) * sizeof(float);
  auto kern = attn_paged_generic_kernel<T, NACC>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_tiles, n_heads);
  const int ifx_rc = launch_pdl(kern, grid, dim3(256), smem, stream, (const T*)q, q_stride, (T*)out, out_stride, kv, b, n_heads, n_kv,
                                head_dim, scale, window);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

template <typename T>
int dispatch_generic(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnBatch b,
                     int n_tiles, int n_heads, int n_kv, int head_dim, float scale, int window, cudaStream_t stream) {
  const int nacc = (head_dim + 31) / 32;
  if (nacc <= 1) return launch_generic<T, 1>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, stream);
  if (nacc <= 2) return launch_generic<T, 2>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, stream);
  if (nacc <= 4) return launch_generic<T, 4>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, stream);
  return launch_generic<T, 8>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, stream);
}
}  // namespace

// Query tiles are 16 tokens of one entry: tile_entry / tile_q0 list them.
// head_dim: any positive size up to 256; n_heads must be a multiple of n_kv.
IFX_API int ifx_attn_paged_generic(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                   void* k_layer, void* v_layer, long long page_stride, int page_size,
                                   const int* block_tables, int bt_stride,
                                   const int* tile_entry, const int* tile_q0, int n_tiles,
                                   const int* entry_q_start, const int* entry_q_len, const int* entry_ctx_start,
                                   int n_heads, int n_kv, int head_dim, float scale, int window,
                                   cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (head_dim < 1 || head_dim > 256 || n_kv < 1 || n_heads % n_kv) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  if (n_heads > 65535) return IFX_ERR_UNSUPPORTED;
  PagedKV kv;
  kv.k = k_layer; kv.v = v_layer; kv.page_stride = page_stride;
  kv.head_stride = page_size * head_dim; kv.page_size = page_size; kv.page_shift = 0;
  while ((1 << kv.page_shift) < page_size) ++kv.page_shift;
  AttnBatch b{block_tables, bt_stride, tile_entry, tile_q0, entry_q_start, entry_q_len, entry_ctx_start};
  if (dtype == IFX_F32)
    return dispatch_generic<float>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, stream);
  if (dtype == IFX_BF16)
    return dispatch_generic<bf16>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, stream);
  return IFX_ERR_UNSUPPORTED;
}
