// bfloat16 paged grouped-query attention on tensor cores: one kernel for prompt
// portions (any number of cached tokens before them) and one for single
// decoded tokens (split over the keys, then merged).
//
// Same formulas as the generic kernel (attention_generic.cu): kv head = head /
// (n_heads / n_kv), s = (q . k) * scale, causal with an optional window,
// float32 online softmax, o = sum p v / sum p.  The reference's counterparts
// are a scalar block-per-query kernel for ratios other than 2/4/8
// (runtime/backends/cuda/kernels/flash_attention.cu:52-173), an mma.sync
// kernel that converts bfloat16 q and k to float16
// (runtime/backends/cuda/kernels/flash_attention_mma.cuh:153-379), and scalar
// decode kernels with a fixed 8-way split (flash_attention.cu:468-570,775-973).
//
// Here q.k and p.v both run as m16n8k16 bfloat16 MMAs with float32
// accumulation; keys and values come from the pages by 16-byte cp.async into
// XOR-swizzled shared memory and are read with ldmatrix.  In the decode kernel
// the 16 rows of an MMA tile are the query heads that share a kv head, so a
// page is read once for all of them.
#include "common.cuh"
#include "rope_math.cuh"
#include <type_traits>

namespace {

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int sz = valid ? 16 : 0;    // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4_at(unsigned (&r)[4], unsigned saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
__device__ __forceinline__ void ldmatrix_x4_trans_at(unsigned (&r)[4], unsigned saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

constexpr float LOG2E = 1.4426950408889634f;

// 2^x by the hardware approximation (about 2 units in the last place of float32); 2^-inf = 0
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// A tile in shared memory: rows of HD bfloat16 = HD/8 chunks of 16 bytes; chunk c of
// row r is stored at chunk (c ^ (r & 7)) so that ldmatrix reads are conflict-free.
template <int HD>
__device__ __forceinline__ bf16* tile_chunk(bf16* tile, int row, int chunk) {
  return tile + row * HD + ((chunk ^ (row & 7)) << 3);
}

// Copy `n_rows` keys (or values) starting at absolute key index `key0` into a tile.
// Rows outside [lo, hi) or in pages that were given back are zero-filled.
template <int HD, int THREADS>
__device__ __forceinline__ void load_kv_tile(bf16* tile, const bf16* base, const PagedKV& kv, const int* bt,
                                             int key0, int n_rows, int lo, int hi, int tid) {
  constexpr int CPR = HD / 8;
  for (int idx = tid; idx < n_rows * CPR; idx += THREADS) {
    const int r = idx / CPR, c = idx - r * CPR;
    const int key = key0 + r;
    bool ok = key >= lo && key < hi;
    const bf16* src = base;
    if (ok) {
      const int page = bt[key >> kv.page_shift];
      ok = page >= 0;
      if (ok) src = base + (size_t)page * kv.page_stride + (size_t)(key & (kv.page_size - 1)) * HD + c * 8;
    }
    cp_async16(tile_chunk<HD>(tile, r, c), src, ok);
  }
}

// Copy 64 keys and their values (absolute key index key0 ..) into two tiles with 128 threads:
// two threads per key, one block-table lookup per thread for both; a pair of lanes covers 32
// contiguous bytes per instruction.  Rows outside [lo, hi) or in pages given back are zero-filled.
// `bt` may point to a copy of the block table in shared memory that starts at logical block
// `bt_first` (the copy removes a global load from the path between two tiles).
template <int HD>
__device__ __forceinline__ void load_kv_tile64(bf16* ktile, bf16* vtile, const bf16* kbase, const bf16* vbase,
                                               const PagedKV& kv, const int* bt, int key0, int lo, int hi, int tid,
                                               int bt_first = 0) {
  constexpr int CPR = HD / 8;
  const int r = tid >> 1, half = tid & 1;
  const int key = key0 + r;
  bool ok = key >= lo && key < hi;
  size_t off = 0;
  if (ok) {
    const int page = bt[(key >> kv.page_shift) - bt_first];
    ok = page >= 0;
    if (ok) off = (size_t)page * kv.page_stride + (size_t)(key & (kv.page_size - 1)) * HD;
  }
  const bf16* ksrc = kbase + off;
  const bf16* vsrc = vbase + off;
  bf16* krow = ktile + r * HD;
  bf16* vrow = vtile + r * HD;
  const int sw = r & 7;
#pragma unroll
  for (int j = 0; j < CPR / 2; ++j) {
    const int c = j * 2 + half;
    cp_async16(krow + ((c ^ sw) << 3), ksrc + c * 8, ok);
    cp_async16(vrow + ((c ^ sw) << 3), vsrc + c * 8, ok);
  }
}

// The same with the row's page already looked up by the caller (page < 0: the row is zero-filled).
template <int HD>
__device__ __forceinline__ void load_kv_tile64_paged(bf16* ktile, bf16* vtile, const bf16* kbase, const bf16* vbase,
                                                     const PagedKV& kv, int page, int key, int tid) {
  constexpr int CPR = HD / 8;
  const int r = tid >> 1, half = tid & 1;
  const bool ok = page >= 0;
  const size_t off = ok ? (size_t)page * kv.page_stride + (size_t)(key & (kv.page_size - 1)) * HD : 0;
  const bf16* ksrc = kbase + off;
  const bf16* vsrc = vbase + off;
  bf16* krow = ktile + r * HD;
  bf16* vrow = vtile + r * HD;
  const int sw = r & 7;
#pragma unroll
  for (int j = 0; j < CPR / 2; ++j) {
    const int c = j * 2 + half;
    cp_async16(krow + ((c ^ sw) << 3), ksrc + c * 8, ok);
    cp_async16(vrow + ((c ^ sw) << 3), vsrc + c * 8, ok);
  }
}

constexpr int BT_CACHE = 1024;      // block-table entries a block keeps in shared memory

struct AttnMeta {
  const int* block_tables; int bt_stride;
  const int* entry_q_start; const int* entry_q_len; const int* entry_ctx_start;
};

// ------------------------------------------------------------------ prompts
// One block: 64 consecutive new tokens of one entry (16 per warp), one head.
template <int HD>
__global__ void __launch_bounds__(128)
attn_prefill_bf16_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                         PagedKV kv, AttnMeta m, const int* __restrict__ tile_entry, const int* __restrict__ tile_q0,
                         int n_heads, int n_kv, float scale, int window) {
  pdl_enter();
  constexpr int BQ = 64, BK = 64, KS = HD / 16, DT = HD / 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* ks = reinterpret_cast<bf16*>(smem_raw);              // [2][BK][HD]
  bf16* vs = ks + 2 * BK * HD;                               // [2][BK][HD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  // tiles run last to first and heads fastest: within a request the later tiles see more
  // keys, and the longest blocks (of every head) should start first
  const int tile = gridDim.y - 1 - blockIdx.y;
  const int e = tile_entry[tile], q0 = tile_q0[tile], head = blockIdx.x;
  const int rows = min(BQ, m.entry_q_len[e] - q0);
  if (rows <= 0) return;
  const int tok0 = m.entry_q_start[e] + q0;
  const int pos0 = m.entry_ctx_start[e] + q0;
  const int kvh = head / (n_heads / n_kv);
  const int* bt = m.block_tables + (size_t)e * m.bt_stride;
  const bf16* kbase = (const bf16*)kv.k + (size_t)kvh * kv.head_stride;
  const bf16* vbase = (const bf16*)kv.v + (size_t)kvh * kv.head_stride;

  // this warp's 16 query rows as A fragments
  const int wr0 = warp * 16;
  unsigned qa[KS][4];
  {
    const bf16* qb = q + (size_t)head * HD;
    const int ra = wr0 + g, rb = wr0 + g + 8;
    const unsigned* pa = reinterpret_cast<const unsigned*>(qb + (size_t)(tok0 + ra) * q_stride);
    const unsigned* pb = reinterpret_cast<const unsigned*>(qb + (size_t)(tok0 + rb) * q_stride);
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      qa[k][0] = ra < rows ? pa[k * 8 + t4] : 0u;
      qa[k][1] = rb < rows ? pb[k * 8 + t4] : 0u;
      qa[k][2] = ra < rows ? pa[k * 8 + 4 + t4] : 0u;
      qa[k][3] = rb < rows ? pb[k * 8 + 4 + t4] : 0u;
    }
  }
  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.0f, 0.0f};
  const float sl2 = scale * LOG2E;

  const int kend = pos0 + rows;                                  // keys [.., kend) may be seen
  const int kfirst = window > 0 ? max(0, pos0 - window + 1) : 0; // first key the first row may see
  const int t_begin = kfirst / BK, t_end = (kend - 1) / BK;
  __shared__ int bt_s[BT_CACHE];                                 // this block's slice of the block table
  int bt_first = 0;
  {
    const int b0 = kfirst >> kv.page_shift, b1 = (kend - 1) >> kv.page_shift;
    if (b1 - b0 < BT_CACHE) {
      for (int i = tid; i <= b1 - b0; i += 128) bt_s[i] = bt[b0 + i];
      bt = bt_s;
      bt_first = b0;
      __syncthreads();
    }
  }
  const int pa_row = pos0 + wr0 + g, pb_row = pa_row + 8;        // positions of this thread's two rows
  const int warp_last = pos0 + min(wr0 + 15, rows - 1);

  // shared-memory byte offsets of this lane's ldmatrix rows, swizzle included (they do not depend on the tile)
  const unsigned ks_addr = (unsigned)__cvta_generic_to_shared(ks), vs_addr = (unsigned)__cvta_generic_to_shared(vs);
  unsigned koff[KS], voff[DT / 2];
  {
    const int j = lane >> 3, r = lane & 7;
#pragma unroll
    for (int k = 0; k < KS; ++k) koff[k] = (unsigned)((((j >> 1) * 8 + r) * HD + (((k * 2 + (j & 1)) ^ r) << 3)) * 2);
#pragma unroll
    for (int dp = 0; dp < DT / 2; ++dp) voff[dp] = (unsigned)((((j & 1) * 8 + r) * HD + (((dp * 2 + (j >> 1)) ^ r) << 3)) * 2);
  }
  load_kv_tile64<HD>(ks, vs, kbase, vbase, kv, bt, t_begin * BK, kfirst, kend, tid, bt_first);
  cp_async_commit();
  for (int t = t_begin; t <= t_end; ++t) {
    const int st = (t - t_begin) & 1;
    if (t < t_end) {
      load_kv_tile64<HD>(ks + (st ^ 1) * BK * HD, vs + (st ^ 1) * BK * HD, kbase, vbase, kv, bt, (t + 1) * BK,
                         kfirst, kend, tid, bt_first);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = t * BK;
    const bool active = wr0 < rows && key0 <= warp_last &&
                        (window <= 0 || key0 + BK > pos0 + wr0 - window + 1);
    if (active) {
      const unsigned kt = ks_addr + (unsigned)(st * BK * HD * 2);
      const unsigned vt = vs_addr + (unsigned)(st * BK * HD * 2);
      float s[BK / 8][4];
#pragma unroll
      for (int n = 0; n < BK / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f; }
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        unsigned kb[BK / 16][4];                                 // the step's four fragments first, then its MMAs
#pragma unroll
        for (int np = 0; np < BK / 16; ++np) ldmatrix_x4_at(kb[np], kt + (unsigned)(np * 16 * HD * 2) + koff[k]);
#pragma unroll
        for (int np = 0; np < BK / 16; ++np) {                   // two n-tiles (16 keys) per ldmatrix.x4
          mma_bf16(s[np * 2], qa[k], kb[np][0], kb[np][1]);
          mma_bf16(s[np * 2 + 1], qa[k], kb[np][2], kb[np][3]);
        }
      }
      // mask (diagonal, window and edge tiles only), row maxima of the raw scores
      const bool need_mask = key0 + BK - 1 > pos0 + wr0 || window > 0 || key0 < kfirst;
      if (need_mask) {
#pragma unroll
        for (int n = 0; n < BK / 8; ++n) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int key = key0 + n * 8 + t4 * 2 + (c & 1);
            const int p = (c & 2) ? pb_row : pa_row;
            const bool vis = key <= p && key < kend && (window <= 0 || key > p - window);
            if (!vis) s[n][c] = -INFINITY;
          }
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < BK / 8; ++n) {
        mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
      }
      // running maxima are kept in raw-score units; exponents are taken of (s - m) * scale * log2(e)
      float alpha[2], msc[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float mnew = fmaxf(mrow[h], mx[h]);
        msc[h] = mnew == -INFINITY ? 0.0f : mnew * sl2;          // a row that has seen nothing yet
        alpha[h] = fast_exp2(mrow[h] * sl2 - msc[h]);            // 2^-inf = 0 on the first visible tile
        mrow[h] = mnew;
      }
      float ls[2] = {0.0f, 0.0f};
#pragma unroll
      for (int n = 0; n < BK / 8; ++n) {
        s[n][0] = fast_exp2(fmaf(s[n][0], sl2, -msc[0]));
        s[n][1] = fast_exp2(fmaf(s[n][1], sl2, -msc[0]));
        s[n][2] = fast_exp2(fmaf(s[n][2], sl2, -msc[1]));
        s[n][3] = fast_exp2(fmaf(s[n][3], sl2, -msc[1]));
        ls[0] += s[n][0] + s[n][1];
        ls[1] += s[n][2] + s[n][3];
      }
      lrow[0] = lrow[0] * alpha[0] + ls[0];
      lrow[1] = lrow[1] * alpha[1] + ls[1];
      if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {   // a maximum moved: rescale o
#pragma unroll
        for (int d = 0; d < DT; ++d) { o[d][0] *= alpha[0]; o[d][1] *= alpha[0]; o[d][2] *= alpha[1]; o[d][3] *= alpha[1]; }
      }
      {
        // value fragments run two ldmatrix ahead of the MMAs that use them
        constexpr int NV = (BK / 16) * (DT / 2);                  // (key step, d pair) in order
        unsigned vb[3][4];
        ldmatrix_x4_trans_at(vb[0], vt + voff[0]);
        if (NV > 1) ldmatrix_x4_trans_at(vb[1], vt + (unsigned)((1 / (DT / 2)) * 16 * HD * 2) + voff[1 % (DT / 2)]);
        unsigned pa[4];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int kk = i / (DT / 2), dp = i % (DT / 2);
          if (dp == 0) {                                          // 16 keys per k-step
            pa[0] = pack_bf16(s[kk * 2][0], s[kk * 2][1]);
            pa[1] = pack_bf16(s[kk * 2][2], s[kk * 2][3]);
            pa[2] = pack_bf16(s[kk * 2 + 1][0], s[kk * 2 + 1][1]);
            pa[3] = pack_bf16(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
          }
          if (i + 2 < NV) {
            const int k2 = (i + 2) / (DT / 2), d2 = (i + 2) % (DT / 2);
            ldmatrix_x4_trans_at(vb[(i + 2) % 3], vt + (unsigned)(k2 * 16 * HD * 2) + voff[d2]);
          }
          mma_bf16(o[dp * 2], pa, vb[i % 3][0], vb[i % 3][1]);   // two d-tiles (16 dims) per ldmatrix.x4.trans
          mma_bf16(o[dp * 2 + 1], pa, vb[i % 3][2], vb[i % 3][3]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 1);
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 2);
  }
  const float inv0 = lrow[0] > 0.0f ? 1.0f / lrow[0] : 0.0f;
  const float inv1 = lrow[1] > 0.0f ? 1.0f / lrow[1] : 0.0f;
  const int ra = wr0 + g, rb = ra + 8;
  bf16* oa = out + (size_t)(tok0 + ra) * out_stride + (size_t)head * HD;
  bf16* ob = out + (size_t)(tok0 + rb) * out_stride + (size_t)head * HD;
#pragma unroll
  for (int d = 0; d < DT; ++d) {
    if (ra < rows) *reinterpret_cast<unsigned*>(oa + d * 8 + t4 * 2) = pack_bf16(o[d][0] * inv0, o[d][1] * inv0);
    if (rb < rows) *reinterpret_cast<unsigned*>(ob + d * 8 + t4 * 2) = pack_bf16(o[d][2] * inv1, o[d][3] * inv1);
  }
}

// ------------------------------------------------------------------- decode
// One block: one decoding entry, up to 8 query heads of one kv head, one split of the keys.
// The product is laid out transposed, S^T = K Q^T and O^T = V^T P^T: the 16 rows of an MMA
// tile are 16 keys (or 16 head dims) and its 8 columns are the query heads that share the kv
// head, so with 7 heads per kv head 7/8 of every MMA is useful work and the accumulator is
// [head_dim x 8] (32 registers).  P^T goes from accumulator layout to operand layout by one
// movmatrix per 8 keys.  The block streams keys and values in tiles of 64 through a ring of
// DSTAGES shared-memory stages (loads run ahead of the math); each of the 4 warps takes 16
// keys of a tile and keeps its own running (max, sum, o), merged at the end.  Partial
// results go to scratch for the merge kernel; with one split the block writes the output.
constexpr int DSTAGES = 3;

__device__ __forceinline__ unsigned movmatrix_trans(unsigned x) {
  unsigned y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

// What the kernel needs to make q, k and v of its token itself (PREP): the product's output before bias and
// rotation, as bfloat16 rows (q) or as float32 partial sums [n_partials][n_tokens][width].
struct QkvPrep {
  const float* bias;        // [width] or null
  const float* cos_t;       // [n_tokens, HD / 2]
  const float* sin_t;
  const int* slot_map;      // [n_tokens]: page * page_size + offset of the token's key and value; null: this layer writes none
  const float* partials;    // or null
  int n_partials;
  long long part_stride;    // n_tokens * width
};

// PREP: the kernel takes the place of the bias/rotation/cache-write kernel for the token it decodes.  Every
// block adds the bias to and rotates the query heads it works on (into shared memory); the block whose
// part of the keys ends with the token's own position does the same for the key, adds the bias to the
// value, writes both to the cache and only then loads that tile.  With more than 8 query heads per kv head
// several blocks write the same bytes.
template <int HD, bool PREP>
__global__ void __launch_bounds__(128)
attn_decode_bf16_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                        PagedKV kv, AttnMeta m, const int* __restrict__ dec_entries,
                        float* __restrict__ part_o, float* __restrict__ part_ml,
                        int n_heads, int n_kv, int head_chunks, float scale, int window, int n_splits, QkvPrep prep) {
  // Up to pdl_wait() below the block reads only what no kernel of the step writes (the step's
  // metadata) and keys and values of tokens older than the one being decoded.
  pdl_launch_dependents();
  constexpr int KS = HD / 16, BK = 64, TK = 16;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* ring = reinterpret_cast<bf16*>(smem_raw);             // [DSTAGES][K|V][BK][HD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  const int e = dec_entries[blockIdx.x];
  const int kvh = blockIdx.y / head_chunks, hc = blockIdx.y - kvh * head_chunks;
  const int split = blockIdx.z;
  const int ratio = n_heads / n_kv;
  const int h0 = kvh * ratio + hc * 8;
  const int nrows = min(8, ratio - hc * 8);                     // query heads of this block
  const int tok = m.entry_q_start[e];
  const int len = m.entry_ctx_start[e] + 1;                     // keys [0, len) exist; the query sits at len - 1
  const int kfirst = window > 0 ? max(0, len - window) : 0;
  const int total = len - kfirst;
  int chunk = (total + n_splits - 1) / n_splits;
  chunk = (chunk + BK - 1) / BK * BK;
  const int kb = kfirst + split * chunk, ke = min(len, kb + chunk);
  const int* bt = m.block_tables + (size_t)e * m.bt_stride;
  const bf16* kbase = (const bf16*)kv.k + (size_t)kvh * kv.head_stride;
  const bf16* vbase = (const bf16*)kv.v + (size_t)kvh * kv.head_stride;
  const int dec = blockIdx.x;
  // this block's slice of the block table, copied to shared memory once
  __shared__ int bt_s[BT_CACHE];
  int bt_first = 0;
  if (kb < ke) {
    const int b0 = kb >> kv.page_shift, b1 = (ke - 1) >> kv.page_shift;
    if (b1 - b0 < BT_CACHE) {
      for (int i = tid; i <= b1 - b0; i += 128) bt_s[i] = bt[b0 + i];
      bt = bt_s;
      bt_first = b0;
      __syncthreads();
    }
  }

  // o[dd]: rows d = dd*16 + g (regs 0,1) and + 8 (regs 2,3); columns heads 2*t4 (regs 0,2) and 2*t4+1 (regs 1,3)
  float o[KS][4];
#pragma unroll
  for (int d = 0; d < KS; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }
  float mcol[2] = {-INFINITY, -INFINITY}, lcol[2] = {0.0f, 0.0f};   // heads 2*t4, 2*t4+1

  const int t_begin = kb / BK, t_end = kb < ke ? (ke - 1) / BK : t_begin - 1, n_t = t_end - t_begin + 1;
  auto first_tiles = [&]() {
#pragma unroll
    for (int p = 0; p < DSTAGES - 1; ++p) {
      if (p < n_t) {
        bf16* st = ring + (size_t)p * 2 * BK * HD;
        load_kv_tile64<HD>(st, st + BK * HD, kbase, vbase, kv, bt, (t_begin + p) * BK, kb, ke, tid, bt_first);
      }
      cp_async_commit();
    }
  };
  // The kernel before this one writes the newest token's key and value (position len - 1).  If none
  // of the first tiles holds it, their copies start before this kernel waits for that one.
  const bool early = kb < ke && min(ke, (t_begin + DSTAGES - 1) * BK) <= len - 1;
  if (early) first_tiles();
  pdl_wait();

  if (kb < ke) {                                                // block-uniform
    unsigned qb[KS][2];                                         // Q^T as the B operand: k = d, n = head g
    if constexpr (PREP) {
      __shared__ __align__(16) bf16 q_s[8 * HD];
      constexpr int HALF = HD / 2, HV = HALF / 8;               // 8-wide groups per half head
      const int width = (n_heads + 2 * n_kv) * HD;
      const bf16* row = q + (size_t)tok * q_stride;
      const float* part = prep.partials ? prep.partials + (size_t)tok * width : nullptr;
      const float* ct = prep.cos_t + (size_t)tok * HALF;
      const float* st = prep.sin_t + (size_t)tok * HALF;
      const int slot = (prep.slot_map && ke == len) ? prep.slot_map[tok] : -1;   // ke == len: the token's own position is ours
      const int q_items = nrows * HV, k_items = slot >= 0 ? HV : 0, v_items = slot >= 0 ? HD / 8 : 0;
      auto items = [&](auto part_tag, auto batch_tag) {
        constexpr bool PART = decltype(part_tag)::value;
        constexpr int NB = decltype(batch_tag)::value;            // slices asked for together
        for (int w = tid; w < q_items + k_items + v_items; w += 128) {
          if (w < q_items + k_items) {
            const bool is_q = w < q_items;
            const int hl = is_q ? w / HV : 0, i = (is_q ? w - hl * HV : w - q_items) * 8;
            const int base = (is_q ? h0 + hl : n_heads + kvh) * HD;
            uint4 lo, hi;
            rope_pairs8<PART, NB>(row, part, prep.n_partials, prep.part_stride, prep.bias, ct, st, base + i, HALF, i, lo, hi);
            bf16* dst = is_q ? q_s + hl * HD
                             : (bf16*)kv.k + (size_t)(slot >> kv.page_shift) * kv.page_stride + (size_t)kvh * kv.head_stride +
                                   (size_t)(slot & (kv.page_size - 1)) * HD;
            *reinterpret_cast<uint4*>(dst + i) = lo;
            *reinterpret_cast<uint4*>(dst + HALF + i) = hi;
          } else {
            const int d = (w - q_items - k_items) * 8;
            bf16* dst = (bf16*)kv.v + (size_t)(slot >> kv.page_shift) * kv.page_stride + (size_t)kvh * kv.head_stride +
                        (size_t)(slot & (kv.page_size - 1)) * HD;
            *reinterpret_cast<uint4*>(dst + d) =
                biased8<PART, NB>(row, part, prep.n_partials, prep.part_stride, prep.bias, (n_heads + n_kv + kvh) * HD + d);
          }
        }
      };
      if (!part) items(std::false_type{}, std::integral_constant<int, 1>{});
      else if (prep.n_partials == 1) items(std::true_type{}, std::integral_constant<int, 1>{});   // (the library's float32 product)
      else items(std::true_type{}, std::integral_constant<int, 4>{});
      if (slot >= 0) __threadfence();                           // the key and value are in memory before the tile that holds them is copied
      __syncthreads();
      const unsigned* pq = reinterpret_cast<const unsigned*>(q_s + (size_t)g * HD);
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        qb[k][0] = g < nrows ? pq[k * 8 + t4] : 0u;
        qb[k][1] = g < nrows ? pq[k * 8 + 4 + t4] : 0u;
      }
    } else {
      const unsigned* pq = reinterpret_cast<const unsigned*>(q + (size_t)tok * q_stride + (size_t)(h0 + g) * HD);
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        qb[k][0] = g < nrows ? pq[k * 8 + t4] : 0u;
        qb[k][1] = g < nrows ? pq[k * 8 + 4 + t4] : 0u;
      }
    }
    const float sl2 = scale * LOG2E;
    if (!early) first_tiles();
    const unsigned ring_addr = (unsigned)__cvta_generic_to_shared(ring);
    unsigned koff[KS], voff[KS];                                // this lane's ldmatrix rows within a stage, swizzle included
    {
      const int j = lane >> 3, r = lane & 7;
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        koff[k] = (unsigned)(((warp * TK + (j & 1) * 8 + r) * HD + (((k * 2 + (j >> 1)) ^ r) << 3)) * 2);
        voff[k] = (unsigned)(((BK + warp * TK + (j >> 1) * 8 + r) * HD + (((k * 2 + (j & 1)) ^ r) << 3)) * 2);
      }
    }
    for (int i = 0; i < n_t; ++i) {
      cp_async_wait<DSTAGES - 2>();                             // tile i has landed (for this thread)
      __syncthreads();                                          // ... for all; and tile i - 1 is no longer read
      {
        const int nx = i + DSTAGES - 1;
        if (nx < n_t) {
          bf16* st = ring + (size_t)(nx % DSTAGES) * 2 * BK * HD;
          load_kv_tile64<HD>(st, st + BK * HD, kbase, vbase, kv, bt, (t_begin + nx) * BK, kb, ke, tid, bt_first);
        }
        cp_async_commit();
      }
      const int key0 = (t_begin + i) * BK + warp * TK;          // this warp's 16 keys of the tile
      if (key0 >= ke || key0 + TK <= kb) continue;              // warp-uniform: nothing of ours in range
      const unsigned stage = ring_addr + (unsigned)((i % DSTAGES) * 2 * BK * HD * 2);
      float s[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};   // (key g | g+8) x (head 2*t4 | 2*t4+1)
      {
        unsigned ka[KS][4];                                     // all key fragments first, then the MMAs
#pragma unroll
        for (int k = 0; k < KS; ++k) ldmatrix_x4_at(ka[k], stage + koff[k]);
#pragma unroll
        for (int k = 0; k < KS; k += 2) {                       // two chains of sums, so an MMA does not wait for the one before it
          mma_bf16(s, ka[k], qb[k][0], qb[k][1]);
          if (k + 1 < KS) mma_bf16(s1, ka[k + 1], qb[k + 1][0], qb[k + 1][1]);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) s[c] += s1[c];
      }
      const bool in0 = key0 + g >= kb && key0 + g < ke, in1 = key0 + g + 8 >= kb && key0 + g + 8 < ke;
      if (!in0) { s[0] = -INFINITY; s[1] = -INFINITY; }
      if (!in1) { s[2] = -INFINITY; s[3] = -INFINITY; }
      float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
      // maxima are kept in raw-score units (and, scaled, in the partial results)
      float alpha[2], msc[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {                             // over the 8 lanes that hold the other keys
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
        const float mnew = fmaxf(mcol[h], mx[h]);
        msc[h] = mnew == -INFINITY ? 0.0f : mnew * sl2;
        alpha[h] = fast_exp2(mcol[h] * sl2 - msc[h]);
        mcol[h] = mnew;
      }
      float p[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) p[c] = fast_exp2(fmaf(s[c], sl2, -msc[c & 1]));
      lcol[0] = lcol[0] * alpha[0] + p[0] + p[2];
      lcol[1] = lcol[1] * alpha[1] + p[1] + p[3];
      if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {   // a maximum moved: rescale o
#pragma unroll
        for (int d = 0; d < KS; ++d) { o[d][0] *= alpha[0]; o[d][1] *= alpha[1]; o[d][2] *= alpha[0]; o[d][3] *= alpha[1]; }
      }
      // P^T as the B operand (k = key, n = head): transpose the two 8x8 blocks
      const unsigned pb0 = movmatrix_trans(pack_bf16(p[0], p[1]));
      const unsigned pb1 = movmatrix_trans(pack_bf16(p[2], p[3]));
      {
        unsigned va[KS][4];                                     // V^T as the A operand: rows d, columns keys
#pragma unroll
        for (int d = 0; d < KS; ++d) ldmatrix_x4_trans_at(va[d], stage + voff[d]);
#pragma unroll
        for (int d = 0; d < KS; ++d) mma_bf16(o[d], va[d], pb0, pb1);
      }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mcol[h] = mcol[h] == -INFINITY ? -INFINITY : mcol[h] * sl2;   // to exponent units for the merges
      lcol[h] += __shfl_xor_sync(0xffffffffu, lcol[h], 4);
      lcol[h] += __shfl_xor_sync(0xffffffffu, lcol[h], 8);
      lcol[h] += __shfl_xor_sync(0xffffffffu, lcol[h], 16);
    }
  }
  // merge the four warps through shared memory (the ring is free now)
  __syncthreads();
  float* red_o = reinterpret_cast<float*>(smem_raw);            // [4][8 heads][HD]
  float* red_ml = red_o + 4 * 8 * HD;                           // [4][8][2]
#pragma unroll
  for (int d = 0; d < KS; ++d) {
    float* r0 = red_o + ((size_t)warp * 8 + t4 * 2) * HD + d * 16 + g;
    r0[0] = o[d][0]; r0[HD] = o[d][1]; r0[8] = o[d][2]; r0[HD + 8] = o[d][3];
  }
  if (g == 0) {
    red_ml[(warp * 8 + t4 * 2) * 2] = mcol[0];     red_ml[(warp * 8 + t4 * 2) * 2 + 1] = lcol[0];
    red_ml[(warp * 8 + t4 * 2 + 1) * 2] = mcol[1]; red_ml[(warp * 8 + t4 * 2 + 1) * 2 + 1] = lcol[1];
  }
  __syncthreads();
  for (int idx = tid; idx < nrows * HD; idx += 128) {
    const int row = idx / HD, d = idx - row * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_ml[(w * 8 + row) * 2]);
    float l = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red_ml[(w * 8 + row) * 2];
      const float f = mw == -INFINITY ? 0.0f : fast_exp2(mw - mm);
      l += red_ml[(w * 8 + row) * 2 + 1] * f;
      acc += red_o[((size_t)w * 8 + row) * HD + d] * f;
    }
    const int head = h0 + row;
    if (n_splits == 1) {
      out[(size_t)tok * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    } else {
      const size_t p = ((size_t)dec * n_heads + head) * n_splits + split;
      part_o[p * HD + d] = acc;
      if (d == 0) { part_ml[p * 2] = mm; part_ml[p * 2 + 1] = l; }
    }
  }
}

// merge the splits: grid (n_dec, n_heads), HD threads.  Up to 16 splits (what the plan gives at the usual
// batch sizes) are loaded in one go, maxima, sums and outputs together, so the block waits for memory once.
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         bf16* __restrict__ out, long long out_stride, const int* __restrict__ dec_entries,
                                         const int* __restrict__ entry_q_start, int n_heads, int head_dim, int n_splits) {
  pdl_launch_dependents();
  const int dec = blockIdx.x, head = blockIdx.y;
  const int tok = entry_q_start[dec_entries[dec]];            // the step's metadata: read before the wait
  pdl_wait();
  const size_t p0 = ((size_t)dec * n_heads + head) * n_splits;
  if (n_splits <= 16) {
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
      float2 ml[16];
      float po[16];
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < n_splits) {
          ml[s] = *reinterpret_cast<const float2*>(part_ml + (p0 + s) * 2);
          po[s] = part_o[(p0 + s) * head_dim + d];
        }
      float mm = -INFINITY;
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < n_splits) mm = fmaxf(mm, ml[s].x);
      float l = 0.0f, acc = 0.0f;
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < n_splits) {
          const float f = ml[s].x == -INFINITY ? 0.0f : fast_exp2(ml[s].x - mm);
          l += ml[s].y * f;
          acc += po[s] * f;
        }
      out[(size_t)tok * out_stride + (size_t)head * head_dim + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    }
    return;
  }
  float mm = -INFINITY;
#pragma unroll 8
  for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, part_ml[(p0 + s) * 2]);
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float l = 0.0f, acc = 0.0f;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[(p0 + s) * 2];
      const float f = ms == -INFINITY ? 0.0f : fast_exp2(ms - mm);
      l += part_ml[(p0 + s) * 2 + 1] * f;
      acc += part_o[(p0 + s) * head_dim + d] * f;
    }
    out[(size_t)tok * out_stride + (size_t)head * head_dim + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
  }
}

// ------------------------------------------------------------------ decode, shared out evenly
// The same attention of single tokens, with the work shared out evenly: the 64-key tiles of all units (a
// unit = entry x kv head x chunk of 8 query heads) form one list, and block b takes the tiles
// [b q, (b + 1) q) of it, q = max(DEC_MIN_TILES, ceil(all tiles / blocks)), whatever units they belong to.
// Every block therefore streams the same number of bytes, however the contexts' lengths differ and
// whether or not the number of units divides the number of blocks the GPU holds.  A unit whose tiles fall
// to several blocks is written as partial results, one per block (piece), and merged by the second
// kernel; a unit that one block does whole is written as output at once.  Each block derives its share
// from the step's metadata alone, before it waits for the kernel before it.
constexpr int DEC_MAX = 1024;        // single tokens in a step that the kernel takes
constexpr int DEC_MIN_TILES = 4;     // a block's share is at least this many tiles

struct DecWalk {                     // a place in the list of tiles: entry d (of dec_entries), unit j of it, tile t of the unit
  int d, j, t, f;                    // f: the place in the whole list
  int len, kfirst, tile0, n_tiles;   // of entry d: keys [kfirst, len) in tiles tile0 .. tile0 + n_tiles - 1
  const int* bt;
};

__device__ __forceinline__ int dec_tiles(int len, int window, int& kfirst) {
  kfirst = window > 0 ? max(0, len - window) : 0;
  return (len - 1) / 64 - kfirst / 64 + 1;
}

// tiles per entry -> P_s[0 .. n_dec] (exclusive prefix; P_s[n_dec] = all of them); 128 threads
__device__ __forceinline__ void dec_prefix(int* P_s, const AttnMeta& m, const int* dec_entries, int n_dec, int window) {
  __shared__ int warp_tot[4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = (n_dec + 127) / 128;
  const int b = min(n_dec, tid * chunk), e = min(n_dec, b + chunk);
  int mine = 0;
  for (int i = b; i < e; ++i) {
    int kf;
    const int t = dec_tiles(m.entry_ctx_start[dec_entries[i]] + 1, window, kf);
    P_s[i + 1] = t;
    mine += t;
  }
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int before = incl - mine;
  for (int w = 0; w < warp; ++w) before += warp_tot[w];
  if (tid == 0) P_s[0] = 0;
  for (int i = b; i < e; ++i) { before += P_s[i + 1]; P_s[i + 1] = before; }   // a thread's own entries only
  __syncthreads();
}

template <int HD>
__global__ void __launch_bounds__(128)
attn_decode_even_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                        PagedKV kv, AttnMeta m, const int* __restrict__ dec_entries, int n_dec,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ piece_count,
                        int n_heads, int n_kv, int head_chunks, float scale, int window, int max_pieces,
                        int* __restrict__ error_flag) {
  pdl_launch_dependents();
  constexpr int KS = HD / 16, BK = 64, TK = 16;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* ring = reinterpret_cast<bf16*>(smem_raw);             // [DSTAGES][K|V][BK][HD]
  __shared__ int P_s[DEC_MAX + 1];
  __shared__ float red[2][32][KS * 4 + 4];                     // two warps' partial results, lane by lane
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  const int ratio = n_heads / n_kv, H = n_kv * head_chunks;
  // Up to pdl_wait() below the block reads only what no kernel of the step writes (the step's metadata)
  // and keys and values of tokens older than the ones being decoded.
  dec_prefix(P_s, m, dec_entries, n_dec, window);
  const int W = H * P_s[n_dec];
  const int share = max(DEC_MIN_TILES, (W + (int)gridDim.x - 1) / (int)gridDim.x);
  const int x0 = (int)blockIdx.x * share, x1 = min(W, x0 + share);
  if (x0 >= x1) {                                              // nothing falls to this block
    pdl_wait();                                                // no kernel of the step ends before the one before it has
    return;
  }

  auto enter = [&](DecWalk& w) {                               // the entry's own figures, on arriving at entry w.d
    if (w.d < 0 || w.d >= n_dec) {                             // cannot happen; never read outside the list
      if (error_flag) atomicExch(error_flag, IFX_DEVICE_ERR_DECODE_PIECES + 1);
      w.d = 0;
    }
    const int e = dec_entries[w.d];
    w.len = m.entry_ctx_start[e] + 1;
    w.n_tiles = dec_tiles(w.len, window, w.kfirst);
    w.tile0 = w.kfirst / BK;
    w.bt = m.block_tables + (size_t)e * m.bt_stride;
  };
  auto advance = [&](DecWalk& w) {
    ++w.f;
    if (++w.t == w.n_tiles) {
      w.t = 0;
      if (++w.j == H) {
        w.j = 0;
        ++w.d;
        if (w.f < x1) enter(w);
      }
    }
  };
  DecWalk ld;                                                  // the next tile to copy
  {
    int lo = 0, hi = n_dec - 1;
    while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (H * P_s[mid] <= x0) lo = mid; else hi = mid - 1; }
    ld.d = lo;
    enter(ld);
    const int rem = x0 - H * P_s[lo];
    ld.j = rem / ld.n_tiles;
    ld.t = rem - ld.j * ld.n_tiles;
    ld.f = x0;
  }
  DecWalk cs = ld;                                             // the tile being worked on

  int ld_page = -1;                                            // the page of this thread's row (tid / 2) of tile ld, or -1: no such key
  auto look_up = [&]() {
    const int key = (ld.tile0 + ld.t) * BK + (tid >> 1);
    ld_page = (ld.f < x1 && key >= ld.kfirst && key < ld.len) ? __ldg(ld.bt + (key >> kv.page_shift)) : -1;
  };
  look_up();
  auto copy_tile = [&](int stage) {                            // all threads: tile ld of the list -> ring[stage]
    const int kvh = ld.j / head_chunks;
    bf16* st = ring + (size_t)stage * 2 * BK * HD;
    load_kv_tile64_paged<HD>(st, st + BK * HD, (const bf16*)kv.k + (size_t)kvh * kv.head_stride,
                             (const bf16*)kv.v + (size_t)kvh * kv.head_stride, kv, ld_page, (ld.tile0 + ld.t) * BK + (tid >> 1), tid);
    advance(ld);
    look_up();                                                 // the next tile's page: the load is under way until its copy starts
  };
  // The first copies start before the wait as long as they hold no token of this step (the last tile of a
  // unit does: the kernel before this one writes it).
  int started = 0;
  while (started < DSTAGES - 1 && ld.f < x1 && ld.t != ld.n_tiles - 1) {
    copy_tile(started);
    cp_async_commit();
    ++started;
  }
  pdl_wait();
  for (; started < DSTAGES - 1; ++started) {
    if (ld.f < x1) copy_tile(started);
    cp_async_commit();
  }

  const float sl2 = scale * LOG2E;
  const unsigned ring_addr = (unsigned)__cvta_generic_to_shared(ring);
  unsigned koff[KS], voff[KS];                                  // this lane's ldmatrix rows within a stage, swizzle included
  {
    const int jj = lane >> 3, r = lane & 7;
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      koff[k] = (unsigned)(((warp * TK + (jj & 1) * 8 + r) * HD + (((k * 2 + (jj >> 1)) ^ r) << 3)) * 2);
      voff[k] = (unsigned)(((BK + warp * TK + (jj >> 1) * 8 + r) * HD + (((k * 2 + (jj & 1)) ^ r) << 3)) * 2);
    }
  }
  // o[dd]: rows d = dd*16 + g (regs 0,1) and + 8 (regs 2,3); columns heads 2*t4 (regs 0,2) and 2*t4+1 (regs 1,3)
  float o[KS][4];
  float mcol[2], lcol[2];
  unsigned qb[KS][2];                                          // Q^T as the B operand: k = d, n = head g
  int tok = 0, h0 = 0, nrows = 0;
  bool fresh = true;                                           // the next tile opens a piece
  for (int i = 0; cs.f < x1; ++i) {
    if (fresh) {
      fresh = false;
      const int kvh = cs.j / head_chunks, hc = cs.j - kvh * head_chunks;
      h0 = kvh * ratio + hc * 8;
      nrows = min(8, ratio - hc * 8);
      tok = m.entry_q_start[dec_entries[cs.d]];
#pragma unroll
      for (int d = 0; d < KS; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }
      mcol[0] = mcol[1] = -INFINITY;
      lcol[0] = lcol[1] = 0.0f;
      const unsigned* pq = reinterpret_cast<const unsigned*>(q + (size_t)tok * q_stride + (size_t)(h0 + g) * HD);
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        qb[k][0] = g < nrows ? pq[k * 8 + t4] : 0u;
        qb[k][1] = g < nrows ? pq[k * 8 + 4 + t4] : 0u;
      }
    }
    cp_async_wait<DSTAGES - 2>();                               // tile i has landed (for this thread)
    __syncthreads();                                            // ... for all; and tile i - 1 is no longer read
    if (ld.f < x1) copy_tile((i + DSTAGES - 1) % DSTAGES);
    cp_async_commit();
    const int kb = cs.kfirst, ke = cs.len;
    const int key0 = (cs.tile0 + cs.t) * BK + warp * TK;        // this warp's 16 keys of the tile
    if (key0 < ke && key0 + TK > kb) {                          // warp-uniform: something of ours is in range
      const unsigned stage = ring_addr + (unsigned)((i % DSTAGES) * 2 * BK * HD * 2);
      float s[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};   // (key g | g+8) x (head 2*t4 | 2*t4+1)
      {
        unsigned ka[KS][4];                                     // all key fragments first, then the MMAs
#pragma unroll
        for (int k = 0; k < KS; ++k) ldmatrix_x4_at(ka[k], stage + koff[k]);
#pragma unroll
        for (int k = 0; k < KS; k += 2) {                       // two chains of sums, so an MMA does not wait for the one before it
          mma_bf16(s, ka[k], qb[k][0], qb[k][1]);
          if (k + 1 < KS) mma_bf16(s1, ka[k + 1], qb[k + 1][0], qb[k + 1][1]);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) s[c] += s1[c];
      }
      const bool in0 = key0 + g >= kb && key0 + g < ke, in1 = key0 + g + 8 >= kb && key0 + g + 8 < ke;
      if (!in0) { s[0] = -INFINITY; s[1] = -INFINITY; }
      if (!in1) { s[2] = -INFINITY; s[3] = -INFINITY; }
      float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
      float alpha[2], msc[2];                                   // maxima are kept in raw-score units
#pragma unroll
      for (int h = 0; h < 2; ++h) {                             // over the 8 lanes that hold the other keys
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
        const float mnew = fmaxf(mcol[h], mx[h]);
        msc[h] = mnew == -INFINITY ? 0.0f : mnew * sl2;
        alpha[h] = fast_exp2(mcol[h] * sl2 - msc[h]);
        mcol[h] = mnew;
      }
      float p[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) p[c] = fast_exp2(fmaf(s[c], sl2, -msc[c & 1]));
      lcol[0] = lcol[0] * alpha[0] + p[0] + p[2];
      lcol[1] = lcol[1] * alpha[1] + p[1] + p[3];
      if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {   // a maximum moved: rescale o
#pragma unroll
        for (int d = 0; d < KS; ++d) { o[d][0] *= alpha[0]; o[d][1] *= alpha[1]; o[d][2] *= alpha[0]; o[d][3] *= alpha[1]; }
      }
      // P^T as the B operand (k = key, n = head): transpose the two 8x8 blocks
      const unsigned pb0 = movmatrix_trans(pack_bf16(p[0], p[1]));
      const unsigned pb1 = movmatrix_trans(pack_bf16(p[2], p[3]));
      {
        unsigned va[KS][4];                                     // V^T as the A operand: rows d, columns keys
#pragma unroll
        for (int d = 0; d < KS; ++d) ldmatrix_x4_trans_at(va[d], stage + voff[d]);
#pragma unroll
        for (int d = 0; d < KS; ++d) mma_bf16(o[d], va[d], pb0, pb1);
      }
    }
    if (cs.t == cs.n_tiles - 1 || cs.f == x1 - 1) {             // the piece ends here (block-uniform): the four warps' results become one
      fresh = true;
      float mm[2], ll[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mm[h] = mcol[h] == -INFINITY ? -INFINITY : mcol[h] * sl2;   // to exponent units
        ll[h] = lcol[h];
        ll[h] += __shfl_xor_sync(0xffffffffu, ll[h], 4);
        ll[h] += __shfl_xor_sync(0xffffffffu, ll[h], 8);
        ll[h] += __shfl_xor_sync(0xffffffffu, ll[h], 16);
      }
      auto put = [&](int slot) {
        float* r = red[slot][lane];
#pragma unroll
        for (int d = 0; d < KS; ++d) { r[d * 4] = o[d][0]; r[d * 4 + 1] = o[d][1]; r[d * 4 + 2] = o[d][2]; r[d * 4 + 3] = o[d][3]; }
        r[KS * 4] = mm[0]; r[KS * 4 + 1] = mm[1]; r[KS * 4 + 2] = ll[0]; r[KS * 4 + 3] = ll[1];
      };
      auto take = [&](int slot) {
        const float* r = red[slot][lane];
        float fa[2], fb[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float mo = r[KS * 4 + h], mn = fmaxf(mm[h], mo);
          fa[h] = mm[h] == -INFINITY ? 0.0f : fast_exp2(mm[h] - mn);
          fb[h] = mo == -INFINITY ? 0.0f : fast_exp2(mo - mn);
          ll[h] = ll[h] * fa[h] + r[KS * 4 + 2 + h] * fb[h];
          mm[h] = mn;
        }
#pragma unroll
        for (int d = 0; d < KS; ++d) {
          o[d][0] = o[d][0] * fa[0] + r[d * 4] * fb[0];
          o[d][1] = o[d][1] * fa[1] + r[d * 4 + 1] * fb[1];
          o[d][2] = o[d][2] * fa[0] + r[d * 4 + 2] * fb[0];
          o[d][3] = o[d][3] * fa[1] + r[d * 4 + 3] * fb[1];
        }
      };
      if (warp >= 2) put(warp - 2);
      __syncthreads();
      if (warp < 2) take(warp);
      __syncthreads();
      if (warp == 1) put(0);
      __syncthreads();
      if (warp == 0) {
        take(0);
        const int xs = H * P_s[cs.d] + cs.j * cs.n_tiles;       // where the unit starts in the list
        const int first = xs / share, pieces = (xs + cs.n_tiles - 1) / share - first + 1;
        bool pieces_ok = true;
        const int piece = (int)blockIdx.x - first;
        if (pieces > max_pieces || piece < 0 || piece >= pieces) {                              // the caller's bound on the contexts was too low: say so, write nothing
          if (error_flag && lane == 0) atomicExch(error_flag, IFX_DEVICE_ERR_DECODE_PIECES);
          pieces_ok = false;
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int hl = 2 * t4 + c;
          if (hl < nrows && g == 0) piece_count[cs.d * n_heads + h0 + hl] = pieces_ok ? pieces : 0;   // for the merge kernel
          if (hl < nrows && pieces_ok) {
            const int head = h0 + hl;
            if (pieces == 1) {
              const float inv = ll[c] > 0.0f ? 1.0f / ll[c] : 0.0f;
              bf16* dst = out + (size_t)tok * out_stride + (size_t)head * HD;
#pragma unroll
              for (int d = 0; d < KS; ++d) {
                dst[d * 16 + g] = __float2bfloat16_rn(o[d][c] * inv);
                dst[d * 16 + g + 8] = __float2bfloat16_rn(o[d][c + 2] * inv);
              }
            } else {
              const size_t pp = ((size_t)cs.d * n_heads + head) * max_pieces + piece;
              float* dst = part_o + pp * HD;
#pragma unroll
              for (int d = 0; d < KS; ++d) { dst[d * 16 + g] = o[d][c]; dst[d * 16 + g + 8] = o[d][c + 2]; }
              if (g == 0) { part_ml[pp * 2] = mm[c]; part_ml[pp * 2 + 1] = ll[c]; }
            }
          }
        }
      }
    }
    advance(cs);
  }
  cp_async_wait<0>();
}

// merge the pieces of the units that several blocks shared: grid (n_dec, n_heads), HD threads.  piece_count
// [n_dec, n_heads]: into how many pieces the attention kernel cut the head's keys (1: it wrote the output itself).
__global__ void attn_decode_even_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int* __restrict__ piece_count, bf16* __restrict__ out,
                                              long long out_stride, const int* __restrict__ dec_entries,
                                              const int* __restrict__ entry_q_start, int n_heads, int head_dim,
                                              int max_pieces) {
  pdl_launch_dependents();
  const int dec = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
  const int tok = entry_q_start[dec_entries[dec]];            // the step's metadata: read before the wait
  pdl_wait();
  const int n_pieces = piece_count[dec * n_heads + head];
  if (n_pieces <= 1) return;
  const size_t p0 = ((size_t)dec * n_heads + head) * max_pieces;
  if (n_pieces <= 16) {
    for (int d = tid; d < head_dim; d += blockDim.x) {
      float2 ml[16];
      float po[16];
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < n_pieces) {
          ml[s] = *reinterpret_cast<const float2*>(part_ml + (p0 + s) * 2);
          po[s] = part_o[(p0 + s) * head_dim + d];
        }
      float mm = -INFINITY;
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < n_pieces) mm = fmaxf(mm, ml[s].x);
      float l = 0.0f, acc = 0.0f;
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < n_pieces) {
          const float f = ml[s].x == -INFINITY ? 0.0f : fast_exp2(ml[s].x - mm);
          l += ml[s].y * f;
          acc += po[s] * f;
        }
      out[(size_t)tok * out_stride + (size_t)head * head_dim + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    }
    return;
  }
  float mm = -INFINITY;
#pragma unroll 8
  for (int s = 0; s < n_pieces; ++s) mm = fmaxf(mm, part_ml[(p0 + s) * 2]);
  for (int d = tid; d < head_dim; d += blockDim.x) {
    float l = 0.0f, acc = 0.0f;
#pragma unroll 8
    for (int s = 0; s < n_pieces; ++s) {
      const float ms = part_ml[(p0 + s) * 2];
      const float f = ms == -INFINITY ? 0.0f : fast_exp2(ms - mm);
      l += part_ml[(p0 + s) * 2 + 1] * f;
      acc += part_o[(p0 + s) * head_dim + d] * f;
    }
    out[(size_t)tok * out_stride + (size_t)head * head_dim + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
  }
}

PagedKV make_kv(void* k_layer, void* v_layer, long long page_stride, int page_size, int head_dim) {
  PagedKV kv;
  kv.k = k_layer; kv.v = v_layer; kv.page_stride = page_stride;
  kv.head_stride = page_size * head_dim; kv.page_size = page_size; kv.page_shift = 0;
  while ((1 << kv.page_shift) < page_size) ++kv.page_shift;
  return kv;
}

template <int HD>
int launch_prefill(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnMeta m,
                   const int* tile_entry, const int* tile_q0, int n_tiles, int n_heads, int n_kv, float scale,
                   int window, cudaStream_t stream) {
  const size_t smem = (size_t)4 * 64 * HD * sizeof(bf16);
  auto kern = attn_prefill_bf16_kernel<HD>;
  {  // dynamic plus static shared memory may pass 48 KB
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int ifx_rc = launch_pdl(kern, dim3(n_heads, n_tiles), dim3(128), smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride, kv, m,
                                                      tile_entry, tile_q0, n_heads, n_kv, scale, window);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

template <int HD, bool PREP>
int launch_decode(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnMeta m,
                  const int* dec_entries, int n_dec, float* part_o, float* part_ml, int n_heads, int n_kv,
                  float scale, int window, int n_splits, QkvPrep prep, cudaStream_t stream) {
  const size_t stage_bytes = (size_t)DSTAGES * 2 * 64 * HD * sizeof(bf16);
  const size_t red_bytes = (size_t)4 * 8 * HD * sizeof(float) + 4 * 8 * 2 * sizeof(float);
  const size_t smem = stage_bytes > red_bytes ? stage_bytes : red_bytes;
  auto kern = attn_decode_bf16_kernel<HD, PREP>;
  {  // dynamic plus static shared memory may pass 48 KB
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int ratio = n_heads / n_kv;
  const int head_chunks = (ratio + 7) / 8;
  int rc = launch_pdl(kern, dim3(n_dec, n_kv * head_chunks, n_splits), dim3(128), smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride, kv, m, dec_entries, part_o, part_ml, n_heads, n_kv,
      head_chunks, scale, window, n_splits, prep);
  if (!rc) rc = IFX_LAUNCH_CHECK();
  if (rc || n_splits == 1) return rc;
  rc = launch_pdl(attn_decode_merge_kernel, dim3(n_dec, n_heads), dim3(HD < 128 ? HD : 128), 0, stream, part_o, part_ml, (bf16*)out, out_stride, dec_entries, m.entry_q_start, n_heads, HD, n_splits);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
// Blocks of the even-share decode kernel that the GPU holds at once (asked once per head size); negative: a CUDA error.
template <int HD>
int even_resident_blocks() {
  static int resident = 0;
  if (!resident) {
    const size_t smem = (size_t)DSTAGES * 2 * 64 * HD * sizeof(bf16);
    auto kern = attn_decode_even_kernel<HD>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return -(int)e;
    int per_sm = 0, dev = 0, sms = 0;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 128, smem)) != cudaSuccess) return -(int)e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return -(int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return -(int)e;
    resident = per_sm * sms > 0 ? per_sm * sms : 1;
  }
  return resident;
}

// Pieces a unit can fall into when no context is longer than max_keys: a block's share is at least
// DEC_MIN_TILES tiles, and at least the unit's own tiles times the units per entry over the blocks.
inline int even_max_pieces(int max_keys, int blocks, int units_per_entry) {
  const int tiles = (max_keys + 63) / 64 + 1;                  // a window may begin in the middle of a tile
  const int by_min = (tiles + DEC_MIN_TILES - 2) / DEC_MIN_TILES + 1, by_blocks = blocks / units_per_entry + 2;
  return by_min < by_blocks ? by_min : by_blocks;
}

template <int HD>
int launch_decode_even(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnMeta m,
                       const int* dec_entries, int n_dec, float* part_o, float* part_ml, int* piece_count, int n_heads,
                       int n_kv, float scale, int window, int max_pieces, int* error_flag, cudaStream_t stream) {
  const int blocks = even_resident_blocks<HD>();
  if (blocks < 0) return -blocks;
  const size_t smem = (size_t)DSTAGES * 2 * 64 * HD * sizeof(bf16);
  const int head_chunks = (n_heads / n_kv + 7) / 8;
  int rc = launch_pdl(attn_decode_even_kernel<HD>, dim3(blocks), dim3(128), smem, stream, (const bf16*)q, q_stride,
                      (bf16*)out, out_stride, kv, m, dec_entries, n_dec, part_o, part_ml, piece_count, n_heads, n_kv, head_chunks,
                      scale, window, max_pieces, error_flag);
  if (!rc) rc = IFX_LAUNCH_CHECK();
  if (rc) return rc;
  rc = launch_pdl(attn_decode_even_merge_kernel, dim3(n_dec, n_heads), dim3(HD < 128 ? HD : 128), 0, stream, (const float*)part_o,
                  (const float*)part_ml, (const int*)piece_count, (bf16*)out, out_stride, dec_entries, m.entry_q_start, n_heads, HD,
                  max_pieces);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
}  // namespace

// head_dim 64 or 128; page_size a power of two; q rows 4-byte aligned.
// Query tiles are 64 tokens of one entry (tile_entry / tile_q0).
IFX_API int ifx_attn_prefill_bf16(const void* q, long long q_stride, void* out, long long out_stride,
                                  void* k_layer, void* v_layer, long long page_stride, int page_size,
                                  const int* block_tables, int bt_stride, const int* tile_entry, const int* tile_q0,
                                  int n_tiles, const int* entry_q_start, const int* entry_q_len,
                                  const int* entry_ctx_start, int n_heads, int n_kv, int head_dim, float scale,
                                  int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (n_kv < 1 || n_heads % n_kv || n_tiles > 65535) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  if ((q_stride & 1) || (out_stride & 1) || ((uintptr_t)q & 3) || ((uintptr_t)out & 3)) return IFX_ERR_ALIGNMENT;
  if ((page_stride & 7) || ((uintptr_t)k_layer & 15) || ((uintptr_t)v_layer & 15)) return IFX_ERR_ALIGNMENT;
  PagedKV kv = make_kv(k_layer, v_layer, page_stride, page_size, head_dim);
  AttnMeta m{block_tables, bt_stride, entry_q_start, entry_q_len, entry_ctx_start};
  if (head_dim == 128)
    return launch_prefill<128>(q, q_stride, out, out_stride, kv, m, tile_entry, tile_q0, n_tiles, n_heads, n_kv, scale, window, stream);
  if (head_dim == 64)
    return launch_prefill<64>(q, q_stride, out, out_stride, kv, m, tile_entry, tile_q0, n_tiles, n_heads, n_kv, scale, window, stream);
  return IFX_ERR_UNSUPPORTED;
}

// Scratch: part_o float32 [n_dec * n_heads * n_splits * head_dim], part_ml float32
// [n_dec * n_heads * n_splits * 2] (unused when n_splits == 1).
IFX_API int ifx_attn_decode_bf16(const void* q, long long q_stride, void* out, long long out_stride,
                                 void* k_layer, void* v_layer, long long page_stride, int page_size,
                                 const int* block_tables, int bt_stride, const int* dec_entries, int n_dec,
                                 const int* entry_q_start, const int* entry_q_len, const int* entry_ctx_start,
                                 float* part_o, float* part_ml, int n_heads, int n_kv, int head_dim, float scale,
                                 int window, int n_splits, cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (n_kv < 1 || n_heads % n_kv || n_splits < 1 || n_splits > 65535) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  if ((q_stride & 1) || ((uintptr_t)q & 3)) return IFX_ERR_ALIGNMENT;
  if ((page_stride & 7) || ((uintptr_t)k_layer & 15) || ((uintptr_t)v_layer & 15)) return IFX_ERR_ALIGNMENT;
  if (n_splits > 1 && (!part_o || !part_ml)) return IFX_ERR_UNSUPPORTED;
  PagedKV kv = make_kv(k_layer, v_layer, page_stride, page_size, head_dim);
  AttnMeta m{block_tables, bt_stride, entry_q_start, entry_q_len, entry_ctx_start};
  if (head_dim == 128)
    return launch_decode<128, false>(q, q_stride, out, out_stride, kv, m, dec_entries, n_dec, part_o, part_ml, n_heads, n_kv, scale, window, n_splits, QkvPrep{}, stream);
  if (head_dim == 64)
    return launch_decode<64, false>(q, q_stride, out, out_stride, kv, m, dec_entries, n_dec, part_o, part_ml, n_heads, n_kv, scale, window, n_splits, QkvPrep{}, stream);
  return IFX_ERR_UNSUPPORTED;
}

// The same for a step of single tokens only, with the work of ifx_qkv_rope_kv_write folded in: qkv is the
// product's output before bias and rotation ([n_tokens, (n_heads + 2 n_kv) * head_dim] bfloat16 rows, or
// float32 partial sums [n_partials][n_tokens][width] of it; the bfloat16 rows are not read then), bias
// float32 [width] or null, cos/sin float32 [n_tokens, head_dim / 2] (the whole head is rotated), slot_map
// [n_tokens] or null for a layer that writes no keys and values.  Every token of the step must be one of the
// decoded entries: nothing else gets its key and value written.
IFX_API int ifx_attn_decode_prep_bf16(const void* qkv, long long qkv_stride, void* out, long long out_stride,
                                      void* k_layer, void* v_layer, long long page_stride, int page_size,
                                      const int* block_tables, int bt_stride, const int* dec_entries, int n_dec,
                                      const int* entry_q_start, const int* entry_q_len, const int* entry_ctx_start,
                                      float* part_o, float* part_ml, int n_heads, int n_kv, int head_dim, float scale,
                                      int window, int n_splits, const float* bias, const float* cos_t,
                                      const float* sin_t, const int* slot_map, const float* partials, int n_partials,
                                      int n_tokens, cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (n_kv < 1 || n_heads % n_kv || n_splits < 1 || n_splits > 65535 || n_tokens < n_dec) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  if ((page_stride & 7) || ((uintptr_t)k_layer & 15) || ((uintptr_t)v_layer & 15)) return IFX_ERR_ALIGNMENT;
  if ((qkv_stride & 7) || (((uintptr_t)qkv | (uintptr_t)bias | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)partials) & 15))
    return IFX_ERR_ALIGNMENT;
  if (!cos_t || !sin_t || (partials && n_partials < 1) || (!partials && !qkv)) return IFX_ERR_UNSUPPORTED;
  if (n_splits > 1 && (!part_o || !part_ml)) return IFX_ERR_UNSUPPORTED;
  PagedKV kv = make_kv(k_layer, v_layer, page_stride, page_size, head_dim);
  AttnMeta m{block_tables, bt_stride, entry_q_start, entry_q_len, entry_ctx_start};
  QkvPrep prep{bias, cos_t, sin_t, slot_map, partials, n_partials, (long long)n_tokens * (n_heads + 2 * n_kv) * head_dim};
  if (head_dim == 128)
    return launch_decode<128, true>(qkv, qkv_stride, out, out_stride, kv, m, dec_entries, n_dec, part_o, part_ml, n_heads, n_kv, scale, window, n_splits, prep, stream);
  if (head_dim == 64)
    return launch_decode<64, true>(qkv, qkv_stride, out, out_stride, kv, m, dec_entries, n_dec, part_o, part_ml, n_heads, n_kv, scale, window, n_splits, prep, stream);
  return IFX_ERR_UNSUPPORTED;
}

namespace {
// Blocks of the decode kernel that the GPU holds at once (asked once per head size); negative: a CUDA error.
template <int HD>
int decode_resident_blocks() {
  static int resident = 0;
  if (!resident) {
    const size_t stage_bytes = (size_t)DSTAGES * 2 * 64 * HD * sizeof(bf16);
    const size_t red_bytes = (size_t)4 * 8 * HD * sizeof(float) + 4 * 8 * 2 * sizeof(float);
    const size_t smem = stage_bytes > red_bytes ? stage_bytes : red_bytes;
    auto kern = attn_decode_bf16_kernel<HD, true>;             // the variant with more static shared memory
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return -(int)e;
    int per_sm = 0, dev = 0, sms = 0;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 128, smem)) != cudaSuccess) return -(int)e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return -(int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return -(int)e;
    resident = per_sm * sms > 0 ? per_sm * sms : 1;
  }
  return resident;
}
}  // namespace

// Into how many parts the decode kernel is best told to cut the keys of n_dec entries whose longest
// context is max_keys: as many as give every block a place on the GPU at once (a second round of
// blocks costs more than longer parts), each part at least four 64-key tiles.  Negative: a CUDA error.
IFX_API int ifx_attn_decode_plan(int n_dec, int n_heads, int n_kv, int head_dim, int max_keys) {
  if (n_dec < 1 || n_kv < 1 || n_heads < n_kv || max_keys < 1) return 1;
  const int resident = head_dim == 128 ? decode_resident_blocks<128>() : head_dim == 64 ? decode_resident_blocks<64>() : 1;
  if (resident < 0) return resident;
  const int base = n_dec * n_kv * ((n_heads / n_kv + 7) / 8);
  int s = resident / base;
  const int by_keys = max_keys / 256;
  if (s > by_keys) s = by_keys;
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  const int tiles = (max_keys + 63) / 64, per = (tiles + s - 1) / s;
  return (tiles + per - 1) / per;                              // no part without a tile
}

// Attention of single tokens with the tiles of all entries shared out evenly over the blocks the GPU holds
// (attn_decode_even_kernel): for steps whose contexts differ much in length.  q is rotated already and the
// step's keys and values are in the cache (ifx_qkv_rope_kv_write).  Scratch: part_o float32 [n_dec * n_heads *
// max_pieces * head_dim], part_ml float32 [n_dec * n_heads * max_pieces * 2], piece_count int [n_dec *
// n_heads]; max_pieces from ifx_attn_decode_even_pieces for a bound on the contexts' lengths (new token
// included; with a window, the window); error_flag: a device int that the kernel sets to 2 if it meets a
// longer context (it then writes nothing for that entry).
IFX_API int ifx_attn_decode_even_bf16(const void* q, long long q_stride, void* out, long long out_stride,
                                      void* k_layer, void* v_layer, long long page_stride, int page_size,
                                      const int* block_tables, int bt_stride, const int* dec_entries, int n_dec,
                                      const int* entry_q_start, const int* entry_q_len, const int* entry_ctx_start,
                                      float* part_o, float* part_ml, int* piece_count, int n_heads, int n_kv,
                                      int head_dim, float scale, int window, int max_pieces, int* error_flag,
                                      cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (n_kv < 1 || n_heads % n_kv || max_pieces < 1 || n_dec > DEC_MAX || !error_flag) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  if ((q_stride & 1) || ((uintptr_t)q & 3)) return IFX_ERR_ALIGNMENT;
  if ((page_stride & 7) || ((uintptr_t)k_layer & 15) || ((uintptr_t)v_layer & 15)) return IFX_ERR_ALIGNMENT;
  if (!part_o || !part_ml || !piece_count || ((uintptr_t)part_ml & 7)) return IFX_ERR_UNSUPPORTED;
  PagedKV kv = make_kv(k_layer, v_layer, page_stride, page_size, head_dim);
  AttnMeta m{block_tables, bt_stride, entry_q_start, entry_q_len, entry_ctx_start};
  if (head_dim == 128)
    return launch_decode_even<128>(q, q_stride, out, out_stride, kv, m, dec_entries, n_dec, part_o, part_ml, piece_count, n_heads, n_kv, scale, window, max_pieces, error_flag, stream);
  if (head_dim == 64)
    return launch_decode_even<64>(q, q_stride, out, out_stride, kv, m, dec_entries, n_dec, part_o, part_ml, piece_count, n_heads, n_kv, scale, window, max_pieces, error_flag, stream);
  return IFX_ERR_UNSUPPORTED;
}

// Blocks that the even-share decode kernel runs (what the GPU holds at once).  Negative: a CUDA error.
IFX_API int ifx_attn_decode_even_blocks(int head_dim) {
  return head_dim == 128 ? even_resident_blocks<128>() : head_dim == 64 ? even_resident_blocks<64>() : 1;
}

// The scratch's pieces per (entry, head) for contexts of at most max_keys keys.  Negative: a CUDA error.
IFX_API int ifx_attn_decode_even_pieces(int n_heads, int n_kv, int head_dim, int max_keys) {
  if (n_kv < 1 || n_heads < n_kv || max_keys < 1) return 1;
  const int blocks = head_dim == 128 ? even_resident_blocks<128>() : head_dim == 64 ? even_resident_blocks<64>() : 1;
  if (blocks < 0) return blocks;
  return even_max_pieces(max_keys, blocks, n_kv * ((n_heads / n_kv + 7) / 8));
}

IFX_STAMP_READER(ifx_stamps_attn)
