// Matrix product for many rows of activations (prompt portions) on the fifth-generation tensor
// cores: out[M, N] = A[M, K] * W[N, K]^T (+ bias), or with a stacked [gate; up] weight
// out[M, I] = silu(A gate^T) * (A up^T), bfloat16 operands, float32 accumulation in tensor memory.
//
// The reference sends every dense projection to cuBLAS and runs SwiGLU as a kernel of its own over
// the [M, 2I] result (runtime/backends/cuda/native/cublas_gemm.cpp:84-102,
// runtime/backends/cuda/native/cuda_kernels.cu:137-149).  Here the product is written out so that the
// activation can sit in its epilogue: the [M, 2I] intermediate never goes to memory.
//
// Two blocks on neighbouring SMs form a cluster and share one output tile of 256 rows x 256
// accumulator columns (cta_group::2); clusters are persistent over the tiles.  Per step of 64 along K
// each block brings 128 rows of A and 128 of the tile's 256 rows of W into its shared memory by TMA
// (32 KB, six stages, the 128-byte-swizzle layout the tensor core reads).  Warp 0 of each block issues
// its TMA loads; warp 1 of the leader (cluster rank 0) issues the MMAs, four tcgen05.mma of M 256, N 256,
// K 16 per step, which read A and the two halves of W from both blocks' shared memory; each block's
// tensor memory gets its 128 rows of the result.  A tile takes 256 of the 512 columns, so the epilogue
// of one tile (warps 2-5: each reads its quarter of the 128 lanes, 32 columns at a time, applies bias or
// SwiGLU and stores its row's 32 values) runs while the MMAs of the next fill the other 256.  With
// SwiGLU the leader's half of W is the gate rows and the other block's the up rows of the same 128
// outputs, so a thread finds gate and up of an output in its own lane.
//
// Barriers (same offsets in both blocks): full[s] counts the bytes of both blocks' copies and lives in
// the leader (the other block's TMA completes on it; no multicast); empty[s] and acc_full[a] are
// arrived on in both blocks by one tcgen05.commit; acc_empty[a] in the leader counts the 256 epilogue
// threads of both blocks.  The pair synchronises as a cluster after set-up and before it frees tensor
// memory, so neither block leaves while the other may still signal it.
//
// Every mbarrier wait is bounded: if one runs out the thread sets *error_flag and the block's abort
// word, the other warps leave their loops, the block waits a moment for TMA copies in flight, and the
// pair frees its tensor memory and returns.
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>

namespace {

constexpr int TK = 64;                  // K per stage: one 128-byte swizzled row of bfloat16
constexpr int G_WAIT_LIMIT = 1 << 20;   // tries of at most 2 microseconds each

__device__ __forceinline__ unsigned g_smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// false: the wait ran out, or (abort_flag given) another warp of the block gave up
__device__ __forceinline__ bool g_wait(unsigned bar, unsigned parity, const volatile int* abort_flag) {
  for (int i = 0; i < G_WAIT_LIMIT; ++i) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(2000u) : "memory");   // a try sleeps 2 microseconds at most
    if (ok) return true;
    if (abort_flag && (i & 255) == 255 && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void g_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned long long g_desc(unsigned saddr) {      // K-major, 128-byte swizzle, 8-row groups of 1024 bytes
  unsigned long long d = 0;
  d |= (unsigned long long)((saddr & 0x3FFFF) >> 4);
  d |= (unsigned long long)(16 >> 4) << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}
__device__ __forceinline__ void g_tmem_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

template <typename T> __device__ __forceinline__ void store_row32(T* dst, const float (&v)[32], int n_valid, bool vec);
template <> __device__ __forceinline__ void store_row32<float>(float* dst, const float (&v)[32], int n_valid, bool vec) {
  if (vec && n_valid == 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < n_valid) dst[i] = v[i];
  }
}
template <> __device__ __forceinline__ void store_row32<bf16>(bf16* dst, const float (&v)[32], int n_valid, bool vec) {
  if (vec && n_valid == 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 p;
      __nv_bfloat162 a = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]), b = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
      __nv_bfloat162 c = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]), d = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
      p.x = *reinterpret_cast<unsigned*>(&a); p.y = *reinterpret_cast<unsigned*>(&b);
      p.z = *reinterpret_cast<unsigned*>(&c); p.w = *reinterpret_cast<unsigned*>(&d);
      reinterpret_cast<uint4*>(dst)[i] = p;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < n_valid) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

constexpr int P_STAGES = 6;
constexpr int P_HALF_BYTES = 128 * TK * 2;            // 16 KB: 128 rows of 128 bytes
constexpr int P_STAGE_BYTES = 2 * P_HALF_BYTES;       // this block's rows of A, then its rows of W
constexpr int P_SMEM = P_STAGES * P_STAGE_BYTES + 1024;
constexpr int P_THREADS = 192;                        // producer warp, MMA warp, 4 epilogue warps
constexpr unsigned LEADER_MASK = 0xFEFFFFFFu;         // a shared-memory address of this block -> the same place in the pair's leader
// kind::f16 instruction descriptor: D float32, A and B bfloat16, both K-major, M 256 (over the pair), N 256
constexpr unsigned P_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(256 >> 4) << 24);   // N (in eighths) goes to bits 17-22

__device__ __forceinline__ unsigned p_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void p_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// One TMA box (64 elements along K x 128 rows) whose first element is (k, row), into this block's shared
// memory; its bytes are counted by the leader's barrier.  The coordinate along K is a multiple of 64
// elements, so the copy starts on a 128-byte boundary.  No multicast.
__device__ __forceinline__ void p_tma_load(unsigned dst, const CUtensorMap* map, int k, int row, unsigned leader_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(dst), "l"(map), "r"(k), "r"(row), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void p_mma(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                      unsigned accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive columns of this thread's lane (the narrow last piece of a tile whose width is not a multiple of 32)
__device__ __forceinline__ void g_tmem_ld16(unsigned taddr, float (&v)[32]) {
  unsigned r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) { v[i] = __uint_as_float(r[i]); v[16 + i] = 0.0f; }
}
__device__ __forceinline__ void p_commit_both(unsigned bar) {      // arrives on this barrier in both blocks of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void p_arrive_leader(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(bar & LEADER_MASK) : "memory");
}

// What the epilogue of mode 3 needs: the product is the stacked q, k, v projection of head size 128, and the
// epilogue adds the bias, rotates the query and key heads (rotate-half, the angles' cosines and sines per
// token), writes the queries to out and the keys and values into the paged cache at each token's slot.
struct QkvEpilogue {
  const float* cos_t;       // [M, 64]
  const float* sin_t;
  const int* slot_map;      // [M]: page * page_size + offset; null or -1: nothing of that token is cached
  bf16* k_cache;            // this layer's keys of page 0 / values of page 0
  bf16* v_cache;
  long long page_stride;    // elements between pages
  int page_size, page_shift, n_heads, n_kv;
};

// MODE 0: out = A W^T (+ bias); 1: SwiGLU of the two halves of W; 2: few rows of A; 3: q, k, v with bias,
// rotation and cache write (tiles of two heads of 128).  In mode 2 the operands
// change places, so that the 256 rows of a tile are rows of the weights and its (few) columns the tokens: the
// kernel is given the weights as map_a (M = their rows) and the activations as map_w (n_out = the tokens, all
// in one tile), K is cut into k_parts parts that are tiles of their own, and the epilogue writes each part's
// sums transposed, as float32 [k_parts][tokens][ldo] part_stride elements apart, for the consumer to add.
template <int MODE, typename TOut>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_umma_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      TOut* __restrict__ out, long long ldo, const float* __restrict__ bias, int M, int n_out, int K,
                      int tile_n, int* __restrict__ error_flag, int k_parts, long long part_stride, QkvEpilogue qe) {
  constexpr bool SWIGLU = MODE == 1, SKINNY = MODE == 2, QKV = MODE == 3;
  pdl_enter();
  extern __shared__ unsigned char g_smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * P_STAGES + 4];    // full[s], empty[s], acc_full[2], acc_empty[2]
  __shared__ unsigned tmem_slot;
  __shared__ int abort_s;
  const unsigned sbase = (g_smem_addr(g_smem_raw) + 1023u) & ~1023u;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned rank = p_cluster_rank();
  const bool leader = rank == 0;
  const unsigned bar_full = g_smem_addr(&bars[0]), bar_empty = g_smem_addr(&bars[P_STAGES]);
  const unsigned bar_acc_full = g_smem_addr(&bars[2 * P_STAGES]), bar_acc_empty = g_smem_addr(&bars[2 * P_STAGES + 2]);
  volatile int* abort_flag = &abort_s;

  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < P_STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_full + 8 * s));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_empty + 8 * s));
    }
    for (int a = 0; a < 2; ++a) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_acc_full + 8 * a));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 256;\n" ::"r"(bar_acc_empty + 8 * a));   // epilogue threads of both blocks
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(g_smem_addr(&tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  p_cluster_sync();                                              // the other block's barriers exist before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem = tmem_slot;

  // tile_n: accumulator columns of a tile (a multiple of 16 up to 256; SwiGLU: 256 = 128 gate + 128 up)
  const int out_cols = SWIGLU ? 128 : tile_n;
  const int m_tiles = (M + 255) / 256, n_tiles = SKINNY ? k_parts : (n_out + out_cols - 1) / out_cols;
  const int tiles = m_tiles * n_tiles, k_steps = (K + TK - 1) / TK;
  const int part_steps = SKINNY ? (k_steps + k_parts - 1) / k_parts : k_steps;   // no part is empty: the host sees to that
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int w_half_rows = tile_n / 2;                            // rows of W this block loads per step
  bool gave_up = false;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      unsigned phase = 0;
      for (int t = pair; t < tiles && !gave_up; t += n_pairs) {
        const int m0 = (t % m_tiles) * 256 + (int)rank * 128;
        const int n0 = SKINNY ? 0 : (t / m_tiles) * out_cols;
        const int w_row = SWIGLU ? (int)rank * n_out + n0 : n0 + (int)rank * w_half_rows;
        const int ks0 = SKINNY ? (t / m_tiles) * part_steps : 0, ks1 = SKINNY ? min(k_steps, ks0 + part_steps) : k_steps;
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!g_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) { gave_up = true; break; }
          const unsigned sa = sbase + stage * P_STAGE_BYTES, sw = sa + P_HALF_BYTES;
          const unsigned full = (bar_full + 8 * stage) & LEADER_MASK;
          if (leader) g_expect_tx(bar_full + 8 * stage, 2 * (P_HALF_BYTES + w_half_rows * 128));
          p_tma_load(sa, &map_a, ks * TK, m0, full);
          p_tma_load(sw, &map_w, ks * TK, w_row, full);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      int stage = 0, count = 0;
      unsigned phase = 0;
      const unsigned idesc = P_IDESC | ((unsigned)(tile_n >> 3) << 17);
      for (int t = pair; t < tiles && !gave_up; t += n_pairs, ++count) {
        const int acc = count & 1;
        const unsigned acc_parity = (unsigned)(count >> 1) & 1u;
        if (!g_wait(bar_acc_empty + 8 * acc, acc_parity ^ 1u, abort_flag)) { gave_up = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned d = tmem + (unsigned)(acc * 256);
        const int ks0 = SKINNY ? (t / m_tiles) * part_steps : 0, ks1 = SKINNY ? min(k_steps, ks0 + part_steps) : k_steps;
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!g_wait(bar_full + 8 * stage, phase, abort_flag)) { gave_up = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned sa = sbase + stage * P_STAGE_BYTES, sw = sa + P_HALF_BYTES;
#pragma unroll
          for (int k = 0; k < TK / 16; ++k) p_mma(d, g_desc(sa + k * 32), g_desc(sw + k * 32), idesc, ks != ks0 || k != 0);
          p_commit_both(bar_empty + 8 * stage);                  // both blocks' stage is free once these MMAs have read it
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!gave_up) p_commit_both(bar_acc_full + 8 * acc);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row_in_tile = (int)rank * 128 + quarter * 32 + lane;
    const bool vec = (ldo % 8 == 0) && ((uintptr_t)out % 16 == 0);
    int count = 0;
    for (int t = pair; t < tiles; t += n_pairs, ++count) {
      const int acc = count & 1;
      const unsigned acc_parity = (unsigned)(count >> 1) & 1u;
      const int m0 = (t % m_tiles) * 256, n0 = SKINNY ? 0 : (t / m_tiles) * out_cols;
      if (!g_wait(bar_acc_full + 8 * acc, acc_parity, abort_flag)) { gave_up = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const unsigned taddr = tmem + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * 256);
      const int row = m0 + row_in_tile;
      TOut* orow = out + (size_t)(row < M ? row : 0) * (SKINNY ? 1 : ldo);
      if (SKINNY) {                                              // this lane's row of the weights is a column of the output
        TOut* opart = orow + (size_t)(t / m_tiles) * part_stride;
#pragma unroll 1
        for (int c = 0; c * 32 < tile_n; ++c) {
          float v[32];
          if (tile_n - c * 32 >= 32) g_tmem_ld32(taddr + c * 32, v);
          else g_tmem_ld16(taddr + c * 32, v);                   // warp-uniform: the tile's last 16 columns
          if (row < M) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int token = c * 32 + i;
              if (token < n_out) opart[(size_t)token * ldo] = (TOut)v[i];   // a warp's lanes write 32 neighbours
            }
          }
        }
      } else if (QKV) {
        // The tile's 256 columns are two heads; this thread has one token's row of both.  Same operations, in
        // the same order, as the kernel that does this after a library product (rope_math.cuh), on the float32
        // sums themselves.
        const int slot = (row < M && qe.slot_map) ? qe.slot_map[row] : -1;
        const float* ct = qe.cos_t + (size_t)(row < M ? row : 0) * 64;
        const float* st = qe.sin_t + (size_t)(row < M ? row : 0) * 64;
        const size_t cache_at = slot >= 0 ? (size_t)(slot >> qe.page_shift) * qe.page_stride +
                                                (size_t)(slot & (qe.page_size - 1)) * 128 : 0;
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
          const int head = n0 / 128 + hh;                          // among the nh + 2 nkv heads of the row
          if (head >= qe.n_heads + 2 * qe.n_kv) break;             // (the same for the whole block)
          const bool is_q = head < qe.n_heads, is_k = !is_q && head < qe.n_heads + qe.n_kv;
          const int kvh = is_q ? 0 : head - qe.n_heads - (is_k ? 0 : qe.n_kv);
          bf16* dst = is_q ? reinterpret_cast<bf16*>(out) + (size_t)(row < M ? row : 0) * ldo + (size_t)head * 128
                           : (is_k ? qe.k_cache : qe.v_cache) + cache_at + (size_t)kvh * qe.page_size * 128;
          const bool wanted = row < M && (is_q || slot >= 0);
          const float* b = bias ? bias + (size_t)head * 128 : nullptr;
          if (is_q || is_k) {
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {                 // pairs (i, i + 64), i in [32 half, 32 half + 32)
              float lo[32], hi[32];
              g_tmem_ld32(taddr + hh * 128 + half * 32, lo);
              g_tmem_ld32(taddr + hh * 128 + 64 + half * 32, hi);
              if (wanted) {
                // 16 bytes a load: a thread reads 128 contiguous bytes of its token's cosines (a line of its own)
                float cs[32], sn[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  *reinterpret_cast<float4*>(cs + 4 * i) = __ldg(reinterpret_cast<const float4*>(ct + half * 32) + i);
                  *reinterpret_cast<float4*>(sn + 4 * i) = __ldg(reinterpret_cast<const float4*>(st + half * 32) + i);
                }
                if (b) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(b + half * 32) + i);
                    const float4 b1 = __ldg(reinterpret_cast<const float4*>(b + 64 + half * 32) + i);
                    lo[4 * i] = __fadd_rn(lo[4 * i], b0.x); lo[4 * i + 1] = __fadd_rn(lo[4 * i + 1], b0.y);
                    lo[4 * i + 2] = __fadd_rn(lo[4 * i + 2], b0.z); lo[4 * i + 3] = __fadd_rn(lo[4 * i + 3], b0.w);
                    hi[4 * i] = __fadd_rn(hi[4 * i], b1.x); hi[4 * i + 1] = __fadd_rn(hi[4 * i + 1], b1.y);
                    hi[4 * i + 2] = __fadd_rn(hi[4 * i + 2], b1.z); hi[4 * i + 3] = __fadd_rn(hi[4 * i + 3], b1.w);
                  }
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  const float x0 = lo[i], x1 = hi[i];
                  lo[i] = __fmaf_rn(x0, cs[i], -__fmul_rn(x1, sn[i]));
                  hi[i] = __fmaf_rn(x0, sn[i], __fmul_rn(x1, cs[i]));
                }
                store_row32<bf16>(dst + half * 32, lo, 32, true);
                store_row32<bf16>(dst + 64 + half * 32, hi, 32, true);
              }
            }
          } else {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              float v[32];
              g_tmem_ld32(taddr + hh * 128 + c * 32, v);
              if (wanted) {
                if (b) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(b + c * 32) + i);
                    v[4 * i] = __fadd_rn(v[4 * i], b0.x); v[4 * i + 1] = __fadd_rn(v[4 * i + 1], b0.y);
                    v[4 * i + 2] = __fadd_rn(v[4 * i + 2], b0.z); v[4 * i + 3] = __fadd_rn(v[4 * i + 3], b0.w);
                  }
                }
                store_row32<bf16>(dst + c * 32, v, 32, true);
              }
            }
          }
        }
      } else if (SWIGLU) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float gate[32], up[32];
          g_tmem_ld32(taddr + c * 32, gate);
          g_tmem_ld32(taddr + 128 + c * 32, up);
#pragma unroll
          for (int i = 0; i < 32; ++i) gate[i] = gate[i] / (1.0f + __expf(-gate[i])) * up[i];
          const int col = n0 + c * 32;
          if (row < M && col < n_out) store_row32<TOut>(orow + col, gate, min(32, n_out - col), vec && (col % 8 == 0));
        }
      } else {
#pragma unroll 1
        for (int c = 0; c * 32 < tile_n; ++c) {
          float v[32];
          if (tile_n - c * 32 >= 32) g_tmem_ld32(taddr + c * 32, v);
          else g_tmem_ld16(taddr + c * 32, v);                   // warp-uniform: the tile's last 16 columns
          const int col = n0 + c * 32;
          if (row < M && col < n_out) {
            if (bias) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += col + i < n_out ? bias[col + i] : 0.0f;
            }
            store_row32<TOut>(orow + col, v, min(min(32, tile_n - c * 32), n_out - col), vec && (col % 8 == 0));
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      p_arrive_leader(bar_acc_empty + 8 * acc);                  // this thread has read its part of the accumulator
    }
  }
  if (gave_up) {                                                 // a wait ran out: tell everyone, let copies in flight land
    atomicExch(error_flag, 1);
    abort_s = 1;
    __nanosleep(2000000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  p_cluster_sync();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}

PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  return fn;
}

// [rows, K] bfloat16, row stride ld elements; boxes of box_rows rows x 64 elements, 128-byte swizzle, zeros outside
int make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
  PFN_cuTensorMapEncodeTiled_v12000 enc = tensor_map_encoder();
  if (!enc) return IFX_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : IFX_ERR_UNSUPPORTED;
}

// Accumulator columns per tile for a plain product: the multiple of 16 (128 to 256) with which the pairs
// of SMs finish soonest.  The kernel runs at the rate at which shared memory is fed from L2 (about 83 GB/s
// per SM measured), so a tile costs its 256 rows of A plus its rows of W; wider wins a tie.
int pick_tile_n(int M, int n_out, int pairs) {
  const int m_tiles = (M + 255) / 256;
  int best = 256;
  long long best_cost = -1;
  for (int tn = 256; tn >= 128; tn -= 16) {
    const long long tiles = (long long)m_tiles * ((n_out + tn - 1) / tn);
    const long long cost = ((tiles + pairs - 1) / pairs) * (256 + tn);
    if (best_cost < 0 || cost < best_cost) { best = tn; best_cost = cost; }
  }
  return best;
}

template <bool SWIGLU, typename TOut>
int launch_gemm_pair(const void* A, long long lda, const void* W, const float* bias, void* out, long long ldo, int M, int n_out,
                     int K, int* error_flag, cudaStream_t stream) {
  auto kern = gemm_umma_pair_kernel<SWIGLU ? 1 : 0, TOut>;
  static int sms = 0;
  if (!sms) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
    if (e != cudaSuccess) return (int)e;
    int dev = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
  }
  const int tile_n = SWIGLU ? 256 : pick_tile_n(M, n_out, sms / 2);
  const int out_cols = SWIGLU ? 128 : tile_n;
  CUtensorMap map_a, map_w;
  int rc = make_map(&map_a, A, M, K, lda, 128);
  if (!rc) rc = make_map(&map_w, W, SWIGLU ? 2ll * n_out : n_out, K, K, tile_n / 2);
  if (rc) return rc;
  const int tiles = ((M + 255) / 256) * ((n_out + out_cols - 1) / out_cols);
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  rc = launch_pdl_cluster(kern, dim3(2 * pairs), dim3(P_THREADS), (size_t)P_SMEM, stream, dim3(2, 1, 1), map_a, map_w, (TOut*)out,
                          ldo, bias, M, n_out, K, tile_n, error_flag, 1, 0ll, QkvEpilogue{});
  return rc ? rc : IFX_LAUNCH_CHECK();
}

// Parts into which the product of a few rows cuts K: as many as give every pair of SMs a tile, each part at
// least 8 steps of 64, none empty.
int skinny_parts(int n_out, int K, int pairs) {
  const int m_tiles = (n_out + 255) / 256, k_steps = (K + TK - 1) / TK;
  int parts = pairs / m_tiles;
  if (parts > k_steps / 8) parts = k_steps / 8;
  if (parts < 1) parts = 1;
  const int per = (k_steps + parts - 1) / parts;
  return (k_steps + per - 1) / per;
}

int device_sms(int* sms) {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
  }
  *sms = n;
  return 0;
}

int launch_gemm_qkv(const void* A, long long lda, const void* W, const float* bias, bf16* q_out, long long ldo, int M, int K,
                    const QkvEpilogue& qe, int* error_flag, cudaStream_t stream) {
  auto kern = gemm_umma_pair_kernel<3, bf16>;
  static bool ready = false;
  if (!ready) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
    if (e != cudaSuccess) return (int)e;
    ready = true;
  }
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc) return rc;
  const int n_out = (qe.n_heads + 2 * qe.n_kv) * 128, tile_n = 256;
  CUtensorMap map_a, map_w;
  rc = make_map(&map_a, A, M, K, lda, 128);
  if (!rc) rc = make_map(&map_w, W, n_out, K, K, tile_n / 2);
  if (rc) return rc;
  const int tiles = ((M + 255) / 256) * ((n_out + tile_n - 1) / tile_n);
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  rc = launch_pdl_cluster(kern, dim3(2 * pairs), dim3(P_THREADS), (size_t)P_SMEM, stream, dim3(2, 1, 1), map_a, map_w, q_out,
                          ldo, bias, M, n_out, K, tile_n, error_flag, 1, 0ll, qe);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

int launch_gemm_skinny(const void* X, long long ldx, const void* W, float* out, long long ldo, int tokens, int n_out, int K,
                       int k_parts, long long part_stride, int* error_flag, cudaStream_t stream) {
  auto kern = gemm_umma_pair_kernel<2, float>;
  static bool ready = false;
  if (!ready) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
    if (e != cudaSuccess) return (int)e;
    ready = true;
  }
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc) return rc;
  const int tile_n = tokens <= 32 ? 32 : (tokens + 15) / 16 * 16;      // the tokens, all in one tile
  CUtensorMap map_w, map_x;
  rc = make_map(&map_w, W, n_out, K, K, 128);
  if (!rc) rc = make_map(&map_x, X, tokens, K, ldx, tile_n / 2);
  if (rc) return rc;
  const int tiles = ((n_out + 255) / 256) * k_parts;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  rc = launch_pdl_cluster(kern, dim3(2 * pairs), dim3(P_THREADS), (size_t)P_SMEM, stream, dim3(2, 1, 1), map_w, map_x, out, ldo,
                          (const float*)nullptr, n_out, tokens, K, tile_n, error_flag, k_parts, part_stride, QkvEpilogue{});
  return rc ? rc : IFX_LAUNCH_CHECK();
}
}  // namespace

// out[M, n_out] = A[M, K] * W^T (+ bias), W [n_out, K] contiguous; or, with swiglu != 0, W [2 * n_out, K] =
// [gate; up] and out = silu(A gate^T) * (A up^T).  A rows lda elements apart; K and lda multiples of 8;
// A and W 16-byte aligned.  out_dtype: float32 or bfloat16.  error_flag: a device word set if a bounded
// wait inside the kernel runs out.
IFX_API int ifx_gemm_umma(const void* A, long long lda, const void* W, const float* bias, void* out, long long ldo,
                          int out_dtype, int M, int n_out, int K, int swiglu, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || n_out <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || !error_flag) return IFX_ERR_UNSUPPORTED;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return IFX_ERR_ALIGNMENT;
  if (swiglu && bias) return IFX_ERR_UNSUPPORTED;
  if (out_dtype == IFX_BF16)
    return swiglu ? launch_gemm_pair<true, bf16>(A, lda, W, bias, out, ldo, M, n_out, K, error_flag, stream)
                  : launch_gemm_pair<false, bf16>(A, lda, W, bias, out, ldo, M, n_out, K, error_flag, stream);
  if (out_dtype == IFX_F32)
    return swiglu ? launch_gemm_pair<true, float>(A, lda, W, bias, out, ldo, M, n_out, K, error_flag, stream)
                  : launch_gemm_pair<false, float>(A, lda, W, bias, out, ldo, M, n_out, K, error_flag, stream);
  return IFX_ERR_UNSUPPORTED;
}

// The product of a few rows (17 to 256 tokens) against weights that must stream from memory once: out
// [k_parts][tokens][n_out] float32 (rows ldo elements apart, parts part_stride) holds partial sums over the
// k_parts parts of K, to be added by the consumer; k_parts from ifx_gemm_umma_skinny_parts.  The weights' rows
// are the 256 rows of the tensor-core tiles and the tokens their columns, so a tile streams 256 rows of W
// through shared memory once for all tokens.  X rows ldx elements apart; K and ldx multiples of 8; X and W
// 16-byte aligned.
IFX_API int ifx_gemm_umma_skinny(const void* X, long long ldx, const void* W, float* out, long long ldo, long long part_stride,
                                 int tokens, int n_out, int K, int k_parts, int* error_flag, cudaStream_t stream) {
  if (tokens <= 0 || n_out <= 0) return 0;
  if (tokens > 256 || K <= 0 || (K & 7) || (ldx & 7) || !error_flag || k_parts < 1) return IFX_ERR_UNSUPPORTED;
  const int k_steps = (K + TK - 1) / TK, per = (k_steps + k_parts - 1) / k_parts;
  if ((k_steps + per - 1) / per != k_parts) return IFX_ERR_UNSUPPORTED;            // a part would be empty
  if (((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)out & 3)) return IFX_ERR_ALIGNMENT;
  return launch_gemm_skinny(X, ldx, W, out, ldo, tokens, n_out, K, k_parts, part_stride, error_flag, stream);
}

IFX_API int ifx_gemm_umma_skinny_parts(int n_out, int K) {
  int sms = 0;
  const int rc = device_sms(&sms);
  if (rc) return -rc;
  return skinny_parts(n_out, K, sms / 2);
}

// The stacked q, k, v projection of a step's tokens with everything that follows it before attention in its
// epilogue: q_out[M, n_heads * 128] (rows ldo elements apart) receives the rotated queries, the paged cache the
// rotated keys and the values at slot_map[token] (page * page_size + offset; -1: not cached).  Head size 128,
// rotate-half over the whole head (cos_t, sin_t float32 [M, 64]), W [(n_heads + 2 n_kv) * 128, K] bfloat16,
// bias float32 of that width or null.  A rows lda elements apart; K, lda, ldo and page_stride multiples of 8;
// every pointer 16-byte aligned.
IFX_API int ifx_gemm_umma_qkv(const void* A, long long lda, const void* W, const float* bias, void* q_out, long long ldo,
                              const float* cos_t, const float* sin_t, const int* slot_map, void* k_layer, void* v_layer,
                              long long page_stride, int page_size, int M, int K, int n_heads, int n_kv, int* error_flag,
                              cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || (ldo & 7) || (page_stride & 7) || !error_flag || n_heads < 1 || n_kv < 0)
    return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1)) || !cos_t || !sin_t) return IFX_ERR_UNSUPPORTED;
  if (n_kv > 0 && (!slot_map || !k_layer || !v_layer)) return IFX_ERR_UNSUPPORTED;
  if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)q_out | (uintptr_t)k_layer | (uintptr_t)v_layer | (uintptr_t)bias |
       (uintptr_t)cos_t | (uintptr_t)sin_t) & 15)
    return IFX_ERR_ALIGNMENT;
  QkvEpilogue qe;
  qe.cos_t = cos_t; qe.sin_t = sin_t; qe.slot_map = n_kv > 0 ? slot_map : nullptr;
  qe.k_cache = (bf16*)k_layer; qe.v_cache = (bf16*)v_layer; qe.page_stride = page_stride;
  qe.page_size = page_size; qe.page_shift = 0;
  while ((1 << qe.page_shift) < page_size) ++qe.page_shift;
  qe.n_heads = n_heads; qe.n_kv = n_kv;
  return launch_gemm_qkv(A, lda, W, bias, (bf16*)q_out, ldo, M, K, qe, error_flag, stream);
}
