// Attention of prompt portions on the fifth-generation tensor cores:
// tcgen05.mma with accumulators in tensor memory, for head size 128.
//
// Same formulas as the other attention kernels (attention_generic.cu): kv head
// = head / (n_heads / n_kv), s = (q . k) * scale, causal with an optional
// window, float32 softmax, o = sum p v / sum p.  The reference's kernel for this
// case is scalar or mma.sync with fp16 operands
// (runtime/backends/cuda/kernels/flash_attention.cu:52-173,
// runtime/backends/cuda/kernels/flash_attention_mma.cuh:153-379).
//
// One block takes 256 consecutive new tokens of one request and one head, as two
// query tiles ("slots") of 128 rows that share every key and value tile the block
// brings in; it has an SM to itself (192 KB of shared memory, all 512 columns of
// tensor memory).
//   * Q (2 x 128 x 128), and per step a tile of 64 keys and 64 values, lie in shared
//     memory in the 128-byte-swizzle layouts the tensor core reads.  Q is written
//     once with 16-byte cp.async.  Keys and values come from the paged cache by
//     TMA (cp.async.bulk.tensor over a 4-D map (dim, slot, kv head, page) of the
//     run's pages): one box per page and 64-dim panel, issued by the lanes of two
//     warps of their own (one for keys, one for values), four stages each ahead of
//     their use, with mbarriers both ways (a stage has landed / a stage has been
//     read by both slots).
//   * Per slot, S = Q K^T is one chain of 8 tcgen05.mma (M 128, N 64, K 16) into 64
//     columns of tensor memory, of which the slot has two (the scores of tile i + 1
//     are computed while the threads work on tile i).  Thread r then owns row r: it
//     reads its scores with tcgen05.ld, keeps the running maximum and sum, and
//     writes P = exp(s - max) as packed bfloat16 back over the scores
//     (tcgen05.st), from where the next MMA takes it as its A operand.
//   * O += P V is 4 tcgen05.mma (M 128, N 128, K 16) with V read in its natural
//     [key][dim] layout (MN-major B operand), accumulating over all key tiles in
//     128 more columns of the slot.  A row's running maximum is moved only when a
//     tile's maximum passes it by more than 8 in exponent units; then (rarely
//     after the first tiles) the thread scales its row of O in tensor memory.
//     The MMAs of the scores two tiles on are issued right behind a tile's P V,
//     and one commit covers both.
// Each slot has a warp whose one thread issues its MMAs: the slot's softmax threads
// arrive on an mbarrier when their row of P is written, and wait on the mbarrier
// that tcgen05.commit arrives on for the next scores.  (One thread issuing for both
// slots measured a quarter slower: an issue waits for room in the tensor core's
// queue, and the other slot's P then waits behind it.)  What bounds the kernel at
// this tile shape is the number of MMA instructions, about 50 cycles each whatever
// their N: 12 a tile and slot.
// Every mbarrier wait is bounded: if one runs out the block sets *error_flag, and
// since every issued copy is waited for before the MMA that reads it, nothing is
// in flight when the block frees its tensor memory and returns.
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>

namespace {

constexpr int UM = 128;          // query rows per slot; a block has two slots (256 consecutive tokens)
constexpr int UN = 64;           // keys per tile
constexpr int UD = 128;          // head size
constexpr int WAIT_LIMIT = 1 << 20;   // tries of at most 2 microseconds each
constexpr int BT_CACHE_U = 1024; // block-table entries a block keeps in shared memory (longer ranges are read where they lie)
constexpr float LOG2E_U = 1.4426950408889634f;

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16_u(unsigned dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ bool mbar_try_wait_u(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"(2000u) : "memory");   // a try sleeps 2 microseconds at most
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_u(unsigned bar, unsigned parity) {
  for (int i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try_wait_u(bar, parity)) return true;
  return false;
}
// shared-memory matrix descriptor: start address, leading / stride byte offsets (in 16-byte units),
// descriptor version 1, 128-byte swizzle
__device__ __forceinline__ unsigned long long umma_desc(unsigned saddr, unsigned lbo_bytes, unsigned sbo_bytes) {
  unsigned long long d = 0;
  d |= (unsigned long long)((saddr & 0x3FFFF) >> 4);
  d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}
// instruction descriptor, kind::f16: D float32, A and B bfloat16, A K-major; B K-major or MN-major
__host__ __device__ constexpr unsigned umma_idesc(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)b_mn_major << 16) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                         unsigned accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// 32 consecutive columns of this thread's tensor-memory lane; the values are valid after tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_nowait(unsigned taddr, unsigned (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// two float32 in one 64-bit register, and arithmetic on both at once
__device__ __forceinline__ unsigned long long pair_f32(float lo, float hi) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpair_f32(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

struct UmmaMeta {
  const int* block_tables; int bt_stride;
  const int* entry_q_start; const int* entry_q_len; const int* entry_ctx_start;
};

// Shared memory (1024-byte aligned): Q of the two query tiles 2 x 32 KB | K 4 x 16 KB | V 4 x 16 KB
constexpr int SQ_BYTES = 2 * UM * 128, SKV_BYTES = 2 * UN * 128;
constexpr int K_STAGES = 4, V_STAGES = 4;
// A block takes 256 consecutive tokens of one request and one head as two query tiles ("slots") of 128 rows,
// which share every key and value tile the block brings in.  Eight softmax warps (one thread per query row of
// the two tiles), a warp per slot that issues its MMAs, a warp that copies keys and one that copies values.
constexpr int U_SOFTMAX = 2 * UM, U_THREADS = U_SOFTMAX + 128;
constexpr int SMEM_UMMA = 2 * SQ_BYTES + (K_STAGES + V_STAGES) * SKV_BYTES;
// Tensor memory, all 512 columns, per slot 256: S of even tiles 64 | S of odd tiles 64 | O 128.  P (64 packed
// bfloat16 = 32 columns) is written over the first half of the scores it was made from.
constexpr unsigned TM_SLOT = 256, TM_S = 0, TM_O = 128;
constexpr int XCH_STRIDE = UD + 4;   // floats a row of the exchange between the two slots of one query tile (O, maximum, sum)

// One TMA box of the paged cache into shared memory: 64 dims (one 128-byte panel row) x box_slots tokens of
// one page and kv head, written in the 128-byte swizzle that the MMA descriptors expect (the swizzle goes by
// the bits of the shared-memory address, so boxes of a few rows line up into one 64-row panel).  The first
// coordinate is 0 or 64 elements, i.e. a multiple of 128 bytes.  A page of -1 (given back behind a window,
// or beyond the request's last key) is outside the tensor and reads as zeros.  No multicast.
__device__ __forceinline__ void tma_load_kv(unsigned dst, const CUtensorMap* map, int dim0, int slot0, int kvh, int page,
                                            unsigned bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
               ::"r"(dst), "l"(map), "r"(dim0), "r"(slot0), "r"(kvh), "r"(page), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(U_THREADS, 1)
attn_prefill_umma_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                         const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         int page_size, int page_shift, UmmaMeta m, const int* __restrict__ tile_entry,
                         const int* __restrict__ tile_q0, int n_heads, int n_kv, float scale, int window,
                         int* __restrict__ error_flag, float* __restrict__ part_o, float* __restrict__ part_ml, int n_splits,
                         int tile_rows) {
  // The kernel before this one (it rotates the queries and writes the new keys and values) is waited for only
  // where its results are first read or the scratch of an earlier launch first written; until then the block
  // reads the step's description, sets up its barriers and gets its tensor memory.
  pdl_launch_dependents();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar_s[2][2];       // per slot and buffer of scores: the tensor core is done
  __shared__ __align__(8) unsigned long long bar_p[2][2];       // per slot and buffer of scores: all 128 rows of P are written
  __shared__ __align__(8) unsigned long long k_full[K_STAGES], k_free[K_STAGES];   // a key stage has landed / was read
  __shared__ __align__(8) unsigned long long v_full[V_STAGES], v_free[V_STAGES];
  __shared__ __align__(8) unsigned long long q_full;            // Q has landed (every softmax thread's copies)
  __shared__ unsigned tmem_slot;
  __shared__ int bt_s[BT_CACHE_U];
  const unsigned sbase = smem_addr(smem_raw);
  if (sbase & 1023u) {                                          // the swizzled tiles need it; never seen, but never assumed
    if (threadIdx.x == 0) atomicExch(error_flag, 1);
    return;
  }
  const unsigned sq0 = sbase, sk0 = sq0 + 2 * SQ_BYTES, sv0 = sk0 + K_STAGES * SKV_BYTES;
  const int tid = threadIdx.x, warp = tid >> 5;
  // tiles run last to first and heads fastest: the longest blocks (of every head) start first
  const int tile = gridDim.y - 1 - blockIdx.y;
  const int e = tile_entry[tile], q0 = tile_q0[tile], head = blockIdx.x;
  const int rows_all = min(tile_rows, m.entry_q_len[e] - q0);       // tile_rows: 256, or 128 (every tile on both slots)
  if (rows_all <= 0) return;
  const int tok0 = m.entry_q_start[e] + q0;
  const int pos0 = m.entry_ctx_start[e] + q0;
  const int kvh = head / (n_heads / n_kv);
  const int* bt = m.block_tables + (size_t)e * m.bt_stride;
  const int rows0 = min(UM, rows_all), rows1 = rows_all - rows0;  // rows of the two slots (the second may have none)
  const int kend = pos0 + rows_all;                              // keys [.., kend) may be seen by the block's last row
  const int kfirst = window > 0 ? max(0, pos0 - window + 1) : 0; // first key the block's first row may see
  // gridDim.z > 1: the key tiles are cut into n_splits consecutive parts, one block each; the parts leave
  // their unnormalised O and (maximum, sum) in scratch for the merge kernel.  Few query tiles over a long
  // context (a short portion of a long prompt) would otherwise leave most of the GPU idle.
  const int split = blockIdx.z;
  const int t_all0 = kfirst / UN, n_all = (kend - 1) / UN - t_all0 + 1;
  const int per_split = (n_all + n_splits - 1) / n_splits;
  const int t_begin = t_all0 + split * per_split, n_t = min(per_split, n_all - split * per_split);
  const size_t part_row0 = (((size_t)tile * n_heads + head) * n_splits + split) * (2 * UM);
  if (n_t <= 0) {                                                // (block-uniform) nothing to do: a part that adds nothing
    pdl_wait();
    if (tid < rows_all) {
      part_ml[(part_row0 + tid) * 2] = -INFINITY;
      part_ml[(part_row0 + tid) * 2 + 1] = 0.0f;
    }
    return;
  }
  // Which of the block's tiles a slot takes part in.  Both begin at the block's first tile (with a window the
  // second slot's first tiles may lie wholly before its rows' windows: they come out masked).  The first slot
  // stops where its last row's keys end, up to two tiles before the second; the second, when it has rows,
  // takes every tile, so it is always the last to read a stage.
  //
  // A block with one query tile only (a short portion, or a portion's last rows) deals its key tiles out to
  // the two slots in turn instead: both hold the same rows, the first takes the even tiles and the second the
  // odd ones, and their two results are put together at the end.
  const bool narrow = rows1 == 0 && n_t >= 2;
  const int n_t0 = narrow ? (n_t + 1) / 2 : max(0, min(n_t, (pos0 + rows0 - 1) / UN + 1 - t_begin));
  const int n_t1 = narrow ? n_t / 2 : (rows1 > 0 ? n_t : 0);

  if (tid == 0) {
    auto init = [](unsigned long long* b, int count) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(b)), "r"(count));
    };
    for (int sl = 0; sl < 2; ++sl)
      for (int i = 0; i < 2; ++i) init(&bar_s[sl][i], 1), init(&bar_p[sl][i], UM);
    for (int i = 0; i < K_STAGES; ++i) init(&k_full[i], 1), init(&k_free[i], 2);
    for (int i = 0; i < V_STAGES; ++i) init(&v_full[i], 1), init(&v_free[i], 2);
    init(&q_full, U_SOFTMAX);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(smem_addr(&tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  int bt_first = 0;
  {
    const int b0 = max(kfirst, t_begin * UN) >> page_shift, b1 = (min(kend, (t_begin + n_t) * UN) - 1) >> page_shift;
    if (b1 - b0 < BT_CACHE_U) {
      for (int i = tid; i <= b1 - b0; i += U_THREADS) bt_s[i] = bt[b0 + i];
      bt = bt_s;
      bt_first = b0;
    }
  }
  pdl_wait();
  // Q of both slots: row r (token tok0 + r), two panels of 64 dims per slot; rows beyond the portion are zero
  for (int idx = tid; idx < 2 * UM * 16 && tid < U_SOFTMAX; idx += U_SOFTMAX) {  // the softmax warps copy it, once
    const int r = idx >> 4, c = idx & 15, sl = r >> 7, rr = r & (UM - 1);
    const bool ok = r < rows_all;
    const bf16* src = q + (size_t)(tok0 + (ok ? r : 0)) * q_stride + (size_t)head * UD + c * 8;
    cp_async16_u(sq0 + sl * SQ_BYTES + (unsigned)(c >> 3) * (UM * 128) + (unsigned)rr * 128u + (unsigned)(((c & 7) ^ (rr & 7)) << 4), src, ok);
  }
  if (tid < U_SOFTMAX) asm volatile("cp.async.commit_group;\n" ::);
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();                                               // bt_s, barriers, tensor-memory address
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem = tmem_slot;
  // Q is waited for only now, and only by those who copy it: the first key and value tiles are on their way
  // meanwhile.  The issuing threads wait on q_full before their first MMA.
  if (tid < U_SOFTMAX) {
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); // Q is visible to the tensor core
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(&q_full)) : "memory");
  }

  // ---- the last two warps copy the key tiles and the value tiles, up to four tiles ahead of their use.  A
  // stage is free once the MMAs of both slots that read it are done (each issuing thread commits onto k_free /
  // v_free).  The boxes of a tile (a page and a 64-dim panel each) are issued by the lanes of the warp side by
  // side, and keys and values by a warp each: issuing a box takes a thread over a hundred cycles, and one warp
  // alone for the sixteen boxes of a step of 16-token pages held the tensor core up.
  if (warp >= U_SOFTMAX / 32 + 2) {
    bool copy_failed = false;
    {
      const int lane = tid & 31;
      const int box_slots = min(page_size, UN);                    // tokens per box: a page, or 64 of a longer page
      const int n_boxes = 2 * (UN / box_slots);                    // boxes of one tile of keys (or values)
      auto copy_tile = [&](const CUtensorMap* map, unsigned sdst, int t, unsigned bar) {
        if (lane == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(SKV_BYTES) : "memory");
        __syncwarp();
        for (int i = lane; i < n_boxes; i += 32) {
          const int b = i >> 1, panel = i & 1;
          const int key = (t_begin + t) * UN + b * box_slots;
          int page = -1;                                           // boxes wholly outside [kfirst, kend) read as zeros
          if (key < kend && key + box_slots > kfirst) page = bt[(key >> page_shift) - bt_first];
          tma_load_kv(sdst + panel * (UN * 128) + (unsigned)b * box_slots * 128u, map, panel * 64, key & (page_size - 1),
                      kvh, page, bar);
        }
      };
      const bool values = warp == U_SOFTMAX / 32 + 3;
      const CUtensorMap* map = values ? &map_v : &map_k;
      const unsigned s0 = values ? sv0 : sk0;
      unsigned long long* full = values ? v_full : k_full;
      unsigned long long* free_ = values ? v_free : k_free;
      const int n_stages = values ? V_STAGES : K_STAGES;
      for (int t = 0; t < n_t; ++t) {
        const int st = t % n_stages;
        if (t >= n_stages && !__all_sync(0xffffffffu, mbar_wait_u(smem_addr(&free_[st]), (unsigned)((t / n_stages - 1) & 1)))) { copy_failed = true; break; }
        copy_tile(map, s0 + st * SKV_BYTES, t, smem_addr(&full[st]));
      }
    }
    // Every copy that was issued is waited for by the issuing thread before its MMA, and the block ends
    // only after the last MMA: nothing is in flight when this warp leaves.  (If a wait ran out, the two
    // barriers below still hold the block together and the error is recorded.)
    const int any = __syncthreads_or(copy_failed);
    if (narrow) __syncthreads();                                 // (the two slots' results are put together here)
    __syncthreads();
    if (any && (tid & 31) == 0) atomicExch(error_flag, 1);
    return;
  }

  constexpr unsigned IDESC_QK = umma_idesc(UM, UN, 0), IDESC_PV = umma_idesc(UM, UD, 1);
  // ---- the ninth and tenth warp: one thread of each issues the MMAs of its slot.  S(t) = Q K(t)^T into the
  // slot's scores buffer t & 1 (8 steps of 16 dims); for tile i, once all the slot's rows of P are written,
  // P V of tile i and then the scores of tile i + 2, which overwrite the scores and P of tile i; one commit on
  // the slot's barrier covers both.  The tensor core works on one slot while the threads of the other are at
  // their scores.
  if (warp == U_SOFTMAX / 32 || warp == U_SOFTMAX / 32 + 1) {
    bool mma_failed = false;
    if ((tid & 31) == 0) {
      const int sl = warp - U_SOFTMAX / 32;
      const int n_mine = sl ? n_t1 : n_t0, n_other = sl ? n_t0 : n_t1;
      const unsigned tm = tmem + sl * TM_SLOT, sq = sq0 + (narrow ? 0 : sl) * SQ_BYTES;
      // the slot's j-th tile among the block's
      auto whole = [&](int j) { return narrow ? 2 * j + sl : j; };
      // a stage goes back to the copy warp after two arrivals: one from each slot, or both from the only
      // slot that reads the tile
      auto hand_back = [&](unsigned long long* bar, int t) {
        umma_commit(smem_addr(bar));
        if (narrow || t >= n_other) umma_commit(smem_addr(bar));
      };
      auto issue_qk = [&](int j) {                                 // the scores of the slot's j-th tile
        const int t = whole(j), st = t % K_STAGES;
        if (!mbar_wait_u(smem_addr(&k_full[st]), (unsigned)((t / K_STAGES) & 1))) { mma_failed = true; return; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned sk = sk0 + st * SKV_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const unsigned long long da = umma_desc(sq + (k >> 2) * (UM * 128) + (k & 3) * 32, 16, 1024);
          const unsigned long long db = umma_desc(sk + (k >> 2) * (UN * 128) + (k & 3) * 32, 16, 1024);
          umma_f16(tm + TM_S + (j & 1) * UN, da, db, IDESC_QK, k > 0);
        }
        hand_back(&k_free[st], t);
        umma_commit(smem_addr(&bar_s[sl][j & 1]));
      };
      if (!mbar_wait_u(smem_addr(&q_full), 0u)) mma_failed = true;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      for (int t = 0; t < 2 && t < n_mine && !mma_failed; ++t) issue_qk(t);
      for (int i = 0; i < n_mine && !mma_failed; ++i) {
        if (!mbar_wait_u(smem_addr(&bar_p[sl][i & 1]), (unsigned)((i >> 1) & 1))) { mma_failed = true; break; }
        const int t = whole(i), st = t % V_STAGES;
        if (!mbar_wait_u(smem_addr(&v_full[st]), (unsigned)((t / V_STAGES) & 1))) { mma_failed = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned sv = sv0 + st * SKV_BYTES;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {                // O += P V, 4 steps of 16 keys; P from tensor memory
          const unsigned long long db = umma_desc(sv + kk * 16 * 128, UN * 128, 1024);   // leading offset = panel stride
          const unsigned acc = (i | kk) != 0;
          asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                       ::"r"(tm + TM_O), "r"(tm + TM_S + (i & 1) * UN + kk * 8), "l"(db), "r"(IDESC_PV), "r"(acc) : "memory");
        }
        hand_back(&v_free[st], t);
        if (i + 2 < n_mine) issue_qk(i + 2);                       // its commit covers this P V as well
        else umma_commit(smem_addr(&bar_s[sl][i & 1]));
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    const int any = __syncthreads_or(mma_failed);
    if (narrow) __syncthreads();
    __syncthreads();                                             // (the softmax warps write the output between these two)
    if (any && (tid & 31) == 0) atomicExch(error_flag, 1);
    return;
  }

  // ---- the softmax threads: thread r of slot sl owns row r of that query tile
  const int sl = tid >> 7, row = tid & (UM - 1);
  const int my_n = sl ? n_t1 : n_t0, my_rows = (sl && !narrow) ? rows1 : rows0;
  const int my_pos0 = pos0 + (narrow ? 0 : sl * UM);
  const int my_kend = my_pos0 + my_rows;
  const int my_kfirst = window > 0 ? max(0, my_pos0 - window + 1) : 0;
  const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;  // this warp's quarter of the 128 lanes
  const unsigned tm_base = tmem + sl * TM_SLOT + lane_base, tm_o = tm_base + TM_O;
  float mrow = -INFINITY, lrow = 0.0f;
  const float sl2 = scale * LOG2E_U;
  const int p_row = my_pos0 + row;                                // this thread's query position
  bool failed = false;

  // O accumulates in tensor memory over all key tiles.  The running maximum of a row is only moved when a
  // tile's maximum passes it by more than RESCALE_STEP (in exponent units): until then P stays below
  // 2^RESCALE_STEP, which bfloat16 P and the float32 accumulator hold easily, and the row of O needs no
  // rescaling.  When it is moved, the thread multiplies its row of O in tensor memory by 2^(old - new).
  //
  // The scores of tile i + 1 are computed by the tensor core while the threads work on tile i (two buffers
  // of scores per slot).  MMAs issued for a slot in iteration i: P V of tile i, then the scores of tile i + 2,
  // then a commit on the barrier of buffer i & 1; so that barrier's completion number i / 2 (parity
  // (i >> 1) & 1) says that the scores of tile i are there, and with them P V up to tile i - 2.
  constexpr float RESCALE_STEP = 8.0f;
  for (int i = 0; i < my_n; ++i) {
    const unsigned tm_s = tm_base + TM_S + (i & 1) * UN;           // scores of this tile; P goes over their first half
    // the outcome of a wait is made the same for the whole warp, whose tensor-memory loads and stores are warp-wide
    if (__all_sync(0xffffffffu, mbar_wait_u(smem_addr(&bar_s[sl][i & 1]), (unsigned)((i >> 1) & 1)))) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int key0 = (t_begin + (narrow ? 2 * i + sl : i)) * UN;
      // this thread's row of scores
      float s[UN];
      {
        unsigned r0[32], r1[32];
        tmem_ld32_nowait(tm_s, r0);
        tmem_ld32_nowait(tm_s + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) { s[c] = __uint_as_float(r0[c]); s[32 + c] = __uint_as_float(r1[c]); }
      }
      if (key0 + UN - 1 > my_pos0 || window > 0 || key0 < my_kfirst || key0 + UN > my_kend) {   // diagonal, window, edges
#pragma unroll
        for (int c = 0; c < UN; ++c) {
          const int key = key0 + c;
          const bool vis = key <= p_row && key < my_kend && (window <= 0 || key > p_row - window);
          if (!vis) s[c] = -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, so the maxima do not wait for one another
#pragma unroll
      for (int c = 0; c < UN; c += 4) {
        mx4[0] = fmaxf(mx4[0], s[c]); mx4[1] = fmaxf(mx4[1], s[c + 1]);
        mx4[2] = fmaxf(mx4[2], s[c + 2]); mx4[3] = fmaxf(mx4[3], s[c + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // the running maximum is kept in raw-score units; exponents are taken of (s - m) * scale * log2(e)
      float alpha = 1.0f;
      if (mrow == -INFINITY) {
        mrow = mx;                                                 // nothing accumulated for this row yet
      } else if ((mx - mrow) * sl2 > RESCALE_STEP) {
        alpha = ex2((mrow - mx) * sl2);
        mrow = mx;
      }
      const float msc = mrow == -INFINITY ? 0.0f : mrow * sl2;     // a row that has seen nothing yet
      // P = 2^(s * sl2 - msc) as packed bfloat16 into tensor memory
      // exponents and the row sum in packed pairs of float32 (one instruction for two values)
      const unsigned long long sl2x2 = pair_f32(sl2, sl2), nmx2 = pair_f32(-msc, -msc);
      unsigned long long ls4[4] = {0ull, 0ull, 0ull, 0ull};        // four chains of (0.0f, 0.0f) sums
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        unsigned pk[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float e0, e1;
          unpair_f32(fma_f32x2(pair_f32(s[h * 16 + 2 * c], s[h * 16 + 2 * c + 1]), sl2x2, nmx2), e0, e1);
          const float p0 = ex2(e0), p1 = ex2(e1);
          ls4[c & 3] = add_f32x2(ls4[c & 3], pair_f32(p0, p1));
          pk[c] = pack2(p0, p1);
        }
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
                     ::"r"(tm_s + h * 8), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]),
                       "r"(pk[6]), "r"(pk[7]) : "memory");
      }
      {
        float lo, hi;
        unpair_f32(add_f32x2(add_f32x2(ls4[0], ls4[1]), add_f32x2(ls4[2], ls4[3])), lo, hi);
        lrow = lrow * alpha + (lo + hi);
      }
      // a moved maximum: this row of O is scaled down; the loads and stores are warp-wide, so the warp does
      // it when any of its rows needs it.  O must then be complete up to tile i - 1: the commit of iteration
      // i - 1 (completion number (i - 1) / 2 + 1 of the other buffer's barrier) says so.
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        if (!__all_sync(0xffffffffu, mbar_wait_u(smem_addr(&bar_s[sl][(i + 1) & 1]), (unsigned)((((i - 1) >> 1) + 1) & 1)))) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (!failed) {
#pragma unroll
          for (int j = 0; j < UD / 32; ++j) {
            unsigned r[32];
            tmem_ld32_nowait(tm_o + j * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
            asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                         ::"r"(tm_o + j * 32), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                           "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                           "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                           "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                         : "memory");
          }
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
    } else {
      failed = true;
    }
    if (failed) break;                                             // the issuing warp's wait for P will run out too
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(&bar_p[sl][i & 1])) : "memory");   // this row of P is written
  }
  // the slot's commit of its last iteration (buffer (n - 1) & 1, completion number (n - 1) / 2 + 1) covers its last P V
  if (my_n > 0 && !failed &&
      !__all_sync(0xffffffffu, mbar_wait_u(smem_addr(&bar_s[sl][(my_n - 1) & 1]), (unsigned)((((my_n - 1) >> 1) + 1) & 1))))
    failed = true;
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  float f0 = 1.0f, f1 = 0.0f;                                     // (one query tile on two slots: see below)
  float m_out = (my_n > 0 && mrow != -INFINITY) ? mrow * sl2 : -INFINITY;       // in exponent units
  const float4* other = nullptr;
  // A slot's result leaves the block: as unnormalised O with the row's maximum and sum for the merge kernel
  // when the keys are cut into parts; else as bfloat16 rows of the output.  Both go through shared memory,
  // the slot's own Q (read for the last time by the MMAs behind the wait above), so that a warp's stores are
  // runs of 256 bytes of a row: a thread storing its own row 16 bytes at a time took three times as long.
  const unsigned so = sq0 + (narrow ? 0 : sl) * SQ_BYTES;         // 128 rows of 256 bytes
  const int lane = tid & 31;
  // this thread's 32 columns j of O out of tensor memory (and, for a query tile on two slots, put together)
  auto load_o = [&](int j, unsigned (&r)[32]) {
    tmem_ld32_nowait(tm_o + j * 32, r);
    tmem_ld_wait();
    if (other) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 o1 = other[j * 8 + c];
        r[c * 4] = __float_as_uint(__uint_as_float(r[c * 4]) * f0 + o1.x * f1);
        r[c * 4 + 1] = __float_as_uint(__uint_as_float(r[c * 4 + 1]) * f0 + o1.y * f1);
        r[c * 4 + 2] = __float_as_uint(__uint_as_float(r[c * 4 + 2]) * f0 + o1.z * f1);
        r[c * 4 + 3] = __float_as_uint(__uint_as_float(r[c * 4 + 3]) * f0 + o1.w * f1);
      }
    }
  };
  // 16 bytes of this thread's row into the staging rows; piece p of row r lies at p ^ (r & 15)
  auto stage = [&](int piece, unsigned a, unsigned b2, unsigned c, unsigned d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n"
                 ::"r"(so + (unsigned)row * 256u + (unsigned)((piece ^ (row & 15)) << 4)), "r"(a), "r"(b2), "r"(c), "r"(d) : "memory");
  };
  // the warp stores the 32 staged rows that its own threads wrote, 256 bytes each, to dst + r * stride_bytes
  auto store_rows = [&](unsigned char* dst, size_t stride_bytes) {
    __syncwarp();
    const int piece = lane & 15;
#pragma unroll 4
    for (int it = 0; it < 16; ++it) {
      const int r = (warp & 3) * 32 + it * 2 + (lane >> 4);
      if (r < my_rows) {
        uint4 v;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(so + (unsigned)r * 256u + (unsigned)((piece ^ (r & 15)) << 4)));
        *reinterpret_cast<uint4*>(dst + (size_t)r * stride_bytes + piece * 16) = v;
      }
    }
    __syncwarp();
  };
  auto emit = [&]() {
    if (n_splits > 1) {
      const size_t prow0 = part_row0 + (narrow ? 0 : sl * UM);     // the slot's first row among the parts' rows
      if (my_n > 0) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {                     // 64 float32 columns (256 bytes a row) at a time
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            unsigned r[32];
            load_o(half * 2 + jj, r);
#pragma unroll
            for (int c = 0; c < 8; ++c) stage(jj * 8 + c, r[c * 4], r[c * 4 + 1], r[c * 4 + 2], r[c * 4 + 3]);
          }
          store_rows(reinterpret_cast<unsigned char*>(part_o + prow0 * UD + half * 64), UD * sizeof(float));
        }
      }
      if (row < my_rows) {
        part_ml[(prow0 + row) * 2] = m_out;
        part_ml[(prow0 + row) * 2 + 1] = my_n > 0 ? lrow : 0.0f;
      }
      return;
    }
    if (my_n <= 0) return;
    const float inv = lrow > 0.0f ? 1.0f / lrow : 0.0f;
#pragma unroll
    for (int j = 0; j < UD / 32; ++j) {
      unsigned r[32];
      load_o(j, r);
#pragma unroll
      for (int c = 0; c < 4; ++c)
        stage(j * 4 + c, pack2(__uint_as_float(r[c * 8]) * inv, __uint_as_float(r[c * 8 + 1]) * inv),
              pack2(__uint_as_float(r[c * 8 + 2]) * inv, __uint_as_float(r[c * 8 + 3]) * inv),
              pack2(__uint_as_float(r[c * 8 + 4]) * inv, __uint_as_float(r[c * 8 + 5]) * inv),
              pack2(__uint_as_float(r[c * 8 + 6]) * inv, __uint_as_float(r[c * 8 + 7]) * inv));
    }
    store_rows(reinterpret_cast<unsigned char*>(out + (size_t)(tok0 + (narrow ? 0 : sl * UM)) * out_stride + (size_t)head * UD),
               (size_t)out_stride * sizeof(bf16));
  };
  int any_failed;
  if (!narrow) {
    // each slot writes as soon as it is done itself: the first, which ends up to two tiles before the second,
    // does not wait for it
    if (!failed) emit();
    any_failed = __syncthreads_or(failed);
  } else {
    // One query tile dealt out to two slots: the second slot hands its row of O, its maximum and its sum to the
    // first through the key stages' shared memory (nothing reads or writes them any more), and the first puts
    // the two together as the merge kernel would: O = O0 f0 + O1 f1 with f = 2^(own maximum - common maximum).
    any_failed = __syncthreads_or(failed);
    float* xch = reinterpret_cast<float*>(smem_raw + 2 * SQ_BYTES);
    float* xrow = xch + (size_t)row * XCH_STRIDE;
    if (sl == 1 && !any_failed) {
#pragma unroll
      for (int j = 0; j < UD / 32; ++j) {
        unsigned r[32];
        tmem_ld32_nowait(tm_o + j * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(xrow + j * 32 + c * 4) = make_uint4(r[c * 4], r[c * 4 + 1], r[c * 4 + 2], r[c * 4 + 3]);
      }
      xrow[UD] = m_out;
      xrow[UD + 1] = lrow;
    }
    __syncthreads();
    if (sl == 0 && !any_failed) {
      const float m1 = xrow[UD], l1 = xrow[UD + 1];
      const float mm = fmaxf(m_out, m1);
      f0 = m_out == -INFINITY ? 0.0f : ex2(m_out - mm);
      f1 = m1 == -INFINITY ? 0.0f : ex2(m1 - mm);
      lrow = lrow * f0 + l1 * f1;
      m_out = mm;
      other = reinterpret_cast<const float4*>(xrow);
      emit();
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
  if (any_failed && tid == 0) atomicExch(error_flag, 1);
}

// The parts of a query tile's keys put together: block (head, tile, group of MERGE_ROWS rows), thread d takes
// column d of the group's rows.  The (maximum, sum) pairs of the group go through shared memory, where one
// thread a row turns them into each part's factor 2^(its maximum - the common maximum) and the row's 1 / sum;
// then every thread loads its column of eight parts at a time before it adds them up (in the order of the
// parts, always), so that the loads do not wait for one another: with one load after the other the kernel
// took longer than the attention it follows.
constexpr int MERGE_ROWS = 8, MERGE_MAX_SPLITS = 64, MERGE_BATCH = 8;
__global__ void __launch_bounds__(UD)
attn_prefill_umma_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                               bf16* __restrict__ out, long long out_stride, UmmaMeta m,
                               const int* __restrict__ tile_entry, const int* __restrict__ tile_q0, int n_heads, int n_splits,
                               int tile_rows) {
  pdl_launch_dependents();
  __shared__ float ml_s[MERGE_ROWS][MERGE_MAX_SPLITS][2];
  __shared__ float f_s[MERGE_ROWS][MERGE_MAX_SPLITS];
  __shared__ float inv_s[MERGE_ROWS];
  const int head = blockIdx.x, tile = blockIdx.y, r0 = blockIdx.z * MERGE_ROWS, d = threadIdx.x;
  const int e = tile_entry[tile], q0 = tile_q0[tile];               // (the step's description: there before any kernel)
  const int rows = min(tile_rows, m.entry_q_len[e] - q0);
  if (r0 >= rows) return;
  const int tok0 = m.entry_q_start[e] + q0;
  pdl_wait();                                                      // the parts are written
  const size_t base = ((size_t)tile * n_heads + head) * n_splits * (2 * UM);
  for (int i = threadIdx.x; i < MERGE_ROWS * n_splits; i += UD) {
    const int rr = i / n_splits, sp = i - rr * n_splits;
    const float2 v = r0 + rr < rows ? *reinterpret_cast<const float2*>(part_ml + (base + (size_t)sp * (2 * UM) + r0 + rr) * 2)
                                    : make_float2(-INFINITY, 0.0f);
    ml_s[rr][sp][0] = v.x;
    ml_s[rr][sp][1] = v.y;
  }
  __syncthreads();
  if (threadIdx.x < MERGE_ROWS) {
    const int rr = threadIdx.x;
    float mm = -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) mm = fmaxf(mm, ml_s[rr][sp][0]);
    float l = 0.0f;
    for (int sp = 0; sp < n_splits; ++sp) {                       // always in the order of the parts
      const float ms = ml_s[rr][sp][0];
      const float f = ms == -INFINITY ? 0.0f : ex2(ms - mm);       // a part that saw nothing: its O was not written
      f_s[rr][sp] = f;
      l += ml_s[rr][sp][1] * f;
    }
    inv_s[rr] = l > 0.0f ? 1.0f / l : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int rr = 0; rr < MERGE_ROWS; ++rr) {
    const int r = r0 + rr;
    if (r >= rows) continue;
    float acc = 0.0f;
    for (int sp0 = 0; sp0 < n_splits; sp0 += MERGE_BATCH) {
      float v[MERGE_BATCH], f[MERGE_BATCH];
#pragma unroll
      for (int k = 0; k < MERGE_BATCH; ++k) {
        const int sp = sp0 + k;
        f[k] = sp < n_splits ? f_s[rr][sp] : 0.0f;
        v[k] = f[k] != 0.0f ? part_o[(base + (size_t)sp * (2 * UM) + r) * UD + d] : 0.0f;
      }
#pragma unroll
      for (int k = 0; k < MERGE_BATCH; ++k) acc += v[k] * f[k];
    }
    out[(size_t)(tok0 + r) * out_stride + (size_t)head * UD + d] = __float2bfloat16_rn(acc * inv_s[rr]);
  }
}
// One run's keys (or values) in the paged cache as a 4-D tensor for TMA: (dim, slot in the page, kv head, page),
// boxes of 64 dims x min(page, 64) slots of one head and page, 128-byte swizzle, zeros outside the tensor.
int make_kv_map(CUtensorMap* map, const void* base, int head_dim, int page_size, int n_kv, int num_pages,
                long long page_stride) {
  static PFN_cuTensorMapEncodeTiled_v12000 enc = nullptr;
  if (!enc) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return IFX_ERR_UNSUPPORTED;
    enc = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)n_kv, (cuuint64_t)num_pages};
  cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)page_size * head_dim * 2, (cuuint64_t)page_stride * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)(page_size < UN ? page_size : UN), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : IFX_ERR_UNSUPPORTED;
}
}  // namespace

// Into how many parts the keys of the query tiles are best cut: 1 when the tiles alone fill the GPU, else as
// many as give every block a place at once, each part at least 8 key tiles of 64.
IFX_API int ifx_attn_prefill_umma_plan(int n_tiles, int n_heads, int max_key_tiles) {
  if (n_tiles < 1 || n_heads < 1) return 1;
  static int resident = 0;
  if (!resident) {
    // one block per SM: a block takes all 512 columns of an SM's tensor memory
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return 1;
    resident = sms > 0 ? sms : 1;
  }
  const long long blocks = (long long)n_tiles * n_heads;
  int s = (int)(resident / blocks);
  if (s > max_key_tiles / 8) s = max_key_tiles / 8;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

// Prompt portions, head_dim 128, query tiles of tile_rows = 256 or 128 tokens of one entry (tile_entry / tile_q0;
// with 128 every tile's key tiles are dealt out to both halves of its block: twice the blocks, for steps whose
// tiles of 256 would leave SMs idle).
// q rows, out rows, k_layer and v_layer 16-byte aligned.  error_flag: a device int set to 1 if a bounded
// wait inside the kernel ran out (the output is then invalid).  n_splits > 1: scratch part_o float32
// [n_tiles * n_heads * n_splits * 256 * 128] (16-byte aligned) and part_ml float32 [n_tiles * n_heads * n_splits * 256 * 2].
IFX_API int ifx_attn_prefill_umma(const void* q, long long q_stride, void* out, long long out_stride,
                                  void* k_layer, void* v_layer, long long page_stride, int page_size,
                                  const int* block_tables, int bt_stride, const int* tile_entry, const int* tile_q0,
                                  int n_tiles, const int* entry_q_start, const int* entry_q_len,
                                  const int* entry_ctx_start, int n_heads, int n_kv, int head_dim, float scale,
                                  int window, int* error_flag, float* part_o, float* part_ml, int n_splits,
                                  int num_pages, int tile_rows, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (head_dim != UD || n_kv < 1 || n_heads % n_kv || n_tiles > 65535 || !error_flag) return IFX_ERR_UNSUPPORTED;
  if (tile_rows != UM && tile_rows != 2 * UM) return IFX_ERR_UNSUPPORTED;
  if (n_splits < 1 || n_splits > MERGE_MAX_SPLITS || (n_splits > 1 && (!part_o || !part_ml))) return IFX_ERR_UNSUPPORTED;
  if (n_splits > 1 && ((uintptr_t)part_o & 15)) return IFX_ERR_ALIGNMENT;
  if (page_size <= 0 || (page_size & (page_size - 1)) || num_pages < 1) return IFX_ERR_UNSUPPORTED;
  if ((q_stride & 7) || (out_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) return IFX_ERR_ALIGNMENT;
  if ((page_stride & 7) || ((uintptr_t)k_layer & 15) || ((uintptr_t)v_layer & 15)) return IFX_ERR_ALIGNMENT;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  CUtensorMap map_k, map_v;
  int ifx_rc = make_kv_map(&map_k, k_layer, head_dim, page_size, n_kv, num_pages, page_stride);
  if (!ifx_rc) ifx_rc = make_kv_map(&map_v, v_layer, head_dim, page_size, n_kv, num_pages, page_stride);
  if (ifx_rc) return ifx_rc;
  UmmaMeta m{block_tables, bt_stride, entry_q_start, entry_q_len, entry_ctx_start};
  cudaError_t e = cudaFuncSetAttribute(attn_prefill_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_UMMA);
  if (e != cudaSuccess) return (int)e;
  ifx_rc = launch_pdl(attn_prefill_umma_kernel, dim3(n_heads, n_tiles, n_splits), dim3(U_THREADS), SMEM_UMMA, stream,
                      (const bf16*)q, q_stride, (bf16*)out, out_stride, map_k, map_v, page_size, page_shift, m,
                      tile_entry, tile_q0, n_heads, n_kv, scale, window, error_flag, part_o, part_ml, n_splits, tile_rows);
  if (!ifx_rc) ifx_rc = IFX_LAUNCH_CHECK();
  if (ifx_rc || n_splits == 1) return ifx_rc;
  ifx_rc = launch_pdl(attn_prefill_umma_merge_kernel, dim3(n_heads, n_tiles, tile_rows / MERGE_ROWS), dim3(UD), 0, stream, (const float*)part_o,
                      (const float*)part_ml, (bf16*)out, out_stride, m, tile_entry, tile_q0, n_heads, n_splits, tile_rows);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}
