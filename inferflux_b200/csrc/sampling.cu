// Token selection from float32 logits: argmax, repetition / frequency /
// presence penalties, and temperature sampling with top-k, top-p and min-p.
//
// Reference behaviour (runtime/backends/cuda/native/gpu_sampler.cu):
//   greedy      argmax over the row (:124-156, one block of 256, ties by thread order)
//   penalties   logit > 0 ? logit / rep : logit * rep;  -= freq * count;  -= pres if count > 0 (:22-48)
//   temperature softmax(logits / T) in three passes by one block (:216-267)
//   top-p       repeated arg-max until the cumulative probability reaches p (:273-330)
//   draw        one thread walks the cumulative sum against one uniform (:374-401)
// Here rows run in parallel, greedy returns the lowest index among equal
// maxima, top-k/top-p/min-p become a probability threshold on the float bit
// pattern, and the uniform comes from a counter-based generator keyed by
// (seed, counter) so a request's draws do not depend on the batch it is in.
// A row that fits the shared memory of a thread-block cluster (up to 409,600
// logits) is read once and held there by up to 8 blocks; the threshold is
// found by a radix search and all masses are added as integers (see
// sample_cluster_kernel).  Longer rows go to one block of 1024 threads per
// row that keeps exp(logit/T - max) in the caller's scratch `weights`
// [n_rows, vocab] float32 and bisects the threshold (sample_kernel).
#include "common.cuh"

namespace {
constexpr int ST = 1024;

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
// uniform in [0, 1) with 24 bits, from (seed, counter)
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long counter) {
  const unsigned long long x = mix64(mix64(seed) ^ (counter * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull));
  return (float)(x >> 40) * (1.0f / 16777216.0f);
}

struct ArgPair { float v; int i; };
__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
  // larger value wins; equal values: lower index wins; NaN never wins
  if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
  return a;
}
// The best pair of the block; every thread of warp 0 gets it.  `scratch` holds 32 pairs.
__device__ ArgPair block_best(ArgPair best, ArgPair* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  best = lane < nwarps ? scratch[lane] : ArgPair{-INFINITY, -1};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  return best;
}
__device__ ArgPair block_argmax(const float* row, int n, ArgPair* scratch) {
  ArgPair best{-INFINITY, -1};
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = row[i];
    if (v == v) best = better(best, ArgPair{v, i});
  }
  return block_best(best, scratch);
}

__global__ void __launch_bounds__(ST) argmax_kernel(const float* __restrict__ logits, long long row_stride,
                                                    int* __restrict__ out, int vocab) {
  pdl_enter();
  __shared__ ArgPair scratch[32];
  const ArgPair b = block_argmax(logits + (size_t)blockIdx.x * row_stride, vocab, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = b.i < 0 ? 0 : b.i;
}

// A wide row in two steps: blocks (part, row) each find the best of a slice of the row, then one
// warp per row picks among the parts.  `slice` is a multiple of 4; with `vec` rows are 16-byte aligned.
constexpr int AP = 256;
__global__ void __launch_bounds__(AP) argmax_part_kernel(const float* __restrict__ logits, long long row_stride,
                                                         int2* __restrict__ part, int vocab, int slice, int vec) {
  pdl_enter();
  __shared__ ArgPair scratch[32];
  const float* row = logits + (size_t)blockIdx.y * row_stride;
  const int lo = blockIdx.x * slice, hi = min(vocab, lo + slice);
  ArgPair best{-INFINITY, -1};
  if (vec) {
    for (int i = lo + threadIdx.x * 4; i < hi; i += AP * 4) {
      if (i + 3 < hi) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        if (v.x == v.x) best = better(best, ArgPair{v.x, i});
        if (v.y == v.y) best = better(best, ArgPair{v.y, i + 1});
        if (v.z == v.z) best = better(best, ArgPair{v.z, i + 2});
        if (v.w == v.w) best = better(best, ArgPair{v.w, i + 3});
      } else {
        for (int j = i; j < hi; ++j) {
          const float v = row[j];
          if (v == v) best = better(best, ArgPair{v, j});
        }
      }
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += AP) {
      const float v = row[i];
      if (v == v) best = better(best, ArgPair{v, i});
    }
  }
  best = block_best(best, scratch);
  if (threadIdx.x == 0) part[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = make_int2(__float_as_int(best.v), best.i);
}
__global__ void __launch_bounds__(32) argmax_final_kernel(const int2* __restrict__ part, int* __restrict__ out, int parts) {
  pdl_enter();
  ArgPair best{-INFINITY, -1};
  for (int p = threadIdx.x; p < parts; p += 32) {
    const int2 v = part[(size_t)blockIdx.x * parts + p];
    best = better(best, ArgPair{__int_as_float(v.x), v.y});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (threadIdx.x == 0) out[blockIdx.x] = best.i < 0 ? 0 : best.i;
}

// recent_ids / recent_counts: [n_rows, max_recent]; n_recent[row] entries are valid, ids distinct.
__global__ void penalties_kernel(float* __restrict__ logits, long long row_stride, const int* __restrict__ recent_ids,
                                 const int* __restrict__ recent_counts, const int* __restrict__ n_recent,
                                 int max_recent, const float* __restrict__ rep, const float* __restrict__ freq,
                                 const float* __restrict__ pres, int vocab) {
  pdl_enter();
  const int row = blockIdx.x;
  float* lg = logits + (size_t)row * row_stride;
  const int n = min(n_recent[row], max_recent);
  for (int k = threadIdx.x; k < n; k += blockDim.x) {
    const int id = recent_ids[(size_t)row * max_recent + k];
    if (id < 0 || id >= vocab) continue;
    const int count = recent_counts[(size_t)row * max_recent + k];
    float v = lg[id];
    const float r = rep[row];
    v = v > 0.0f ? v / r : v * r;
    v -= freq[row] * (float)count;
    if (count > 0) v -= pres[row];
    lg[id] = v;
  }
}

// The same penalties from the tokens themselves, kept on the device: ring [n_slots, ring_size] holds each
// request's tokens in order of arrival, written round and round; totals[slot] = how many were written in
// all.  Row r belongs to the request in slots[r] (negative: no penalties for this row) and counts its
// latest min(last_n[r], total, ring_size) tokens.  A thread per token: the first occurrence of an id within
// the window applies the penalties for all of them.
__global__ void penalties_ring_kernel(float* __restrict__ logits, long long row_stride, const int* __restrict__ ring,
                                      int ring_size, const int* __restrict__ totals, const int* __restrict__ slots,
                                      const int* __restrict__ last_n, const float* __restrict__ rep,
                                      const float* __restrict__ freq, const float* __restrict__ pres, int vocab) {
  pdl_enter();
  extern __shared__ int window[];                       // [ring_size]
  const int row = blockIdx.x;
  const int slot = slots[row];
  if (slot < 0) return;
  const int total = totals[slot];
  const int n = min(min(last_n[row], total), ring_size);
  for (int t = threadIdx.x; t < n; t += blockDim.x) window[t] = ring[(size_t)slot * ring_size + (total - 1 - t) % ring_size];
  __syncthreads();
  float* lg = logits + (size_t)row * row_stride;
  for (int t = threadIdx.x; t < n; t += blockDim.x) {
    const int id = window[t];
    if (id < 0 || id >= vocab) continue;
    int count = 0;
    bool first = true;
    for (int u = 0; u < n; ++u)
      if (window[u] == id) { ++count; if (u < t) first = false; }
    if (!first) continue;
    float v = lg[id];
    const float r = rep[row];
    v = v > 0.0f ? v / r : v * r;
    v -= freq[row] * (float)count;
    v -= pres[row];
    lg[id] = v;
  }
}

// ring[slots[r]] gets ids[r] as its next token (rows with a negative slot are skipped)
__global__ void ring_append_kernel(int* __restrict__ ring, int ring_size, int* __restrict__ totals,
                                   const int* __restrict__ slots, const int* __restrict__ ids, int n_rows) {
  pdl_enter();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n_rows) return;
  const int slot = slots[row];
  if (slot < 0) return;
  const int t = totals[slot];
  ring[(size_t)slot * ring_size + t % ring_size] = ids[row];
  totals[slot] = t + 1;
}

// sum / count over the entries whose weight bits are >= bits
__device__ __forceinline__ void block_sum_count_ge(const float* w, int n, unsigned bits, float* red,
                                                   float* sum_out, int* count_out) {
  float s = 0.0f;
  int c = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = w[i];
    if (__float_as_uint(v) >= bits) { s += v; ++c; }
  }
  *sum_out = block_sum(s, red);
  *count_out = (int)(block_sum((float)c, red) + 0.5f);   // exact below 2^24 entries
}

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, long long row_stride, float* __restrict__ weights,
              const float* __restrict__ temperature, const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const unsigned long long* __restrict__ seeds,
              const unsigned long long* __restrict__ counters, int* __restrict__ out, int vocab) {
  pdl_enter();
  __shared__ ArgPair ascratch[32];
  __shared__ float red[32];
  __shared__ float seg_prefix[ST];
  __shared__ int chosen;
  const int row = blockIdx.x;
  const float* lg = logits + (size_t)row * row_stride;
  const float temp = temperature[row];
  const ArgPair top = block_argmax(lg, vocab, ascratch);
  if (temp <= 0.0f || top.i < 0) {
    if (threadIdx.x == 0) out[row] = top.i < 0 ? 0 : top.i;
    return;
  }
  float* w = weights + (size_t)row * vocab;
  const float inv_t = 1.0f / temp;
  const float mx = top.v * inv_t;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = lg[i];
    w[i] = (v == v) ? expf(v * inv_t - mx) : 0.0f;     // in [0, 1], the maximum is exactly 1
  }
  __syncthreads();
  unsigned thr = 0u;                                    // keep entries with weight bits >= thr
  float kept_sum;
  int kept_count;
  const int k = top_k[row];
  if (k > 0 && k < vocab) {                             // largest threshold that keeps at least k entries
    unsigned lo = 0u, hi = 0x3F800000u;                 // bits of 0.0 .. 1.0
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1u) / 2u;
      block_sum_count_ge(w, vocab, mid, red, &kept_sum, &kept_count);
      if (kept_count >= k) lo = mid; else hi = mid - 1u;
    }
    thr = lo;
  }
  const float mp = min_p[row];
  if (mp > 0.0f) thr = max(thr, __float_as_uint(fminf(mp, 1.0f)));
  const float p = top_p[row];
  if (p > 0.0f && p < 1.0f) {                           // largest threshold whose kept mass is >= p of the mass kept so far
    float base_sum;
    block_sum_count_ge(w, vocab, thr, red, &base_sum, &kept_count);
    const float need = p * base_sum;
    unsigned lo = thr, hi = 0x3F800000u;
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1u) / 2u;
      block_sum_count_ge(w, vocab, mid, red, &kept_sum, &kept_count);
      if (kept_sum >= need) lo = mid; else hi = mid - 1u;
    }
    thr = lo;
  }
  // inverse CDF over the kept entries, in index order: thread t owns one contiguous segment
  const int seg = (vocab + ST - 1) / ST;
  const int begin = min(vocab, (int)threadIdx.x * seg), end = min(vocab, begin + seg);
  float mine = 0.0f;
  for (int i = begin; i < end; ++i) {
    const float v = w[i];
    if (__float_as_uint(v) >= thr) mine += v;
  }
  seg_prefix[threadIdx.x] = mine;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  if (threadIdx.x == 0) {                                // 1024 additions: exclusive prefix, fixed order
    float run = 0.0f;
    for (int t = 0; t < ST; ++t) { const float s = seg_prefix[t]; seg_prefix[t] = run; run += s; }
    red[0] = run;
  }
  __syncthreads();
  const float total = red[0];
  const float target = uniform01(seeds[row], counters[row]) * total;
  const float before = seg_prefix[threadIdx.x];
  const bool last_seg = (threadIdx.x == ST - 1);
  const float after = last_seg ? INFINITY : seg_prefix[threadIdx.x + 1];
  if (mine > 0.0f && before <= target && target < after) {
    float run = before;
    int pick = -1, last_kept = -1;
    for (int i = begin; i < end; ++i) {
      const float v = w[i];
      if (__float_as_uint(v) >= thr && v > 0.0f) {
        run += v;
        last_kept = i;
        if (target < run) { pick = i; break; }
      }
    }
    if (pick < 0) pick = last_kept;
    if (pick >= 0) atomicMax(&chosen, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[row] = chosen >= 0 ? chosen : top.i;
}

// ------------------------------------------------------------------ a row on a cluster
// The same draw for rows that fit the shared memory of a thread-block cluster (8 blocks hold up to 409,600
// logits): every block keeps its slice of the row in shared memory, so the row is read from memory once and
// every later pass runs on chip.  The threshold for top-k / top-p is found by a radix search over the float
// bit pattern (three levels of 1,024 bins, histograms added across the cluster through distributed shared
// memory) instead of 30 bisection passes each, and all masses are summed as 64-bit fixed-point integers
// (weight * 2^39, the maximum weight is exactly 1), so the result does not depend on the order of any sum
// nor on how many blocks share the row.
constexpr int SC_THREADS = 1024, SC_BINS = 1024, SC_MAX_CL = 8;
constexpr int SC_MAX_SLICE = 51200;                     // floats of a row one block keeps (200 KB)

struct SampleShared {
  unsigned limb[3][SC_BINS];                            // counts, or masses in three 13-bit limbs: 32-bit shared-memory adds
  unsigned long long hist[2][SC_BINS];                  // the limbs put together; two buffers: one is read by the cluster
                                                        // while the next fills
  unsigned long long warp_tot[32];
  unsigned long long part_base, part_total, bcast;      // what this block tells the others
  ArgPair best;
  ArgPair ascratch[32];
};

__device__ __forceinline__ unsigned long long weight_fix(float w) { return __float2ull_rz(w * 549755813888.0f); }   // * 2^39

__device__ __forceinline__ unsigned cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the address of the same shared-memory object in block `rank` of the cluster
template <typename T>
__device__ __forceinline__ const T* cluster_peer(const T* p, unsigned rank) {
  unsigned long long out;
  asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"((unsigned long long)p), "r"(rank));
  return reinterpret_cast<const T*>(out);
}

// inclusive sum over the block in thread order; every thread gets its own prefix
__device__ __forceinline__ unsigned long long block_scan_incl_u64(unsigned long long v, unsigned long long* warp_tot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();                                      // warp_tot may still be read from the call before
  if (lane == 31) warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {                                      // the warps' totals -> what lies before each warp
    const unsigned long long own = warp_tot[lane];
    unsigned long long t = own;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long u = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += u;
    }
    warp_tot[lane] = t - own;
  }
  __syncthreads();
  return v + warp_tot[warp];
}
__device__ __forceinline__ unsigned long long block_total_u64(unsigned long long v, unsigned long long* warp_tot) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long t = warp_tot[threadIdx.x & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// The largest threshold T >= floor_bits such that the entries with bits >= T number (COUNT) or weigh (fixed
// point) at least `target`; floor_bits if even that does not reach it.  w: this block's n weights.
template <bool COUNT>
__device__ unsigned radix_threshold(SampleShared& sh, const float* w, int n, unsigned floor_bits,
                                    unsigned long long target, int& buffer, int cl) {
  const int tid = threadIdx.x;
  unsigned prefix = 0;                                  // the bits above the level's ten, once decided
  unsigned long long above = 0;                         // count / mass of the entries above the prefix's range
  for (int lev = 0; lev < 3; ++lev) {
    const int shift = 20 - 10 * lev;
    unsigned long long* h = sh.hist[buffer & 1];
    ++buffer;
    sh.limb[0][tid] = 0;
    if (!COUNT) { sh.limb[1][tid] = 0; sh.limb[2][tid] = 0; }
    __syncthreads();
    for (int i = tid; i < n; i += SC_THREADS) {
      const float v = w[i];
      const unsigned b = __float_as_uint(v);
      if (b >= floor_bits && (lev == 0 || (b >> (shift + 10)) == prefix)) {
        const unsigned key = (b >> shift) & (SC_BINS - 1);
        if (COUNT) {
          atomicAdd(&sh.limb[0][key], 1u);
        } else {                                        // a slice has at most 51,200 entries: no limb's sum passes 2^32
          const unsigned long long q = weight_fix(v);
          if (q) {
            atomicAdd(&sh.limb[0][key], (unsigned)(q & 0x1FFFu));
            atomicAdd(&sh.limb[1][key], (unsigned)((q >> 13) & 0x1FFFu));
            atomicAdd(&sh.limb[2][key], (unsigned)(q >> 26));
          }
        }
      }
    }
    __syncthreads();
    h[tid] = COUNT ? (unsigned long long)sh.limb[0][tid]
                   : (unsigned long long)sh.limb[0][tid] + ((unsigned long long)sh.limb[1][tid] << 13) +
                         ((unsigned long long)sh.limb[2][tid] << 26);
    cluster_sync_all();
    const int bin = SC_BINS - 1 - tid;                  // thread order = bins from the top
    unsigned long long part[SC_MAX_CL];
#pragma unroll
    for (int r = 0; r < SC_MAX_CL; ++r) part[r] = r < cl ? cluster_peer(h, r)[bin] : 0ull;   // all loads in flight together
    unsigned long long tot = 0;
#pragma unroll
    for (int r = 0; r < SC_MAX_CL; ++r) tot += part[r];
    const unsigned long long reach = block_scan_incl_u64(tot, sh.warp_tot) + above;    // entries in this bin and above it
    const int n_reach = __syncthreads_count(reach >= target);                          // they are the last n_reach threads
    const int chosen = n_reach > 0 ? n_reach - 1 : 0;
    if (n_reach > 0 && n_reach < SC_BINS && tid == SC_BINS - n_reach - 1) sh.bcast = reach;   // the bins above the chosen one
    __syncthreads();
    if (n_reach > 0 && n_reach < SC_BINS) above = sh.bcast;
    prefix = (prefix << 10) | (unsigned)chosen;
    __syncthreads();                                    // bcast is free again
  }
  return prefix > floor_bits ? prefix : floor_bits;
}

__global__ void __launch_bounds__(SC_THREADS, 2)        // two blocks per SM: 32 registers a thread
sample_cluster_kernel(const float* __restrict__ logits, long long row_stride, const float* __restrict__ temperature,
                      const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                      const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
                      int* __restrict__ out, int vocab, int cl, int slice) {
  pdl_enter();
  extern __shared__ __align__(16) float w_s[];          // this block's slice of the row: logits, then weights
  __shared__ SampleShared sh;
  const int tid = threadIdx.x;
  const int row = blockIdx.x / cl;
  const int rank = (int)cluster_rank();
  const int begin = min(vocab, rank * slice), n = min(vocab, begin + slice) - begin;
  const float* lg = logits + (size_t)row * row_stride + begin;
  // the slice into shared memory, and its best logit
  ArgPair best{-INFINITY, -1};
  if ((((uintptr_t)lg) & 15) == 0) {
    for (int i = tid * 4; i < n; i += SC_THREADS * 4) {
      if (i + 4 <= n) {
        const float4 v = *reinterpret_cast<const float4*>(lg + i);
        *reinterpret_cast<float4*>(w_s + i) = v;
        if (v.x == v.x) best = better(best, ArgPair{v.x, begin + i});
        if (v.y == v.y) best = better(best, ArgPair{v.y, begin + i + 1});
        if (v.z == v.z) best = better(best, ArgPair{v.z, begin + i + 2});
        if (v.w == v.w) best = better(best, ArgPair{v.w, begin + i + 3});
      } else {
        for (int j = i; j < n; ++j) { const float v = lg[j]; w_s[j] = v; if (v == v) best = better(best, ArgPair{v, begin + j}); }
      }
    }
  } else {
    for (int i = tid; i < n; i += SC_THREADS) { const float v = lg[i]; w_s[i] = v; if (v == v) best = better(best, ArgPair{v, begin + i}); }
  }
  best = block_best(best, sh.ascratch);
  if (tid == 0) sh.best = best;
  cluster_sync_all();
  ArgPair top{-INFINITY, -1};
  {
    ArgPair peer[SC_MAX_CL];
#pragma unroll
    for (int r = 0; r < SC_MAX_CL; ++r) peer[r] = r < cl ? *cluster_peer(&sh.best, r) : ArgPair{-INFINITY, -1};
#pragma unroll
    for (int r = 0; r < SC_MAX_CL; ++r) top = better(top, peer[r]);                 // in rank order: the lowest index among equals
  }
  const float temp = temperature[row];
  if (temp <= 0.0f || top.i < 0) {
    if (rank == 0 && tid == 0) out[row] = top.i < 0 ? 0 : top.i;
    cluster_sync_all();                                 // no block leaves while another may still read its shared memory
    return;
  }
  const float inv_t = 1.0f / temp;
  const float mx = top.v * inv_t;
  for (int i = tid; i < n; i += SC_THREADS) {
    const float v = w_s[i];
    w_s[i] = (v == v) ? expf(v * inv_t - mx) : 0.0f;    // in [0, 1], the maximum is exactly 1
  }
  __syncthreads();
  int buffer = 0;
  unsigned thr = 0u;                                    // keep entries with weight bits >= thr
  const int k = top_k[row];
  if (k > 0 && k < vocab) thr = radix_threshold<true>(sh, w_s, n, 0u, (unsigned long long)k, buffer, cl);
  const float mp = min_p[row];
  if (mp > 0.0f) thr = max(thr, __float_as_uint(fminf(mp, 1.0f)));
  const float p = top_p[row];
  if (p > 0.0f && p < 1.0f) {                           // the largest threshold whose kept mass is >= p of the mass kept so far
    unsigned long long mine = 0;
    for (int i = tid; i < n; i += SC_THREADS) { const float v = w_s[i]; if (__float_as_uint(v) >= thr) mine += weight_fix(v); }
    mine = block_total_u64(mine, sh.warp_tot);
    if (tid == 0) sh.part_base = mine;
    cluster_sync_all();
    unsigned long long base = 0;
#pragma unroll
    for (int r = 0; r < SC_MAX_CL; ++r) base += r < cl ? *cluster_peer(&sh.part_base, r) : 0ull;
    unsigned long long need = (unsigned long long)((double)p * (double)base);
    if (need < 1) need = 1;
    thr = radix_threshold<false>(sh, w_s, n, thr, need, buffer, cl);
  }
  // inverse CDF over the kept entries in index order: first the block that holds the target, then the thread, then the entry
  unsigned long long mine = 0;
  for (int i = tid; i < n; i += SC_THREADS) { const float v = w_s[i]; if (__float_as_uint(v) >= thr) mine += weight_fix(v); }
  const unsigned long long block_total = block_total_u64(mine, sh.warp_tot);
  if (tid == 0) sh.part_total = block_total;
  cluster_sync_all();
  unsigned long long total = 0, offset = 0;
#pragma unroll
  for (int r = 0; r < SC_MAX_CL; ++r) {
    const unsigned long long t = r < cl ? *cluster_peer(&sh.part_total, r) : 0ull;
    if (r < rank) offset += t;
    total += t;
  }
  const unsigned long long target = (unsigned long long)((double)uniform01(seeds[row], counters[row]) * (double)total);   // < total
  if (target >= offset && target - offset < block_total) {                    // block-uniform
    const unsigned long long local = target - offset;
    const int seg = (n + SC_THREADS - 1) / SC_THREADS;
    const int sb = min(n, tid * seg), se = min(n, sb + seg);
    unsigned long long s = 0;
    for (int i = sb; i < se; ++i) { const float v = w_s[i]; if (__float_as_uint(v) >= thr) s += weight_fix(v); }
    const unsigned long long incl = block_scan_incl_u64(s, sh.warp_tot), before = incl - s;
    if (s > 0 && before <= local && local < incl) {     // exactly one thread
      unsigned long long run = before;
      int pick = se - 1;
      for (int i = sb; i < se; ++i) {
        const float v = w_s[i];
        if (__float_as_uint(v) >= thr) {
          run += weight_fix(v);
          if (local < run) { pick = i; break; }
        }
      }
      out[row] = begin + pick;
    }
  }
  cluster_sync_all();
}

// Blocks per row for the cluster kernel (a power of two up to 8), or 0 if the row does not fit
inline int sample_cluster_blocks(int vocab) {
  int cl = 1;
  while (cl < SC_MAX_CL && (vocab + cl - 1) / cl > 8192) cl <<= 1;
  return ((vocab + cl - 1) / cl + 3) / 4 * 4 <= SC_MAX_SLICE ? cl : 0;
}

int launch_sample_cluster(const float* logits, long long row_stride, const float* temperature, const int* top_k,
                          const float* top_p, const float* min_p, const unsigned long long* seeds,
                          const unsigned long long* counters, int* out, int n_rows, int vocab, int cl, cudaStream_t stream) {
  const int slice = ((vocab + cl - 1) / cl + 3) / 4 * 4;
  const size_t smem = (size_t)slice * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int rc = launch_pdl_cluster(sample_cluster_kernel, dim3(n_rows * cl), dim3(SC_THREADS), smem, stream, dim3(cl, 1, 1),
                                    logits, row_stride, temperature, top_k, top_p, min_p, seeds, counters, out, vocab, cl, slice);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
}  // namespace

// out[row] = lowest index of the largest value of the row (0 for a row of NaNs).  `part` is scratch of
// n_rows * parts pairs of ints (8-byte aligned) for rows cut into `parts` slices, or null with parts <= 1.
IFX_API int ifx_argmax(const float* logits, long long row_stride, int* out, int n_rows, int vocab, void* part, int parts,
                       cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0) return IFX_ERR_UNSUPPORTED;
  int ifx_rc;
  if (parts <= 1 || !part) {
    ifx_rc = launch_pdl(argmax_kernel, dim3(n_rows), dim3(ST), 0, stream, logits, row_stride, out, vocab);
    return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
  }
  if (((uintptr_t)part & 7) || n_rows > 65535) return IFX_ERR_ALIGNMENT;
  const int slice = ((vocab + parts - 1) / parts + 3) / 4 * 4;
  const int vec = ((uintptr_t)logits & 15) == 0 && (row_stride & 3) == 0;
  ifx_rc = launch_pdl(argmax_part_kernel, dim3(parts, n_rows), dim3(AP), 0, stream, logits, row_stride, (int2*)part, vocab, slice, vec);
  if (!ifx_rc) ifx_rc = IFX_LAUNCH_CHECK();
  if (ifx_rc) return ifx_rc;
  ifx_rc = launch_pdl(argmax_final_kernel, dim3(n_rows), dim3(32), 0, stream, (const int2*)part, out, parts);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_apply_penalties(float* logits, long long row_stride, const int* recent_ids, const int* recent_counts,
                                const int* n_recent, int max_recent, const float* rep, const float* freq,
                                const float* pres, int n_rows, int vocab, cudaStream_t stream) {
  if (n_rows <= 0 || max_recent <= 0) return 0;
  const int ifx_rc = launch_pdl(penalties_kernel, dim3(n_rows), dim3(128), 0, stream, logits, row_stride, recent_ids, recent_counts, n_recent, max_recent,
                                               rep, freq, pres, vocab);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

// Penalties from the device-resident token rings (penalties_ring_kernel), and the rings' update with the
// tokens just sampled.  ring_size at most 4096.
IFX_API int ifx_apply_penalties_ring(float* logits, long long row_stride, const int* ring, int ring_size,
                                     const int* totals, const int* slots, const int* last_n, const float* rep,
                                     const float* freq, const float* pres, int n_rows, int vocab, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (ring_size < 1 || ring_size > 4096) return IFX_ERR_UNSUPPORTED;
  const int threads = ring_size < 256 ? (ring_size + 31) / 32 * 32 : 256;
  const int ifx_rc = launch_pdl(penalties_ring_kernel, dim3(n_rows), dim3(threads), (size_t)ring_size * sizeof(int), stream, logits,
                                row_stride, ring, ring_size, totals, slots, last_n, rep, freq, pres, vocab);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_ring_append(int* ring, int ring_size, int* totals, const int* slots, const int* ids, int n_rows,
                            cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (ring_size < 1) return IFX_ERR_UNSUPPORTED;
  const int ifx_rc = launch_pdl(ring_append_kernel, dim3((n_rows + 127) / 128), dim3(128), 0, stream, ring, ring_size, totals, slots, ids,
                                n_rows);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_sample(const float* logits, long long row_stride, float* weights, const float* temperature,
                       const int* top_k, const float* top_p, const float* min_p, const unsigned long long* seeds,
                       const unsigned long long* counters, int* out, int n_rows, int vocab, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab >= (1 << 24)) return IFX_ERR_UNSUPPORTED;
  if (const int cl = sample_cluster_blocks(vocab))     // rows that fit a cluster's shared memory; the scratch is not used
    return launch_sample_cluster(logits, row_stride, temperature, top_k, top_p, min_p, seeds, counters, out, n_rows, vocab, cl, stream);
  const int ifx_rc = launch_pdl(sample_kernel, dim3(n_rows), dim3(ST), 0, stream, logits, row_stride, weights, temperature, top_k, top_p, min_p, seeds,
                                           counters, out, vocab);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- no allocation
// ifx_sample_static: ifx_sample for callers that cannot allocate (see sample_static.h).
// The scratch that ifx_sample takes from its caller lives here instead.
#include "sample_static.h"

namespace {
// exp(logit / T - max) of the rows of the call in progress; shared by all calls on the device
static __device__ __align__(256) float g_sample_static_weights[(size_t)IFX_SAMPLE_STATIC_MAX_ROWS *
                                                               IFX_SAMPLE_STATIC_MAX_VOCAB];
constexpr int kMaxDevices = 64;
float* g_sample_static_ptr[kMaxDevices] = {};   // device address of the array, per device, once looked up
}  // namespace

extern "C" const char* ifx_sample_static_message(int code) {
  switch (code) {
    case 0: return "success";
    case IFX_ERR_STATIC_TOO_LARGE:
      return "ifx_sample_static: n_rows or vocab is beyond the built-in scratch "
             "(at most 8 rows of at most 262144 logits); use ifx_sample with a buffer of your own";
    case IFX_ERR_UNSUPPORTED: return "ifx_sample_static: unsupported argument (vocab must be below 2^24, device index below 64)";
    default: return cudaGetErrorString((cudaError_t)code);
  }
}

extern "C" int ifx_sample_static(const float* logits, long long row_stride, const float* temperature,
                                 const int* top_k, const float* top_p, const float* min_p,
                                 const unsigned long long* seeds, const unsigned long long* counters, int* out,
                                 int n_rows, int vocab, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_rows > IFX_SAMPLE_STATIC_MAX_ROWS || vocab > IFX_SAMPLE_STATIC_MAX_VOCAB) return IFX_ERR_STATIC_TOO_LARGE;
  if (vocab < 1) return IFX_ERR_UNSUPPORTED;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return IFX_ERR_UNSUPPORTED;
  float* scratch = g_sample_static_ptr[dev];
  if (!scratch) {
    // In host code the array's name is only a handle; the kernel needs its address on this device.
    e = cudaGetSymbolAddress((void**)&scratch, g_sample_static_weights);
    if (e != cudaSuccess) return (int)e;
    g_sample_static_ptr[dev] = scratch;
  }
  // rows are packed [n_rows, vocab]; every element a row reads is written first, so nothing is cleared
  const int ifx_rc = launch_pdl(sample_kernel, dim3(n_rows), dim3(ST), 0, stream, logits, row_stride, scratch, temperature, top_k, top_p, min_p, seeds,
                                           counters, out, vocab);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

IFX_STAMP_READER(ifx_stamps_sampling)
