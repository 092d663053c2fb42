// A second implementation of every operation of the model, on the host, in
// plain loops: no CUDA, no library, no vector tricks.  Tensors are float32;
// every sum (dot products, mean squares, softmax denominators, cumulative
// probabilities) runs in index order in a double accumulator and is rounded to
// float32 once.  It exists to be disagreed with: the CUDA kernels are tested
// against it and against a PyTorch restatement written separately, and the
// whole-model forward below steps over a paged cache of its own, so it also
// checks the cache logic of the engine against something that shares no code
// with it.  Nothing on the serving path calls this file.
//
// Formulas follow vjsingh1984/inferflux (paths within that project):
//   embedding            runtime/backends/cuda/native/cuda_kernels.cu:599-614
//   RMSNorm (+ add)      cuda_kernels.cu:469-501, :541-579   (weight after the rsqrt scale)
//   biases               cuda_kernels.cu:694-723
//   rotate-half RoPE     cuda_kernels.cu:69-115              (f = theta^(-2i/d), pairs (i, i + d/2))
//   attention            runtime/backends/cuda/kernels/flash_attention.cu:70-71,85,127-171
//                        (kv head = head / ratio, scale after the dot, key j visible iff j <= query position)
//   SiLU * up            cuda_kernels.cu:137-149
//   penalties            runtime/backends/cuda/native/gpu_sampler.cu:22-48
//   softmax, top-p       gpu_sampler.cu:216-267, :273-330
// Its own host-side oracles in the reference are tests/unit/test_native_forward.cpp:64-99
// (rotation) and :1364-1405 (naive causal GQA attention).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#define HR_API extern "C" __attribute__((visibility("default")))

namespace {

inline float dot(const float* a, const float* b, int n) {
  double s = 0.0;
  for (int i = 0; i < n; ++i) s += (double)a[i] * (double)b[i];
  return (float)s;
}

// element (page, head, slot, d) of one run's keys (or values): page0 is the run's [kv_head][slot][head_dim]
// block inside page 0, pages lie page_stride elements apart
inline long cache_at(long page, int head, int slot, int d, long page_stride, int page_size, int head_dim) {
  return page * page_stride + ((long)head * page_size + slot) * head_dim + d;
}

void rms_norm_row(const float* x, const float* w, float eps, float* y, int h) {
  double ss = 0.0;
  for (int i = 0; i < h; ++i) ss += (double)x[i] * (double)x[i];
  const float r = 1.0f / std::sqrt((float)(ss / h) + eps);
  for (int i = 0; i < h; ++i) y[i] = x[i] * r * w[i];
}

}  // namespace

HR_API void hr_embed_gather(const float* table, const int* ids, float* out, int n, int hidden) {
  for (int t = 0; t < n; ++t)
    for (int i = 0; i < hidden; ++i) out[(long)t * hidden + i] = table[(long)ids[t] * hidden + i];
}

// residual [n, hidden] += sum of the n_partials slices of delta ([n_partials][n][hidden]; null = nothing to add);
// out (null = none) gets the normed rows: all n, or the n_rows listed in rows (then the residual is left as it is
// and the sum is formed for those rows only).
HR_API void hr_add_rmsnorm(float* residual, const float* delta, int n_partials, const float* weight, float eps,
                           float* out, const int* rows, int n_rows, int n, int hidden) {
  std::vector<float> tmp(hidden);
  const int count = rows ? n_rows : n;
  for (int r = 0; r < count; ++r) {
    const int row = rows ? rows[r] : r;
    float* res = residual + (long)row * hidden;
    for (int i = 0; i < hidden; ++i) {
      float v = res[i];
      if (delta) {
        double d = 0.0;
        for (int p = 0; p < n_partials; ++p) d += (double)delta[((long)p * n + row) * hidden + i];
        v = v + (float)d;
      }
      tmp[i] = v;
    }
    if (!rows) std::memcpy(res, tmp.data(), sizeof(float) * hidden);
    if (out) rms_norm_row(tmp.data(), weight, eps, out + (long)r * hidden, hidden);
  }
}

// gate_up [m, 2 * inter] = [gate | up] -> out [m, inter] = gate / (1 + exp(-gate)) * up
HR_API void hr_swiglu(const float* gate_up, float* out, int m, int inter) {
  for (int r = 0; r < m; ++r)
    for (int i = 0; i < inter; ++i) {
      const float g = gate_up[(long)r * 2 * inter + i], u = gate_up[(long)r * 2 * inter + inter + i];
      out[(long)r * inter + i] = g / (1.0f + std::exp(-g)) * u;
    }
}

// y [m, n] = a [m, k] . w [n, k]^T (+ bias [n])
HR_API void hr_gemm(const float* a, const float* w, const float* bias, float* y, int m, int n, int k) {
  for (int r = 0; r < m; ++r)
    for (int c = 0; c < n; ++c) {
      float v = dot(a + (long)r * k, w + (long)c * k, k);
      y[(long)r * n + c] = bias ? v + bias[c] : v;
    }
}

// cos, sin [n, half] of position * inv_freq[i], angles in double
HR_API void hr_rope_table(const int* positions, const double* inv_freq, float* cos_out, float* sin_out, int n,
                          int half) {
  for (int t = 0; t < n; ++t)
    for (int i = 0; i < half; ++i) {
      const double a = (double)positions[t] * inv_freq[i];
      cos_out[(long)t * half + i] = (float)std::cos(a);
      sin_out[(long)t * half + i] = (float)std::sin(a);
    }
}

// qkv [n, (n_heads + 2 n_kv) * head_dim]: + bias (null = none); q and k heads rotated over their first 2 * half
// dimensions, pairs (i, i + half); q written back in place, k and v to cache slot slot_map[t] (< 0 = not stored).
HR_API void hr_qkv_rope_kv_write(float* qkv, const float* bias, const float* cos_t, const float* sin_t, int half,
                                 const int* slot_map, float* k_page0, float* v_page0, long page_stride, int page_size,
                                 int n, int n_heads, int n_kv, int head_dim) {
  const int width = (n_heads + 2 * n_kv) * head_dim;
  std::vector<float> row(width);
  for (int t = 0; t < n; ++t) {
    float* x = qkv + (long)t * width;
    for (int i = 0; i < width; ++i) row[i] = bias ? x[i] + bias[i] : x[i];
    for (int h = 0; h < n_heads + n_kv; ++h) {
      float* v = row.data() + (long)h * head_dim;
      for (int i = 0; i < half; ++i) {
        const float c = cos_t[(long)t * half + i], s = sin_t[(long)t * half + i];
        const float x0 = v[i], x1 = v[i + half];
        v[i] = x0 * c - x1 * s;
        v[i + half] = x0 * s + x1 * c;
      }
    }
    std::memcpy(x, row.data(), sizeof(float) * (long)n_heads * head_dim);
    if (n_kv == 0 || !slot_map || slot_map[t] < 0) continue;
    const long page = slot_map[t] / page_size;
    const int slot = slot_map[t] % page_size;
    for (int h = 0; h < n_kv; ++h)
      for (int d = 0; d < head_dim; ++d) {
        const long at = cache_at(page, h, slot, d, page_stride, page_size, head_dim);
        k_page0[at] = row[(long)(n_heads + h) * head_dim + d];
        v_page0[at] = row[(long)(n_heads + n_kv + h) * head_dim + d];
      }
  }
}

// Causal grouped-query attention over the paged cache.  Entry e brings q_len[e] query rows starting at row
// q_start[e]; its first query stands at position ctx_start[e]; the keys of positions 0 .. its own position are in
// the pages named by block_tables[e]; window > 0 hides keys more than window - 1 positions behind the query.
HR_API void hr_attention_paged(const float* q, long q_stride, float* out, long out_stride, const float* k_page0,
                               const float* v_page0, long page_stride, int page_size, const int* block_tables,
                               int table_width, const int* entry_q_start, const int* entry_q_len,
                               const int* entry_ctx_start, int n_entries, int n_heads, int n_kv, int head_dim,
                               float scale, int window) {
  const int ratio = n_heads / n_kv;
  std::vector<float> s;
  std::vector<double> acc(head_dim);
  for (int e = 0; e < n_entries; ++e)
    for (int i = 0; i < entry_q_len[e]; ++i) {
      const long row = entry_q_start[e] + i;
      const int pos = entry_ctx_start[e] + i;
      const int lo = window > 0 ? std::max(0, pos - window + 1) : 0;
      for (int h = 0; h < n_heads; ++h) {
        const int kh = h / ratio;
        const float* qv = q + row * q_stride + (long)h * head_dim;
        s.assign(pos - lo + 1, 0.0f);
        float top = -std::numeric_limits<float>::infinity();
        for (int j = lo; j <= pos; ++j) {
          const long page = block_tables[(long)e * table_width + j / page_size];
          const float* kv = k_page0 + cache_at(page, kh, j % page_size, 0, page_stride, page_size, head_dim);
          s[j - lo] = dot(qv, kv, head_dim) * scale;
          top = std::max(top, s[j - lo]);
        }
        double denom = 0.0;
        std::fill(acc.begin(), acc.end(), 0.0);
        for (int j = lo; j <= pos; ++j) {
          const float p = std::exp(s[j - lo] - top);
          denom += p;
          const long page = block_tables[(long)e * table_width + j / page_size];
          const float* vv = v_page0 + cache_at(page, kh, j % page_size, 0, page_stride, page_size, head_dim);
          for (int d = 0; d < head_dim; ++d) acc[d] += (double)p * (double)vv[d];
        }
        for (int d = 0; d < head_dim; ++d) out[row * out_stride + (long)h * head_dim + d] = (float)(acc[d] / denom);
      }
    }
}

// the lowest index among equal maxima; NaN never wins
HR_API void hr_argmax(const float* logits, long row_stride, int* out, int rows, int vocab) {
  for (int r = 0; r < rows; ++r) {
    int best = -1;
    for (int i = 0; i < vocab; ++i) {
      const float v = logits[(long)r * row_stride + i];
      if (std::isnan(v)) continue;
      if (best < 0 || v > logits[(long)r * row_stride + best]) best = i;
    }
    out[r] = best < 0 ? 0 : best;
  }
}

// for each listed id: logit > 0 ? logit / rep : logit * rep; -= freq * count; -= pres when count > 0
HR_API void hr_apply_penalties(float* logits, const int* ids, const int* counts, const int* n_recent, int width,
                               const float* rep, const float* freq, const float* pres, int rows, int vocab) {
  for (int r = 0; r < rows; ++r)
    for (int k = 0; k < n_recent[r]; ++k) {
      const int t = ids[(long)r * width + k], c = counts[(long)r * width + k];
      float v = logits[(long)r * vocab + t];
      v = v > 0.0f ? v / rep[r] : v * rep[r];
      v -= freq[r] * (float)c;
      if (c > 0) v -= pres[r];
      logits[(long)r * vocab + t] = v;
    }
}

// softmax(logits / temperature) restricted to the top_k largest (ties with the k-th kept), then to those within
// min_p of the largest, then to the smallest set of the largest whose mass reaches top_p (ties at the cut kept);
// zero elsewhere, not renormalised.  probs [vocab] in double.
HR_API void hr_kept_probabilities(const float* logits, int vocab, float temperature, int top_k, float top_p,
                                  float min_p, double* probs) {
  double top = -std::numeric_limits<double>::infinity();
  for (int i = 0; i < vocab; ++i) top = std::max(top, (double)logits[i] / temperature);
  double denom = 0.0;
  for (int i = 0; i < vocab; ++i) {
    probs[i] = std::exp((double)logits[i] / temperature - top);
    denom += probs[i];
  }
  for (int i = 0; i < vocab; ++i) probs[i] /= denom;
  std::vector<double> sorted(probs, probs + vocab);
  std::sort(sorted.begin(), sorted.end(), [](double a, double b) { return a > b; });
  if (top_k > 0 && top_k < vocab) {
    const double kth = sorted[top_k - 1];
    for (int i = 0; i < vocab; ++i)
      if (probs[i] < kth) probs[i] = 0.0;
  }
  if (min_p > 0.0f) {
    const double cut = (double)min_p * sorted[0];
    for (int i = 0; i < vocab; ++i)
      if (probs[i] < cut) probs[i] = 0.0;
  }
  if (top_p > 0.0f && top_p < 1.0f) {
    sorted.assign(probs, probs + vocab);
    std::sort(sorted.begin(), sorted.end(), [](double a, double b) { return a > b; });
    double total = 0.0;
    for (int i = 0; i < vocab; ++i) total += sorted[i];
    const double need = (double)top_p * total;
    double run = 0.0;
    int below = 0;                      // how many of the largest have a cumulative mass still short of need
    for (int i = 0; i < vocab; ++i) {
      run += sorted[i];
      if (run < need) ++below;
    }
    const double cut = sorted[std::min(below + 1, vocab) - 1];
    for (int i = 0; i < vocab; ++i)
      if (probs[i] < cut) probs[i] = 0.0;
  }
}

// the counter-based uniform in [0, 1) with 24 bits that the sampling kernels draw for (seed, counter)
HR_API double hr_uniform01(uint64_t seed, uint64_t counter) {
  auto mix = [](uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  };
  const uint64_t x = mix(mix(seed) ^ (counter * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull));
  return (double)(x >> 40) / 16777216.0;
}

// the token whose interval of the cumulative kept probability (in index order, renormalised) holds u
HR_API int hr_inverse_cdf(const double* probs, int vocab, double u) {
  double total = 0.0;
  for (int i = 0; i < vocab; ++i) total += probs[i];
  double run = 0.0;
  int last = 0;
  for (int i = 0; i < vocab; ++i) {
    if (probs[i] <= 0.0) continue;
    run += probs[i];
    last = i;
    if (u * total < run) return i;
  }
  return last;
}

// ------------------------------------------------------------------ whole model
struct HrLayer {
  const float *input_norm, *wq, *wk, *wv, *bq, *bk, *bv, *wo, *post_norm, *w_gate, *w_up, *w_down;
  int window;          // 0 = every key
  int pad;
};

struct HrModel {
  int hidden, n_heads, n_kv, head_dim, inter, vocab, n_layers, pad;
  float eps;
  float pad2;
  double theta;
  const float *embed, *final_norm, *lm_head;   // lm_head = embed when the head is tied
  const HrLayer* layers;
};

// One step over the host model's own paged cache: pool [page][layer][k|v][kv_head][slot][head_dim] float32.
// tokens [n] flattened over the entries; entry e brings q_len[e] tokens at positions ctx_start[e] ...; its pages
// are block_tables[e][...] (every position up to its last new token must have a page).  logits [n_want, vocab]
// for the rows listed in want_rows.  Returns 0, or a negative number if a page is missing.
HR_API int hr_model_step(const HrModel* m, float* pool, int page_size, const int* tokens, int n,
                         const int* entry_q_start, const int* entry_q_len, const int* entry_ctx_start, int n_entries,
                         const int* block_tables, int table_width, const int* want_rows, int n_want, float* logits) {
  const int H = m->hidden, nh = m->n_heads, nkv = m->n_kv, hd = m->head_dim, I = m->inter;
  const int qw = (nh + 2 * nkv) * hd, half = hd / 2;
  const long run_stride = 2L * nkv * page_size * hd, page_stride = (long)m->n_layers * run_stride;
  std::vector<int> positions(n), slot_map(n);
  for (int e = 0; e < n_entries; ++e)
    for (int i = 0; i < entry_q_len[e]; ++i) {
      const int pos = entry_ctx_start[e] + i, t = entry_q_start[e] + i;
      const int page = block_tables[(long)e * table_width + pos / page_size];
      if (page < 0) return -1;
      positions[t] = pos;
      slot_map[t] = page * page_size + pos % page_size;
    }
  std::vector<double> inv_freq(half);
  for (int i = 0; i < half; ++i) inv_freq[i] = 1.0 / std::pow(m->theta, 2.0 * i / hd);
  std::vector<float> cos_t((long)n * half), sin_t((long)n * half);
  hr_rope_table(positions.data(), inv_freq.data(), cos_t.data(), sin_t.data(), n, half);
  std::vector<float> residual((long)n * H), x((long)n * H), qkv((long)n * qw), attn((long)n * nh * hd),
      delta((long)n * H), gate_up((long)n * 2 * I), act((long)n * I);
  hr_embed_gather(m->embed, tokens, residual.data(), n, H);
  bool pending = false;
  for (int l = 0; l < m->n_layers; ++l) {
    const HrLayer& L = m->layers[l];
    hr_add_rmsnorm(residual.data(), pending ? delta.data() : nullptr, 1, L.input_norm, m->eps, x.data(), nullptr, 0,
                   n, H);
    for (int t = 0; t < n; ++t) {
      float* row = qkv.data() + (long)t * qw;
      hr_gemm(x.data() + (long)t * H, L.wq, L.bq, row, 1, nh * hd, H);
      hr_gemm(x.data() + (long)t * H, L.wk, L.bk, row + (long)nh * hd, 1, nkv * hd, H);
      hr_gemm(x.data() + (long)t * H, L.wv, L.bv, row + (long)(nh + nkv) * hd, 1, nkv * hd, H);
    }
    float* k0 = pool + (long)l * run_stride;
    float* v0 = k0 + (long)nkv * page_size * hd;
    hr_qkv_rope_kv_write(qkv.data(), nullptr, cos_t.data(), sin_t.data(), half, slot_map.data(), k0, v0, page_stride,
                         page_size, n, nh, nkv, hd);
    hr_attention_paged(qkv.data(), qw, attn.data(), (long)nh * hd, k0, v0, page_stride, page_size, block_tables,
                       table_width, entry_q_start, entry_q_len, entry_ctx_start, n_entries, nh, nkv, hd,
                       1.0f / std::sqrt((float)hd), L.window);
    hr_gemm(attn.data(), L.wo, nullptr, delta.data(), n, H, nh * hd);
    hr_add_rmsnorm(residual.data(), delta.data(), 1, L.post_norm, m->eps, x.data(), nullptr, 0, n, H);
    for (int t = 0; t < n; ++t) {
      hr_gemm(x.data() + (long)t * H, L.w_gate, nullptr, gate_up.data() + (long)t * 2 * I, 1, I, H);
      hr_gemm(x.data() + (long)t * H, L.w_up, nullptr, gate_up.data() + (long)t * 2 * I + I, 1, I, H);
    }
    hr_swiglu(gate_up.data(), act.data(), n, I);
    hr_gemm(act.data(), L.w_down, nullptr, delta.data(), n, H, I);
    pending = true;
  }
  if (n_want == 0) return 0;
  std::vector<float> last((long)n_want * H);
  hr_add_rmsnorm(residual.data(), pending ? delta.data() : nullptr, 1, m->final_norm, m->eps, last.data(), want_rows,
                 n_want, n, H);
  hr_gemm(last.data(), m->lm_head, nullptr, logits, n_want, m->vocab, H);
  return 0;
}
