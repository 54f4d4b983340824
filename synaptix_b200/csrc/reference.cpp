// Plain C++ counterparts of the kernels, for the CPU: one function per operation, naive loops, one element at a
// time, 32-bit math where the kernels have it and 64-bit sums where a kernel's order of addition is its own
// business.  They take the same arguments as the kernels' exported functions (host pointers, no stream), so a
// test calls both with the same data.  Nothing on the product path calls them: they say what each kernel
// computes, in the manner of the reference's CPU kernels (crates/synaptix-kernels-cpu/src/lib.rs), and the tests
// compare every CUDA kernel with them.
//
// bfloat16 is the upper half of a float32, rounded to nearest even (a NaN stays a NaN).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#define SX_F32 0
#define SX_BF16 1
#define SX_ERR_DTYPE 10001
#define SX_ERR_SIZE 10002
#define SX_PAGE 64

namespace {

inline float bf16_to_f32(uint16_t v) {
  uint32_t b = (uint32_t)v << 16;
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {
  uint32_t b;
  std::memcpy(&b, &f, 4);
  if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x0040u);      // NaN, kept quiet
  b += 0x7fffu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}
inline float load(const void* p, size_t i, int dt) {
  return dt == SX_F32 ? static_cast<const float*>(p)[i] : bf16_to_f32(static_cast<const uint16_t*>(p)[i]);
}
inline void store(void* p, size_t i, int dt, float v) {
  if (dt == SX_F32) static_cast<float*>(p)[i] = v;
  else static_cast<uint16_t*>(p)[i] = f32_to_bf16(v);
}
inline bool known(int dt) { return dt == SX_F32 || dt == SX_BF16; }

// the key that orders floats as unsigned integers (the sampling kernel cuts by it)
inline uint32_t order_key(float f) {     // larger float, larger key; a NaN counts as -inf
  if (f != f) f = -INFINITY;
  uint32_t b;
  std::memcpy(&b, &f, 4);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Philox4x32-10, key (seed lo, seed hi), counter (c0, c1, 0, 0) (crates/synaptix-ops/src/rng.rs:1-97)
uint32_t philox_word(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, int word) {
  uint32_t c[4] = {c0, c1, 0u, 0u};
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0, hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c[word & 3];
}

}  // namespace

extern "C" {

// out[t, :] = float(table[ids[t], :]); an id outside the table gives zeros
int sx_ref_embed_gather(const void* table, int dt, const int* ids, float* out, int n_tokens, int H, int V) {
  if (!known(dt)) return SX_ERR_DTYPE;
  for (int t = 0; t < n_tokens; ++t) {
    const int id = ids[t];
    for (int i = 0; i < H; ++i) out[(size_t)t * H + i] = (id >= 0 && id < V) ? load(table, (size_t)id * H + i, dt) : 0.f;
  }
  return 0;
}

// v = h[t] (+ delta[t]); if write_h: h[t] = v; y[r] = v * rsqrt(mean(v^2) + eps) * w, t = rows ? rows[r] : r
// (crates/synaptix-models/llm/common/src/model.rs:209-244)
int sx_ref_add_rmsnorm(float* h, const void* delta, const float* w, float eps, void* y, const int* rows, int R, int H,
                       int dt, int write_h) {
  if (!known(dt)) return SX_ERR_DTYPE;
  std::vector<float> v(H);
  for (int r = 0; r < R; ++r) {
    const size_t t = rows ? rows[r] : r;
    double ss = 0.0;
    for (int i = 0; i < H; ++i) {
      v[i] = h[t * H + i] + (delta ? load(delta, t * H + i, dt) : 0.f);
      if (delta && write_h) h[t * H + i] = v[i];
      ss += (double)v[i] * v[i];
    }
    const float inv = 1.0f / std::sqrt((float)(ss / H) + eps);
    for (int i = 0; i < H; ++i) store(y, (size_t)r * H + i, dt, v[i] * inv * w[i]);
  }
  return 0;
}

int sx_ref_residual_add(float* h, const void* delta, long long n, int dt) {
  if (!known(dt)) return SX_ERR_DTYPE;
  for (long long i = 0; i < n; ++i) h[i] += load(delta, (size_t)i, dt);
  return 0;
}

// C[m, n] = sum_k A[m, k] * W[n, k]
int sx_ref_gemm(const void* A, int a_dt, const void* W, int w_dt, void* C, int c_dt, int M, int N, int K) {
  if (!known(a_dt) || !known(w_dt) || !known(c_dt)) return SX_ERR_DTYPE;
  if (K <= 0) return SX_ERR_SIZE;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      double s = 0.0;
      for (int k = 0; k < K; ++k) s += (double)load(A, (size_t)m * K + k, a_dt) * load(W, (size_t)n * K + k, w_dt);
      store(C, (size_t)m * N + n, c_dt, (float)s);
    }
  return 0;
}

// out[t, i] = silu(gu[t, i]) * gu[t, I + i]
int sx_ref_silu_mul(const void* gu, void* out, int n_tokens, int I, int dt) {
  if (!known(dt)) return SX_ERR_DTYPE;
  for (int t = 0; t < n_tokens; ++t)
    for (int i = 0; i < I; ++i) {
      const float g = load(gu, (size_t)t * 2 * I + i, dt), u = load(gu, (size_t)t * 2 * I + I + i, dt);
      store(out, (size_t)t * I + i, dt, g / (1.f + std::exp(-g)) * u);
    }
  return 0;
}

// Heads of the fused projection qkv[t] = [q heads | k heads | v heads]: q and k heads get an RMSNorm over the head
// (gain wq / wk, skipped when null) and a rotate-half rotation of their first rotary_dim elements by
// pos * inv_freq[i] (skipped when inv_freq is null); q goes to q_out[t, head, :], k and v into the token's place
// in its sequence's page (crates/synaptix-models/llm/common/src/model.rs:300-420).
int sx_ref_qkv_prepare(const void* qkv, void* q_out, void* k_pages, void* v_pages, const float* wq, const float* wk,
                       const float* inv_freq, int rotary_dim, float eps, const int* positions, const int* seq_of_token,
                       const int* block_table, int maxp, int n_tokens, int nh, int nkv, int hd, int n_pages, int dt) {
  if (!known(dt)) return SX_ERR_DTYPE;
  if (hd <= 0 || (rotary_dim & 1) || rotary_dim > hd) return SX_ERR_SIZE;
  const int half = inv_freq ? rotary_dim / 2 : 0;
  const size_t row = (size_t)(nh + 2 * nkv) * hd;
  std::vector<float> x(hd);
  for (int t = 0; t < n_tokens; ++t) {
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_of_token[t] * maxp + (pos >> 6)];
    const bool page_ok = page >= 0 && page < n_pages;
    for (int head = 0; head < nh + 2 * nkv; ++head) {
      const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
      void* dst;
      size_t at;
      if (is_q) {
        dst = q_out;
        at = ((size_t)t * nh + head) * hd;
      } else {
        dst = is_k ? k_pages : v_pages;
        if (!dst || !page_ok) continue;
        const int kvh = is_k ? head - nh : head - nh - nkv;
        at = (((size_t)page * nkv + kvh) * SX_PAGE + (pos & 63)) * hd;
      }
      double ss = 0.0;
      for (int i = 0; i < hd; ++i) {
        x[i] = load(qkv, (size_t)t * row + (size_t)head * hd + i, dt);
        ss += (double)x[i] * x[i];
      }
      if (is_q || is_k) {
        const float* w = is_q ? wq : wk;
        if (w) {
          const float inv = 1.0f / std::sqrt((float)(ss / hd) + eps);
          for (int i = 0; i < hd; ++i) x[i] = x[i] * inv * w[i];
        }
        for (int p = 0; p < half; ++p) {
          const float ang = (float)pos * inv_freq[p];
          const float c = std::cos(ang), s = std::sin(ang);
          const float a = x[p], b = x[p + half];
          x[p] = a * c - b * s;
          x[p + half] = a * s + b * c;
        }
      }
      for (int i = 0; i < hd; ++i) store(dst, at + i, dt, x[i]);
    }
  }
  return 0;
}

// Attention of every token's query heads over its sequence's keys lo..pos in the paged cache,
// lo = window > 0 ? max(0, pos - window + 1) : 0; query head h reads kv head h / (nh / nkv); softmax of
// q.k * scale over those keys, times the values (crates/synaptix-models/llm/common/src/model.rs:420-520).
int sx_ref_attn(const void* q, const void* k_pages, const void* v_pages, void* out, const int* positions,
                const int* seq_of_token, const int* block_table, int maxp, int n_tokens, int nh, int nkv, int hd,
                float scale, int window, int dt) {
  if (!known(dt)) return SX_ERR_DTYPE;
  if (hd <= 0 || nkv <= 0 || nh % nkv != 0) return SX_ERR_SIZE;
  std::vector<double> p, acc(hd);
  for (int t = 0; t < n_tokens; ++t) {
    const int pos = positions[t];
    const int* bt = block_table + (size_t)seq_of_token[t] * maxp;
    const int lo = window > 0 ? std::max(0, pos - window + 1) : 0;
    for (int h = 0; h < nh; ++h) {
      const int kvh = h / (nh / nkv);
      p.assign(pos - lo + 1, 0.0);
      double mx = -INFINITY;
      for (int j = lo; j <= pos; ++j) {
        const size_t kr = (((size_t)bt[j >> 6] * nkv + kvh) * SX_PAGE + (j & 63)) * hd;
        double d = 0.0;
        for (int i = 0; i < hd; ++i) d += (double)load(q, ((size_t)t * nh + h) * hd + i, dt) * load(k_pages, kr + i, dt);
        p[j - lo] = d * scale;
        mx = std::max(mx, p[j - lo]);
      }
      double l = 0.0;
      std::fill(acc.begin(), acc.end(), 0.0);
      for (int j = lo; j <= pos; ++j) {
        const double e = std::exp(p[j - lo] - mx);
        l += e;
        const size_t vr = (((size_t)bt[j >> 6] * nkv + kvh) * SX_PAGE + (j & 63)) * hd;
        for (int i = 0; i < hd; ++i) acc[i] += e * load(v_pages, vr + i, dt);
      }
      for (int i = 0; i < hd; ++i) store(out, ((size_t)t * nh + h) * hd + i, dt, (float)(acc[i] / l));
    }
  }
  return 0;
}

// index of each row's maximum; among equal maxima the last one; a NaN never wins (a row of NaNs gives V - 1)
// (crates/synaptix-infer/src/sampling/greedy.rs:8-12)
int sx_ref_argmax_rows(const float* logits, int* out, int R, int V) {
  if (V <= 0) return SX_ERR_SIZE;
  for (int r = 0; r < R; ++r) {
    float bv = -INFINITY;
    int bi = -1;
    for (int i = 0; i < V; ++i) {
      float v = logits[(size_t)r * V + i];
      if (v != v) v = -INFINITY;
      if (v >= bv) { bv = v; bi = i; }
    }
    out[r] = bi < 0 ? V - 1 : bi;
  }
  return 0;
}

// Penalties over the last `last_n` (0 = all) tokens of each row's context hist[r, 0..hist_len[r]): repetition
// once per occurrence (logit > 0 ? logit / rep : logit * rep), presence and frequency once per distinct token
// (crates/synaptix-infer/src/sampling/repetition.rs:7-77)
int sx_ref_penalties(float* logits, const int* hist, const int* hist_len, int hist_stride, int last_n, float rep,
                     float presence, float frequency, int R, int V) {
  std::vector<int> cnt(V);
  for (int r = 0; r < R; ++r) {
    std::fill(cnt.begin(), cnt.end(), 0);
    const int n = hist_len[r];
    const int start = (last_n > 0 && last_n < n) ? n - last_n : 0;
    for (int i = start; i < n; ++i) {
      const int t = hist[(size_t)r * hist_stride + i];
      if (t >= 0 && t < V) ++cnt[t];
    }
    for (int i = 0; i < V; ++i) {
      if (!cnt[i]) continue;
      float x = logits[(size_t)r * V + i];
      if (rep != 1.0f)
        for (int k = 0; k < cnt[i]; ++k) x = x > 0.f ? x / rep : x * rep;
      if (presence != 0.f || frequency != 0.f) x -= presence + frequency * (float)cnt[i];
      logits[(size_t)r * V + i] = x;
    }
  }
  return 0;
}

// Greedy if temperature <= 0.  Else x = logit / temperature; top-k keeps the k largest (with everything equal to
// the k-th); top-p keeps the shortest run of largest values whose probability mass exceeds top_p (of what top-k
// kept; equals of the last one included); min-p keeps exp(x - max) >= min_p; then the token whose interval of the
// cumulative kept mass, in index order, holds u * total, u = Philox word (seed; step / 4, seq_index; step % 4) / 2^32
// (crates/synaptix-infer/src/sampling/{top_k,top_p,min_p,multinomial}.rs).  keep_out [R, V], if given, gets 1
// where a token was kept.
int sx_ref_sample_rows(const float* logits, int* out, int R, int V, float temperature, int top_k, float top_p, float min_p,
                       unsigned long long seed, const int* seq_index, const int* step, float* u_out,
                       unsigned char* keep_out) {
  if (V <= 0) return SX_ERR_SIZE;
  if (!(temperature > 0.f)) return sx_ref_argmax_rows(logits, out, R, V);
  std::vector<float> x(V);
  std::vector<int> order(V);
  std::vector<char> keep(V);
  for (int r = 0; r < R; ++r) {
    float mx = -INFINITY;
    for (int i = 0; i < V; ++i) {
      x[i] = temperature != 1.0f ? logits[(size_t)r * V + i] / temperature : logits[(size_t)r * V + i];
      if (x[i] == x[i]) mx = std::max(mx, x[i]);
      order[i] = i;
    }
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return order_key(x[a]) > order_key(x[b]); });
    for (int i = 0; i < V; ++i) keep[i] = x[i] > -INFINITY;
    if (top_k > 0 && top_k < V) {
      const uint32_t kth = order_key(x[order[top_k - 1]]);
      for (int i = 0; i < V; ++i) keep[i] = keep[i] && order_key(x[i]) >= kth;
    }
    if (top_p < 1.0f) {
      double total = 0.0;
      for (int i = 0; i < V; ++i)
        if (keep[i]) total += std::exp(x[i] - mx);
      const double thresh = (double)top_p * total;
      double run = 0.0;
      int j = 0;
      uint32_t last_key = 0u;
      bool cut = false;
      while (j < V) {                                   // groups of equal values, largest first
        const uint32_t key = order_key(x[order[j]]);
        int e = j;
        while (e < V && order_key(x[order[e]]) == key) {
          if (keep[order[e]]) run += std::exp(x[order[e]] - mx);
          ++e;
        }
        j = e;
        if (run > thresh) { last_key = key; cut = true; break; }
      }
      if (cut)
        for (int i = 0; i < V; ++i) keep[i] = keep[i] && order_key(x[i]) >= last_key;
    }
    if (min_p > 0.f)
      for (int i = 0; i < V; ++i) keep[i] = keep[i] && std::exp(x[i] - mx) >= min_p;
    double total = 0.0;
    for (int i = 0; i < V; ++i) {
      if (keep[i]) total += std::exp(x[i] - mx);
      if (keep_out) keep_out[(size_t)r * V + i] = keep[i] ? 1 : 0;
    }
    const uint32_t word = philox_word((uint32_t)(seed & 0xffffffffull), (uint32_t)(seed >> 32), (uint32_t)(step[r] >> 2),
                                      (uint32_t)seq_index[r], step[r] & 3);
    const float u = (float)(double)word / 4294967296.0f;
    if (u_out) u_out[r] = u;
    const double target = (double)u * total;
    double run = 0.0;
    int pick = -1, last = -1;
    for (int i = 0; i < V; ++i) {
      if (!keep[i]) continue;
      last = i;
      run += std::exp(x[i] - mx);
      if (target < run) { pick = i; break; }
    }
    out[r] = pick >= 0 ? pick : (last >= 0 ? last : V - 1);
  }
  return 0;
}

// The decode loop's two bookkeeping steps.  Begin: a row whose control word is not negative runs that token instead of
// the one sampled for it in the step before (and its history, if one is kept, ends with that token).  Advance: every
// live row (advance_by != 0; all rows when advance_by is null) takes its sampled token as the next input, appends it
// to its history, and moves one position and one word of its random stream on; rows that pad the batch stay put.
int sx_ref_decode_begin(int* token_ids, const int* control, int* history, const int* hist_len, int hist_cap, int S) {
  for (int s = 0; s < S; ++s) {
    const int t = control[s];
    if (t < 0) continue;
    token_ids[s] = t;
    if (history) {
      const int n = hist_len[s];
      if (n > 0 && n <= hist_cap) history[(size_t)s * hist_cap + n - 1] = t;
    }
  }
  return 0;
}
int sx_ref_decode_advance(int* token_ids, const int* sampled, int* positions, int* seq_past, int* seq_lens, int* rng_step,
                          const int* advance_by, int* history, int* hist_len, int hist_cap, int S) {
  for (int s = 0; s < S; ++s) {
    if (advance_by && advance_by[s] == 0) continue;
    const int t = sampled[s];
    token_ids[s] = t;
    positions[s] += 1;
    seq_past[s] += 1;
    seq_lens[s] += 1;
    if (rng_step) rng_step[s] += 1;
    if (history) {
      const int n = hist_len[s];
      if (n < hist_cap) {
        history[(size_t)s * hist_cap + n] = t;
        hist_len[s] = n + 1;
      }
    }
  }
  return 0;
}

}  // extern "C"
