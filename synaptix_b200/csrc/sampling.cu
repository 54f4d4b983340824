// Sampling on the device, over rows of logits [R, V] (float32): one block a row, or, for wide vocabularies, a row
// spread over a thread-block cluster (argmax: over blocks of a first kernel, with a second to finish).
//
// What is computed follows the reference's host-side pipeline
// (crates/synaptix-models/llm/common/src/generate.rs:304-340):
//   repetition penalty -> presence/frequency penalty -> temperature -> top-k -> top-p -> min-p
//   -> argmax if temperature <= 0, else a multinomial draw
// with the processors of crates/synaptix-infer/src/sampling/{repetition,logit_processor,top_k,
// top_p,min_p,greedy,multinomial}.rs and the Philox4x32-10 generator of
// crates/synaptix-ops/src/rng.rs:1-97.  The reference sorts on the host; here the top-k and
// top-p cut-offs are found by bisection on the values' bit patterns, with reductions in a
// fixed order, so a row's result depends on nothing but the row.  Where the reference's
// result depends on its sort (a NaN among the logits; equal values at a cut-off), here a
// NaN counts as -inf and all values equal to the cut-off are kept.
#include "common.cuh"

#define SAMPLE_THREADS 1024

// order-preserving map float -> uint32 (larger float, larger key); NaN is treated as -inf
__device__ __forceinline__ uint32_t order_key(float x) {
  if (x != x) x = -INFINITY;
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ int block_sum_int(int v, int* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += red[i];
    red[32] = s;
  }
  __syncthreads();
  return red[32];
}

// ---------------------------------------------------------------------------------------
// argmax per row; among equal maxima the LAST index wins, as Rust's Iterator::max_by does
// (crates/synaptix-infer/src/sampling/greedy.rs:8-12)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void argmax_combine(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i > bi)) { bv = v; bi = i; }
}

__device__ int block_argmax(const float* __restrict__ row, int V, float inv_t_div, bool divide,
                            float* red_v, int* red_i) {
  float bv = -INFINITY;
  int bi = -1;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = row[i];
    if (divide) v = v / inv_t_div;
    if (v != v) v = -INFINITY;
    argmax_combine(bv, bi, v, i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { red_v[warp] = bv; red_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = red_v[0];
    int i = red_i[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) argmax_combine(v, i, red_v[w], red_i[w]);
    red_i[32] = i < 0 ? V - 1 : i;
    red_v[32] = v;
  }
  __syncthreads();
  return red_i[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS) argmax_rows_kernel(const float* __restrict__ logits,
                                                                     int* __restrict__ out, int V) {
  __shared__ float red_v[33];
  __shared__ int red_i[33];
  const int r = blockIdx.x;
  const int i = block_argmax(logits + (size_t)r * V, V, 1.f, false, red_v, red_i);
  if (threadIdx.x == 0) out[r] = i;
}

extern "C" int sx_argmax_rows(const float* logits, int* out, int R, int V, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return SX_ERR_SIZE;
  argmax_rows_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, out, V);
  return sx_launch_status();
}

// The same in two kernels, for wide vocabularies: one block per row scans 150 thousand logits
// in a long serial loop per thread; here each row is cut into chunks scanned by blocks of their own
// (partial maxima to scratch [R, chunks] values and indices), and a small kernel finishes.
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* __restrict__ logits, float* __restrict__ pv,
                                                             int* __restrict__ pi, int V, int chunk) {
  __shared__ float red_v[33];
  __shared__ int red_i[33];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.y, c = blockIdx.x;
  const int b = c * chunk, e = min(V, b + chunk);
  const float* row = logits + (size_t)r * V;
  float bv = -INFINITY;
  int bi = -1;
  for (int i = b + threadIdx.x; i < e; i += 256) {
    float v = row[i];
    if (v != v) v = -INFINITY;
    argmax_combine(bv, bi, v, i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { red_v[warp] = bv; red_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = red_v[0];
    int i = red_i[0];
    for (int w = 1; w < 8; ++w) argmax_combine(v, i, red_v[w], red_i[w]);
    pv[(size_t)r * gridDim.x + c] = v;
    pi[(size_t)r * gridDim.x + c] = i;
  }
}

__global__ void __launch_bounds__(32) argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi,
                                                          int* __restrict__ out, int chunks, int V) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  float bv = -INFINITY;
  int bi = -1;
  for (int c = threadIdx.x; c < chunks; c += 32) argmax_combine(bv, bi, pv[(size_t)r * chunks + c], pi[(size_t)r * chunks + c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  if (threadIdx.x == 0) out[r] = bi < 0 ? V - 1 : bi;
}

// scratch_v float [R * chunks], scratch_i int [R * chunks]; chunks <= 1024
extern "C" int sx_argmax_rows_chunked(const float* logits, int* out, float* scratch_v, int* scratch_i, int R, int V,
                                      int chunks, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || chunks <= 0 || chunks > 1024 || R > 65535) return SX_ERR_SIZE;
  const int chunk = (V + chunks - 1) / chunks;
  int rc = sx_launch(argmax_partial_kernel, dim3(chunks, R), dim3(256), 0, stream, logits, scratch_v, scratch_i, V, chunk);
  if (rc) return rc;
  return sx_launch(argmax_final_kernel, dim3(R), dim3(32), 0, stream, (const float*)scratch_v, (const int*)scratch_i, out, chunks, V);
}

// ---------------------------------------------------------------------------------------
// penalties over a window of each row's context (crates/synaptix-infer/src/sampling/
// repetition.rs:7-77).  hist is [R, hist_stride]; row r's context is hist[r, 0..hist_len[r]);
// the window is its last `last_n` tokens (0 = all).  Repetition: once per OCCURRENCE,
// logit > 0 ? logit / p : logit * p.  Presence/frequency: once per distinct token,
// logit -= presence + frequency * count.  counts is scratch [R, V] int32, ALL ZERO on entry and on exit: the
// kernel touches only the entries of tokens in the window (a pass over the whole vocabulary to clear and to
// read the counts cost 100 us a row at 151,936 logits, one block's bandwidth).  First every occurrence adds one
// to its token's count; then every occurrence swaps its token's count for zero, and the one that gets a
// positive count back applies the penalties for that token.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS) penalties_kernel(
    float* __restrict__ logits, int* __restrict__ counts, const int* __restrict__ hist,
    const int* __restrict__ hist_len, int hist_stride, int last_n, float rep, float presence,
    float frequency, int V) {
  const int r = blockIdx.x;
  float* row = logits + (size_t)r * V;
  int* cnt = counts + (size_t)r * V;
  const int n = hist_len[r];
  const int start = (last_n > 0 && last_n < n) ? n - last_n : 0;
  const int* hr = hist + (size_t)r * hist_stride;
  for (int i = start + threadIdx.x; i < n; i += blockDim.x) {
    const int t = hr[i];
    if (t >= 0 && t < V) atomicAdd(&cnt[t], 1);
  }
  __syncthreads();
  for (int i = start + threadIdx.x; i < n; i += blockDim.x) {
    const int t = hr[i];
    if (t < 0 || t >= V) continue;
    const int c = atomicExch(&cnt[t], 0);
    if (c == 0) continue;
    float x = row[t];
    if (rep != 1.0f)
      for (int k = 0; k < c; ++k) x = x > 0.f ? x / rep : x * rep;
    if (presence != 0.f || frequency != 0.f) x -= presence + frequency * (float)c;
    row[t] = x;
  }
}

extern "C" int sx_penalties(float* logits, int* counts, const int* hist, const int* hist_len,
                            int hist_stride, int last_n, float rep, float presence, float frequency,
                            int R, int V, cudaStream_t stream) {
  if (R <= 0) return 0;
  penalties_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, counts, hist, hist_len, hist_stride, last_n,
                                                      rep, presence, frequency, V);
  return sx_launch_status();
}

// ---------------------------------------------------------------------------------------
// Philox4x32-10 (crates/synaptix-ops/src/rng.rs:1-97): key = (seed lo, seed hi); the
// reference draws word number `step` of one stream per request, i.e. block step/4, word
// step%4 with counter (block, 0, 0, 0).  Here counter[1] carries the request's index in its
// call, so rows of a batch have independent streams and request 0 equals the reference's.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t philox_word(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, int word) {
  uint32_t c[4] = {c0, c1, 0u, 0u};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c[word & 3];
}

// ---------------------------------------------------------------------------------------
// temperature / top-k / top-p / min-p / multinomial, one block per row.
//
// Every cut-off is found by bisection on the values' keys, FOUR BITS a pass: a pass counts (top-k) or weighs
// (top-p) the values against 15 thresholds at once, so a cut-off costs 8 passes over the row instead of 32, and a
// pass reads the row 16 bytes a thread with several loads on the way (one 4-byte load at a time left a block at
// 20 GB/s: a draw with top-k and top-p took 2 ms for 151,936 logits, whatever the number of rows).  When top-k
// keeps few values (at most SAMPLE_LIST of them, ties included) they are gathered into shared memory in index
// order and top-p, min-p and the draw work on that list.  Counts are integers and sums are added in a fixed
// order (a thread's own elements, lanes by butterfly, warps in index order), so a row's result depends on
// nothing but the row.
// ---------------------------------------------------------------------------------------
#define SAMPLE_LIST 2048
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)

// f(i, x) for every element of the row, x = logit / temperature; 16-byte loads, four of them on the way
template <typename F>
__device__ __forceinline__ void sample_for_each(const float* __restrict__ row, int V, float temperature, bool divide, F f) {
  const int tid = threadIdx.x;
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2;
    for (int j0 = tid; j0 < n4; j0 += 4 * SAMPLE_THREADS) {
      float4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u * SAMPLE_THREADS;
        q[u] = j < n4 ? r4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u * SAMPLE_THREADS;
        if (j < n4) {
          const float e[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
          for (int c = 0; c < 4; ++c) f(4 * j + c, divide ? e[c] / temperature : e[c]);
        }
      }
    }
  } else {
    for (int i = tid; i < V; i += SAMPLE_THREADS) f(i, divide ? row[i] / temperature : row[i]);
  }
}
// the same over a list in shared memory
template <typename F>
__device__ __forceinline__ void sample_for_list(const float* xv, int n, F f) {
  for (int i = threadIdx.x; i < n; i += SAMPLE_THREADS) f(i, xv[i]);
}

// 15 block-wide sums at once, each in a fixed order; every thread gets them in out[15].  red: [SAMPLE_WARPS][16] + [16]
template <typename T>
__device__ __forceinline__ void block_sum15(const T (&v)[15], T* red, T (&out)[15]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T w[15];
#pragma unroll
  for (int j = 0; j < 15; ++j) {
    w[j] = v[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w[j] += __shfl_xor_sync(0xffffffffu, w[j], o);
  }
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < 15; ++j) red[warp * 16 + j] = w[j];
  }
  __syncthreads();
  if (threadIdx.x < 15) {
    T sum = 0;
    for (int i = 0; i < SAMPLE_WARPS; ++i) sum += red[i * 16 + threadIdx.x];
    red[SAMPLE_WARPS * 16 + threadIdx.x] = sum;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 15; ++j) out[j] = red[SAMPLE_WARPS * 16 + j];
}

// Largest key t with count(key >= t) >= k over the elements the walk visits (0 if even key 1 has fewer), and that count
template <typename W>
__device__ __forceinline__ uint32_t sample_kth_key(W walk, int k, int* red, int& kept) {
  uint32_t t = 0u;
  kept = 0;
  for (int shift = 28; shift >= 0; shift -= 4) {
    int c[15];
#pragma unroll
    for (int j = 0; j < 15; ++j) c[j] = 0;
    walk([&](int, float x) {
      const uint32_t key = order_key(x);
#pragma unroll
      for (int j = 0; j < 15; ++j) c[j] += key >= (t | ((uint32_t)(j + 1) << shift));
    });
    int tot[15];
    block_sum15(c, red, tot);
    int best = 0;
#pragma unroll
    for (int j = 0; j < 15; ++j)
      if (tot[j] >= k) { best = j + 1; kept = tot[j]; }
    t |= (uint32_t)best << shift;
  }
  return t;
}

// Largest key t with mass(key > t) > thresh, the mass being sum of exp(x - mx) over visited elements with live(x)
template <typename W, typename L>
__device__ __forceinline__ uint32_t sample_mass_key(W walk, L live, float mx, float thresh, float* red) {
  uint32_t t = 0u;
  for (int shift = 28; shift >= 0; shift -= 4) {
    float g[15];
#pragma unroll
    for (int j = 0; j < 15; ++j) g[j] = 0.f;
    walk([&](int, float x) {
      if (!live(x)) return;
      const uint32_t key = order_key(x);
      const float e = expf(x - mx);
#pragma unroll
      for (int j = 0; j < 15; ++j) g[j] += key > (t | ((uint32_t)(j + 1) << shift)) ? e : 0.f;
    });
    float tot[15];
    block_sum15(g, red, tot);
    int best = 0;
#pragma unroll
    for (int j = 0; j < 15; ++j)
      if (tot[j] > thresh) best = j + 1;
    t |= (uint32_t)best << shift;
  }
  return t;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_rows_kernel(
    const float* __restrict__ logits, int* __restrict__ out, int V, float temperature, int top_k,
    float top_p, float min_p, uint32_t seed_lo, uint32_t seed_hi, const int* __restrict__ seq_index,
    const int* __restrict__ step, float* __restrict__ u_out) {
  __shared__ float red[33];
  __shared__ float red_v[33];
  __shared__ int red_i[33];
  __shared__ float red15f[SAMPLE_WARPS * 16 + 16];
  __shared__ int red15i[SAMPLE_WARPS * 16 + 16];
  __shared__ float chunk_excl[SAMPLE_THREADS];
  __shared__ float list_x[SAMPLE_LIST];
  __shared__ int list_i[SAMPLE_LIST];
  __shared__ int found;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * V;

  if (!(temperature > 0.f)) {       // greedy
    const int i = block_argmax(row, V, 1.f, false, red_v, red_i);
    if (tid == 0) out[r] = i;
    return;
  }
  const bool divide = temperature != 1.0f;
  auto walk_row = [&](auto f) { sample_for_each(row, V, temperature, divide, f); };

  // maximum
  float mx = -INFINITY;
  walk_row([&](int, float v) { if (v == v) mx = fmaxf(mx, v); });
  mx = block_max(mx, red);

  // top-k: largest key tk with count(key >= tk) >= k
  uint32_t tk = 0u;
  int n_list = -1;                  // >= 0: the kept values are in the list
  if (top_k > 0 && top_k < V) {
    int kept = 0;
    tk = sample_kth_key(walk_row, top_k, red15i, kept);
    if (kept > 0 && kept <= SAMPLE_LIST) {
      // gather them in index order: every thread its own contiguous run of the row
      const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
      const int b0 = min(V, tid * chunk), e0 = min(V, b0 + chunk);
      int mine = 0;
      for (int i = b0; i < e0; ++i) {
        const float v = divide ? row[i] / temperature : row[i];
        mine += order_key(v) >= tk && v > -INFINITY;
      }
      // exclusive scan over the threads: lanes, then warps in order
      const int lane = tid & 31, warp = tid >> 5;
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      __syncthreads();
      if (lane == 31) red_i[warp] = incl;
      __syncthreads();
      if (tid == 0) {
        int run = 0;
        for (int w = 0; w < SAMPLE_WARPS; ++w) { const int c = red_i[w]; red_i[w] = run; run += c; }
        red_i[32] = run;
      }
      __syncthreads();
      int at = red_i[warp] + incl - mine;
      n_list = red_i[32];           // <= kept: values equal to -inf are not listed
      for (int i = b0; i < e0; ++i) {
        const float v = divide ? row[i] / temperature : row[i];
        if (order_key(v) >= tk && v > -INFINITY) { list_x[at] = v; list_i[at] = i; ++at; }
      }
      __syncthreads();
    }
  }

  bool use_tp = false;
  uint32_t tp = 0u;
  const int chunk_row = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  int pick_index = -1;              // thread 0 holds the result
  if (n_list >= 0) {
    // ------------------------------------------------------------ the kept values are few: work on the list
    auto walk_list = [&](auto f) { sample_for_list(list_x, n_list, f); };
    if (top_p < 1.0f) {
      float sm = 0.f, g0 = 0.f;
      walk_list([&](int, float v) { const float e = expf(v - mx); sm += e; if (order_key(v) > 0u) g0 += e; });
      sm = block_sum(sm, red);
      g0 = block_sum(g0, red);
      const float thresh = top_p * sm;
      if (g0 > thresh) {
        use_tp = true;
        tp = sample_mass_key(walk_list, [](float) { return true; }, mx, thresh, red15f);
      }
    }
    auto kept_l = [&](float v) { return (!use_tp || order_key(v) > tp) && (!(min_p > 0.f) || expf(v - mx) >= min_p); };
    const int chunk = (n_list + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int b = min(n_list, tid * chunk), e = min(n_list, b + chunk);
    float cs = 0.f;
    for (int i = b; i < e; ++i)
      if (kept_l(list_x[i])) cs += expf(list_x[i] - mx);
    chunk_excl[tid] = cs;
    if (tid == 0) found = -1;
    __syncthreads();
    if (tid == 0) {
      float run = 0.f;
      for (int t = 0; t < SAMPLE_THREADS; ++t) { const float c = chunk_excl[t]; chunk_excl[t] = run; run += c; }
      red[32] = run;
    }
    __syncthreads();
    const float total = red[32];
    const uint32_t word = philox_word(seed_lo, seed_hi, (uint32_t)(step[r] >> 2), (uint32_t)seq_index[r], step[r] & 3);
    const float u = (float)(double)word / 4294967296.0f;          // (multinomial.rs:30-32)
    if (tid == 0 && u_out) u_out[r] = u;
    const float target = u * total;
    const float lo = chunk_excl[tid];
    if (cs > 0.f && target >= lo && target < lo + cs) {
      float run = lo;
      int pick = -1, last = -1;
      for (int i = b; i < e; ++i) {
        if (!kept_l(list_x[i])) continue;
        last = i;
        run += expf(list_x[i] - mx);
        if (target < run) { pick = i; break; }
      }
      atomicMax(&found, pick < 0 ? last : pick);      // at most one thread gets here with target in its range
    }
    __syncthreads();
    const int first_try = found;
    __syncthreads();
    if (first_try < 0) {                // u == 1 or rounding past the end: the last kept value
      int last = -1;
      for (int i = b; i < e; ++i)
        if (kept_l(list_x[i])) last = i;
      if (last >= 0) atomicMax(&found, last);
      __syncthreads();
    }
    if (tid == 0) pick_index = found < 0 ? V - 1 : list_i[found];
    if (tid == 0) out[r] = pick_index;
    return;
  }

  // -------------------------------------------------------------- no top-k, or it keeps many: work on the row
  auto in_k = [&](float v) { return order_key(v) >= tk && v > -INFINITY; };
  if (top_p < 1.0f) {
    float sm = 0.f, g0 = 0.f;
    walk_row([&](int, float v) {
      if (!in_k(v)) return;
      const float e = expf(v - mx);
      sm += e;
      if (order_key(v) > 0u) g0 += e;       // mass(key > 0) is everything except keys equal to 0 (never a finite value)
    });
    sm = block_sum(sm, red);
    g0 = block_sum(g0, red);
    const float thresh = top_p * sm;
    if (g0 > thresh) {
      use_tp = true;
      tp = sample_mass_key(walk_row, in_k, mx, thresh, red15f);
    }
  }
  // min-p: with the maximum's probability as reference, keep exp(x - max) >= min_p
#define KEPT(v) (order_key(v) >= tk && (!use_tp || order_key(v) > tp) && (v) > -INFINITY && \
                 (!(min_p > 0.f) || expf((v) - mx) >= min_p))
#define XVAL(i) (divide ? row[i] / temperature : row[i])

  // multinomial over the kept values: contiguous chunks per thread, exclusive scan of chunk sums
  const int b = min(V, tid * chunk_row), e = min(V, b + chunk_row);
  float cs = 0.f;
  for (int i = b; i < e; ++i) {
    const float v = XVAL(i);
    if (KEPT(v)) cs += expf(v - mx);
  }
  chunk_excl[tid] = cs;
  if (tid == 0) found = -1;
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int t = 0; t < SAMPLE_THREADS; ++t) {
      const float c = chunk_excl[t];
      chunk_excl[t] = run;
      run += c;
    }
    red[32] = run;
  }
  __syncthreads();
  const float total = red[32];
  const uint32_t word = philox_word(seed_lo, seed_hi, (uint32_t)(step[r] >> 2), (uint32_t)seq_index[r], step[r] & 3);
  // u = (word as f64 as f32) / (u32::MAX as f32)   (multinomial.rs:30-32)
  const float u = (float)(double)word / 4294967296.0f;
  if (tid == 0 && u_out) u_out[r] = u;
  const float target = u * total;
  const float lo = chunk_excl[tid];
  if (cs > 0.f && target >= lo && target < lo + cs) {
    float run = lo;
    int pick = -1, last = -1;
    for (int i = b; i < e; ++i) {
      const float v = XVAL(i);
      if (!KEPT(v)) continue;
      last = i;
      run += expf(v - mx);
      if (target < run) { pick = i; break; }
    }
    if (pick < 0) pick = last;        // rounding at the chunk's end
    atomicMax(&found, pick);          // at most one thread gets here with target in its range
  }
  __syncthreads();
  const int first_try = found;
  __syncthreads();
  if (first_try < 0) {                // u == 1 or rounding past the end: last kept index
    int last = -1;
    for (int i = b; i < e; ++i) {
      const float v = XVAL(i);
      if (KEPT(v)) last = i;
    }
    if (last >= 0) atomicMax(&found, last);
    __syncthreads();
  }
  if (tid == 0) out[r] = found < 0 ? V - 1 : found;
#undef XVAL
#undef KEPT
}

// ---------------------------------------------------------------------------------------
// The same draw with a row spread over a CLUSTER of blocks, for wide vocabularies.
//
// One block per row leaves all but a few SMs idle and walks 150 thousand logits with one SM's issue rate: after
// the loads were widened the passes were bound by instructions (a pass of 15 compare-and-adds per value took
// 60 us a row).  Here the row is cut into contiguous parts, one per block of a cluster; a block turns its part
// into keys ONCE (the division by the temperature included) and keeps them in shared memory, so every later pass
// reads shared memory.  A pass sorts each value into one of 16 bins (its next four key bits relative to the
// threshold found so far), a thread adding into bins of its own in shared memory, so a value costs a handful of
// instructions instead of 15 compare-and-adds; suffix sums of the bins give the 15 counts or masses.  Blocks
// exchange their partial results through one another's shared memory: every block writes its words, one
// cluster barrier, every block reads all of them and combines them in rank order, so all blocks hold the same
// bits and take the same branches.  Two buffers in turn make one barrier an exchange enough.
// The draw walks the kept values in index order: rank by rank, and in a block thread by thread over contiguous runs.
// ---------------------------------------------------------------------------------------
#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)
#define SC_MAX_CLUSTER 8
#define SC_KEY_NEG_INF 0x007fffffu      // order_key(-inf): no key is smaller

__device__ __forceinline__ float key_value(uint32_t key) {     // order_key's inverse
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
__device__ __forceinline__ uint32_t cluster_load_u32(const uint32_t* local, uint32_t rank) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(local), r, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];\n" : "=r"(v) : "r"(r) : "memory");
  return v;
}

struct ScShared {
  uint32_t xch[2][16];                    // this block's words of the running exchange, two buffers in turn
  uint32_t gath[SC_MAX_CLUSTER][16];      // every block's words of the last exchange
  uint32_t red[SC_WARPS * 16];
  float excl[SC_THREADS];
  int found[2];
};

// Every block has written n <= 16 words into sh.xch[parity]; afterwards sh.gath[c][j] holds block c's word j.
__device__ __forceinline__ void sc_exchange(ScShared& sh, int& parity, int n, int C) {
  cluster_sync_all();
  const int tid = threadIdx.x;
  if (tid < C * 16) {
    const int c = tid >> 4, j = tid & 15;
    if (j < n) sh.gath[c][j] = cluster_load_u32(&sh.xch[parity][j], (uint32_t)c);
  }
  __syncthreads();
  parity ^= 1;
}

// 15 sums over the block, lanes by butterfly and warps in index order, left in sh.xch[parity][0..15)
template <typename T>
__device__ __forceinline__ void sc_block_sum15(const T (&v)[15], ScShared& sh, int parity) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T* red = reinterpret_cast<T*>(sh.red);
#pragma unroll
  for (int j = 0; j < 15; ++j) {
    T w = v[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if (lane == 0) red[warp * 16 + j] = w;
  }
  __syncthreads();
  if (threadIdx.x < 15) {
    T sum = 0;
    for (int i = 0; i < SC_WARPS; ++i) sum += red[i * 16 + threadIdx.x];
    reinterpret_cast<T*>(sh.xch[parity])[threadIdx.x] = sum;
  }
}

// one float summed over the block and then over the cluster, the same bits in every block
__device__ __forceinline__ float sc_cluster_sum(float v, ScShared& sh, int& parity, int C) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* red = reinterpret_cast<float*>(sh.red);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < SC_WARPS; ++i) s += red[i];
    sh.xch[parity][0] = __float_as_uint(s);
  }
  sc_exchange(sh, parity, 1, C);
  float s = 0.f;
  for (int c = 0; c < C; ++c) s += __uint_as_float(sh.gath[c][0]);
  return s;
}

__global__ void __launch_bounds__(SC_THREADS) sample_rows_cluster_kernel(
    const float* __restrict__ logits, int* __restrict__ out, int V, int part, float temperature, int top_k,
    float top_p, float min_p, uint32_t seed_lo, uint32_t seed_hi, const int* __restrict__ seq_index,
    const int* __restrict__ step, float* __restrict__ u_out) {
  extern __shared__ __align__(16) uint32_t sc_dyn[];
  __shared__ ScShared sh;
  uint32_t* keys = sc_dyn;                                   // [part]
  uint32_t* bins = sc_dyn + part;                            // [16][SC_THREADS]; part is a multiple of 4
  float* bins_f = reinterpret_cast<float*>(bins);
  const int tid = threadIdx.x;
  const int C = (int)gridDim.x, rank = (int)cluster_rank(), r = blockIdx.y;
  const float* row = logits + (size_t)r * V;
  const int begin = min(V, rank * part), n = min(V, begin + part) - begin;
  const bool divide = temperature != 1.0f;
  int parity = 0;

  // ---- this block's part as keys, and the row's maximum
  uint32_t kmax = SC_KEY_NEG_INF;
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(row + begin);
    uint4* k4 = reinterpret_cast<uint4*>(keys);
    const int n4 = n >> 2;
#pragma unroll 4
    for (int j = tid; j < n4; j += SC_THREADS) {
      const float4 q = r4[j];
      uint4 k;
      k.x = order_key(divide ? q.x / temperature : q.x);
      k.y = order_key(divide ? q.y / temperature : q.y);
      k.z = order_key(divide ? q.z / temperature : q.z);
      k.w = order_key(divide ? q.w / temperature : q.w);
      k4[j] = k;
      kmax = max(max(kmax, k.x), max(k.y, max(k.z, k.w)));
    }
  } else {
    for (int i = tid; i < n; i += SC_THREADS) {
      const float x = row[begin + i];
      const uint32_t k = order_key(divide ? x / temperature : x);
      keys[i] = k;
      kmax = max(kmax, k);
    }
  }
  {
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    if (lane == 0) sh.red[warp] = kmax;
    __syncthreads();                                         // the keys are written, too
    if (tid == 0) {
      uint32_t m = sh.red[0];
      for (int i = 1; i < SC_WARPS; ++i) m = max(m, sh.red[i]);
      sh.xch[parity][0] = m;
    }
    sc_exchange(sh, parity, 1, C);
    kmax = sh.gath[0][0];
    for (int c = 1; c < C; ++c) kmax = max(kmax, sh.gath[c][0]);
  }
  const float mx = key_value(kmax);

  // ---- top-k: the largest key tk with count(key >= tk) >= k
  uint32_t tk = 0u;
  if (top_k > 0 && top_k < V) {
    for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
      for (int b = 1; b < 16; ++b) bins[b * SC_THREADS + tid] = 0u;
      for (int i = tid; i < n; i += SC_THREADS) {
        const uint32_t key = keys[i];
        if (key >= tk) {
          const uint32_t b = min((key - tk) >> shift, 15u);
          if (b) bins[b * SC_THREADS + tid] += 1u;
        }
      }
      int c[15];
      int run = 0;
#pragma unroll
      for (int b = 15; b >= 1; --b) { run += (int)bins[b * SC_THREADS + tid]; c[b - 1] = run; }
      sc_block_sum15(c, sh, parity);
      sc_exchange(sh, parity, 15, C);
      int best = 0;
#pragma unroll
      for (int j = 0; j < 15; ++j) {
        int tot = 0;
        for (int cc = 0; cc < C; ++cc) tot += (int)sh.gath[cc][j];
        if (tot >= top_k) best = j + 1;
      }
      tk |= (uint32_t)best << shift;
    }
  }
  const uint32_t low = max(tk, SC_KEY_NEG_INF + 1u);          // kept by top-k, and not -inf

  // ---- top-p: the largest key tp with mass(key > tp) > top_p * mass(all kept by top-k)
  bool use_tp = false;
  uint32_t tp = 0u;
  if (top_p < 1.0f) {
    float sm = 0.f;
    for (int i = tid; i < n; i += SC_THREADS) {
      const uint32_t key = keys[i];
      if (key >= low) sm += expf(key_value(key) - mx);
    }
    sm = sc_cluster_sum(sm, sh, parity, C);
    const float thresh = top_p * sm;
    if (sm > thresh) {
      use_tp = true;
      for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
        for (int b = 1; b < 16; ++b) bins_f[b * SC_THREADS + tid] = 0.f;
        for (int i = tid; i < n; i += SC_THREADS) {
          const uint32_t key = keys[i];
          if (key >= low && key - 1u >= tp) {                // key > tp + j * 2^shift  <=>  bin of (key - 1) >= j
            const uint32_t b = min((key - 1u - tp) >> shift, 15u);
            if (b) bins_f[b * SC_THREADS + tid] += expf(key_value(key) - mx);
          }
        }
        float g[15];
        float run = 0.f;
#pragma unroll
        for (int b = 15; b >= 1; --b) { run += bins_f[b * SC_THREADS + tid]; g[b - 1] = run; }
        sc_block_sum15(g, sh, parity);
        sc_exchange(sh, parity, 15, C);
        int best = 0;
#pragma unroll
        for (int j = 0; j < 15; ++j) {
          float tot = 0.f;
          for (int cc = 0; cc < C; ++cc) tot += __uint_as_float(sh.gath[cc][j]);
          if (tot > thresh) best = j + 1;
        }
        tp |= (uint32_t)best << shift;
      }
    }
  }

  // ---- the draw over the kept values, in index order
  auto kept = [&](uint32_t key) {
    return key >= low && (!use_tp || key > tp) && (!(min_p > 0.f) || expf(key_value(key) - mx) >= min_p);
  };
  const int chunk = (n + SC_THREADS - 1) / SC_THREADS;
  const int b0 = min(n, tid * chunk), e0 = min(n, b0 + chunk);
  float cs = 0.f;
  int last = -1;
  for (int i = b0; i < e0; ++i) {
    const uint32_t key = keys[i];
    if (kept(key)) { cs += expf(key_value(key) - mx); last = i; }
  }
  sh.excl[tid] = cs;
  if (tid == 0) { sh.found[0] = -1; sh.found[1] = -1; }
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int t = 0; t < SC_THREADS; ++t) { const float c = sh.excl[t]; sh.excl[t] = run; run += c; }
    sh.xch[parity][0] = __float_as_uint(run);
  }
  sc_exchange(sh, parity, 1, C);
  float base = 0.f, total = 0.f;
  for (int c = 0; c < C; ++c) {
    if (c == rank) base = total;
    total += __uint_as_float(sh.gath[c][0]);
  }
  const uint32_t word = philox_word(seed_lo, seed_hi, (uint32_t)(step[r] >> 2), (uint32_t)seq_index[r], step[r] & 3);
  const float u = (float)(double)word / 4294967296.0f;          // (multinomial.rs:30-32)
  const float target = u * total;
  const float lo = base + sh.excl[tid];
  if (cs > 0.f && target >= lo) {
    // the last kept value of every run that starts at or before the target: the answer if no run claims the
    // target (u == 1, or rounding between two runs' ends)
    atomicMax(&sh.found[1], begin + last);
    if (target < lo + cs) {
      float run = lo;
      int pick = last;
      for (int i = b0; i < e0; ++i) {
        const uint32_t key = keys[i];
        if (!kept(key)) continue;
        run += expf(key_value(key) - mx);
        if (target < run) { pick = i; break; }
      }
      atomicMax(&sh.found[0], begin + pick);
    }
  }
  __syncthreads();
  if (tid < 2) sh.xch[parity][tid] = (uint32_t)sh.found[tid];
  sc_exchange(sh, parity, 2, C);
  if (rank == 0 && tid == 0) {
    int claim = -1, before = -1;
    for (int c = 0; c < C; ++c) { claim = max(claim, (int)sh.gath[c][0]); before = max(before, (int)sh.gath[c][1]); }
    out[r] = claim >= 0 ? claim : (before >= 0 ? before : V - 1);
    if (u_out) u_out[r] = u;
  }
  // no block leaves while another may still read its words
  cluster_sync_all();
}

static size_t sc_smem_bytes(int part) { return ((size_t)part + 16 * SC_THREADS) * sizeof(uint32_t); }

// blocks a row: 0 = this row width goes to the one-block kernel
static int sc_pick_cluster(int V) {
  if (V < 8192) return 0;
  const int part = (((V + SC_MAX_CLUSTER - 1) / SC_MAX_CLUSTER) + 3) & ~3;
  return sc_smem_bytes(part) + sizeof(ScShared) + 1024 <= 227u * 1024u ? SC_MAX_CLUSTER : 0;
}

extern "C" int sx_sample_rows_cluster(const float* logits, int* out, int R, int V, float temperature, int top_k,
                                      float top_p, float min_p, unsigned long long seed, const int* seq_index,
                                      const int* step, float* u_out, int cluster, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || !(temperature > 0.f) || R > 65535) return SX_ERR_SIZE;
  if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return SX_ERR_SIZE;
  const int part = (((V + cluster - 1) / cluster) + 3) & ~3;
  const size_t smem = sc_smem_bytes(part);
  if (smem + sizeof(ScShared) + 1024 > 227u * 1024u) return SX_ERR_SIZE;
  auto kern = sample_rows_cluster_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)cluster, (unsigned)R);
  cfg.blockDim = dim3(SC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, logits, out, V, part, temperature, top_k, top_p, min_p,
                                 (uint32_t)(seed & 0xffffffffull), (uint32_t)(seed >> 32), seq_index, step, u_out);
}

extern "C" int sx_sample_rows_block(const float* logits, int* out, int R, int V, float temperature, int top_k,
                                    float top_p, float min_p, unsigned long long seed, const int* seq_index,
                                    const int* step, float* u_out, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return SX_ERR_SIZE;
  sample_rows_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(
      logits, out, V, temperature, top_k, top_p, min_p, (uint32_t)(seed & 0xffffffffull),
      (uint32_t)(seed >> 32), seq_index, step, u_out);
  return sx_launch_status();
}

extern "C" int sx_sample_rows(const float* logits, int* out, int R, int V, float temperature, int top_k,
                              float top_p, float min_p, unsigned long long seed, const int* seq_index,
                              const int* step, float* u_out, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return SX_ERR_SIZE;
  if (temperature > 0.f && R <= 65535) {
    const int cluster = sc_pick_cluster(V);
    if (cluster) return sx_sample_rows_cluster(logits, out, R, V, temperature, top_k, top_p, min_p, seed, seq_index, step, u_out, cluster, stream);
  }
  return sx_sample_rows_block(logits, out, R, V, temperature, top_k, top_p, min_p, seed, seq_index, step, u_out, stream);
}
