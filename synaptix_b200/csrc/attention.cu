// Attention over the paged cache for bfloat16, on tensor cores: scores and P*V as
// mma.sync.m16n8k16 with 32-bit accumulation, softmax in 32-bit in the exp2 domain,
// keys and values brought page by page (64 keys) into shared memory by cp.async.
//
//   prefill  one block per (64 query rows of one sequence, query head); each of 4 warps owns
//            16 query rows and walks over the sequence's pages up to its diagonal.
//   decode   one block per (split of a sequence's pages, kv head, sequence): the G = nh/nkv
//            query heads that share the kv head are the rows of ONE fragment, so every key and
//            value byte is read once for all of them; the 4 warps split the 64 keys of a page,
//            keep their own running maximum and sum, and are merged at the end.  With more than
//            one split, un-normalised partial results go to scratch memory and a second kernel
//            merges them.
//
// The reference's prefill kernel has the same FA-2 scheme for contiguous caches
// (crates/synaptix-kernels-cuda/src/cu/fused/attention/flash_splitq.cu:49-52,187-600); its decode
// kernel is scalar and re-reads K/V for every query head
// (crates/synaptix-kernels-cuda/src/cu/fused/attention/flash_decode.cu:92-205,340-387).
//
// Masking: key j is visible to the query at position p iff j <= p and (window == 0 or
// j > p - window).  Rows of a page at or beyond the sequence's length are zero-filled in shared
// memory (never read from the cache), so stale or non-finite cache contents cannot leak.
#include "common.cuh"

#include "attn_tile.cuh"

// =======================================================================================
// decode: grid (n_splits, nkv, S), one query token per sequence (token index = sequence index)
// =======================================================================================
// PREP: q is the raw fused projection [S, (nh + 2 nkv) HD] of the step's tokens, and the kernel does what
// qkv_prepare_kernel does on the way: per-head RMSNorm of the group's query heads and of the new key, rotation by
// the token's position, the new key and value into the cache (by the block whose pages hold the token's place,
// which also puts them into its staged page), so that a decode step needs no kernel for it.
struct AtPrep {
  const float* wq;          // [HD] gains of the q and k norms, or null
  const float* wk;
  const float* inv_freq;    // [HD / 2] or null (no rotation)
  float eps;
  int write;                // 0: this layer reads a cache another layer wrote (the token's key and value are there)
  int n_pages;
};

template <int HD, bool PREP>
__global__ void __launch_bounds__(AT_THREADS) attn_decode_kernel(
    const bf16* __restrict__ q, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    const int* __restrict__ seq_lens, const int* __restrict__ block_table, int maxp, int nh, int nkv,
    float scale_log2, int window, int n_splits, int* __restrict__ counters, const AtPrep prep) {
  using L = AtLayout<HD>;
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ __align__(16) bf16 q_s[PREP ? 16 * HD : 8];       // the group's prepared query heads
  __shared__ __align__(16) bf16 kv_new[PREP ? 2 * HD : 8];     // the token's prepared key and value
  if (!PREP) { pdl_wait(); pdl_trigger(); }
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int G = nh / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int len = seq_lens[seq];
  const int pos = len - 1;                                   // the query's position
  const int lo = window > 0 ? max(0, len - window) : 0;      // first visible key
  const int p_first = lo >> 6, p_end = (len + 63) >> 6;
  const int total = p_end - p_first;
  const int per = (total + n_splits - 1) / n_splits;
  const int p0 = p_first + split * per, p1 = min(p_end, p0 + per);
  const int* bt = block_table + (size_t)seq * maxp;

  // does this block hold the page of the token's own place?  (PREP with a cache to write: it prepares the new
  // key and value, writes them to the cache and patches them into its staged page)
  const int p_last = pos >> 6;
  const bool has_last = PREP && prep.write && p0 <= p_last && p_last < p1;
  const int npages = max(0, p1 - p0);
  // rows of a page that come from the cache: with has_last the token's own row does not (it is not there yet)
  auto rows_of = [&](int pg) { return min(64, (has_last ? len - 1 : len) - pg * 64); };
  auto first_pages = [&]() {
#pragma unroll
    for (int st = 0; st < AT_STAGES_DECODE - 1; ++st) {
      if (st < npages) load_page<HD>(smem + st * L::STAGE, k_pages, v_pages, bt[p0 + st], kvh, nkv, rows_of(p0 + st));
      cp_async_commit();
    }
  };
  if (PREP) {
    // The first pages are asked for while the product before this kernel still runs: what they hold (every row
    // but the token's own, which this kernel makes) and the lengths and block tables were written at least two
    // launches ago, and a kernel behind a programmatic launch starts only when the one before its predecessor
    // has ended.
    first_pages();
    constexpr int half = HD / 2;
    const int heads = nh + 2 * nkv;
    const bf16* tok = q + (size_t)seq * heads * HD;
    float cs[2] = {1.f, 1.f}, sn[2] = {0.f, 0.f};
    const int p = 2 * lane;                                   // this lane's pairs (p, p + half), (p + 1, p + 1 + half)
    if (prep.inv_freq && p < half) {
      sincosf((float)pos * prep.inv_freq[p], &sn[0], &cs[0]);
      sincosf((float)pos * prep.inv_freq[p + 1], &sn[1], &cs[1]);
    }
    // the gains of the two norms at this lane's four places: weights, like the angles fetched before the wait
    float gq[4] = {1.f, 1.f, 1.f, 1.f}, gk[4] = {1.f, 1.f, 1.f, 1.f};
    if (p < half) {
      if (prep.wq) { gq[0] = prep.wq[p]; gq[1] = prep.wq[p + 1]; gq[2] = prep.wq[p + half]; gq[3] = prep.wq[p + 1 + half]; }
      if (prep.wk) { gk[0] = prep.wk[p]; gk[1] = prep.wk[p + 1]; gk[2] = prep.wk[p + half]; gk[3] = prep.wk[p + 1 + half]; }
    }
    bf16* k_row = nullptr;
    bf16* v_row = nullptr;
    if (has_last) {
      const int page = bt[p_last];
      if (page >= 0 && page < prep.n_pages) {                 // the host guarantees a page; never write outside
        const size_t at = (((size_t)page * nkv + kvh) * SX_PAGE + (pos & 63)) * HD;
        k_row = k_pages + at;
        v_row = v_pages + at;
      }
    }
    pdl_wait();                                               // the projection comes from the kernel before
    pdl_trigger();
    // jobs: the G query heads of the group, then (has_last) the key head and the value head
    const int jobs = G + (has_last ? 2 : 0);
    for (int j = warp; j < jobs; j += AT_THREADS / 32) {
      const bool is_q = j < G, is_k = j == G;
      const bf16* src = tok + (size_t)(is_q ? kvh * G + j : (is_k ? nh + kvh : nh + nkv + kvh)) * HD;
      if (!is_q && !is_k) {                                   // value: copy
        for (int i = lane * 8; i < HD; i += 256) {
          const uint4 v = *reinterpret_cast<const uint4*>(src + i);
          *reinterpret_cast<uint4*>(kv_new + HD + i) = v;
          if (v_row) *reinterpret_cast<uint4*>(v_row + i) = v;
        }
        continue;
      }
      const float* w = is_q ? prep.wq : prep.wk;
      float2 x1 = make_float2(0.f, 0.f), x2 = x1;
      if (p < half) {
        x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + p));
        x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + p + half));
      }
      float inv = 1.f;
      if (w) inv = rsqrtf(warp_sum(x1.x * x1.x + x1.y * x1.y + x2.x * x2.x + x2.y * x2.y) / (float)HD + prep.eps);
      if (p < half) {
        const float a0 = x1.x * inv * (is_q ? gq[0] : gk[0]), a1 = x1.y * inv * (is_q ? gq[1] : gk[1]);
        const float b0 = x2.x * inv * (is_q ? gq[2] : gk[2]), b1 = x2.y * inv * (is_q ? gq[3] : gk[3]);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a0 * cs[0] - b0 * sn[0], a1 * cs[1] - b1 * sn[1]);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(a0 * sn[0] + b0 * cs[0], a1 * sn[1] + b1 * cs[1]);
        bf16* dst = is_q ? q_s + j * HD : kv_new;
        *reinterpret_cast<__nv_bfloat162*>(dst + p) = lo;
        *reinterpret_cast<__nv_bfloat162*>(dst + p + half) = hi;
        if (is_k && k_row) {
          *reinterpret_cast<__nv_bfloat162*>(k_row + p) = lo;
          *reinterpret_cast<__nv_bfloat162*>(k_row + p + half) = hi;
        }
      }
    }
    __syncthreads();
  }

  // query fragments: row r of the fragment is query head kvh*G + r (rows >= G are zero)
  uint32_t qf[HD / 16][4];
  {
    const bf16* qb = PREP ? q_s : q + ((size_t)seq * nh + (size_t)kvh * G) * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const int c = ks * 16 + 2 * t;
      qf[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qb + (size_t)g * HD + c) : 0u;
      qf[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (size_t)(g + 8) * HD + c) : 0u;
      qf[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qb + (size_t)g * HD + c + 8) : 0u;
      qf[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (size_t)(g + 8) * HD + c + 8) : 0u;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  if (!PREP) first_pages();
  for (int i = 0; i < npages; ++i) {
    cp_async_wait<AT_STAGES_DECODE - 2>();
    __syncthreads();
    const int nx = i + AT_STAGES_DECODE - 1;
    if (nx < npages)
      load_page<HD>(smem + (nx % AT_STAGES_DECODE) * L::STAGE, k_pages, v_pages, bt[p0 + nx], kvh, nkv, rows_of(p0 + nx));
    cp_async_commit();
    if (PREP && has_last && p0 + i == p_last) {               // the token's key and value into their row of the staged page
      unsigned char* stw = smem + (i % AT_STAGES_DECODE) * L::STAGE + (pos & 63) * L::ROW;
      if (threadIdx.x < HD / 8) *reinterpret_cast<uint4*>(stw + threadIdx.x * 16) = reinterpret_cast<const uint4*>(kv_new)[threadIdx.x];
      else if (threadIdx.x < HD / 4)
        *reinterpret_cast<uint4*>(stw + L::TILE + (threadIdx.x - HD / 8) * 16) = reinterpret_cast<const uint4*>(kv_new + HD)[threadIdx.x - HD / 8];
      __syncthreads();
    }
    const unsigned char* st = smem + (i % AT_STAGES_DECODE) * L::STAGE;
    // this warp's 16 keys of the page; all fragment rows sit at the same position
    const int jb = (p0 + i) * 64;
    if (jb + 63 > pos || (window > 0 && jb <= pos - window))
      attend_tile<HD, 2, true>(qf, st, st + L::TILE, warp * 16, jb, pos, pos, window, scale_log2, m, l, o);
    else      // the whole page is visible: no comparisons
      attend_tile<HD, 2, false>(qf, st, st + L::TILE, warp * 16, jb, pos, pos, window, scale_log2, m, l, o);
  }
  cp_async_wait<0>();
  __syncthreads();

  // the running maxima are of raw scores; the merges below work in the scaled (log2) domain
  m[0] *= scale_log2;
  m[1] *= scale_log2;
  // rows' sums over the 4 lanes that share a row
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  // merge the 4 warps through shared memory (the stage buffers are free now)
  float* wo = reinterpret_cast<float*>(smem);                 // [4][16][HD]
  float* wml = wo + 4 * 16 * HD;                              // [4][16][2]
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    const int c = n * 8 + 2 * t;
    wo[(warp * 16 + g) * HD + c] = o[n][0];
    wo[(warp * 16 + g) * HD + c + 1] = o[n][1];
    wo[(warp * 16 + g + 8) * HD + c] = o[n][2];
    wo[(warp * 16 + g + 8) * HD + c + 1] = o[n][3];
  }
  if (t == 0) {
    wml[(warp * 16 + g) * 2] = m[0];
    wml[(warp * 16 + g) * 2 + 1] = l[0];
    wml[(warp * 16 + g + 8) * 2] = m[1];
    wml[(warp * 16 + g + 8) * 2 + 1] = l[1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += AT_THREADS) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, wml[(w * 16 + r) * 2]);
    float Lsum = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = wml[(w * 16 + r) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      Lsum += wml[(w * 16 + r) * 2 + 1] * f;
      O += wo[(w * 16 + r) * HD + d] * f;
    }
    const int head = kvh * G + r;
    if (n_splits == 1) {
      out[((size_t)seq * nh + head) * HD + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
    } else {
      const size_t pi = ((size_t)seq * nh + head) * n_splits + split;
      part_o[pi * HD + d] = O;
      if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = Lsum; }
    }
  }
  if (n_splits == 1 || counters == nullptr) return;      // without counters a second kernel merges

  // The block that finishes last for this (sequence, kv head) merges all splits, in split order.
  // counters[seq * nkv + kvh] counts finished blocks and is set back to zero by the last one, so
  // the array only has to be zero before the very first launch.
  __shared__ int s_last;
  __threadfence();                                       // this block's partials are visible before it counts
  __syncthreads();
  if (threadIdx.x == 0) {
    int* c = counters + (size_t)seq * nkv + kvh;
    const int done = atomicAdd(c, 1);
    s_last = (done == n_splits - 1);
    if (s_last) *c = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();                                       // and the others' partials before they are read
  float* fac = reinterpret_cast<float*>(smem);           // [G][n_splits] maxima, then weights
  float* ls = fac + G * n_splits;                        // [G][n_splits] sums
  float* gl = ls + G * n_splits;                         // [G] merged sums
  for (int idx = threadIdx.x; idx < G * n_splits; idx += AT_THREADS) {
    const int r = idx / n_splits, i = idx % n_splits;
    const float2 ml = reinterpret_cast<const float2*>(part_ml)[((size_t)seq * nh + kvh * G + r) * n_splits + i];
    fac[idx] = ml.x;
    ls[idx] = ml.y;
  }
  __syncthreads();
  for (int r = warp; r < G; r += 4) {                    // one warp per head: maximum, weights, sum
    float M = -INFINITY;
    for (int i = lane; i < n_splits; i += 32) M = fmaxf(M, fac[r * n_splits + i]);
    M = warp_max(M);
    float L = 0.f;
    for (int i = lane; i < n_splits; i += 32) {
      const float mi = fac[r * n_splits + i];
      const float f = (mi == -INFINITY) ? 0.f : exp2f(mi - M);
      fac[r * n_splits + i] = f;
      L += ls[r * n_splits + i] * f;
    }
    L = warp_sum(L);
    if (lane == 0) gl[r] = L;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += AT_THREADS) {
    const int r = idx / HD, d = idx % HD;
    const size_t row = (size_t)seq * nh + kvh * G + r;
    const float* po = part_o + row * n_splits * HD + d;
    const float* f = fac + r * n_splits;
    float O = 0.f;
#pragma unroll 8
    for (int i = 0; i < n_splits; ++i) O += po[(size_t)i * HD] * f[i];
    const float L = gl[r];
    out[row * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
  }
}

#include "attn_merge.cuh"

// =======================================================================================
// prefill: grid (n_tiles, nh); tile i covers query rows tile_q0[i] .. +63 of sequence tile_seq[i]
// =======================================================================================
template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 3) attn_prefill_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
    bf16* __restrict__ out, const int* __restrict__ tile_seq, const int* __restrict__ tile_q0,
    const int* __restrict__ cu_seqlens, const int* __restrict__ seq_past, const int* __restrict__ seq_lens,
    const int* __restrict__ block_table, int maxp, int nh, int nkv, float scale_log2, int window) {
  using L = AtLayout<HD, AT_STAGES_PREFILL>;
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_trigger();
  // tiles late in a sequence see more keys: they are started first, so that the short ones fill the tail
  const int tile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int kvh = h / (nh / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int t_begin = cu_seqlens[seq], n_new = cu_seqlens[seq + 1] - t_begin;
  const int past = seq_past[seq], len = seq_lens[seq];
  const int rows = min(64, n_new - q0);                       // query rows of this tile
  const int* bt = block_table + (size_t)seq * maxp;

  // this warp's rows, their packed token indices and positions
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
  const bool ok_lo = r_lo < rows, ok_hi = r_hi < rows;
  const int pos_lo = ok_lo ? past + q0 + r_lo : -1, pos_hi = ok_hi ? past + q0 + r_hi : -1;
  uint32_t qf[HD / 16][4];
  {
    const bf16* qlo = q + ((size_t)(t_begin + q0 + (ok_lo ? r_lo : 0)) * nh + h) * HD;
    const bf16* qhi = q + ((size_t)(t_begin + q0 + (ok_hi ? r_hi : 0)) * nh + h) * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const int c = ks * 16 + 2 * t;
      qf[ks][0] = ok_lo ? *reinterpret_cast<const uint32_t*>(qlo + c) : 0u;
      qf[ks][1] = ok_hi ? *reinterpret_cast<const uint32_t*>(qhi + c) : 0u;
      qf[ks][2] = ok_lo ? *reinterpret_cast<const uint32_t*>(qlo + c + 8) : 0u;
      qf[ks][3] = ok_hi ? *reinterpret_cast<const uint32_t*>(qhi + c + 8) : 0u;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  // pages the tile can see: from the first key visible to its first row to the last row's position
  const int first_pos = past + q0, last_pos = past + q0 + rows - 1;
  const int lo_key = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int p0 = lo_key >> 6, p1 = (last_pos >> 6) + 1;
  const int npages = p1 - p0;
  // this warp needs pages up to its own last row only
  const int warp_last = past + q0 + min(rows - 1, warp * 16 + 15);
  const bool warp_on = warp * 16 < rows;
  const int warp_first = past + q0 + warp * 16;

#pragma unroll
  for (int st = 0; st < AT_STAGES_PREFILL - 1; ++st) {
    if (st < npages) load_page<HD>(smem + st * L::STAGE, k_pages, v_pages, bt[p0 + st], kvh, nkv, min(64, len - (p0 + st) * 64));
    cp_async_commit();
  }
  for (int i = 0; i < npages; ++i) {
    cp_async_wait<AT_STAGES_PREFILL - 2>();
    __syncthreads();
    const int nx = i + AT_STAGES_PREFILL - 1;
    if (nx < npages)
      load_page<HD>(smem + (nx % AT_STAGES_PREFILL) * L::STAGE, k_pages, v_pages, bt[p0 + nx], kvh, nkv, min(64, len - (p0 + nx) * 64));
    cp_async_commit();
    const unsigned char* st = smem + (i % AT_STAGES_PREFILL) * L::STAGE;
    const int jbase = (p0 + i) * 64;
    if (warp_on && jbase <= warp_last) {
      // visible to every row of this warp without a comparison: ends before the warp's first row's
      // position and starts after the window's lower edge of its last row
      if (jbase + 63 > warp_first || (window > 0 && jbase <= warp_last - window))
        attend_tile<HD, 8, true>(qf, st, st + L::TILE, 0, jbase, pos_lo, pos_hi, window, scale_log2, m, l, o);
      else
        attend_tile<HD, 8, false>(qf, st, st + L::TILE, 0, jbase, pos_lo, pos_hi, window, scale_log2, m, l, o);
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  const float inv_lo = l[0] > 0.f ? 1.f / l[0] : 0.f, inv_hi = l[1] > 0.f ? 1.f / l[1] : 0.f;
  bf16* olo = out + ((size_t)(t_begin + q0 + r_lo) * nh + h) * HD;
  bf16* ohi = out + ((size_t)(t_begin + q0 + r_hi) * nh + h) * HD;
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    const int c = n * 8 + 2 * t;
    if (ok_lo) *reinterpret_cast<uint32_t*>(olo + c) = pack_bf16(o[n][0] * inv_lo, o[n][1] * inv_lo);
    if (ok_hi) *reinterpret_cast<uint32_t*>(ohi + c) = pack_bf16(o[n][2] * inv_hi, o[n][3] * inv_hi);
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
template <int HD, bool PREP>
static int decode_launch(const bf16* q, bf16* k, bf16* v, bf16* out, float* part_o, float* part_ml,
                         const int* seq_lens, const int* bt, int maxp, int S, int nh, int nkv, float scale_log2,
                         int window, int n_splits, int* counters, const AtPrep& prep, cudaStream_t stream) {
  using L = AtLayout<HD>;
  const size_t merge_bytes = (size_t)(4 * 16 * HD + 4 * 16 * 2) * sizeof(float);
  const size_t last_bytes = (size_t)(2 * 16 * n_splits + 16) * sizeof(float);
  size_t smem = L::SMEM > merge_bytes ? L::SMEM : merge_bytes;
  if (last_bytes > smem) counters = nullptr;             // too many splits for the in-kernel merge
  auto kern = attn_decode_kernel<HD, PREP>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(n_splits, nkv, S);
  int rc = sx_launch(kern, grid, dim3(AT_THREADS), smem, stream, q, k, v, out, part_o, part_ml, seq_lens, bt, maxp, nh, nkv,
                     scale_log2, window, n_splits, counters, prep);
  if (rc || n_splits == 1 || counters) return rc;
  return sx_launch(attn_merge_kernel<HD>, dim3(S * nh), dim3(HD), 2 * n_splits * sizeof(float), stream,
                   (const float*)part_o, (const float*)part_ml, out, n_splits);
}

// q [S, nh, hd] (one token per sequence), out [S, nh*hd]; part_o f32 [S*nh*n_splits*hd] and
// part_ml f32 [S*nh*n_splits*2] are scratch (unused when n_splits == 1).
static int attn_decode_any(const void* q, const void* k_pages, const void* v_pages, void* out, float* part_o,
                           float* part_ml, const int* seq_lens, const int* block_table, int maxp, int S, int nh,
                           int nkv, int hd, float scale, int window, int n_splits, int* counters, const AtPrep* prep,
                           cudaStream_t stream) {
  if (S <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 16 || n_splits < 1 || nkv > 65535 || S > 65535) return SX_ERR_SIZE;
  // the merge keeps two floats a split in shared memory: refused before anything is launched
  if (n_splits > AT_MAX_SPLITS) return SX_ERR_SIZE;
  if (n_splits > 1 && (!part_o || !part_ml)) return SX_ERR_SIZE;
  const float sl = scale * 1.4426950408889634f;
  const bf16* qb = (const bf16*)q;
  bf16 *kb = (bf16*)const_cast<void*>(k_pages), *vb = (bf16*)const_cast<void*>(v_pages), *ob = (bf16*)out;
  const AtPrep none = {nullptr, nullptr, nullptr, 0.f, 0, 0};
#define AT_GO(HD)                                                                                                            \
  return prep ? decode_launch<HD, true>(qb, kb, vb, ob, part_o, part_ml, seq_lens, block_table, maxp, S, nh, nkv, sl, window, \
                                        n_splits, counters, *prep, stream)                                                     \
              : decode_launch<HD, false>(qb, kb, vb, ob, part_o, part_ml, seq_lens, block_table, maxp, S, nh, nkv, sl, window, \
                                         n_splits, counters, none, stream)
  if (hd == 128) AT_GO(128);
  if (hd == 64) AT_GO(64);
  if (hd == 32) AT_GO(32);
#undef AT_GO
  return SX_ERR_SIZE;
}

// the splits are merged by a second kernel
extern "C" int sx_attn_decode(const void* q, const void* k_pages, const void* v_pages, void* out, float* part_o,
                              float* part_ml, const int* seq_lens, const int* block_table, int maxp, int S, int nh,
                              int nkv, int hd, float scale, int window, int n_splits, cudaStream_t stream) {
  return attn_decode_any(q, k_pages, v_pages, out, part_o, part_ml, seq_lens, block_table, maxp, S, nh, nkv, hd, scale,
                         window, n_splits, nullptr, nullptr, stream);
}

// The same for a step's raw fused projection qkv [S, (nh + 2 nkv) hd]: per-head RMSNorm of q and k (gains wq, wk in
// float32, or null), rotate-half rotation of the whole head by seq_lens[s] - 1 (inv_freq [hd / 2], or null), the new
// key and value written into the cache (write != 0; pages [n_pages, nkv, 64, hd]) happen inside the attention kernel.
extern "C" int sx_attn_decode_prep(const void* qkv, void* k_pages, void* v_pages, void* out, float* part_o, float* part_ml,
                                   const float* wq, const float* wk, const float* inv_freq, float eps, int write,
                                   long long n_pages, const int* seq_lens, const int* block_table, int maxp, int S, int nh,
                                   int nkv, int hd, float scale, int window, int n_splits, cudaStream_t stream) {
  if (((uintptr_t)qkv & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return SX_ERR_ALIGN;
  if (n_pages <= 0 || n_pages > 0x7fffffffLL) return SX_ERR_SIZE;
  const AtPrep prep = {wq, wk, inv_freq, eps, write, (int)n_pages};
  return attn_decode_any(qkv, k_pages, v_pages, out, part_o, part_ml, seq_lens, block_table, maxp, S, nh, nkv, hd, scale,
                         window, n_splits, nullptr, &prep, stream);
}

// the splits are merged inside the kernel by whichever block of a (sequence, kv head) finishes last;
// counters int32 [S * nkv] must be zero before the first launch and is left zero by every launch
extern "C" int sx_attn_decode_fused(const void* q, const void* k_pages, const void* v_pages, void* out, float* part_o,
                                    float* part_ml, int* counters, const int* seq_lens, const int* block_table,
                                    int maxp, int S, int nh, int nkv, int hd, float scale, int window, int n_splits,
                                    cudaStream_t stream) {
  return attn_decode_any(q, k_pages, v_pages, out, part_o, part_ml, seq_lens, block_table, maxp, S, nh, nkv, hd, scale,
                         window, n_splits, counters, nullptr, stream);
}

// ---------------------------------------------------------------------------------------
// The same decode attention with its scratch inside the library (see no_alloc.h for whom
// this is meant and what it promises).  Only this function and the array below are new; the
// kernels and the launch path are the ones sx_attn_decode uses.
// ---------------------------------------------------------------------------------------
#include "no_alloc.h"
#include <atomic>

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer a kernel can use.
static __device__ __align__(256) unsigned char sx_noalloc_scratch[SX_NOALLOC_SCRATCH_BYTES];

#define SX_NOALLOC_MAX_DEVICES 64

// the array's device address on the current device, looked up once per device; host threads that make
// their first call at the same time both look it up and store the same value
static int noalloc_scratch_address(float** out_ptr) {
  static std::atomic<float*> addr[SX_NOALLOC_MAX_DEVICES];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= SX_NOALLOC_MAX_DEVICES) return SX_ERR_SIZE;
  float* a = addr[dev].load(std::memory_order_acquire);
  if (!a) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, sx_noalloc_scratch);      // the copy of the array that lives on `dev`
    if (e != cudaSuccess) return (int)e;
    a = reinterpret_cast<float*>(p);
    addr[dev].store(a, std::memory_order_release);
  }
  *out_ptr = a;
  return 0;
}

extern "C" unsigned long long sx_attn_decode_noalloc_capacity(void) { return SX_NOALLOC_SCRATCH_BYTES; }

extern "C" int sx_attn_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                      const int* seq_lens, const int* block_table, int maxp, int S, int nh, int nkv,
                                      int hd, float scale, int window, int n_splits, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || nh / nkv > 16 || n_splits < 1 || nkv > 65535 || S > 65535) return SX_ERR_SIZE;
  if (hd != 128 && hd != 64 && hd != 32) return SX_ERR_SIZE;
  if (n_splits > AT_MAX_SPLITS) return SX_ERR_SIZE;
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (n_splits > 1) {
    const unsigned long long slots = (unsigned long long)S * nh * n_splits;
    const unsigned long long need = slots * (unsigned long long)(hd + 2) * sizeof(float);
    if (need > SX_NOALLOC_SCRATCH_BYTES) return SX_ERR_NOALLOC_TOO_LARGE;
    float* base = nullptr;
    const int rc = noalloc_scratch_address(&base);
    if (rc) return rc;
    part_o = base;                          // [slots][hd]
    part_ml = base + slots * hd;            // [slots][2]; slots * hd * 4 bytes keeps it 8-byte aligned
  }
  return sx_attn_decode(q, k_pages, v_pages, out, part_o, part_ml, seq_lens, block_table, maxp, S, nh, nkv, hd, scale,
                        window, n_splits, stream);
}

template <int HD>
static int prefill_launch(const bf16* q, const bf16* k, const bf16* v, bf16* out, const int* tile_seq, const int* tile_q0,
                          int n_tiles, const int* cu, const int* past, const int* lens, const int* bt, int maxp, int nh,
                          int nkv, float scale_log2, int window, cudaStream_t stream) {
  using L = AtLayout<HD, AT_STAGES_PREFILL>;
  auto kern = attn_prefill_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(n_tiles, nh);
  return sx_launch(kern, grid, dim3(AT_THREADS), L::SMEM, stream, q, k, v, out, tile_seq, tile_q0, cu, past, lens, bt, maxp, nh,
                   nkv, scale_log2, window);
}

// q [T, nh, hd] packed tokens, out [T, nh*hd]; tile_seq/tile_q0 [n_tiles] list 64-row query tiles.
extern "C" int sx_attn_prefill(const void* q, const void* k_pages, const void* v_pages, void* out,
                               const int* tile_seq, const int* tile_q0, int n_tiles, const int* cu_seqlens,
                               const int* seq_past, const int* seq_lens, const int* block_table, int maxp, int nh,
                               int nkv, int hd, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh > 65535) return SX_ERR_SIZE;
  const float sl = scale * 1.4426950408889634f;
  const bf16 *qb = (const bf16*)q, *kb = (const bf16*)k_pages, *vb = (const bf16*)v_pages;
  if (hd == 128) return prefill_launch<128>(qb, kb, vb, (bf16*)out, tile_seq, tile_q0, n_tiles, cu_seqlens, seq_past, seq_lens, block_table, maxp, nh, nkv, sl, window, stream);
  if (hd == 64) return prefill_launch<64>(qb, kb, vb, (bf16*)out, tile_seq, tile_q0, n_tiles, cu_seqlens, seq_past, seq_lens, block_table, maxp, nh, nkv, sl, window, stream);
  if (hd == 32) return prefill_launch<32>(qb, kb, vb, (bf16*)out, tile_seq, tile_q0, n_tiles, cu_seqlens, seq_past, seq_lens, block_table, maxp, nh, nkv, sl, window, stream);
  return SX_ERR_SIZE;
}
