// Attention of single-token steps over the paged cache (bfloat16, head size 64 or 128): pages by TMA,
// a warp per page.
//
// A decode step reads every cached key and value once, so this kernel has to keep HBM busy and nothing
// else.  The cp.async kernel of attention.cu spends most of its instructions on moving a page (2,048
// 16-byte copies with their addresses per page) and on bookkeeping that it repeats for every 16 keys
// (four warps split a page), and with two blocks of four warps an SM that is what bounds it: measured
// 486 instructions a warp a page, 1.6 us a page a block, whatever HBM could deliver.  Here
//   * one elected lane of a producer warp (the whole warp walks the pages) brings a page with 2 (head size 64) or 4 (128) TMA copies
//     (cp.async.bulk.tensor.4d over the cache [pages, kv heads, 64, head size], 128-byte swizzle)
//     into 3 stages; full/empty mbarriers per stage, no block-wide barrier in the loop;
//   * each of the 3 compute warps takes WHOLE pages (page i of the block's range goes to warp i % 3, through
//     stage i % 3: a stage has one consumer, so the parities of its barriers are counted by one warp and the
//     producer alone, and a wait can never be for a phase further than one ahead):
//     scores of 64 keys as 8 key tiles x (head size / 16) mma.sync.m16n8k16, one softmax update and one
//     rescale of the output per page instead of four, P V as 4 x (head size / 8) MMAs; fragments come
//     from the swizzled stage by ldmatrix with the XOR applied to the address;
//   * the output is rescaled only when a row's maximum moved.
// The G = nh / nkv query heads that share the kv head are the rows of one fragment, so every cache byte
// is read once for all of them.  grid (splits, kv heads, sequences): a block takes a contiguous share of
// the sequence's visible pages.  With one split the block writes the result itself.  With 2, 4, 8 or 16 splits
// the blocks of a (sequence, kv head) form a thread-block cluster (CLUSTER): each leaves its un-normalised sums
// with maximum and denominator in its own shared memory, and after a barrier over the cluster every block
// merges a share of the outputs, reading the others' shared memory (distributed shared memory): no scratch in
// global memory, no second kernel, one kernel boundary less in a decode step.  Any other number of splits goes
// through scratch and a second kernel (attn_merge.cuh) that adds the splits up.
//
// With PREP the kernel takes the step's fused q/k/v projection as it left the product and does what head
// preparation does on the way: per-head RMSNorm of q and k, rotate-half rotation by the token's position,
// the new key and value into the cache (by the block that holds the token's own page, which also patches
// them into its staged page).  Rows of the last page beyond the sequence's length are never used as they
// come from the cache: keys there are masked, values are zeroed in shared memory.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the library's status word
// (sx_attn_decode_status) and the block leaves.
//
// The reference's decode kernel is scalar and re-reads K/V for every query head
// (crates/synaptix-kernels-cuda/src/cu/fused/attention/flash_decode.cu:92-205,340-387).
#include "common.cuh"

#include <cuda.h>

#include "attn_merge.cuh"

#define AD_COMPUTE_WARPS 3
#define AD_THREADS 128                  // 3 compute warps + the producer warp
#define AD_STAGES 3                     // = AD_COMPUTE_WARPS: stage w belongs to compute warp w (see the kernel)
#define AD_SPIN_LIMIT (1u << 26)
#define AD_CHUNK (64 * 128)             // bytes of [64 keys][64 values]: one swizzled column half of a page

template <int HD> struct AdLayout {
  static constexpr int HALVES = HD / 64;
  static constexpr int TILE = HALVES * AD_CHUNK;       // K (or V) of one page
  static constexpr int STAGE = 2 * TILE;               // K then V
  static constexpr int SMEM = AD_STAGES * STAGE + 1024;  // + room to align the ring to 1,024 bytes (the swizzle's period)
};

struct AdPrep {
  const float* wq;          // [HD] gains of the q and k norms, or null
  const float* wk;
  const float* inv_freq;    // [HD / 2] or null (no rotation)
  float eps;
  int write;                // 0: this layer reads a cache another layer wrote (the token's key and value are there)
  int n_pages;
};

__device__ __forceinline__ uint32_t ad_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ad_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void ad_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ad_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool ad_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < AD_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
// one lane of the (converged) warp
__device__ __forceinline__ bool ad_elect_one() {
  uint32_t is_leader;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(is_leader));
  return is_leader != 0;
}
__device__ __forceinline__ void ad_tma_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void ad_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ad_ldsm(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ad_ldsm_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ float ad_ex2(float x) {      // 2^x on the special-function unit; -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t ad_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset, inside a page's K or V tile, of 16-byte chunk `c16` (8 values) of key row `key`: column halves of
// 64 values are AD_CHUNK apart, a row of a half is 128 bytes, and TMA's 128-byte swizzle XORs the chunk index
// with the row index modulo 8.
__device__ __forceinline__ uint32_t ad_off(int key, int c16) {
  return (uint32_t)((c16 >> 3) * AD_CHUNK + key * 128 + (((c16 & 7) ^ (key & 7)) << 4));
}

// One page (64 keys) for one warp: scores, masking, online softmax, O += P V.
//   qf  query fragments [HD/16][4];  kt / vt  shared-memory addresses of the page's K and V tiles
//   jbase  absolute index of the page's first key;  pos  the query's position (keys beyond are masked)
template <int HD, bool MASKED>
__device__ __forceinline__ void ad_attend_page(const uint32_t (&qf)[HD / 16][4], uint32_t kt, uint32_t vt, int jbase,
                                               int pos, int window, float scale_log2, float (&m)[2], float (&l)[2],
                                               float (&o)[HD / 8][4]) {
  const int lane = threadIdx.x & 31, t = lane & 3;
  const int lrow = lane & 7, lmat = lane >> 3;
  float s[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
  // S = Q K^T: one ldmatrix.x4 brings a key tile's fragments for two k-steps (32 values of the head).  The lane's
  // address is ad_off(tile * 8 + lrow, d * 4 + lmat) written so that everything but two lane values is a constant:
  // the row's low bits are lrow whatever the tile, and the chunk index d * 4 + lmat differs between even and odd d
  // in bit 2 only, which the swizzle's XOR carries to bit 6 of the address.
  const uint32_t kx0 = kt + (uint32_t)(lrow * 128 + ((lmat ^ lrow) << 4));
  const uint32_t kx1 = kt + (uint32_t)(lrow * 128 + (((lmat + 4) ^ lrow) << 4));
#pragma unroll
  for (int d = 0; d < HD / 32; ++d) {
#pragma unroll
    for (int k0 = 0; k0 < 8; k0 += 4) {
      uint32_t b[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        ad_ldsm(b[j][0], b[j][1], b[j][2], b[j][3], ((d & 1) ? kx1 : kx0) + (d >> 1) * AD_CHUNK + (k0 + j) * 1024);
#pragma unroll
      for (int j = 0; j < 4; ++j) ad_mma(s[k0 + j], qf[2 * d], b[j][0], b[j][1]);
#pragma unroll
      for (int j = 0; j < 4; ++j) ad_mma(s[k0 + j], qf[2 * d + 1], b[j][2], b[j][3]);
    }
  }
  float mx[2] = {m[0], m[1]};
#pragma unroll
  for (int kt8 = 0; kt8 < 8; ++kt8) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (MASKED) {
        const int j = jbase + kt8 * 8 + 2 * t + (e & 1);
        const bool vis = j <= pos && (window == 0 || j > pos - window);
        if (!vis) s[kt8][e] = -INFINITY;
      }
      mx[e >> 1] = fmaxf(mx[e >> 1], s[kt8][e]);
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
  }
  // the output and the sums are rescaled only if some row's maximum moved (decided for the whole warp)
  if (__any_sync(0xffffffffu, mx[0] != m[0] || mx[1] != m[1])) {
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      corr[r] = (mx[r] == -INFINITY) ? 1.f : ad_ex2((m[r] - mx[r]) * scale_log2);
      l[r] *= corr[r];
      m[r] = mx[r];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
  }
  float ms[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) ms[r] = (mx[r] == -INFINITY) ? 0.f : mx[r] * scale_log2;   // nothing visible yet: 2^(-inf - 0) = 0
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int kt8 = 0; kt8 < 8; ++kt8) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = ad_ex2(fmaf(s[kt8][e], scale_log2, -ms[e >> 1]));
      s[kt8][e] = p;
      sum[e >> 1] += p;
    }
  }
  l[0] += sum[0];                // per-thread partial sums; the lanes of a row are added at the end
  l[1] += sum[1];
  // O += P V: 16 keys a step; V fragments by transposing ldmatrix
  const uint32_t vx = vt + (uint32_t)(((lmat & 1) * 8 + lrow) * 128 + (((lmat >> 1) ^ lrow) << 4));
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    uint32_t pa[4];
    pa[0] = ad_pack(s[2 * kk][0], s[2 * kk][1]);
    pa[1] = ad_pack(s[2 * kk][2], s[2 * kk][3]);
    pa[2] = ad_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    pa[3] = ad_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    // matrices of one ldmatrix.x4.trans: (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15).
    // The lane's address is ad_off(kk * 16 + (lmat & 1) * 8 + lrow, n * 2 + (lmat >> 1)): the chunk's low bits
    // (n & 3) * 2 + (lmat >> 1) XOR lrow are ((n & 3) * 2) XOR a lane value, so the lane's part is one register.
#pragma unroll
    for (int n = 0; n < HD / 16; ++n) {
      uint32_t b0, b1, b2, b3;
      ad_ldsm_t(b0, b1, b2, b3, (vx ^ (uint32_t)((n & 3) * 32)) + (n >> 2) * AD_CHUNK + kk * 2048);
      ad_mma(o[2 * n], pa, b0, b1);
      ad_mma(o[2 * n + 1], pa, b2, b3);
    }
  }
}

template <int HD, bool PREP, bool CLUSTER>
__global__ void __launch_bounds__(AD_THREADS, 2) attn_decode_tma_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    const bf16* __restrict__ q, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, bf16* __restrict__ out,
    float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ seq_lens,
    const int* __restrict__ block_table, int maxp, int nh, int nkv, float scale_log2, int window, int n_splits,
    const AdPrep prep, int* __restrict__ status) {
  using L = AdLayout<HD>;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(16) bf16 q_s[PREP ? 16 * HD : 8];       // the group's prepared query heads
  __shared__ __align__(16) bf16 kv_new[PREP ? 2 * HD : 8];     // the token's prepared key and value
  __shared__ __align__(8) uint64_t bars[2 * AD_STAGES];         // full[stage], empty[stage]
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t ring_a = ad_smem(ring);
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int G = nh / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  auto full = [&](int s) { return ad_smem(&bars[s]); };
  auto empty = [&](int s) { return ad_smem(&bars[AD_STAGES + s]); };
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < AD_STAGES; ++s) {
      ad_mbar_init(full(s), 1);
      ad_mbar_init(empty(s), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (!PREP) { pdl_wait(); pdl_trigger(); }
  __syncthreads();

  // lengths and block tables were written at least two launches ago (see below), so they are read before the wait
  const int len = seq_lens[seq];
  const int pos = len - 1;                                   // the query's position
  const int lo = window > 0 ? max(0, len - window) : 0;      // first visible key
  const int p_first = lo >> 6, p_end = max((len + 63) >> 6, p_first + 1);
  const int total = p_end - p_first;
  const int per = (total + n_splits - 1) / n_splits;
  const int p0 = p_first + split * per, p1 = min(p_end, p0 + per);
  const int npages = max(0, p1 - p0);
  const int* bt = block_table + (size_t)seq * maxp;
  const int p_last = pos < 0 ? 0 : pos >> 6;                 // the page of the token's own place (the sequence's last)
  const bool has_last = p0 <= p_last && p_last < p1;
  const bool writes = PREP && prep.write;

  if (warp == AD_COMPUTE_WARPS) {
    // ------------------------------------------------------------------ producer
    // The first pages are asked for while the product before this kernel still runs: what they hold (every row
    // but the token's own, which this kernel makes) and the lengths and block tables were written at least two
    // launches ago, and a kernel behind a programmatic launch starts only when the one before its predecessor
    // has ended.
    // (The whole warp walks the pages and one elected lane issues: addresses computed in uniform control flow
    // stay in uniform registers, which the copy instruction takes its operands from.)
    const bool leader = ad_elect_one();
    for (int i = 0; i < npages; ++i) {
      const int st = i % AD_STAGES, use = i / AD_STAGES;
      if (use > 0 && !__all_sync(0xffffffffu, ad_mbar_wait(empty(st), (use - 1) & 1))) {
        if (leader) sx_set_status(status, 1);
        break;
      }
      const int page = bt[p0 + i];
      const uint32_t dst = ring_a + st * L::STAGE, bar = full(st);
      if (leader) {
        ad_mbar_expect_tx(bar, L::STAGE);
#pragma unroll
        for (int h = 0; h < L::HALVES; ++h) {
          ad_tma_4d(dst + h * AD_CHUNK, &map_k, h * 64, 0, kvh, page, bar);
          ad_tma_4d(dst + L::TILE + h * AD_CHUNK, &map_v, h * 64, 0, kvh, page, bar);
        }
      }
      __syncwarp();
    }
    if (CLUSTER) {                  // every thread of the cluster takes part in its two barriers
      cluster_sync_all();
      cluster_sync_all();
    }
    return;
  }

  // -------------------------------------------------------------------- compute warps
  if (PREP) {
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
    if (writes && has_last) {
      const int page = bt[p_last];
      if (page >= 0 && page < prep.n_pages) {                 // the host guarantees a page; never write outside
        const size_t at = (((size_t)page * nkv + kvh) * SX_PAGE + (pos & 63)) * HD;
        k_row = k_pages + at;
        v_row = v_pages + at;
      }
    }
    pdl_wait();                                               // the projection comes from the kernel before
    pdl_trigger();
    // jobs: the G query heads of the group, then (the block with the token's page) the key head and the value head
    const int jobs = G + (writes && has_last ? 2 : 0);
    for (int j = warp; j < jobs; j += AD_COMPUTE_WARPS) {
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
        const __nv_bfloat162 lo2 = __floats2bfloat162_rn(a0 * cs[0] - b0 * sn[0], a1 * cs[1] - b1 * sn[1]);
        const __nv_bfloat162 hi2 = __floats2bfloat162_rn(a0 * sn[0] + b0 * cs[0], a1 * sn[1] + b1 * cs[1]);
        bf16* dst = is_q ? q_s + j * HD : kv_new;
        *reinterpret_cast<__nv_bfloat162*>(dst + p) = lo2;
        *reinterpret_cast<__nv_bfloat162*>(dst + p + half) = hi2;
        if (is_k && k_row) {
          *reinterpret_cast<__nv_bfloat162*>(k_row + p) = lo2;
          *reinterpret_cast<__nv_bfloat162*>(k_row + p + half) = hi2;
        }
      }
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(AD_COMPUTE_WARPS * 32) : "memory");       // the compute warps only
  }

  // query fragments: row r of the fragment is query head kvh * G + r (rows >= G are zero)
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

  bool ok = true;
  for (int i = warp; i < npages; i += AD_COMPUTE_WARPS) {
    const int st = warp;                                      // i % AD_STAGES: this warp's own stage
    if (!ad_mbar_wait(full(st), (i / AD_STAGES) & 1)) { if (lane == 0) sx_set_status(status, 2); ok = false; break; }
    unsigned char* stage = ring + st * L::STAGE;
    const uint32_t kt = ring_a + st * L::STAGE, vt = kt + L::TILE;
    const int pg = p0 + i, jb = pg * 64;
    if (pg == p_last) {
      // The sequence's last page.  Its rows beyond the token's place hold whatever the cache held: the keys there
      // are masked, the values are set to zero (a value that is not finite would survive a zero weight).  The
      // token's own row is patched in from what this block prepared when the cache does not hold it yet.
      const int own = pos < 0 ? -1 : (pos & 63);           // (an empty sequence: every value row is zeroed)
      for (int c = lane; c < (63 - own) * (HD / 8); c += 32) {
        const int r = own + 1 + c / (HD / 8), c16 = c % (HD / 8);
        *reinterpret_cast<uint4*>(stage + L::TILE + ad_off(r, c16)) = make_uint4(0u, 0u, 0u, 0u);
      }
      if (writes && own >= 0) {
        for (int c = lane; c < 2 * (HD / 8); c += 32) {
          const int isv = c / (HD / 8), c16 = c % (HD / 8);
          *reinterpret_cast<uint4*>(stage + isv * L::TILE + ad_off(own, c16)) =
              reinterpret_cast<const uint4*>(kv_new + isv * HD)[c16];
        }
      }
      __syncwarp();
    }
    if (jb + 63 > pos || (window > 0 && jb <= pos - window))
      ad_attend_page<HD, true>(qf, kt, vt, jb, pos, window, scale_log2, m, l, o);
    else      // the whole page is visible: no comparisons
      ad_attend_page<HD, false>(qf, kt, vt, jb, pos, window, scale_log2, m, l, o);
    __syncwarp();
    if (lane == 0) {
      // generic-proxy writes to the stage (the patches above) are ordered before the TMA copy that refills it
      if (pg == p_last) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      ad_mbar_arrive(empty(st));
    }
  }
  // every page that was asked for has been consumed by some warp once all compute warps are here
  asm volatile("bar.sync 1, %0;\n" ::"n"(AD_COMPUTE_WARPS * 32) : "memory");
  (void)ok;

  // the running maxima are of raw scores; the merges below work in the scaled (log2) domain
  m[0] *= scale_log2;
  m[1] *= scale_log2;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  // merge the compute warps through shared memory (the ring is free now)
  float* wo = reinterpret_cast<float*>(ring);                 // [warps][16][HD]
  float* wml = wo + AD_COMPUTE_WARPS * 16 * HD;               // [warps][16][2]
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    const int c = n * 8 + 2 * t;
    *reinterpret_cast<float2*>(wo + (warp * 16 + g) * HD + c) = make_float2(o[n][0], o[n][1]);
    *reinterpret_cast<float2*>(wo + (warp * 16 + g + 8) * HD + c) = make_float2(o[n][2], o[n][3]);
  }
  if (t == 0) {
    wml[(warp * 16 + g) * 2] = m[0];
    wml[(warp * 16 + g) * 2 + 1] = l[0];
    wml[(warp * 16 + g + 8) * 2] = m[1];
    wml[(warp * 16 + g + 8) * 2 + 1] = l[1];
  }
  asm volatile("bar.sync 1, %0;\n" ::"n"(AD_COMPUTE_WARPS * 32) : "memory");
  // this block's result: O [G][HD], then (M, L) [G][2], behind the warps' results in the ring
  float* res = wml + AD_COMPUTE_WARPS * 16 * 2;
  float* res_ml = res + 16 * HD;
  for (int idx = threadIdx.x; idx < G * HD; idx += AD_COMPUTE_WARPS * 32) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < AD_COMPUTE_WARPS; ++w) M = fmaxf(M, wml[(w * 16 + r) * 2]);
    float Lsum = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < AD_COMPUTE_WARPS; ++w) {
      const float mw = wml[(w * 16 + r) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      Lsum += wml[(w * 16 + r) * 2 + 1] * f;
      O += wo[(w * 16 + r) * HD + d] * f;
    }
    const int head = kvh * G + r;
    if (n_splits == 1) {
      out[((size_t)seq * nh + head) * HD + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
    } else if (CLUSTER) {
      res[r * HD + d] = O;
      if (d == 0) { res_ml[r * 2] = M; res_ml[r * 2 + 1] = Lsum; }
    } else {
      const size_t pi = ((size_t)seq * nh + head) * n_splits + split;
      part_o[pi * HD + d] = O;
      if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = Lsum; }
    }
  }
  if (CLUSTER && n_splits > 1) {
    // The cluster is the n_splits blocks of this (sequence, kv head); its rank is the split.  After the barrier
    // every block's result lies in its shared memory; block k merges outputs k, k + n_splits, ... of the G * HD
    // (head, value) pairs, in rank order, reading the others' results from afar.
    cluster_sync_all();
    for (int idx = split + n_splits * (int)threadIdx.x; idx < G * HD; idx += n_splits * AD_COMPUTE_WARPS * 32) {
      const int r = idx / HD, d = idx % HD;
      float M = -INFINITY;
      for (int k = 0; k < n_splits; ++k) M = fmaxf(M, cluster_load_f32(res_ml + r * 2, k));
      float Lsum = 0.f, O = 0.f;
      for (int k = 0; k < n_splits; ++k) {
        const float mk = cluster_load_f32(res_ml + r * 2, k);
        const float f = (mk == -INFINITY) ? 0.f : exp2f(mk - M);
        Lsum += cluster_load_f32(res_ml + r * 2 + 1, k) * f;
        if (f != 0.f) O += cluster_load_f32(res + r * HD + d, k) * f;
      }
      out[((size_t)seq * nh + kvh * G + r) * HD + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
    }
    cluster_sync_all();             // nobody leaves while its shared memory may still be read
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*ad_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static ad_encode_fn ad_get_encode() {
  static ad_encode_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = (ad_encode_fn)p;
  }
  return fn;
}
// cache pages [n_pages, nkv, 64, hd]: boxes of one page's 64 tokens x 64 values of one kv head
static int ad_map_pages(CUtensorMap* map, const void* pages, long long n_pages, int nkv, int hd) {
  ad_encode_fn enc = ad_get_encode();
  if (!enc) return SX_ERR_SIZE;
  cuuint64_t dims[4] = {(cuuint64_t)hd, SX_PAGE, (cuuint64_t)nkv, (cuuint64_t)n_pages};
  cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)SX_PAGE * hd * 2, (cuuint64_t)nkv * SX_PAGE * hd * 2};
  cuuint32_t box[4] = {64, SX_PAGE, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(pages), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

static int* ad_status_word() {
  static int* p = nullptr;
  if (!p) p = sx_status_word_alloc();
  return p;
}

template <int HD, bool PREP>
static int ad_launch(const CUtensorMap& mk, const CUtensorMap& mv, const bf16* q, bf16* k, bf16* v, bf16* out, float* part_o,
                     float* part_ml, const int* seq_lens, const int* bt, int maxp, int S, int nh, int nkv, float scale_log2,
                     int window, int n_splits, const AdPrep& prep, int* status, cudaStream_t stream) {
  using L = AdLayout<HD>;
  static_assert(AD_STAGES == AD_COMPUTE_WARPS, "a stage has one consumer");
  static_assert(AD_STAGES * L::STAGE >= (AD_COMPUTE_WARPS + 1) * (16 * HD + 16 * 2) * (int)sizeof(float),
                "the ring holds the warps' results and the block's");
  // 2, 4, 8 or 16 splits: the splits of a (sequence, kv head) are a cluster and merge among themselves
  if (part_o == nullptr && n_splits > 1) {
    auto kern = attn_decode_tma_kernel<HD, PREP, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM);
    if (e != cudaSuccess) return (int)e;
    return sx_launch_cluster(kern, dim3(n_splits, nkv, S), dim3(AD_THREADS), (size_t)L::SMEM, stream, n_splits, mk, mv, q, k,
                             v, out, part_o, part_ml, seq_lens, bt, maxp, nh, nkv, scale_log2, window, n_splits, prep, status);
  }
  auto kern = attn_decode_tma_kernel<HD, PREP, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM);
  if (e != cudaSuccess) return (int)e;
  int rc = sx_launch(kern, dim3(n_splits, nkv, S), dim3(AD_THREADS), (size_t)L::SMEM, stream, mk, mv, q, k, v, out, part_o,
                     part_ml, seq_lens, bt, maxp, nh, nkv, scale_log2, window, n_splits, prep, status);
  if (rc || n_splits == 1) return rc;
  return sx_launch(attn_merge_kernel<HD>, dim3(S * nh), dim3(HD), 2 * n_splits * sizeof(float), stream,
                   (const float*)part_o, (const float*)part_ml, out, n_splits);
}

// q: [S, nh, hd] prepared queries against a cache that holds the step's keys and values, or (prep_on != 0) the
// step's fused projection [S, (nh + 2 nkv) hd]: per-head RMSNorm of q and k (gains wq, wk in float32, or null),
// rotate-half rotation of the whole head by seq_lens[s] - 1 (inv_freq [hd / 2], or null), and (write != 0) the new
// key and value into the cache happen inside the kernel.  k_pages / v_pages [n_pages, nkv, 64, hd]; out [S, nh * hd];
// part_o f32 [S * nh * n_splits * hd] and part_ml f32 [S * nh * n_splits * 2] are scratch (unused with one split).
// Without scratch (both null) and 2, 4, 8 or 16 splits, the splits of a (sequence, kv head) run as a thread-block
// cluster and merge through one another's shared memory; other split counts need the scratch.  Head size 64 or 128.
extern "C" int sx_attn_decode_tma(const void* q, void* k_pages, void* v_pages, void* out, float* part_o, float* part_ml,
                                  int prep_on, const float* wq, const float* wk, const float* inv_freq, float eps,
                                  int write, long long n_pages, const int* seq_lens, const int* block_table, int maxp,
                                  int S, int nh, int nkv, int hd, float scale, int window, int n_splits,
                                  cudaStream_t stream) {
  if (S <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 16 || n_splits < 1 || nkv > 65535 || S > 65535) return SX_ERR_SIZE;
  if (hd != 64 && hd != 128) return SX_ERR_SIZE;
  if (n_splits > AT_MAX_SPLITS) return SX_ERR_SIZE;
  const bool clustered = n_splits == 2 || n_splits == 4 || n_splits == 8 || n_splits == 16;
  if (n_splits > 1 && (!part_o || !part_ml) && !(clustered && !part_o && !part_ml)) return SX_ERR_SIZE;
  if (n_pages <= 0 || n_pages > 0x7fffffffLL) return SX_ERR_SIZE;
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return SX_ERR_ALIGN;
  int* status = ad_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  CUtensorMap mk, mv;
  int rc = ad_map_pages(&mk, k_pages, n_pages, nkv, hd);
  if (rc) return rc;
  if ((rc = ad_map_pages(&mv, v_pages, n_pages, nkv, hd))) return rc;
  const float sl = scale * 1.4426950408889634f;
  const AdPrep prep = {wq, wk, inv_freq, eps, write, (int)n_pages};
  const bf16* qb = (const bf16*)q;
  bf16 *kb = (bf16*)k_pages, *vb = (bf16*)v_pages, *ob = (bf16*)out;
#define AD_GO(HD)                                                                                                          \
  return prep_on ? ad_launch<HD, true>(mk, mv, qb, kb, vb, ob, part_o, part_ml, seq_lens, block_table, maxp, S, nh, nkv, sl, \
                                       window, n_splits, prep, status, stream)                                              \
                 : ad_launch<HD, false>(mk, mv, qb, kb, vb, ob, part_o, part_ml, seq_lens, block_table, maxp, S, nh, nkv, sl, \
                                        window, n_splits, prep, status, stream)
  if (hd == 128) AD_GO(128);
  AD_GO(64);
#undef AD_GO
}

// Reads the status word in host memory: no device call.  It tells of kernels the host has already waited for
// (0, or which bounded wait ran out: 1 the producer's, 2 a compute warp's).  With reset != 0 the word goes back to 0.
extern "C" int sx_attn_decode_status(int* host_value, int reset) {
  int* p = ad_status_word();
  if (!p) return (int)cudaErrorMemoryAllocation;
  *host_value = *(volatile int*)p;
  if (reset) *(volatile int*)p = 0;
  return 0;
}
