// Device code shared by the attention kernels: fragment helpers, the shared-memory layout of a
// staged cache page, the page loader and the tile routine (scores, masking, online softmax, P*V).
// Included by attention.cu.
#pragma once
#include "common.cuh"

#define AT_THREADS 128
#define AT_STAGES_DECODE 3      // pages in flight per block: decode streams the cache, three stages keep HBM busy
#define AT_STAGES_PREFILL 2     // prompt steps reuse pages from L2; two stages leave room for three blocks per SM

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;      // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <int HD, int STAGES = AT_STAGES_DECODE> struct AtLayout {
  static constexpr int ROW = HD * 2 + 16;              // bytes of a padded row: ldmatrix rows hit distinct banks
  static constexpr int TILE = 64 * ROW;                // one page of K (or V)
  static constexpr int STAGE = 2 * TILE;               // K then V
  static constexpr int SMEM = STAGES * STAGE;
};

// one page (64 keys) of K and V of (page, kvh) -> stage; rows >= valid_rows are zero-filled
template <int HD>
__device__ __forceinline__ void load_page(unsigned char* stage, const bf16* __restrict__ k_pages,
                                          const bf16* __restrict__ v_pages, int page, int kvh, int nkv, int valid_rows) {
  using L = AtLayout<HD>;
  constexpr int CH = HD / 8;                           // 16-byte chunks per row
  const size_t base = ((size_t)page * nkv + kvh) * SX_PAGE * HD;
  for (int c = threadIdx.x; c < 64 * CH; c += AT_THREADS) {
    const int r = c / CH, ch = c % CH;
    const bool ok = r < valid_rows;
    const size_t off = base + (size_t)(ok ? r : 0) * HD + ch * 8;
    cp_async16(smem_addr(stage + r * L::ROW + ch * 16), k_pages + off, ok);
    cp_async16(smem_addr(stage + L::TILE + r * L::ROW + ch * 16), v_pages + off, ok);
  }
}

// ---------------------------------------------------------------------------------------
// Scores of one 16-row query fragment against NKT key tiles (8 keys each) starting at key
// row `key0` of the staged page, masking, online softmax update, and O += P V.
//   qf     query fragments [HD/16][4]
//   pos_lo/pos_hi  absolute positions of fragment rows g and g + 8 (keys beyond are masked);
//                  a negative position masks the whole row
//   jbase  absolute index of the page's first key
// ---------------------------------------------------------------------------------------
template <int HD, int NKT, bool MASKED>
__device__ __forceinline__ void attend_tile(const uint32_t (&qf)[HD / 16][4], const unsigned char* kst,
                                            const unsigned char* vst, int key0, int jbase, int pos_lo, int pos_hi,
                                            int window, float scale_log2, float (&m)[2], float (&l)[2],
                                            float (&o)[HD / 8][4]) {
  using L = AtLayout<HD>;
  const int lane = threadIdx.x & 31, t = lane & 3;
  float s[NKT][4];
#pragma unroll
  for (int i = 0; i < NKT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;

  // S = Q K^T.  One ldmatrix.x4 brings a key tile's fragments for two k-steps (32 of the head
  // dim).  Key tiles are taken in groups (of 4 when there are that many) so that consecutive MMAs
  // write different accumulators: a dependent pair is then a whole group of MMAs apart.
  const int lrow = lane & 7, lmat = lane >> 3;
  constexpr int KG = NKT >= 4 ? 4 : NKT;
#pragma unroll
  for (int d = 0; d < HD / 32; ++d) {
#pragma unroll
    for (int k0 = 0; k0 < NKT; k0 += KG) {
      uint32_t b[KG][4];
#pragma unroll
      for (int j = 0; j < KG; ++j)
        ldsm_x4(b[j][0], b[j][1], b[j][2], b[j][3],
                smem_addr(kst + (key0 + (k0 + j) * 8 + lrow) * L::ROW + lmat * 16) + d * 64);
#pragma unroll
      for (int j = 0; j < KG; ++j) mma16816(s[k0 + j], qf[2 * d], b[j][0], b[j][1]);
#pragma unroll
      for (int j = 0; j < KG; ++j) mma16816(s[k0 + j], qf[2 * d + 1], b[j][2], b[j][3]);
    }
  }
  // running maximum of the raw scores (the scale is positive, so it can be applied later inside
  // the exponent: p = 2^(s * scale - m * scale), one FFMA and one EX2 per score).  A page that lies
  // wholly inside every row's visible range (MASKED == false) needs no comparisons at all.
  float mx[2] = {m[0], m[1]};
#pragma unroll
  for (int kt = 0; kt < NKT; ++kt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (MASKED) {
        const int j = jbase + key0 + kt * 8 + 2 * t + (e & 1);
        const int p = (e < 2) ? pos_lo : pos_hi;
        const bool vis = j <= p && (window == 0 || j > p - window);
        if (!vis) s[kt][e] = -INFINITY;
      }
      mx[e >> 1] = fmaxf(mx[e >> 1], s[kt][e]);
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
  }
  float corr[2], ms[2], sum[2] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    corr[r] = (mx[r] == -INFINITY) ? 1.f : exp2f((m[r] - mx[r]) * scale_log2);
    ms[r] = (mx[r] == -INFINITY) ? 0.f : mx[r] * scale_log2;      // a row with nothing visible yet: 2^(-inf - 0) = 0
  }
#pragma unroll
  for (int kt = 0; kt < NKT; ++kt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = exp2f(fmaf(s[kt][e], scale_log2, -ms[e >> 1]));
      s[kt][e] = p;
      sum[e >> 1] += p;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] = l[r] * corr[r] + sum[r];      // per-thread partial sums; lanes of a row are added at the end
    m[r] = mx[r];
  }
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    o[n][0] *= corr[0]; o[n][1] *= corr[0];
    o[n][2] *= corr[1]; o[n][3] *= corr[1];
  }
  // O += P V : 16 keys a step; V fragments by transposing ldmatrix
#pragma unroll
  for (int kk = 0; kk < NKT / 2; ++kk) {
    uint32_t pa[4];
    pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    // matrices of one ldmatrix.x4.trans: (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
    const uint32_t vaddr = smem_addr(vst + (key0 + kk * 16 + (lmat & 1) * 8 + lrow) * L::ROW + (lmat >> 1) * 16);
#pragma unroll
    for (int n = 0; n < HD / 16; ++n) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_trans(b0, b1, b2, b3, vaddr + n * 32);
      mma16816(o[2 * n], pa, b0, b1);
      mma16816(o[2 * n + 1], pa, b2, b3);
    }
  }
}

