// A run of decoder layers for a step of single tokens (at most 8 sequences, bfloat16) as ONE
// persistent kernel: one block per SM, launched cooperatively, every layer's work split over all
// blocks, and the phases of a layer separated by barriers across the grid.
//
// Why.  A decode step reads every weight once, so its floor is the time HBM needs.  A layer built
// from separate kernels loses several microseconds at every kernel boundary: the next kernel's
// first weights are only asked for when it starts.  Here every thread walks through ITS share of
// ALL matrices of ALL layers as one sequence and keeps DS_DEPTH steps of it in flight (cp.async
// into a ring in shared memory that only this thread reads back).  The sequence does not stop at a
// phase's end, so while the block stands at a barrier or runs attention, the ring already holds
// the first weights of the next product: HBM stays busy across phase boundaries.
//
// Phases of a layer (a barrier across the grid after each):
//   1  qkv = rmsnorm(h) * gain  Wqkv^T                                             -> float32 scratch
//   2  per-head RMSNorm of q and k, rotate-half rotation, q -> scratch, k and v -> cache pages
//   3  attention over the cache, split over pages; the block that finishes a (sequence, kv head)
//      last merges the splits                                                      -> scratch
//   4  h += attn Wo^T
//   5  act = silu(x Wg^T) * (x Wu^T),  x = rmsnorm(h) * gain2                      -> scratch
//   6  h += act Wd^T
// The residual stream h is float32 and updated in place.  A norm needs no reduction of its own: the
// product that writes h also writes each block's partial sum of squares per row; after the barrier
// every block adds the partial sums (in block order) and writes x = bf16(h * inv * gain) to shared memory.  All sums run in a fixed order (no atomics on
// data), so a step gives the same bits every time.
//
// Work split of a product.  Block c owns the contiguous output rows [rows*c/G, rows*(c+1)/G), cut
// evenly into tiles of at most 16 rows (8 gate + 8 up rows for the gated product).  The 8 warps split
// k between them; a warp's step is 32 k-values of a tile: every thread copies 16 bytes of two
// rows, which are the fragments of two mma.sync.m16n8k16 under the "16 bytes of k per thread" map
// of skinny_gemm_kernel (decode.cu).  The products of normalised rows (many tiles) keep x in shared
// memory and run tile by tile; the products into h (at most 3 tiles) run k-major and fetch their
// activation fragments from L2 a few steps ahead.  The warps' partial sums are added through shared
// memory in warp order.  The code is kept small on purpose: a first version with 48 unrolled
// element bodies per product ran out of the instruction cache and was four times slower.
//
// Everything one block wrote and another reads (h, the scratch arrays, the cache) is read with
// loads that bypass L1 (ld.global.cg, cp.async.cg), since L1 is not coherent between SMs.
//
// The wait at a grid barrier is bounded.  A wait that runs out writes a code to the status word,
// raises the block's abort flag and the block leaves; the other blocks then run out at their next
// barrier.  The host reads the status word with sx_decode_stream_status.
//
// The reference runs a layer as separate launches (crates/synaptix-models/llm/common/src/model.rs:
// 1179-1199, 1670-1734); it has no counterpart of this kernel.
#include "common.cuh"
#include "attn_tile.cuh"

#define DS_WARPS 8
#define DS_THREADS (DS_WARPS * 32)
#define DS_CTHREADS DS_THREADS
#ifndef DS_DEPTH
#define DS_DEPTH 14                                  // steps (2 x 16 bytes) every thread keeps in flight
#endif
#define DS_MAXT 3                                    // most tiles of a product into h (their sums are live at once)
#define DS_XPD 4                                     // activation fragments a thread has on the way (products into h)
#define DS_RING_BYTES (DS_DEPTH * 2 * DS_THREADS * 16)      // 114,688
#define DS_SHARED_BYTES (3 * 2 * 64 * (128 * 2 + 16))      // 104,448: attention stages / the warps' partial sums
#define DS_MISC_BYTES 1024
#define DS_SMEM (DS_RING_BYTES + DS_SHARED_BYTES + DS_MISC_BYTES)
#define DS_MAX_ROWS 8
#define DS_GRID_LIMIT (1u << 23)

// One layer run.  The layout is mirrored by a ctypes structure on the host.
struct SxStreamLayer {
  const bf16* w_qkv;      // [(nh + 2 nkv) hd, H]
  const bf16* w_o;        // [H, nh hd]
  const bf16* w_gu;       // [2 I, H]: gate rows, then up rows
  const bf16* w_down;     // [H, I]
  const float* g_in;      // [H]
  const float* g_post;    // [H]
  const float* g_q;       // [hd] or null
  const float* g_k;       // [hd] or null
  const float* inv_freq;  // [hd / 2] or null (no rotation)
  bf16* k_pages;          // [n_pages, nkv, 64, hd]
  bf16* v_pages;
  float eps_in, eps_post, eps_qk, scale_log2;
  int window, group, write_cache, n_pages;
};

struct SxStreamArgs {
  const SxStreamLayer* layers;
  int n_layers, M, H, nh, nkv, I, n_splits, pad0;
  float* h;                       // [M, H] float32, in place
  const int* positions;           // [M]
  const int* seq_lens;            // [M] after this step
  const int* block_table[4];      // per storage group [M, maxp]
  int maxp[4];
  float* qkv;                     // scratch [M, (nh + 2 nkv) hd]
  bf16* q;                        // [M, nh, hd]
  float* part_o;                  // [M, nh, n_splits, hd]
  float* part_ml;                 // [M, nh, n_splits, 2]
  bf16* attn;                     // [M, nh hd]
  bf16* act;                      // [M, I]
  float* ssq;                     // [2][blocks][8] partial sums of squares of h's rows
  int* counters;                  // [M, nkv] zero between launches
  unsigned* barrier;              // zero at launch
  int* status;
  unsigned long long* prof;       // null, or [blocks][n_layers][16] time stamps (ns) of the phases, for tuning
};

enum { DS_OK = 0, DS_FAIL_GRID = 3 };
enum { DS_EPI_QKV = 0, DS_EPI_ADD_H = 1, DS_EPI_SILU = 2 };

__device__ __forceinline__ uint32_t ds_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ds_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ds_stamp(const SxStreamArgs& a, int li, int k) {
  if (a.prof != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    a.prof[((size_t)blockIdx.x * a.n_layers + li) * 16 + k] = t;
  }
}
__device__ __forceinline__ void ds_csync() { asm volatile("bar.sync 1, %0;\n" ::"n"(DS_THREADS) : "memory"); }   // all warps
__device__ __forceinline__ void ds_tsync() { asm volatile("bar.sync 2, %0;\n" ::"n"(AT_THREADS) : "memory"); }    // the attention team (warps 0..3)

// the shape of product `ph` (0 q/k/v, 1 o, 2 gate/up, 3 down) of a layer
struct DsGeo {
  const bf16* W;
  int rows, K, rpt;      // output rows split over the grid; k; most rows of a tile
};
template <int HD>
__device__ __forceinline__ DsGeo ds_geo(const SxStreamArgs& a, const SxStreamLayer& L, int ph) {
  DsGeo g;
  switch (ph) {
    case 0: g.W = L.w_qkv; g.rows = (a.nh + 2 * a.nkv) * HD; g.K = a.H; g.rpt = 16; break;
    case 1: g.W = L.w_o; g.rows = a.H; g.K = a.nh * HD; g.rpt = 16; break;
    case 2: g.W = L.w_gu; g.rows = a.I; g.K = a.H; g.rpt = 8; break;
    default: g.W = L.w_down; g.rows = a.H; g.K = a.I; g.rpt = 16; break;
  }
  return g;
}
// this block's rows of a product, its tiles, and this warp's k-steps of a tile
struct DsPlan {
  int r0, r1, ntiles, q, last_rows, s_begin, s_end;
};
__device__ __forceinline__ DsPlan ds_plan(const DsGeo& geo) {
  DsPlan p;
  p.r0 = (int)((long long)geo.rows * blockIdx.x / gridDim.x);
  p.r1 = (int)((long long)geo.rows * (blockIdx.x + 1) / gridDim.x);
  const int rows = p.r1 - p.r0;
  p.ntiles = (rows + geo.rpt - 1) / geo.rpt;
  p.q = p.ntiles ? (rows + p.ntiles - 1) / p.ntiles : 0;
  p.last_rows = p.ntiles ? rows - (p.ntiles - 1) * p.q : 0;
  const int nsteps = geo.K >> 5, per = (nsteps + DS_WARPS - 1) / DS_WARPS;
  p.s_begin = min(nsteps, (int)(threadIdx.x >> 5) * per);
  p.s_end = min(nsteps, p.s_begin + per);
  return p;
}

// ---------------------------------------------------------------------------------------
// This thread's walk through the weights, one element (a k-step of a tile: 16 bytes of two rows)
// at a time: layers, products, and inside a product either tile by tile (products of normalised
// rows) or k-major (products into h).  ask() issues the copies of the element the walk stands on
// into a ring slot and moves on; the common path is a handful of instructions.
// ---------------------------------------------------------------------------------------
template <int HD>
struct DsWalk {
  const unsigned char* cur;       // address of the element's 16 bytes of the "lo" row
  const unsigned char* outer;     // cur at the start of the inner loop
  long long in_stride, out_stride, hi_off;
  int in_i, in_n, out_i, out_n;
  int ntiles, q, last_rows, hi_idx, g;
  int li, ph;
  bool tile_inner, done;

  __device__ __forceinline__ void load_phase(const SxStreamArgs& a) {     // inlined: otherwise the walk lives in local memory (measured 2x slower)
    for (;;) {
      if (li >= a.n_layers) { done = true; return; }
      const DsGeo geo = ds_geo<HD>(a, a.layers[li], ph);
      const DsPlan pl = ds_plan(geo);
      if (pl.ntiles > 0 && pl.s_begin < pl.s_end) {
        const int lane = threadIdx.x & 31, t = lane & 3;
        g = lane >> 2;
        const long long row_bytes = (long long)geo.K * 2;
        const long long tile_stride = (long long)pl.q * row_bytes;
        hi_idx = ph == 2 ? g : g + 8;
        hi_off = ph == 2 ? (long long)a.I * row_bytes : 8 * row_bytes;
        ntiles = pl.ntiles; q = pl.q; last_rows = pl.last_rows;
        tile_inner = (ph & 1) != 0;                      // products into h run k-major
        const int nst = pl.s_end - pl.s_begin;
        if (tile_inner) { in_n = pl.ntiles; in_stride = tile_stride; out_n = nst; out_stride = 64; }
        else { in_n = nst; in_stride = 64; out_n = pl.ntiles; out_stride = tile_stride; }
        in_i = out_i = 0;
        outer = reinterpret_cast<const unsigned char*>(geo.W) + (long long)(pl.r0 + g) * row_bytes + (long long)pl.s_begin * 64 + t * 16;
        cur = outer;
        return;
      }
      if (++ph == 4) { ph = 0; ++li; }
    }
  }
  __device__ __forceinline__ void init(const SxStreamArgs& a) {
    li = 0; ph = 0; done = false;
    load_phase(a);
  }
  __device__ __forceinline__ void ask(const SxStreamArgs& a, uint32_t slot_addr) {
    if (!done) {
      const int tile = tile_inner ? in_i : out_i;
      const int rows_in = tile == ntiles - 1 ? last_rows : q;
      if (g < rows_in) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(slot_addr), "l"(cur) : "memory");
      if (hi_idx < rows_in) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(slot_addr + DS_THREADS * 16), "l"(cur + hi_off) : "memory");
      cur += in_stride;
      if (++in_i == in_n) {
        in_i = 0;
        outer += out_stride;
        cur = outer;
        if (++out_i == out_n) {
          if (++ph == 4) { ph = 0; ++li; }
          load_phase(a);
        }
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");        // one group per element, empty or not
  }
};

// ---------------------------------------------------------------------------------------
// the barrier across the grid, called by all threads; false = gave up
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ bool ds_grid_sync(const SxStreamArgs& a, unsigned& epoch, volatile int* abort_flag) {
  ds_csync();
  ++epoch;
  if (threadIdx.x == 0) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(a.barrier) : "memory");
    const unsigned target = epoch * gridDim.x;
    bool ok = false;
    for (uint32_t i = 0; i < DS_GRID_LIMIT; ++i) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(a.barrier) : "memory");
      if (v >= target) { ok = true; break; }
      if ((i & 255u) == 255u) {
        int st;
        asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];\n" : "=r"(st) : "l"(a.status) : "memory");
        if (st != 0) break;
      }
    }
    if (!ok) {
      atomicCAS(a.status, 0, DS_FAIL_GRID);
      *abort_flag = 1;
    }
  }
  ds_csync();
  return *abort_flag == 0;
}

// this block's share of the sums of squares of h's rows (columns [H c/G, H (c+1)/G)), set 0: before the first layer
__device__ __forceinline__ void ds_first_ssq(const SxStreamArgs& a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = (int)((long long)a.H * blockIdx.x / gridDim.x), c1 = (int)((long long)a.H * (blockIdx.x + 1) / gridDim.x);
  if (warp < a.M) {
    float s = 0.f;
    for (int n = c0 + lane; n < c1; n += 32) {
      const float v = __ldcg(a.h + (size_t)warp * a.H + n);
      s += v * v;
    }
    s = warp_sum(s);
    if (lane == 0) a.ssq[(size_t)blockIdx.x * DS_MAX_ROWS + warp] = s;
  }
}

// bytes between the rows of x in shared memory: 64 modulo 128, so that the two rows a quarter-warp reads hit different banks
__device__ __forceinline__ int ds_xstride(int K) { return ((K * 2 + 127) / 128) * 128 + 64; }

// x = bf16(h * inv * gain) for all rows into shared memory; inv from the blocks' partial sums of
// squares (set `which`), added in block order by one warp per row
__device__ __forceinline__ void ds_build_x(const SxStreamArgs& a, int which, float eps, const float* __restrict__ gain,
                                           unsigned char* xs, int xstride, float* inv) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < a.M) {
    const float* p = a.ssq + ((size_t)which * gridDim.x) * DS_MAX_ROWS + warp;
    float s = 0.f;
    for (int c = lane; c < (int)gridDim.x; c += 32) s += __ldcg(p + (size_t)c * DS_MAX_ROWS);
    s = warp_sum(s);
    if (lane == 0) inv[warp] = rsqrtf(s / (float)a.H + eps);
  }
  ds_csync();
  const int n4 = a.H >> 2, total = a.M * n4;
  for (int i0 = threadIdx.x; i0 < total; i0 += 4 * DS_THREADS) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * DS_THREADS;
      if (i < total) v[u] = __ldcg(reinterpret_cast<const float4*>(a.h) + i);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * DS_THREADS;
      if (i < total) {
        const int b = i / n4, c = i - b * n4;
        const float4 gn = __ldg(reinterpret_cast<const float4*>(gain) + c);
        const float s = inv[b];
        uint2 o;
        o.x = pack_bf16(v[u].x * s * gn.x, v[u].y * s * gn.y);
        o.y = pack_bf16(v[u].z * s * gn.z, v[u].w * s * gn.w);
        *reinterpret_cast<uint2*>(xs + (size_t)b * xstride + (size_t)c * 8) = o;
      }
    }
  }
  ds_csync();
}

__device__ __forceinline__ void ds_wait_slot(uint32_t sa, uint4& va, uint4& vb) {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(DS_DEPTH - 1) : "memory");
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(va.x), "=r"(va.y), "=r"(va.z), "=r"(va.w) : "r"(sa));
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(vb.x), "=r"(vb.y), "=r"(vb.z), "=r"(vb.w) : "r"(sa + DS_THREADS * 16));
}

// ---------------------------------------------------------------------------------------
// A product of the normalised rows x (in shared memory), tile by tile.  epi: DS_EPI_QKV or DS_EPI_SILU.
// Every warp leaves its partial sums of a tile in `red`; after a group of tiles they are added in
// warp order and written out.
// ---------------------------------------------------------------------------------------
template <int HD>
__device__ __forceinline__ void ds_product_x(const SxStreamArgs& a, const DsGeo& geo, int epi, const unsigned char* xs,
                                             int xstride, unsigned char* ring, float* red, int red_tiles,
                                             DsWalk<HD>& wk, int& slot) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int M = a.M;
  const DsPlan pl = ds_plan(geo);
  const uint32_t ring0 = ds_smem(ring) + threadIdx.x * 16;
  const uint32_t x0 = ds_smem(xs) + g * xstride + t * 16;
  for (int g0 = 0; g0 < pl.ntiles; g0 += red_tiles) {
    const int tg = min(red_tiles, pl.ntiles - g0);
    for (int tt = 0; tt < tg; ++tt) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int st = pl.s_begin; st < pl.s_end; ++st) {
        const uint32_t sa = ring0 + slot * (2 * DS_THREADS * 16);
        uint4 va, vb, xv = make_uint4(0u, 0u, 0u, 0u);
        ds_wait_slot(sa, va, vb);
        wk.ask(a, sa);
        slot = slot + 1 == DS_DEPTH ? 0 : slot + 1;
        if (g < M) asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(xv.x), "=r"(xv.y), "=r"(xv.z), "=r"(xv.w) : "r"(x0 + st * 64));
        ds_mma(acc, va.x, vb.x, va.y, vb.y, xv.x, xv.y);
        ds_mma(acc, va.z, vb.z, va.w, vb.w, xv.z, xv.w);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) red[((tt * DS_WARPS + warp) * 4 + j) * 32 + lane] = acc[j];
    }
    ds_csync();
    for (int tt = warp; tt < tg; tt += DS_WARPS) {
      float c[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < DS_WARPS; ++w) v += red[((tt * DS_WARPS + w) * 4 + j) * 32 + lane];
        c[j] = v;
      }
      const int tile = g0 + tt;
      const int tile_r = pl.r0 + tile * pl.q;
      const int rows_in = tile == pl.ntiles - 1 ? pl.last_rows : pl.q;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int b = t * 2 + j;
        if (b >= M) continue;
        if (epi == DS_EPI_SILU) {
          if (g < rows_in) a.act[(size_t)b * a.I + tile_r + g] = __float2bfloat16_rn(c[j] / (1.f + expf(-c[j])) * c[2 + j]);
        } else {
          if (g < rows_in) a.qkv[(size_t)b * geo.rows + tile_r + g] = c[j];
          if (g + 8 < rows_in) a.qkv[(size_t)b * geo.rows + tile_r + g + 8] = c[2 + j];
        }
      }
    }
    ds_csync();                                    // red is free again
  }
}

// ---------------------------------------------------------------------------------------
// A product into h: h += x W^T for bf16 rows x in global memory, at most DS_MAXT tiles, k-major; the
// block's share of the new rows' sums of squares goes to set `ssq_set`.
// ---------------------------------------------------------------------------------------
template <int HD>
__device__ __forceinline__ void ds_product_h(const SxStreamArgs& a, const DsGeo& geo, const bf16* __restrict__ x, int ssq_set,
                                             unsigned char* ring, float* red, float* ssq_t, DsWalk<HD>& wk, int& slot) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int M = a.M, K = geo.K;
  const DsPlan pl = ds_plan(geo);
  const uint32_t ring0 = ds_smem(ring) + threadIdx.x * 16;
  const int tg = pl.ntiles;                          // <= DS_MAXT (the host checks)
  const uint4* xrow = reinterpret_cast<const uint4*>(x + (size_t)g * K + t * 8);      // + 4 per step

  float acc[DS_MAXT][4];
#pragma unroll
  for (int i = 0; i < DS_MAXT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  uint4 xq[DS_XPD];
#pragma unroll
  for (int u = 0; u < DS_XPD; ++u) {
    xq[u] = make_uint4(0u, 0u, 0u, 0u);
    if (pl.s_begin + u < pl.s_end && g < M) xq[u] = __ldcg(xrow + (size_t)(pl.s_begin + u) * 4);
  }
  for (int s = pl.s_begin; s < pl.s_end; s += DS_XPD) {
#pragma unroll
    for (int u = 0; u < DS_XPD; ++u) {
      const int st = s + u;
      if (st < pl.s_end) {
        const uint4 xv = xq[u];
        xq[u] = make_uint4(0u, 0u, 0u, 0u);
        if (st + DS_XPD < pl.s_end && g < M) xq[u] = __ldcg(xrow + (size_t)(st + DS_XPD) * 4);
#pragma unroll
        for (int tt = 0; tt < DS_MAXT; ++tt) {
          if (tt < tg) {
            const uint32_t sa = ring0 + slot * (2 * DS_THREADS * 16);
            uint4 va, vb;
            ds_wait_slot(sa, va, vb);
            wk.ask(a, sa);
            slot = slot + 1 == DS_DEPTH ? 0 : slot + 1;
            ds_mma(acc[tt], va.x, vb.x, va.y, vb.y, xv.x, xv.y);
            ds_mma(acc[tt], va.z, vb.z, va.w, vb.w, xv.z, xv.w);
          }
        }
      }
    }
  }
#pragma unroll
  for (int tt = 0; tt < DS_MAXT; ++tt)
    if (tt < tg) {
#pragma unroll
      for (int j = 0; j < 4; ++j) red[((tt * DS_WARPS + warp) * 4 + j) * 32 + lane] = acc[tt][j];
    }
  ds_csync();
  if (warp < tg) {
    const int tt = warp;
    float c[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < DS_WARPS; ++w) v += red[((tt * DS_WARPS + w) * 4 + j) * 32 + lane];
      c[j] = v;
    }
    const int tile_r = pl.r0 + tt * pl.q;
    const int rows_in = tt == pl.ntiles - 1 ? pl.last_rows : pl.q;
    float sq[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int b = t * 2 + j;
      if (b >= M) continue;
      if (g < rows_in) {
        float* p = a.h + (size_t)b * a.H + tile_r + g;
        const float v = __ldcg(p) + c[j];
        *p = v;
        sq[j] += v * v;
      }
      if (g + 8 < rows_in) {
        float* p = a.h + (size_t)b * a.H + tile_r + g + 8;
        const float v = __ldcg(p) + c[2 + j];
        *p = v;
        sq[j] += v * v;
      }
    }
    // this tile's share of the rows' sums of squares: over the 8 row lanes, in a fixed order
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      sq[j] += __shfl_xor_sync(0xffffffffu, sq[j], 4);
      sq[j] += __shfl_xor_sync(0xffffffffu, sq[j], 8);
      sq[j] += __shfl_xor_sync(0xffffffffu, sq[j], 16);
    }
    if (g == 0) {
      ssq_t[tt * DS_MAX_ROWS + t * 2] = sq[0];
      ssq_t[tt * DS_MAX_ROWS + t * 2 + 1] = sq[1];
    }
  }
  ds_csync();                                      // red is free again; ssq_t is whole
  if (threadIdx.x < DS_MAX_ROWS) {
    float s = 0.f;
    for (int tt = 0; tt < tg; ++tt) s += ssq_t[tt * DS_MAX_ROWS + threadIdx.x];
    a.ssq[((size_t)ssq_set * gridDim.x + blockIdx.x) * DS_MAX_ROWS + threadIdx.x] = s;
  }
}

// ---------------------------------------------------------------------------------------
// phase 2: one warp per (token, head of the fused projection).  A lane owns the rotation pairs
// p = 64 k + 2 lane + {0, 1} (the whole head is rotated: rotary_dim == HD).
// ---------------------------------------------------------------------------------------
template <int HD>
__device__ __forceinline__ void ds_prepare(const SxStreamArgs& a, const SxStreamLayer& L) {
  constexpr int PQ = (HD / 2 + 63) / 64, half = HD / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = a.nh + 2 * a.nkv;
  const int items = a.M * heads;
  const int* bt = a.block_table[L.group];
  const int maxp = a.maxp[L.group];
  for (int item = blockIdx.x * DS_WARPS + warp; item < items; item += gridDim.x * DS_WARPS) {
    const int b = item / heads, head = item % heads;
    const bool is_q = head < a.nh, is_k = !is_q && head < a.nh + a.nkv;
    const int kvh = is_q ? 0 : (is_k ? head - a.nh : head - a.nh - a.nkv);
    const float* src = a.qkv + (size_t)b * heads * HD + (size_t)head * HD;
    const int pos = a.positions[b];
    bf16* dst;
    if (is_q) {
      dst = a.q + ((size_t)b * a.nh + head) * HD;
    } else {
      if (!L.write_cache) continue;
      const int page = bt[(size_t)b * maxp + (pos >> 6)];
      if (page < 0 || page >= L.n_pages) continue;          // the host guarantees a page; never write outside
      dst = (is_k ? L.k_pages : L.v_pages) + (((size_t)page * a.nkv + kvh) * SX_PAGE + (pos & 63)) * HD;
    }
    if (!is_q && !is_k) {
      for (int i = lane * 4; i < HD; i += 128) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + i));
        uint2 o;
        o.x = pack_bf16(v.x, v.y);
        o.y = pack_bf16(v.z, v.w);
        *reinterpret_cast<uint2*>(dst + i) = o;
      }
      continue;
    }
    const float* w = is_q ? L.g_q : L.g_k;
    float2 x1[PQ], x2[PQ];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < PQ; ++k) {
      const int p = 64 * k + 2 * lane;
      x1[k] = x2[k] = make_float2(0.f, 0.f);
      if (p < half) {
        x1[k] = __ldcg(reinterpret_cast<const float2*>(src + p));
        x2[k] = __ldcg(reinterpret_cast<const float2*>(src + p + half));
        ss += x1[k].x * x1[k].x + x1[k].y * x1[k].y + x2[k].x * x2[k].x + x2[k].y * x2[k].y;
      }
    }
    float inv = 1.f;
    if (w) inv = rsqrtf(warp_sum(ss) / (float)HD + L.eps_qk);
#pragma unroll
    for (int k = 0; k < PQ; ++k) {
      const int p = 64 * k + 2 * lane;
      if (p < half) {
        float cs[2] = {1.f, 1.f}, sn[2] = {0.f, 0.f}, g1[2] = {1.f, 1.f}, g2[2] = {1.f, 1.f};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (L.inv_freq) sincosf((float)pos * __ldg(L.inv_freq + p + j), &sn[j], &cs[j]);
          if (w) { g1[j] = __ldg(w + p + j); g2[j] = __ldg(w + p + j + half); }
        }
        const float a0 = x1[k].x * inv * g1[0], a1 = x1[k].y * inv * g1[1];
        const float b0 = x2[k].x * inv * g2[0], b1 = x2[k].y * inv * g2[1];
        *reinterpret_cast<uint32_t*>(dst + p) = pack_bf16(a0 * cs[0] - b0 * sn[0], a1 * cs[1] - b1 * sn[1]);
        *reinterpret_cast<uint32_t*>(dst + p + half) = pack_bf16(a0 * sn[0] + b0 * cs[0], a1 * sn[1] + b1 * cs[1]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// phase 3: attention of the step's tokens over the cache, by warps 0..3 of every block.
// An item is (split of a sequence's pages, kv head, sequence); the scheme is that of
// attn_decode_kernel (attention.cu) with its in-kernel merge by the last block to finish.
// ---------------------------------------------------------------------------------------
template <int HD>
__device__ __forceinline__ void ds_attention(const SxStreamArgs& a, const SxStreamLayer& L, unsigned char* smem, int* s_last) {
  using AL = AtLayout<HD>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int G = a.nh / a.nkv, n_splits = a.n_splits;
  const int items = a.M * a.nkv * n_splits;
  const int window = L.window;
  const float scale_log2 = L.scale_log2;
  const int maxp = a.maxp[L.group];
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int split = item % n_splits, kvh = (item / n_splits) % a.nkv, seq = item / (n_splits * a.nkv);
    const int len = a.seq_lens[seq];
    const int pos = len - 1;
    const int lo = window > 0 ? max(0, len - window) : 0;
    const int p_first = lo >> 6, p_end = (len + 63) >> 6;
    const int total = p_end - p_first;
    const int per = (total + n_splits - 1) / n_splits;
    const int p0 = p_first + split * per, p1 = min(p_end, p0 + per);
    const int* bt = a.block_table[L.group] + (size_t)seq * maxp;

    uint32_t qf[HD / 16][4];
    {
      const bf16* qb = a.q + ((size_t)seq * a.nh + (size_t)kvh * G) * HD;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const int c = ks * 16 + 2 * t;
        qf[ks][0] = g < G ? __ldcg(reinterpret_cast<const unsigned*>(qb + (size_t)g * HD + c)) : 0u;
        qf[ks][1] = g + 8 < G ? __ldcg(reinterpret_cast<const unsigned*>(qb + (size_t)(g + 8) * HD + c)) : 0u;
        qf[ks][2] = g < G ? __ldcg(reinterpret_cast<const unsigned*>(qb + (size_t)g * HD + c + 8)) : 0u;
        qf[ks][3] = g + 8 < G ? __ldcg(reinterpret_cast<const unsigned*>(qb + (size_t)(g + 8) * HD + c + 8)) : 0u;
      }
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    const int npages = max(0, p1 - p0);
#pragma unroll
    for (int st = 0; st < AT_STAGES_DECODE - 1; ++st) {
      if (st < npages) load_page<HD>(smem + st * AL::STAGE, L.k_pages, L.v_pages, bt[p0 + st], kvh, a.nkv, min(64, len - (p0 + st) * 64));
      cp_async_commit();
    }
    for (int i = 0; i < npages; ++i) {
      cp_async_wait<AT_STAGES_DECODE - 2>();
      ds_tsync();
      const int nx = i + AT_STAGES_DECODE - 1;
      if (nx < npages)
        load_page<HD>(smem + (nx % AT_STAGES_DECODE) * AL::STAGE, L.k_pages, L.v_pages, bt[p0 + nx], kvh, a.nkv, min(64, len - (p0 + nx) * 64));
      cp_async_commit();
      const unsigned char* st = smem + (i % AT_STAGES_DECODE) * AL::STAGE;
      const int jb = (p0 + i) * 64;
      if (jb + 63 > pos || (window > 0 && jb <= pos - window))
        attend_tile<HD, 2, true>(qf, st, st + AL::TILE, warp * 16, jb, pos, pos, window, scale_log2, m, l, o);
      else
        attend_tile<HD, 2, false>(qf, st, st + AL::TILE, warp * 16, jb, pos, pos, window, scale_log2, m, l, o);
    }
    cp_async_wait<0>();
    ds_tsync();

    m[0] *= scale_log2;
    m[1] *= scale_log2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
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
    ds_tsync();
    for (int idx = threadIdx.x; idx < G * HD; idx += AT_THREADS) {
      const int r = idx / HD, d = idx % HD;
      float Mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) Mx = fmaxf(Mx, wml[(w * 16 + r) * 2]);
      float Lsum = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = wml[(w * 16 + r) * 2];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - Mx);
        Lsum += wml[(w * 16 + r) * 2 + 1] * f;
        O += wo[(w * 16 + r) * HD + d] * f;
      }
      const int head = kvh * G + r;
      if (n_splits == 1) {
        a.attn[((size_t)seq * a.nh + head) * HD + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
      } else {
        const size_t pi = ((size_t)seq * a.nh + head) * n_splits + split;
        a.part_o[pi * HD + d] = O;
        if (d == 0) { a.part_ml[pi * 2] = Mx; a.part_ml[pi * 2 + 1] = Lsum; }
      }
    }
    if (n_splits == 1) { ds_tsync(); continue; }

    // the block that finishes last for this (sequence, kv head) merges all splits, in split order
    __threadfence();
    ds_tsync();
    if (threadIdx.x == 0) {
      int* c = a.counters + (size_t)seq * a.nkv + kvh;
      const int done = atomicAdd(c, 1);
      *s_last = (done == n_splits - 1);
      if (*s_last) *c = 0;
    }
    ds_tsync();
    if (!*s_last) { ds_tsync(); continue; }
    __threadfence();
    float* fac = reinterpret_cast<float*>(smem);           // [G][n_splits] maxima, then weights
    float* ls = fac + G * n_splits;
    float* gl = ls + G * n_splits;
    for (int idx = threadIdx.x; idx < G * n_splits; idx += AT_THREADS) {
      const int r = idx / n_splits, i = idx % n_splits;
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml) + ((size_t)seq * a.nh + kvh * G + r) * n_splits + i);
      fac[idx] = ml.x;
      ls[idx] = ml.y;
    }
    ds_tsync();
    for (int r = warp; r < G; r += 4) {
      float Mx = -INFINITY;
      for (int i = lane; i < n_splits; i += 32) Mx = fmaxf(Mx, fac[r * n_splits + i]);
      Mx = warp_max(Mx);
      float Ls = 0.f;
      for (int i = lane; i < n_splits; i += 32) {
        const float mi = fac[r * n_splits + i];
        const float f = (mi == -INFINITY) ? 0.f : exp2f(mi - Mx);
        fac[r * n_splits + i] = f;
        Ls += ls[r * n_splits + i] * f;
      }
      Ls = warp_sum(Ls);
      if (lane == 0) gl[r] = Ls;
    }
    ds_tsync();
    for (int idx = threadIdx.x; idx < G * HD; idx += AT_THREADS) {
      const int r = idx / HD, d = idx % HD;
      const size_t row = (size_t)seq * a.nh + kvh * G + r;
      const float* po = a.part_o + row * n_splits * HD + d;
      const float* f = fac + r * n_splits;
      float O = 0.f;
#pragma unroll 8
      for (int i = 0; i < n_splits; ++i) O += __ldcg(po + (size_t)i * HD) * f[i];
      const float Ls = gl[r];
      a.attn[row * HD + d] = __float2bfloat16_rn(Ls > 0.f ? O / Ls : 0.f);
    }
    ds_tsync();                                            // the stage buffers are free for the next item
  }
}

// ---------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(DS_THREADS, 1) decode_stream_kernel(const __grid_constant__ SxStreamArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* ring = smem_raw;
  unsigned char* shared = ring + DS_RING_BYTES;
  float* inv = reinterpret_cast<float*>(shared + DS_SHARED_BYTES);         // [8]
  float* ssq_t = inv + DS_MAX_ROWS;                                        // [DS_MAXT][8]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ssq_t + DS_MAXT * DS_MAX_ROWS);
  int* s_last = const_cast<int*>(abort_flag) + 1;
  const int warp = threadIdx.x >> 5;
  // products of normalised rows: x at the start of `shared`, the warps' partial sums behind it
  const int xstride = ds_xstride(a.H);
  const int x_bytes = ((a.M * xstride + 127) / 128) * 128;
  float* red_x = reinterpret_cast<float*>(shared + x_bytes);
  const int red_tiles = (DS_SHARED_BYTES - x_bytes) / (DS_WARPS * 4 * 32 * 4);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *s_last = 0;
  }
  // the first DS_DEPTH elements of this thread's walk are asked for before anything else
  DsWalk<HD> wk;
  wk.init(a);
  {
    const uint32_t ring0 = ds_smem(ring) + threadIdx.x * 16;
#pragma unroll 1
    for (int i = 0; i < DS_DEPTH; ++i) wk.ask(a, ring0 + i * (2 * DS_THREADS * 16));
  }
  int slot = 0;
  unsigned epoch = 0;
  __syncthreads();
  ds_first_ssq(a);
  bool ok = ds_grid_sync(a, epoch, abort_flag);

  for (int li = 0; li < a.n_layers && ok; ++li) {
    const SxStreamLayer& L = a.layers[li];
#pragma unroll 1
    for (int half = 0; half < 2 && ok; ++half) {
      // a product of normalised rows: q/k/v, or gate/up
      ds_stamp(a, li, half * 8 + 0);
      ds_build_x(a, half, half ? L.eps_post : L.eps_in, half ? L.g_post : L.g_in, shared, xstride, inv);
      ds_stamp(a, li, half * 8 + 1);
      ds_product_x<HD>(a, ds_geo<HD>(a, L, half * 2), half ? DS_EPI_SILU : DS_EPI_QKV, shared, xstride, ring, red_x, red_tiles, wk, slot);
      ds_stamp(a, li, half * 8 + 2);
      if (!(ok = ds_grid_sync(a, epoch, abort_flag))) break;
      ds_stamp(a, li, half * 8 + 3);
      if (half == 0) {
        ds_prepare<HD>(a, L);
        ds_stamp(a, li, 4);
        if (!(ok = ds_grid_sync(a, epoch, abort_flag))) break;
        ds_stamp(a, li, 5);
        if (warp < 4) ds_attention<HD>(a, L, shared, s_last);
        ds_stamp(a, li, 6);
        if (!(ok = ds_grid_sync(a, epoch, abort_flag))) break;
        ds_stamp(a, li, 7);
      }
      // a product into h: o (sums of squares for the second norm), or down (for the next layer's first norm)
      ds_product_h<HD>(a, ds_geo<HD>(a, L, half * 2 + 1), half ? a.act : a.attn, half ? 0 : 1, ring,
                       reinterpret_cast<float*>(shared), ssq_t, wk, slot);
      ds_stamp(a, li, half ? 12 : 13);
      if (!(li + 1 == a.n_layers && half == 1)) ok = ds_grid_sync(a, epoch, abort_flag);
      ds_stamp(a, li, half ? 14 : 15);
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");        // no copy may be in flight when the block ends
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static size_t ds_align(size_t v) { return (v + 255) & ~(size_t)255; }

#define DS_MAX_BLOCKS 512
struct DsScratch {
  size_t qkv, q, part_o, part_ml, attn, act, ssq, counters, barrier, status, total;
};
// the layout holds DS_MAX_ROWS rows whatever M is, so one piece of memory serves every launch;
// max_items bounds M * nkv * n_splits of launches with more than one split
static DsScratch ds_scratch_layout(int nh, int nkv, int hd, int I, int max_items) {
  const size_t R = DS_MAX_ROWS, G = nh / nkv;
  DsScratch s;
  size_t o = 0;
  s.counters = o; o = ds_align(o + R * nkv * sizeof(int));
  s.barrier = o; o = ds_align(o + sizeof(unsigned));
  s.status = o; o = ds_align(o + sizeof(int));
  s.ssq = o; o = ds_align(o + (size_t)2 * DS_MAX_BLOCKS * R * sizeof(float));
  s.qkv = o; o = ds_align(o + R * (nh + 2 * nkv) * hd * sizeof(float));
  s.q = o; o = ds_align(o + R * nh * hd * sizeof(bf16));
  s.part_o = o; o = ds_align(o + (size_t)max_items * G * hd * sizeof(float));
  s.part_ml = o; o = ds_align(o + (size_t)max_items * G * 2 * sizeof(float));
  s.attn = o; o = ds_align(o + R * nh * hd * sizeof(bf16));
  s.act = o; o = ds_align(o + R * I * sizeof(bf16));
  s.total = o;
  return s;
}

// blocks of the cooperative grid on the current device (0: the kernel does not fit)
template <int HD>
static int ds_grid_blocks() {
  auto kern = decode_stream_kernel<HD>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DS_SMEM) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int dev = 0, sms = 0, per = 0, coop = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  if (!coop) return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, kern, DS_THREADS, DS_SMEM) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return per > 0 ? sms : 0;
}

extern "C" int sx_decode_stream_blocks(int hd) {
  static int cached[2] = {-1, -1};
  const int which = hd == 128 ? 0 : (hd == 64 ? 1 : -1);
  if (which < 0) return 0;
  if (cached[which] < 0) cached[which] = which == 0 ? ds_grid_blocks<128>() : ds_grid_blocks<64>();
  return cached[which];
}

// bytes of scratch a launch with these sizes needs; the caller hands over that much ZEROED memory
// once and keeps it for all launches (the kernel leaves the counters zero; the barrier word is
// cleared on the stream before every launch)
extern "C" unsigned long long sx_decode_stream_scratch_bytes(int nh, int nkv, int hd, int I, int max_items) {
  if (nkv <= 0 || nh % nkv || max_items < 0) return 0;
  return ds_scratch_layout(nh, nkv, hd, I, max_items).total;
}

// h [M, H] float32 is updated in place by n_layers layer runs.  layers: device array of SxStreamLayer.
// block_tables: host array of 4 device pointers (unused groups null), maxp: host array of 4 ints.
// prof: null, or device memory for blocks * n_layers * 16 time stamps (a tuning aid).
// Refuses (SX_ERR_SIZE) what the kernel does not take; the caller then runs the layers kernel by kernel.
extern "C" int sx_decode_stream(const void* layers, int n_layers, int M, int H, int nh, int nkv, int hd, int I,
                                float* h, const int* positions, const int* seq_lens, const void* const* block_tables,
                                const int* maxp, void* scratch, unsigned long long scratch_bytes, int max_items,
                                int n_splits, void* prof, cudaStream_t stream) {
  if (n_layers <= 0 || M <= 0) return 0;
  if (M > DS_MAX_ROWS || (hd != 128 && hd != 64) || nkv <= 0 || nh % nkv || nh / nkv > 16) return SX_ERR_SIZE;
  if ((H & 31) || (I & 31) || ((nh * hd) & 31) || H < 32) return SX_ERR_SIZE;
  // x of the products of normalised rows stays in shared memory, with room for one tile's partial sums behind it
  if ((size_t)DS_MAX_ROWS * (((H * 2 + 127) / 128) * 128 + 64) + 128 + DS_WARPS * 4 * 32 * 4 > DS_SHARED_BYTES) return SX_ERR_SIZE;
  if (n_splits < 1 || n_splits > 512 || (n_splits > 1 && (long long)M * nkv * n_splits > max_items)) return SX_ERR_SIZE;
  if (((size_t)(nh / nkv) * n_splits * 2 + nh / nkv) * sizeof(float) > DS_SHARED_BYTES) return SX_ERR_SIZE;
  const int blocks = sx_decode_stream_blocks(hd);
  if (blocks <= 0 || blocks > DS_MAX_BLOCKS) return SX_ERR_SIZE;
  if ((H + blocks - 1) / blocks > 16 * DS_MAXT) return SX_ERR_SIZE;      // the products into h keep all their tiles live
  const DsScratch lay = ds_scratch_layout(nh, nkv, hd, I, max_items);
  if (scratch_bytes < lay.total || ((uintptr_t)scratch & 255)) return SX_ERR_SIZE;
  unsigned char* sc = (unsigned char*)scratch;

  SxStreamArgs a;
  a.layers = (const SxStreamLayer*)layers;
  a.n_layers = n_layers; a.M = M; a.H = H; a.nh = nh; a.nkv = nkv; a.I = I; a.n_splits = n_splits; a.pad0 = 0;
  a.h = h; a.positions = positions; a.seq_lens = seq_lens;
  for (int i = 0; i < 4; ++i) { a.block_table[i] = (const int*)block_tables[i]; a.maxp[i] = maxp[i]; }
  a.qkv = (float*)(sc + lay.qkv); a.q = (bf16*)(sc + lay.q);
  a.part_o = (float*)(sc + lay.part_o); a.part_ml = (float*)(sc + lay.part_ml);
  a.attn = (bf16*)(sc + lay.attn); a.act = (bf16*)(sc + lay.act); a.ssq = (float*)(sc + lay.ssq);
  a.prof = (unsigned long long*)prof;
  a.counters = (int*)(sc + lay.counters); a.barrier = (unsigned*)(sc + lay.barrier); a.status = (int*)(sc + lay.status);

  cudaError_t e = cudaMemsetAsync(a.barrier, 0, sizeof(unsigned), stream);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(DS_THREADS);
  cfg.dynamicSmemBytes = DS_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (hd == 128) return (int)cudaLaunchKernelEx(&cfg, decode_stream_kernel<128>, a);
  return (int)cudaLaunchKernelEx(&cfg, decode_stream_kernel<64>, a);
}

// the status word inside the scratch memory: 0, or 3 when a wait at a grid barrier ran out
extern "C" int sx_decode_stream_status(const void* scratch, int nh, int nkv, int hd, int I, int max_items, int* host_value) {
  const DsScratch lay = ds_scratch_layout(nh, nkv, hd, I, max_items);
  return (int)cudaMemcpy(host_value, (const unsigned char*)scratch + lay.status, sizeof(int), cudaMemcpyDeviceToHost);
}
