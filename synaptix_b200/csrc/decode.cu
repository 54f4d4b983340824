// Weight-streaming matrix products for decode steps (few rows of activations, bfloat16).
//
//   y[b, n] = sum_k x[b, k] * W[n, k]      b < M <= 16,  W [N, K] row-major,  32-bit accumulation
//
// A decode step reads every weight once, so these kernels are bound by HBM, not by math.
// The reference has a warp-per-row GEMV for one row of activations only and falls to a 32x32
// GEMM tile for more (crates/synaptix-kernels-cuda/src/best_cu/gemv/mma_gemv.cu:19-133,
// crates/synaptix-kernels-cuda/src/cuda_backend.rs:738-754); here one kernel serves 1..16 rows
// and reads W once for all of them.
//
// Shape of the kernel.  The roles of the operands are swapped: 16 rows of W are the M side of
// mma.sync.m16n8k16 and 8 rows of activations its N side, so a warp owns 16 output columns for
// all M activation rows.  Every thread loads 16 contiguous bytes of a W row (8 k-values) straight
// from global memory into the registers of two MMAs: since a dot product does not care in which
// order k is visited, the k-values that thread (g, t) holds are declared to be "its" fragment
// columns, and the activation fragment is loaded with the same map.  No shared-memory staging,
// no ldmatrix: the only traffic is W once from HBM and x from L1/L2.
//   warp tile   16 rows of W x (K / KS) of k, KS warps of a block split K and add up through
//               shared memory in warp order (fixed order, no atomics)
//   epilogues   bf16 or f32 store;  SiLU(gate)*up for a stacked [gate; up] matrix, where a
//               warp's 16 rows are 8 gate rows and the 8 matching up rows;
//               optional RMSNorm prologue: x = rmsnorm(h + delta) * gain computed per block
//               (h float32), so that the norm needs no kernel and no round trip of x.
//   RMSNorm split between producer and consumer (SkNorm): the product whose result is a branch of the
//               residual stream adds it into h (float32, in place), writes x~ = bf16(h * gain) of the NEXT norm
//               and one partial sum of squares of h per row and 16-column tile (EPI_RESID); the product that
//               consumes x~ multiplies its own results by rsqrt(sum of the partials / K + eps) per row.  A row's
//               norm then costs no kernel, no pass over h and no reduction in anybody's critical path.
#include "common.cuh"

#define SK_WARPS 8
#define XS_ROWS 2          // rows of activations the norm prologue takes
#define SK_THREADS (SK_WARPS * 32)
#define SK_DEPTH 4          // steps (of 2 x 16 bytes) every thread keeps in flight; 4 measured best (more blocks per SM beat deeper rings)

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SILU_MUL = 2, EPI_RESID = 3 };

struct SkNorm {
  // consumer side: the rows of x lack the factor rsqrt(sum_i ssq_in[b * n_in + i] / K + eps_in); null: they do not
  const float* ssq_in;
  int n_in;
  float eps_in;
  // producer side (EPI_RESID): h [M, N] += result; out = bf16(h * gain_next); ssq_out [M, ceil(N / 16)]
  float* h_io;
  const float* gain_next;
  float* ssq_out;
};

// NT: activation rows in tiles of 8 (M <= 8 NT);  KS: warps that split K;  RT = SK_WARPS / KS row tiles per block
// XS: activations are read from shared memory (filled by the norm prologue) instead of global memory
template <int NT, int KS, int EPI, bool XS>
__global__ void __launch_bounds__(KS > SK_WARPS ? KS * 32 : SK_THREADS) skinny_gemm_kernel(
    const bf16* __restrict__ x, const bf16* __restrict__ W, void* __restrict__ out, int M, int N, int K,
    // norm prologue (XS only): x = rmsnorm(h_in + delta) * gain; block 0 writes h_in + delta to h_out
    const float* __restrict__ h_in, const bf16* __restrict__ delta, float* __restrict__ h_out,
    const float* __restrict__ gain, float eps, const SkNorm nrm) {
  constexpr int WARPS = KS > SK_WARPS ? KS : SK_WARPS;      // 16 warps split K for matrices with few rows
  constexpr int THREADS = WARPS * 32;
  constexpr int RT = WARPS / KS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* red = reinterpret_cast<float*>(smem_raw);                        // [WARPS][NT][4][32]
  bf16* xs = reinterpret_cast<bf16*>(smem_raw + (KS > 1 ? WARPS * NT * 4 * 32 * sizeof(float) : 0));  // [NT*8][K]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rt = warp / KS, ks = warp % KS;

  // rows of W this warp owns
  const int tile = blockIdx.x * RT + rt;
  int row_lo, row_hi;          // W rows behind fragment rows g and g + 8
  bool tile_ok;
  if (EPI == EPI_SILU_MUL) {   // N = 2 I stacked [gate; up]; the tile is 8 gate rows and their up rows
    const int I = N / 2;
    const int i = tile * 8 + g;
    tile_ok = tile * 8 < I;
    row_lo = min(i, I - 1);
    row_hi = I + min(i, I - 1);
  } else {
    tile_ok = tile * 16 < N;
    row_lo = min(tile * 16 + g, N - 1);
    row_hi = min(tile * 16 + g + 8, N - 1);
  }
  const int nsteps = K >> 5;                       // 32 k-values a step
  const int per = (nsteps + KS - 1) / KS;
  const int s_begin = ks * per, s_end = min(nsteps, s_begin + per);
  const bf16* wlo = W + (size_t)row_lo * K + t * 8;
  const bf16* whi = W + (size_t)row_hi * K + t * 8;
  // Every thread keeps SK_DEPTH steps of its own weights in flight, copied asynchronously
  // (cp.async, 16 bytes) into a ring in shared memory that only this thread reads back: no
  // registers are held while the data travels, no barrier is needed, and all of a warp's first
  // SK_DEPTH steps are asked for in ONE round trip to HBM instead of one round per batch of loads.
  // The first steps are asked for before anything else, so that HBM is busy during the prologue.
  uint4* ring = reinterpret_cast<uint4*>(smem_raw + (KS > 1 ? WARPS * NT * 4 * 32 * sizeof(float) : 0) +
                                         (XS ? (size_t)XS_ROWS * K * sizeof(bf16) : 0));      // [SK_DEPTH][2][THREADS]
  const uint32_t ring_base = (uint32_t)__cvta_generic_to_shared(ring) + threadIdx.x * 16;
  auto ask = [&](int step, int slot) {
    if (step < s_end && tile_ok) {
      const uint32_t dst = ring_base + slot * (2 * THREADS * 16);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(wlo + (size_t)step * 32) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + THREADS * 16), "l"(whi + (size_t)step * 32) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");        // one group per step, empty or not
  };
#pragma unroll
  for (int i = 0; i < SK_DEPTH; ++i) ask(s_begin + i, i);
  // the norm's gains are weights too: fetched before the wait
  float4 gn[XS ? 4 : 1];
  if (XS) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = threadIdx.x + k * THREADS;
      gn[k] = i < (K >> 2) ? __ldg(reinterpret_cast<const float4*>(gain) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  // the next norm's gains of this warp's columns (EPI_RESID) are weights as well
  float gnext[2] = {0.f, 0.f};
  if (EPI == EPI_RESID && tile_ok) {
    gnext[0] = __ldg(nrm.gain_next + row_lo);
    gnext[1] = __ldg(nrm.gain_next + row_hi);
  }
  pdl_wait();          // the weights depend on no earlier kernel; everything below may
  pdl_trigger();

  // The rows' factors (consumer side of SkNorm): one warp per row adds the partial sums, lane i those at i, i + 32,
  // ... in that order, then the lanes' butterfly.  The partial sums are asked for here and added after the main
  // loop, so that the trip to L2 is not in the way of the first weights.
  __shared__ float row_factor[NT * 8];
  constexpr int PRE = 8;
  float pre[PRE];
  const bool pre_ok = nrm.ssq_in && nrm.n_in <= 32 * PRE && M <= WARPS;
  if (pre_ok && warp < M) {
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int idx = lane + 32 * i;
      pre[i] = idx < nrm.n_in ? nrm.ssq_in[(size_t)warp * nrm.n_in + idx] : 0.f;
    }
  }

  if (XS) {
    // RMSNorm prologue by the whole block, one row after the other, the row held in registers:
    // one round of loads, one reduction, 32-bit throughout.  K <= 4096, M <= XS_ROWS.
    __shared__ float xs_red[WARPS];
    const int n4 = K >> 2;
    for (int b = 0; b < M; ++b) {
      const float4* hr = reinterpret_cast<const float4*>(h_in + (size_t)b * K);
      const uint2* dr = delta ? reinterpret_cast<const uint2*>(delta + (size_t)b * K) : nullptr;
      float4 v[4];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * THREADS;
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
          v[k] = hr[i];
          if (dr) {
            const uint2 d = dr[i];
            const __nv_bfloat162 d0 = *reinterpret_cast<const __nv_bfloat162*>(&d.x);
            const __nv_bfloat162 d1 = *reinterpret_cast<const __nv_bfloat162*>(&d.y);
            v[k].x += __low2float(d0); v[k].y += __high2float(d0); v[k].z += __low2float(d1); v[k].w += __high2float(d1);
          }
          ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
      }
      ss = warp_sum(ss);
      __syncthreads();                              // xs_red of the previous row has been read
      if (lane == 0) xs_red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) tot += xs_red[w];
      const float inv = rsqrtf(tot / (float)K + eps);
      bf16* xr = xs + (size_t)b * K;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * THREADS;
        if (i < n4) {
          if (blockIdx.x == 0 && h_out) reinterpret_cast<float4*>(h_out + (size_t)b * K)[i] = v[k];
          __nv_bfloat162 o0 = __floats2bfloat162_rn(v[k].x * inv * gn[k].x, v[k].y * inv * gn[k].y);
          __nv_bfloat162 o1 = __floats2bfloat162_rn(v[k].z * inv * gn[k].z, v[k].w * inv * gn[k].w);
          uint2 o;
          o.x = *reinterpret_cast<uint32_t*>(&o0); o.y = *reinterpret_cast<uint32_t*>(&o1);
          reinterpret_cast<uint2*>(xr)[i] = o;
        }
      }
    }
    __syncthreads();
  }

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  if (tile_ok) {
    int slot = 0;
    auto step = [&](int sc, const uint4 (&xv)[NT]) {
      asm volatile("cp.async.wait_group %0;\n" ::"n"(SK_DEPTH - 1) : "memory");   // step sc has landed
      const uint4 va = ring[(slot * 2) * THREADS + threadIdx.x];
      const uint4 vb = ring[(slot * 2 + 1) * THREADS + threadIdx.x];
      ask(sc + SK_DEPTH, slot);                       // the slot is free again: next step into it
      slot = slot + 1 == SK_DEPTH ? 0 : slot + 1;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma_bf16_16816(acc[nt], va.x, vb.x, va.y, vb.y, xv[nt].x, xv[nt].y);
        mma_bf16_16816(acc[nt], va.z, vb.z, va.w, vb.w, xv[nt].z, xv[nt].w);
      }
    };
    // Activations from global memory (up to 16 rows: the registers allow it) are asked for XD steps ahead into a
    // ring of registers, always before the wait for a step's weights: a step's 64 bytes of a row are a trip to L2
    // that would otherwise stand between the arrival of the weights and their use.
    constexpr bool XAHEAD = !XS && NT <= 2;
    constexpr int XD = 1;        // steps ahead; 4 (as deep as the weights) measured slower: 475 against 489 tok/s at one row
    if (XAHEAD) {
      uint4 xr[XD][NT];
      auto ask_x = [&](int sc, uint4 (&dst)[NT]) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int b = nt * 8 + g;
          dst[nt] = make_uint4(0u, 0u, 0u, 0u);
          if (sc < s_end && b < M) dst[nt] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * K + sc * 32 + t * 8));
        }
      };
#pragma unroll
      for (int u = 0; u < XD; ++u) ask_x(s_begin + u, xr[u]);
      for (int sc = s_begin; sc < s_end; sc += XD) {
#pragma unroll
        for (int u = 0; u < XD; ++u) {
          if (sc + u < s_end) {
            uint4 xc[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) xc[nt] = xr[u][nt];
            ask_x(sc + u + XD, xr[u]);
            step(sc + u, xc);
          }
        }
      }
    } else {
      for (int sc = s_begin; sc < s_end; ++sc) {
        uint4 xv[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int b = nt * 8 + g;
          xv[nt] = make_uint4(0u, 0u, 0u, 0u);
          if (XS) { if (b < M) xv[nt] = *reinterpret_cast<const uint4*>(xs + (size_t)b * K + sc * 32 + t * 8); }
          else if (b < M) xv[nt] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b * K + sc * 32 + t * 8));
        }
        step(sc, xv);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");

  if (nrm.ssq_in) {
    if (pre_ok) {
      if (warp < M) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < PRE; ++i) ss += pre[i];
        ss = warp_sum(ss);
        if (lane == 0) row_factor[warp] = rsqrtf(ss / (float)K + nrm.eps_in);
      }
    } else {
      for (int b = warp; b < M; b += WARPS) {
        float ss = 0.f;
        for (int i = lane; i < nrm.n_in; i += 32) ss += nrm.ssq_in[(size_t)b * nrm.n_in + i];
        ss = warp_sum(ss);
        if (lane == 0) row_factor[b] = rsqrtf(ss / (float)K + nrm.eps_in);
      }
    }
    if (KS == 1) __syncthreads();      // with KS > 1 the barrier of the add-up below orders it
  }

  // EPI_RESID: the residual stream's values of this warp's results, asked for before the add-up hides the trip
  float hv[EPI == EPI_RESID ? NT : 1][4];
  if (EPI == EPI_RESID && ks == 0 && tile_ok) {
    const int n0 = tile * 16 + g, n1 = n0 + 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int b = nt * 8 + t * 2 + j;
        hv[nt][j] = (b < M && n0 < N) ? nrm.h_io[(size_t)b * N + n0] : 0.f;
        hv[nt][2 + j] = (b < M && n1 < N) ? nrm.h_io[(size_t)b * N + n1] : 0.f;
      }
  }

  // add up the KS partial sums of a row tile in warp order
  if (KS > 1) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) red[((warp * NT + nt) * 4 + j) * 32 + lane] = acc[nt][j];
    __syncthreads();
    if (ks != 0) return;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = acc[nt][j];
        for (int w = 1; w < KS; ++w) v += red[(((warp + w) * NT + nt) * 4 + j) * 32 + lane];
        acc[nt][j] = v;
      }
  }
  if (!tile_ok) return;

  // fragment element (j): row g (j < 2) or g + 8 of the tile, activation row nt*8 + t*2 + (j & 1)
  if (nrm.ssq_in) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int b = nt * 8 + t * 2 + j;
        const float f = b < M ? row_factor[b] : 0.f;
        acc[nt][j] *= f;
        acc[nt][2 + j] *= f;
      }
  }
  if (EPI == EPI_RESID) {
    const int n0 = tile * 16 + g, n1 = n0 + 8;
    const int tiles = (N + 15) >> 4;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int b = nt * 8 + t * 2 + j;             // uniform over the 8 lanes that share t
        float ss = 0.f;
        if (b < M) {
          if (n0 < N) {
            const float v = hv[nt][j] + acc[nt][j];
            nrm.h_io[(size_t)b * N + n0] = v;
            reinterpret_cast<bf16*>(out)[(size_t)b * N + n0] = __float2bfloat16_rn(v * gnext[0]);
            ss += v * v;
          }
          if (n1 < N) {
            const float v = hv[nt][2 + j] + acc[nt][2 + j];
            nrm.h_io[(size_t)b * N + n1] = v;
            reinterpret_cast<bf16*>(out)[(size_t)b * N + n1] = __float2bfloat16_rn(v * gnext[1]);
            ss += v * v;
          }
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        ss += __shfl_xor_sync(0xffffffffu, ss, 8);
        ss += __shfl_xor_sync(0xffffffffu, ss, 16);
        if (g == 0 && b < M) nrm.ssq_out[(size_t)b * tiles + tile] = ss;
      }
    }
  } else {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int b = nt * 8 + t * 2 + j;
      if (b >= M) continue;
      if (EPI == EPI_SILU_MUL) {
        const int I = N / 2;
        const int i = tile * 8 + g;
        if (i < I) {
          const float gate = acc[nt][j], up = acc[nt][2 + j];
          reinterpret_cast<bf16*>(out)[(size_t)b * I + i] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
        }
      } else {
        const int n0 = tile * 16 + g, n1 = n0 + 8;
        if (EPI == EPI_F32) {
          if (n0 < N) reinterpret_cast<float*>(out)[(size_t)b * N + n0] = acc[nt][j];
          if (n1 < N) reinterpret_cast<float*>(out)[(size_t)b * N + n1] = acc[nt][2 + j];
        } else {
          if (n0 < N) reinterpret_cast<bf16*>(out)[(size_t)b * N + n0] = __float2bfloat16_rn(acc[nt][j]);
          if (n1 < N) reinterpret_cast<bf16*>(out)[(size_t)b * N + n1] = __float2bfloat16_rn(acc[nt][2 + j]);
        }
      }
    }
  }
  }
}

template <int NT, int KS, int EPI, bool XS>
static int skinny_launch(const bf16* x, const bf16* W, void* out, int M, int N, int K, const float* h_in,
                         const bf16* delta, float* h_out, const float* gain, float eps, const SkNorm& nrm, cudaStream_t stream) {
  constexpr int WARPS = KS > SK_WARPS ? KS : SK_WARPS, THREADS = WARPS * 32;
  constexpr int RT = WARPS / KS;
  const int tiles = (EPI == EPI_SILU_MUL) ? (N / 2 + 7) / 8 : (N + 15) / 16;
  const int grid = (tiles + RT - 1) / RT;
  size_t smem = (KS > 1 ? (size_t)WARPS * NT * 4 * 32 * sizeof(float) : 0) +
                (XS ? (size_t)XS_ROWS * K * sizeof(bf16) : 0) + (size_t)SK_DEPTH * 2 * THREADS * 16;
  auto kern = skinny_gemm_kernel<NT, KS, EPI, XS>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return SX_ERR_SIZE;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return sx_launch(kern, dim3(grid), dim3(THREADS), smem, stream, x, W, out, M, N, K, h_in, delta, h_out, gain, eps, nrm);
}

// 8 warps split K, or 16 (blocks of 16 warps); 1, 2 and 4 measured slower everywhere and are not built
template <int NT, int EPI, bool XS>
static int skinny_pick_ks(int ks, const bf16* x, const bf16* W, void* out, int M, int N, int K, const float* h_in,
                          const bf16* delta, float* h_out, const float* gain, float eps, const SkNorm& nrm, cudaStream_t stream) {
  switch (ks) {
    case 16: return skinny_launch<NT, 16, EPI, XS>(x, W, out, M, N, K, h_in, delta, h_out, gain, eps, nrm, stream);
    case 8: return skinny_launch<NT, 8, EPI, XS>(x, W, out, M, N, K, h_in, delta, h_out, gain, eps, nrm, stream);
    default: return SX_ERR_SIZE;
  }
}

// up to 16 rows (more go to the tcgen05 product, which takes every K this kernel takes)
template <int EPI, bool XS>
static int skinny_pick_nt(int ks, const bf16* x, const bf16* W, void* out, int M, int N, int K, const float* h_in,
                          const bf16* delta, float* h_out, const float* gain, float eps, const SkNorm& nrm, cudaStream_t stream) {
  if (M <= 8) return skinny_pick_ks<1, EPI, XS>(ks, x, W, out, M, N, K, h_in, delta, h_out, gain, eps, nrm, stream);
  if (M <= 16) return skinny_pick_ks<2, EPI, XS>(ks, x, W, out, M, N, K, h_in, delta, h_out, gain, eps, nrm, stream);
  return SX_ERR_SIZE;
}

// x [M, K] bf16 (or, with h_in, computed as rmsnorm(h_in + delta) * gain), W [N, K] bf16.
// epi 0: out bf16 [M, N];  1: out f32 [M, N];  2: W is [gate; up] stacked, out bf16 [M, N/2] = silu(gate) * up.
// ks: warps that split K (8, or 16 with blocks of 16 warps).  Requires K % 32 == 0, 16-byte aligned x and W, M <= 16
// (M <= XS_ROWS = 2 with the norm prologue).
extern "C" int sx_skinny_gemm(const void* x, const void* W, void* out, int M, int N, int K, int epi, int ks,
                              const float* h_in, const void* delta, float* h_out, const float* gain, float eps,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 31) || M > 16) return SX_ERR_SIZE;
  if (epi == EPI_SILU_MUL && (N & 1)) return SX_ERR_SIZE;
  if (((uintptr_t)W & 15) || (x && ((uintptr_t)x & 15))) return SX_ERR_ALIGN;
  const bf16* xb = (const bf16*)x;
  const bf16* wb = (const bf16*)W;
  const bf16* db = (const bf16*)delta;
  const SkNorm none = {nullptr, 0, 0.f, nullptr, nullptr, nullptr};
  if (h_in) {
    if (M > XS_ROWS || K > 4096 || (K & 3)) return SX_ERR_SIZE;   // the prologue holds a row in registers
    switch (epi) {
      case EPI_BF16: return skinny_pick_nt<EPI_BF16, true>(ks, xb, wb, out, M, N, K, h_in, db, h_out, gain, eps, none, stream);
      case EPI_F32: return skinny_pick_nt<EPI_F32, true>(ks, xb, wb, out, M, N, K, h_in, db, h_out, gain, eps, none, stream);
      case EPI_SILU_MUL: return skinny_pick_nt<EPI_SILU_MUL, true>(ks, xb, wb, out, M, N, K, h_in, db, h_out, gain, eps, none, stream);
      default: return SX_ERR_DTYPE;
    }
  }
  switch (epi) {
    case EPI_BF16: return skinny_pick_nt<EPI_BF16, false>(ks, xb, wb, out, M, N, K, nullptr, nullptr, nullptr, nullptr, 0.f, none, stream);
    case EPI_F32: return skinny_pick_nt<EPI_F32, false>(ks, xb, wb, out, M, N, K, nullptr, nullptr, nullptr, nullptr, 0.f, none, stream);
    case EPI_SILU_MUL: return skinny_pick_nt<EPI_SILU_MUL, false>(ks, xb, wb, out, M, N, K, nullptr, nullptr, nullptr, nullptr, 0.f, none, stream);
    default: return SX_ERR_DTYPE;
  }
}

// The same product with an RMSNorm split between the product before it and itself (see SkNorm above).
//   ssq_in [M, n_in] (or null): x lacks the factor rsqrt(sum_i ssq_in[b, i] / K + eps_in) per row; the results get it.
//   epi 3: h_io f32 [M, N] += x W^T in place, out bf16 [M, N] = h_io * gain_next, ssq_out f32 [M, ceil(N / 16)] =
//          sums of squares of h_io over each 16-column tile.  Other epilogues as in sx_skinny_gemm.
extern "C" int sx_skinny_gemm_norm(const void* x, const void* W, void* out, int M, int N, int K, int epi, int ks,
                                   const float* ssq_in, int n_in, float eps_in, float* h_io, const float* gain_next,
                                   float* ssq_out, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 31) || M > 16 || !x) return SX_ERR_SIZE;
  if (epi == EPI_SILU_MUL && (N & 1)) return SX_ERR_SIZE;
  if (ssq_in && n_in <= 0) return SX_ERR_SIZE;
  if (epi == EPI_RESID && (!h_io || !gain_next || !ssq_out)) return SX_ERR_SIZE;
  if (((uintptr_t)W & 15) || ((uintptr_t)x & 15)) return SX_ERR_ALIGN;
  const bf16* xb = (const bf16*)x;
  const bf16* wb = (const bf16*)W;
  const SkNorm nrm = {ssq_in, n_in, eps_in, h_io, gain_next, ssq_out};
  switch (epi) {
    case EPI_BF16: return skinny_pick_nt<EPI_BF16, false>(ks, xb, wb, out, M, N, K, nullptr, nullptr, nullptr, nullptr, 0.f, nrm, stream);
    case EPI_F32: return skinny_pick_nt<EPI_F32, false>(ks, xb, wb, out, M, N, K, nullptr, nullptr, nullptr, nullptr, 0.f, nrm, stream);
    case EPI_SILU_MUL: return skinny_pick_nt<EPI_SILU_MUL, false>(ks, xb, wb, out, M, N, K, nullptr, nullptr, nullptr, nullptr, 0.f, nrm, stream);
    case EPI_RESID: return skinny_pick_nt<EPI_RESID, false>(ks, xb, wb, out, M, N, K, nullptr, nullptr, nullptr, nullptr, 0.f, nrm, stream);
    default: return SX_ERR_DTYPE;
  }
}
