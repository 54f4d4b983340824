// C[M, N] = X[M, K] * W[N, K]^T for a few dozen rows of X (decode steps of 17 to 256 sequences): the weight
// matrix streams from HBM once, through TMA, and is the M side of the tcgen05 instruction.
//
// With so few rows the product is bound by reading W, and a 128-row tile of X would be mostly padding.  So the
// operands swap: a block takes 128 ROWS OF W (the instruction's M = 128) and all rows of X (the instruction's
// N = the row count rounded up to 16), and the accumulator in tensor memory is C transposed: lane = column
// of C, column = row of C.  K is cut over the blocks of a thread-block cluster (1, 2, 4 or 8), so that a narrow
// matrix still gives every SM a block and each block streams its own part of W; the blocks of a cluster leave
// their float32 partial tiles in their own shared memory and add them up, each block a share of the columns,
// reading the others' through distributed shared memory, in block order (with up to 32 rows of X the blocks
// send their parts to the block that adds them up instead: one cluster barrier less).  No workspace in global
// memory and no second kernel.  The reference's products for decode steps are mma.sync tiles
// (crates/synaptix-kernels-cuda/src/best_cu/gemm/gemm_bf16.cu:37-61); it has no such path.
//
//   warp 0   producer: per 64-wide slice of K one TMA load of W (128 rows x 64; for a stacked [gate; up] matrix 64
//            gate rows and the 64 matching up rows) and one of X (all rows x 64) into a ring of stages.  The
//            first ring of W is asked for BEFORE the wait for the kernel before: weights are nobody's result.
//   warp 1   allocates the tensor memory; one lane issues 4 tcgen05.mma (K = 16 each) per stage
//   warps 2-5 read the accumulator and lay it into shared memory as P[row of C][column of the tile]
//   all      after a cluster barrier: the sum over the cluster's blocks, the epilogue, the store
// Epilogues: bfloat16 or float32 store; SiLU(gate) * up; both optionally times a factor per row of C,
// rsqrt(sum(ssq[row]) / K + eps) (rows of X that lack their RMSNorm factor); or h += C in the float32
// residual stream with bf16(h * gain) and partial sums of squares of h as outputs (what the next norm needs).
// Rows of W beyond N, rows of X beyond M and the tail of K are zero-filled by TMA: every size with K % 8 == 0.
// Every wait on an mbarrier is bounded; a wait that runs out sets *status and the block still meets the
// cluster's barriers and frees its tensor memory.
#include "tcgen05.cuh"

#define WS_THREADS 192
#define WS_BK 64
#define WS_W_BYTES (128 * WS_BK * 2)          // 16 KB of W per stage
#define WS_MAX_ROWS 256
#define WS_MAX_STAGES 8

enum { WS_EPI_BF16 = 0, WS_EPI_F32 = 1, WS_EPI_SILU_MUL = 2, WS_EPI_RESIDUAL = 3 };

struct WsEpilogue {
  const float* ssq_in;   // [M, n_ssq] partial sums of squares behind the row factors, or null
  int n_ssq;
  float eps;
  float* h;              // residual stream [M, N] (WS_EPI_RESIDUAL)
  const float* gain;     // [N]
  float* ssq_out;        // [M, tiles * splits]
};

__device__ __forceinline__ float4 ws_cluster_load4(const float* local, uint32_t rank) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(local), r;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(r) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t ws_cluster_addr(const float* local, uint32_t rank) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(local), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(rank));
  return r;
}
__device__ __forceinline__ void ws_cluster_store(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(WS_THREADS, 2) gemm_ws_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x,
                                                                void* __restrict__ out, int M, int N, int K, int nmma,
                                                                int stages, int splits, int tmem_cols, int push, WsEpilogue ep,
                                                                int* __restrict__ status) {
  extern __shared__ unsigned char ws_smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ws_smem_raw) + 1023) & ~(uintptr_t)1023);
  const int x_bytes = nmma * WS_BK * 2;
  const int stage_bytes = WS_W_BYTES + x_bytes;
  const int ring_bytes = stages * stage_bytes;
  const int p_bytes = M * 128 * 4;
  // pull: the partial tile P lies over the ring; push: a buffer of its own behind the ring receives the cluster's parts
  unsigned char* after = tiles + (push ? ring_bytes + p_bytes : (ring_bytes > p_bytes ? ring_bytes : p_bytes));
  float* R = reinterpret_cast<float*>(tiles + ring_bytes);                  // [splits][M][128 / splits] (push)
  uint64_t* bars = reinterpret_cast<uint64_t*>(after);                      // full[S], empty[S], accum
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * WS_MAX_STAGES + 1);
  float* row_factor = reinterpret_cast<float*>(tmem_slot + 2);              // [WS_MAX_ROWS]
  float* P = reinterpret_cast<float*>(tiles);                               // [M][128] once the ring is done with
  const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + WS_MAX_STAGES), accum = tc_smem(bars + 2 * WS_MAX_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_out = (EPI == WS_EPI_SILU_MUL) ? N / 2 : N;
  constexpr int tile_cols = (EPI == WS_EPI_SILU_MUL) ? 64 : 128;            // columns of C per tile
  const int tile = blockIdx.x / splits, part = blockIdx.x - tile * splits;  // part == the block's rank in its cluster
  const int n0 = tile * tile_cols;
  const int nkb_all = (K + WS_BK - 1) / WS_BK;
  const int kb0 = (int)((long long)nkb_all * part / splits), kb1 = (int)((long long)nkb_all * (part + 1) / splits);
  const int nkb = kb1 - kb0;                                                // the host keeps splits <= nkb_all: >= 1

  // Warp 0 sets the barriers up and asks for the first ring of W at once: before the tensor memory is there, and
  // before the wait for the kernel before (weights are nobody's result).
  const bool leader = warp == 0 && tc_elect_one();
  const uint32_t tiles_addr = tc_smem(tiles);
  const int pre = nkb < stages ? nkb : stages;
  if (warp == 0) {
    if (lane == 0) {
      for (int s = 0; s < stages; ++s) {
        tc_mbar_init(full0 + 8 * s, 1);
        tc_mbar_init(empty0 + 8 * s, 1);
      }
      tc_mbar_init(accum, 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_x) : "memory");
    }
    __syncwarp();
    for (int kb = 0; kb < pre; ++kb) {
      const uint32_t w_dst = tiles_addr + kb * stage_bytes, bar = full0 + 8 * kb;
      const int kx = (kb0 + kb) * WS_BK;
      if (leader) {
        tc_mbar_expect_tx(bar, stage_bytes);
        if (EPI == WS_EPI_SILU_MUL) {
          tc_tma_load_2d(w_dst, &map_w, kx, n0, bar);                           // 64 gate rows
          tc_tma_load_2d(w_dst + WS_W_BYTES / 2, &map_w, kx, N / 2 + n0, bar);  // 64 up rows
        } else {
          tc_tma_load_2d(w_dst, &map_w, kx, n0, bar);
        }
      }
    }
    __syncwarp();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)), "r"((uint32_t)tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // (the whole warp walks the ring, one elected lane issues: see the MMA warp)
    pdl_wait();
    pdl_trigger();
    for (int kb = 0; kb < pre; ++kb)
      if (leader) tc_tma_load_2d(tiles_addr + kb * stage_bytes + WS_W_BYTES, &map_x, (kb0 + kb) * WS_BK, 0, full0 + 8 * kb);
    for (int kb = pre; kb < nkb; ++kb) {
      const int s = kb % stages;
      const bool ok = __all_sync(0xffffffffu, tc_mbar_wait(empty0 + 8 * s, ((kb / stages) & 1) ^ 1));
      if (!ok) {
        if (leader) sx_set_status(status, 1);
        break;
      }
      const uint32_t w_dst = tiles_addr + s * stage_bytes, bar = full0 + 8 * s;
      const int kx = (kb0 + kb) * WS_BK;
      if (leader) {
        tc_mbar_expect_tx(bar, stage_bytes);
        if (EPI == WS_EPI_SILU_MUL) {
          tc_tma_load_2d(w_dst, &map_w, kx, n0, bar);
          tc_tma_load_2d(w_dst + WS_W_BYTES / 2, &map_w, kx, N / 2 + n0, bar);
        } else {
          tc_tma_load_2d(w_dst, &map_w, kx, n0, bar);
        }
        tc_tma_load_2d(w_dst + WS_W_BYTES, &map_x, kx, 0, bar);
      }
      __syncwarp();
    }
    __syncwarp();
  } else if (warp == 1) {
    pdl_wait();
    pdl_trigger();
    // The whole warp walks the ring (so that addresses and descriptors are computed in uniform control flow and
    // stay in uniform registers); one elected lane issues.
    const uint32_t idesc = tc_instr_desc(128, nmma);
    const bool issuer = tc_elect_one();
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % stages;
      const bool ok = __all_sync(0xffffffffu, tc_mbar_wait(full0 + 8 * s, (kb / stages) & 1));
      if (!ok) {
        if (issuer) sx_set_status(status, 2);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t w_addr = tiles_addr + s * stage_bytes, x_addr = w_addr + WS_W_BYTES;
      const uint64_t dw = tc_smem_desc(w_addr), dx = tc_smem_desc(x_addr);
      const uint32_t acc = kb != 0;
      if (issuer) {
#pragma unroll
        for (int k = 0; k < WS_BK / 16; ++k)          // 32 bytes further along K: 2 in the descriptor's 16-byte units
          tc_mma(tmem_base, dw + 2 * k, dx + 2 * k, idesc, acc | (k != 0));
        tc_commit(empty0 + 8 * s);
      }
      __syncwarp();
    }
    if (issuer) tc_commit(accum);
    __syncwarp();
  } else {
    pdl_wait();
    pdl_trigger();
    // The rows' factors, while the product runs.  The 128 threads share the rows (1, 2, 4 ... threads a row, neighbours
    // in a warp), each adds its part of the row's partial sums with 16-byte loads, many on the way at once, and
    // the parts are added by shuffles: a fixed order.  (One thread a row walking 160 partial sums one after the
    // other cost 8 us at 64 rows, a warp a row as much: what counts is how many loads are on the way.)
    if (ep.ssq_in != nullptr) {
      const int e = threadIdx.x - 64;
      int tpr = 1;
      while (tpr < 32 && 2 * tpr * M <= WS_THREADS - 64) tpr *= 2;
      // (more rows than threads: a thread takes rows e, e + 128, ...)
      const int rows_a_pass = (WS_THREADS - 64) / tpr, m_end = (M + rows_a_pass - 1) / rows_a_pass * rows_a_pass;
      for (int m = e / tpr, sub = e - (e / tpr) * tpr; m < m_end; m += rows_a_pass) {
        float s = 0.f;
        if (m < M) {
          const float* row = ep.ssq_in + (size_t)m * ep.n_ssq;
          if ((ep.n_ssq & 3) == 0 && ((uintptr_t)ep.ssq_in & 15) == 0) {
            const float4* r4 = reinterpret_cast<const float4*>(row);
#pragma unroll 8
            for (int j = sub; j < (ep.n_ssq >> 2); j += tpr) {
              const float4 f = r4[j];
              s += (f.x + f.y) + (f.z + f.w);
            }
          } else {
#pragma unroll 8
            for (int j = sub; j < ep.n_ssq; j += tpr) s += row[j];
          }
        }
        for (int d = tpr >> 1; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
        if (m < M && sub == 0) row_factor[m] = rsqrtf(s / (float)K + ep.eps);
      }
    }
    const int quarter = warp & 3;                     // warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    if (tc_mbar_wait(accum, 0)) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
      const int n = quarter * 32 + lane;                 // this thread's row of the W tile
      if (push) {
        // every value goes straight into the shared memory of the block that will add this column up
        const int cpo = 128 / splits;                    // values a row of C an owner receives from one block
        int owner, j;
        if (EPI == WS_EPI_SILU_MUL) {
          const int half = cpo >> 1, c = n & 63;
          owner = c / half;
          j = (n >> 6) * half + c % half;                // gate values first, then up values
        } else {
          owner = n / cpo;
          j = n % cpo;
        }
        const uint32_t dst = ws_cluster_addr(R + (size_t)part * M * cpo + j, (uint32_t)owner);
        for (int c0 = 0; c0 < nmma; c0 += 16) {
          uint32_t v[16];
          tc_ld16(t_row + c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c0 + i < M) ws_cluster_store(dst + (uint32_t)((c0 + i) * cpo * 4), __uint_as_float(v[i]));
        }
      } else {
        float* dst = P + n;
        for (int c0 = 0; c0 < nmma; c0 += 16) {
          uint32_t v[16];
          tc_ld16(t_row + c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c0 + i < M) dst[(size_t)(c0 + i) * 128] = __uint_as_float(v[i]);
        }
      }
    } else {
      if (lane == 0) sx_set_status(status, 3);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  if (splits > 1) cluster_sync_all();                 // every block's P is complete and visible
  else __syncthreads();
  if (warp == 1) {                                    // the accumulator has been read: the tensor memory goes back now
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
  }

  // the sum over the cluster's blocks and the epilogue: this block takes tile_cols / splits columns of every row
  {
    const int cols_per = tile_cols / splits;          // 128 .. 8
    const int g4 = cols_per / 4;                      // groups of four columns a row: 32 .. 2
    const int items = M * g4;
    for (int base = warp * 32; base < items; base += WS_THREADS) {
      const int idx = base + lane;
      const bool valid = idx < items;
      const int m = valid ? idx / g4 : 0;
      const int c = part * cols_per + (valid ? idx - m * g4 : 0) * 4;       // column within the tile
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      if (valid && push) {
        const int cpo = 128 / splits, col4 = c - part * cols_per;
        for (int z = 0; z < splits; ++z) {            // what every block sent, in block order
          const float* src = R + ((size_t)z * M + m) * cpo + col4;
          const float4 f = *reinterpret_cast<const float4*>(src);
          a.x += f.x; a.y += f.y; a.z += f.z; a.w += f.w;
          if (EPI == WS_EPI_SILU_MUL) {
            const float4 u = *reinterpret_cast<const float4*>(src + cols_per);
            b.x += u.x; b.y += u.y; b.z += u.z; b.w += u.w;
          }
        }
      } else if (valid) {
        for (int z = 0; z < splits; ++z) {
          const float4 f = ws_cluster_load4(P + (size_t)m * 128 + c, (uint32_t)z);
          a.x += f.x; a.y += f.y; a.z += f.z; a.w += f.w;
          if (EPI == WS_EPI_SILU_MUL) {
            const float4 u = ws_cluster_load4(P + (size_t)m * 128 + 64 + c, (uint32_t)z);
            b.x += u.x; b.y += u.y; b.z += u.z; b.w += u.w;
          }
        }
      }
      float o[4] = {a.x, a.y, a.z, a.w};
      const float rf = (valid && ep.ssq_in != nullptr) ? row_factor[m] : 1.f;
      if (EPI == WS_EPI_SILU_MUL) {
        const float u[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float g = o[j] * rf;
          o[j] = g / (1.f + __expf(-g)) * (u[j] * rf);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] *= rf;
      }
      const int n = n0 + c;
      const int cols = valid ? min(4, n_out - n) : 0;                      // <= 0: beyond the matrix
      const size_t at = (size_t)m * n_out + n;
      const bool vec = cols == 4 && (n_out & 3) == 0;
      if (EPI == WS_EPI_RESIDUAL) {
        float sq = 0.f;
        if (cols > 0) {
          float hv[4] = {0.f, 0.f, 0.f, 0.f}, gv[4] = {0.f, 0.f, 0.f, 0.f};
          if (vec) {
            const float4 h4 = *reinterpret_cast<const float4*>(ep.h + at);
            const float4 g4v = *reinterpret_cast<const float4*>(ep.gain + n);
            hv[0] = h4.x; hv[1] = h4.y; hv[2] = h4.z; hv[3] = h4.w;
            gv[0] = g4v.x; gv[1] = g4v.y; gv[2] = g4v.z; gv[3] = g4v.w;
          } else {
            for (int j = 0; j < cols; ++j) { hv[j] = ep.h[at + j]; gv[j] = ep.gain[n + j]; }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            hv[j] += o[j];
            if (j < cols) sq += hv[j] * hv[j];
          }
          bf16* xo = reinterpret_cast<bf16*>(out) + at;
          if (vec) {
            *reinterpret_cast<float4*>(ep.h + at) = make_float4(hv[0], hv[1], hv[2], hv[3]);
            __nv_bfloat162 lo = __floats2bfloat162_rn(hv[0] * gv[0], hv[1] * gv[1]), hi = __floats2bfloat162_rn(hv[2] * gv[2], hv[3] * gv[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(xo) = pk;
          } else {
            for (int j = 0; j < cols; ++j) { ep.h[at + j] = hv[j]; xo[j] = __float2bfloat16_rn(hv[j] * gv[j]); }
          }
        }
        // the row's sum of squares over this block's columns: the g4 lanes of a row are neighbours
        for (int d = g4 >> 1; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
        if (valid && (idx - m * g4) == 0) ep.ssq_out[(size_t)m * (gridDim.x) + blockIdx.x] = sq;
      } else if (cols > 0) {
        if (EPI == WS_EPI_F32) {
          float* dst = reinterpret_cast<float*>(out) + at;
          if (vec) *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
          else
            for (int j = 0; j < cols; ++j) dst[j] = o[j];
        } else {
          bf16* dst = reinterpret_cast<bf16*>(out) + at;
          if (vec) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst) = pk;
          } else {
            for (int j = 0; j < cols; ++j) dst[j] = __float2bfloat16_rn(o[j]);
          }
        }
      }
    }
  }

  if (splits > 1 && !push) cluster_sync_all();        // nobody reads this block's P any more
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static int* ws_status_word() {
  static int* p = nullptr;
  if (!p) p = sx_status_word_alloc();
  return p;
}

static int ws_sm_count() {
  static int n[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!n[dev]) {
    if (cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n[dev] <= 0) n[dev] = 148;
  }
  return n[dev];
}

// Shared memory a block takes with a ring of `stages` (the partial tile lies over the ring), and how many blocks of
// that size an SM holds (228 KB an SM, 1 KB of it per resident block).
// With few rows the blocks of a cluster SEND their partial results to the block that adds a column up (a buffer of
// M x 128 floats behind the ring receives them): one cluster barrier and no remote loads.  With more rows that buffer
// would cost ring stages, and the partial tile stays where it is (over the ring) for the others to fetch: two barriers.
#define WS_PUSH_MAX_ROWS 32
static size_t ws_smem_bytes(int M, int nmma, int stages, bool push) {
  const size_t ring = (size_t)stages * (WS_W_BYTES + nmma * WS_BK * 2), p_bytes = (size_t)M * 128 * 4;
  return 1024 + (push ? ring + p_bytes : (ring > p_bytes ? ring : p_bytes)) + (2 * WS_MAX_STAGES + 1) * sizeof(uint64_t) + 8 +
         WS_MAX_ROWS * sizeof(float) + 16;
}
static int ws_blocks_per_sm(int M, int nmma, int stages) {
  return (int)(233472 / (ws_smem_bytes(M, nmma, stages, M <= WS_PUSH_MAX_ROWS) + 1024));
}

// The deepest ring (up to what lets two blocks share an SM) with which all `blocks` blocks are on the GPU at once;
// 0 if there is none of at least 2 stages.  A block that has to wait for a place runs behind all the others.
static int ws_pick_stages(int M, int nmma, long long blocks) {
  const int sms = ws_sm_count();
  // (a partial tile of more than 100 KB leaves room for one block an SM whatever the ring: the ring may be as large)
  const size_t room = (size_t)M * 128 * 4 > 100 * 1024 ? 200 * 1024 : 100 * 1024;
  int stages = (int)(room / (WS_W_BYTES + nmma * WS_BK * 2));
  if (stages > WS_MAX_STAGES) stages = WS_MAX_STAGES;
  const long long per_sm = (blocks + sms - 1) / sms;
  while (stages >= 2 && ws_blocks_per_sm(M, nmma, stages) < per_sm) --stages;
  return stages >= 2 ? stages : 0;
}

// Blocks of a cluster that share a tile's K: the fewest of 1, 2, 4, 8 that give (nearly) every SM a block, each
// block keeping at least two 64-wide slices.  (Measured at 64 rows: 6144 x 2560 best with 4, 2560 x 4096 and
// 2560 x 9728 with 8; more blocks than that cost more than they stream.)  Then, if that is more than one block an
// SM (the stacked 19456 x 2560: 152 tiles on 148 SMs), twice as many blocks with shallower rings, as long as they
// are all on the GPU at once and keep 16 slices each: most SMs would otherwise hold ONE block, whose ring of 3 or
// 4 stages is too few bytes on the way for a loaded HBM (27.5 us with 1 block a tile and 4 stages, 23.9 with 2 and 3).
static int ws_pick_splits(int M, int tiles, int nkb) {
  const int sms = ws_sm_count(), want = sms * 7 / 8;
  const int nmma = (M + 15) / 16 * 16;
  int s = 1;
  while (s < 8 && tiles * s < want && nkb / (2 * s) >= 2) s *= 2;
  if (s < 8 && (long long)tiles * s > sms && nkb / (2 * s) >= 16) {
    const int st = ws_pick_stages(M, nmma, (long long)tiles * 2 * s);
    if (st >= (nmma <= 64 ? 3 : 2)) s *= 2;
  }
  return s;
}

extern "C" int sx_gemm_ws_plan(int M, int N, int K, int epi, int* out2) {
  if (M <= 0 || N <= 0 || K <= 0) return SX_ERR_SIZE;
  const int n_out = epi == WS_EPI_SILU_MUL ? N / 2 : N;
  const int tile_cols = epi == WS_EPI_SILU_MUL ? 64 : 128;
  const int tiles = (n_out + tile_cols - 1) / tile_cols;
  out2[0] = tiles;
  out2[1] = ws_pick_splits(M, tiles, (K + WS_BK - 1) / WS_BK);
  return 0;
}

template <int EPI>
static int ws_launch(const void* X, const void* W, void* out, int M, int N, int K, int splits, int stages,
                     const WsEpilogue& ep, cudaStream_t stream) {
  int* status = ws_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  const int n_out = EPI == WS_EPI_SILU_MUL ? N / 2 : N;
  const int tile_cols = EPI == WS_EPI_SILU_MUL ? 64 : 128;
  const long long tiles = ((long long)n_out + tile_cols - 1) / tile_cols;
  if (tiles * splits > 0x7fffffffLL) return SX_ERR_SIZE;
  const int nmma = (M + 15) / 16 * 16;
  int tmem_cols = 32;
  while (tmem_cols < nmma) tmem_cols *= 2;
  CUtensorMap mw, mx;
  int rc = tc_make_map_rows(&mw, W, N, K, EPI == WS_EPI_SILU_MUL ? 64 : 128);
  if (rc) return rc;
  if ((rc = tc_make_map_rows(&mx, X, M, K, nmma))) return rc;
  // the ring: given, or the deepest with which every block is on the GPU at once (at most what lets two share an SM)
  const int stage_bytes = WS_W_BYTES + nmma * WS_BK * 2;
  if (stages <= 0) stages = ws_pick_stages(M, nmma, tiles * splits);
  if (stages <= 0) stages = (int)(((size_t)M * 128 * 4 > 100 * 1024 ? 200 * 1024 : 100 * 1024) / stage_bytes);
  if (stages > WS_MAX_STAGES) stages = WS_MAX_STAGES;
  if (stages > (220 * 1024) / stage_bytes) stages = (220 * 1024) / stage_bytes;
  if (stages < 2) stages = 2;
  const int push = splits > 1 && M <= WS_PUSH_MAX_ROWS;
  const size_t smem = ws_smem_bytes(M, nmma, stages, push != 0);
  auto kern = gemm_ws_kernel<EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return sx_launch_cluster(kern, dim3((unsigned)(tiles * splits)), dim3(WS_THREADS), smem, stream, splits, mw, mx, out, M, N, K, nmma,
                           stages, splits, tmem_cols, push, ep, status);
}

// X [M, K], W [N, K] bfloat16 row-major, 16-byte aligned, K % 8 == 0, 1 <= M <= 256.
// epi 0: out bf16 [M, N]; 1: out f32 [M, N]; 2: W = [gate; up] stacked, out bf16 [M, N/2];
// 3: h [M, N] float32 += the product in place, out bf16 [M, N] = bf16(h * gain), ssq_out [M, tiles * splits] the sums
//    of squares of the new h over each block's columns (sx_gemm_ws_plan gives tiles and splits).
// ssq_in (epi 0-2, may be null): [M, n_ssq] float32; row m of the result is multiplied by rsqrt(sum(ssq_in[m]) / K + eps).
// splits: blocks of a cluster that share a tile's K (1, 2, 4 or 8); 0 lets the library choose.
// stages: depth of the ring (2 to 8, as far as shared memory holds them); 0 = what lets two blocks share an SM.
extern "C" int sx_gemm_ws(const void* X, const void* W, void* out, int M, int N, int K, int epi, int splits, int stages,
                          const float* ssq_in, int n_ssq, float eps, float* h, const float* gain, float* ssq_out,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > WS_MAX_ROWS || K <= 0 || (K & 7)) return SX_ERR_SIZE;
  if (epi == WS_EPI_SILU_MUL && (N & 1)) return SX_ERR_SIZE;
  if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return SX_ERR_ALIGN;
  const int nkb = (K + WS_BK - 1) / WS_BK;
  const int n_out = epi == WS_EPI_SILU_MUL ? N / 2 : N;
  const int tile_cols = epi == WS_EPI_SILU_MUL ? 64 : 128;
  if (splits == 0) splits = ws_pick_splits(M, (n_out + tile_cols - 1) / tile_cols, nkb);
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return SX_ERR_SIZE;
  while (splits > nkb) splits /= 2;
  WsEpilogue ep;
  ep.ssq_in = ssq_in; ep.n_ssq = n_ssq; ep.eps = eps; ep.h = h; ep.gain = gain; ep.ssq_out = ssq_out;
  switch (epi) {
    case WS_EPI_BF16: return ws_launch<WS_EPI_BF16>(X, W, out, M, N, K, splits, stages, ep, stream);
    case WS_EPI_F32: return ws_launch<WS_EPI_F32>(X, W, out, M, N, K, splits, stages, ep, stream);
    case WS_EPI_SILU_MUL: return ws_launch<WS_EPI_SILU_MUL>(X, W, out, M, N, K, splits, stages, ep, stream);
    case WS_EPI_RESIDUAL:
      if (!h || !gain || !ssq_out || ssq_in) return SX_ERR_SIZE;
      return ws_launch<WS_EPI_RESIDUAL>(X, W, out, M, N, K, splits, stages, ep, stream);
    default: return SX_ERR_DTYPE;
  }
}

// 0, or which bounded wait ran out (1 producer, 2 MMA issuer, 3 the warps that read the accumulator).  Reads the
// word in host memory: no device call.  With reset != 0 the word goes back to 0.
extern "C" int sx_gemm_ws_status(int* host_value, int reset) {
  int* p = ws_status_word();
  if (!p) return (int)cudaErrorMemoryAllocation;
  *host_value = *(volatile int*)p;
  if (reset) *(volatile int*)p = 0;
  return 0;
}
