// C[M, N] = A[M, K] * W[N, K]^T for bfloat16 on the 5th-generation tensor cores (sm_100a):
// operands staged in shared memory by TMA (128-byte swizzle), tcgen05.mma issued by one thread,
// accumulator in tensor memory, read back with tcgen05.ld for the epilogue.
//
// This is the matrix product of prompt steps (hundreds to thousands of rows).  The reference's
// kernels for it are mma.sync/ldmatrix tiles, some fed by TMA, tuned for sm_120a
// (crates/synaptix-kernels-cuda/src/best_cu/gemm/gemm_bf16.cu:37-61,1678-2013); it has no
// tcgen05 path.
//
// One block computes one 128 x 256 tile of C.
//   warp 0   producer: for every 64-wide slice of K, one TMA load of A (128 rows x 64) and two of
//            W (128 rows x 64 each) into a ring of STAGES stages, signalled through mbarriers
//   warp 1   allocates 256 columns of tensor memory; one lane issues 4 tcgen05.mma (K = 16
//            each) per stage, and tcgen05.commit hands the stage back to the producer
//   warps 2-5 epilogue: each reads its 32 lanes of the accumulator in chunks of 32 columns,
//            converts and stores
// Rows of A beyond M, rows of W beyond N and the tail of K are zero-filled by TMA, so every size
// with K % 8 == 0 is taken.  Epilogues: bfloat16 store; float32 store; SiLU(gate) * up for a
// stacked [gate; up] matrix (the two W loads of a stage then fetch 128 gate rows and the 128
// matching up rows, and the tile of C is 128 x 128).
// Every wait on an mbarrier is bounded; a wait that runs out sets *status, and the block still
// frees its tensor memory before it ends.
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_A_BYTES (TC_BM * TC_BK * 2)            // 16 KB
#define TC_THREADS 192
// (the epilogue that prepares heads has eight epilogue warps, one group of four per head of the tile)
template <int EPI> struct TcThreads { static constexpr int N = EPI == 4 ? 320 : TC_THREADS; };
#define TC_RED_ROWS 6

enum { TC_EPI_BF16 = 0, TC_EPI_F32 = 1, TC_EPI_SILU_MUL = 2, TC_EPI_PARTIAL = 3, TC_EPI_QKV = 4 };

// TC_EPI_QKV: the product is the fused q/k/v projection of a prompt step with heads of 128, and its epilogue is the head
// preparation (what sx_qkv_prepare does to the projection): a 128 x 256 tile holds two whole heads of 128 tokens, an
// epilogue thread owns a token, so the RMSNorm over a head and the rotation of its halves stay inside a thread.  Query heads
// go to q_out [M, nh * 128], keys and values into the token's place in its sequence's page.  Values are rounded to bfloat16
// first, as the projection's own output would be.  cs / sn [M, 64]: cosines and sines of position * inv_freq (null: no rotation).
struct TcQkv {
  bf16* q_out;
  bf16* k_pages;
  bf16* v_pages;
  const float* wq;
  const float* wk;
  const float* cs;
  const float* sn;
  const int* positions;
  const int* seq_of_token;
  const int* block_table;
  int maxp, nh, nkv, n_pages;
  float eps;
};

// BN: columns of W per block (256, or 128 for the split-K form); stages fill the shared memory
template <int BN> struct TcShape {
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
};

template <int EPI, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_w,
                                                                void* __restrict__ out, int M, int N, int K,
                                                                int* __restrict__ status) {
  constexpr int TC_BN = BN, TC_STAGES = TcShape<BN>::STAGES, TC_B_BYTES = TcShape<BN>::B_BYTES,
                TC_STAGE_BYTES = TcShape<BN>::STAGE_BYTES;
  extern __shared__ unsigned char tc_smem_raw[];
  // the swizzled tiles must start on a 1024-byte boundary
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * TC_STAGE_BYTES);   // full[S], empty[S], accum
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 1);
  const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + TC_STAGES), accum = tc_smem(bars + 2 * TC_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_out = (EPI == TC_EPI_SILU_MUL) ? N / 2 : N;                 // columns of C
  const int tile_n = (EPI == TC_EPI_SILU_MUL) ? TC_BN / 2 : TC_BN;        // columns of C per block
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * tile_n;
  // split-K: block z of gridDim.z takes a contiguous range of the 64-wide slices of K and (with
  // TC_EPI_PARTIAL) writes its float32 partial tile to out[z][M][N]; the host gives every z a non-empty range
  const int nkb_all = (K + TC_BK - 1) / TC_BK;
  const int kper = (nkb_all + gridDim.z - 1) / gridDim.z;
  const int kb0 = blockIdx.z * kper;
  const int nkb = max(0, min(nkb_all, kb0 + kper) - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      tc_mbar_init(full0 + 8 * s, 1);
      tc_mbar_init(empty0 + 8 * s, 1);
    }
    tc_mbar_init(accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)), "r"((uint32_t)TC_BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();          // barriers and tensor memory are set up; the operands may come from the kernel before
  pdl_trigger();

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % TC_STAGES;
        if (!tc_mbar_wait(empty0 + 8 * s, ((kb / TC_STAGES) & 1) ^ 1)) { sx_set_status(status, 1); break; }
        tc_mbar_expect_tx(full0 + 8 * s, TC_STAGE_BYTES);
        const uint32_t a_dst = tc_smem(tiles + s * TC_STAGE_BYTES), b_dst = a_dst + TC_A_BYTES;
        const int kx = (kb0 + kb) * TC_BK;
        tc_tma_load_2d(a_dst, &map_a, kx, m0, full0 + 8 * s);
        if (EPI == TC_EPI_SILU_MUL) {
          tc_tma_load_2d(b_dst, &map_w, kx, n0, full0 + 8 * s);                        // gate rows
          tc_tma_load_2d(b_dst + TC_B_BYTES / 2, &map_w, kx, N / 2 + n0, full0 + 8 * s);  // up rows
        } else {
#pragma unroll
          for (int j = 0; j < TC_BN / 128; ++j)
            tc_tma_load_2d(b_dst + j * (128 * TC_BK * 2), &map_w, kx, n0 + j * 128, full0 + 8 * s);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc_instr_desc(TC_BM, TC_BN);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % TC_STAGES;
        if (!tc_mbar_wait(full0 + 8 * s, (kb / TC_STAGES) & 1)) { sx_set_status(status, 2); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t a_addr = tc_smem(tiles + s * TC_STAGE_BYTES), b_addr = a_addr + TC_A_BYTES;
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k)
          tc_mma(tmem_base, tc_smem_desc(a_addr + k * 32), tc_smem_desc(b_addr + k * 32), idesc, (kb | k) != 0);
        tc_commit(empty0 + 8 * s);          // the stage is free once these MMAs have read it
      }
      tc_commit(accum);                     // the accumulator is complete once all MMAs are done
    }
    __syncwarp();
  } else {
    // epilogue warps 2..5: warp w may touch tensor-memory lanes 32*(w%4) .. +31
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    if (tc_mbar_wait(accum, 0)) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
      const bool vec_ok = (n_out % 8) == 0;
#pragma unroll 1
      for (int c0 = 0; c0 < tile_n; c0 += 32) {
        uint32_t v[32];
        tc_ld32(t_row + c0, v);
        uint32_t u[32];
        if (EPI == TC_EPI_SILU_MUL) tc_ld32(t_row + TC_BN / 2 + c0, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (row >= M || n0 + c0 >= n_out) continue;
        float f[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          f[i] = __uint_as_float(v[i]);
          if (EPI == TC_EPI_SILU_MUL) f[i] = f[i] / (1.f + expf(-f[i])) * __uint_as_float(u[i]);
        }
        const int ncol = min(32, n_out - (n0 + c0));
        if (EPI == TC_EPI_F32 || EPI == TC_EPI_PARTIAL) {
          float* dst = reinterpret_cast<float*>(out) + ((size_t)(EPI == TC_EPI_PARTIAL ? blockIdx.z : 0) * M + row) * n_out + n0 + c0;
          if (ncol == 32 && (n_out % 4) == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
          } else {
            for (int i = 0; i < ncol; ++i) dst[i] = f[i];
          }
        } else {
          bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)row * n_out + n0 + c0;
          if (ncol == 32 && vec_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 p;
              __nv_bfloat162 t0 = __floats2bfloat162_rn(f[8 * i], f[8 * i + 1]), t1 = __floats2bfloat162_rn(f[8 * i + 2], f[8 * i + 3]);
              __nv_bfloat162 t2 = __floats2bfloat162_rn(f[8 * i + 4], f[8 * i + 5]), t3 = __floats2bfloat162_rn(f[8 * i + 6], f[8 * i + 7]);
              p.x = *reinterpret_cast<uint32_t*>(&t0); p.y = *reinterpret_cast<uint32_t*>(&t1);
              p.z = *reinterpret_cast<uint32_t*>(&t2); p.w = *reinterpret_cast<uint32_t*>(&t3);
              reinterpret_cast<uint4*>(dst)[i] = p;
            }
          } else {
            for (int i = 0; i < ncol; ++i) dst[i] = __float2bfloat16_rn(f[i]);
          }
        }
      }
    } else {
      if (lane == 0) sx_set_status(status, 3);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)TC_BN) : "memory");
  }
}

// =======================================================================================
// The persistent form for many rows: one block per SM walks over the 128 x 256 tiles of C
// (tile t -> row tile t % tiles_m, column tile t / tiles_m, so that blocks running at the same
// time share W tiles through L2).  Tensor memory holds TWO accumulators (2 x 256 columns): while
// the epilogue warps read tile i out of one, the MMA warp is already filling the other with tile
// i + 1, and the TMA ring runs ahead across tiles.  Barriers: full/empty per stage, and
// acc_full/acc_empty per accumulator.  When the tiles do not fill a round of all SMs (a nearly empty last
// round, or fewer tiles than SMs as in steps of a few dozen rows), those tiles are cut over K (TcPlan below).
// =======================================================================================
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

template <int EPI>
__device__ __forceinline__ void tc_store_chunk(const uint32_t (&v)[32], const uint32_t (&u)[32], void* __restrict__ out,
                                               int row, int col, int n_out) {
  float f[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    f[i] = __uint_as_float(v[i]);
    if (EPI == TC_EPI_SILU_MUL) f[i] = f[i] / (1.f + __expf(-f[i])) * __uint_as_float(u[i]);
  }
  const int ncol = min(32, n_out - col);
  if (EPI == TC_EPI_F32) {
    float* dst = reinterpret_cast<float*>(out) + (size_t)row * n_out + col;
    if (ncol == 32 && (n_out % 4) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) if (i < ncol) dst[i] = f[i];
    }
  } else {
    bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)row * n_out + col;
    if (ncol == 32 && (n_out % 8) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 p;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(f[8 * i], f[8 * i + 1]), t1 = __floats2bfloat162_rn(f[8 * i + 2], f[8 * i + 3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(f[8 * i + 4], f[8 * i + 5]), t3 = __floats2bfloat162_rn(f[8 * i + 6], f[8 * i + 7]);
        p.x = *reinterpret_cast<uint32_t*>(&t0); p.y = *reinterpret_cast<uint32_t*>(&t1);
        p.z = *reinterpret_cast<uint32_t*>(&t2); p.w = *reinterpret_cast<uint32_t*>(&t3);
        reinterpret_cast<uint4*>(dst)[i] = p;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) if (i < ncol) dst[i] = __float2bfloat16_rn(f[i]);
    }
  }
}

// The work of the persistent kernel.  The tiles are numbered m-fastest.  The first n_whole of them are
// computed whole, block c taking tiles c, c + G, ...  The remaining R = n_tiles - n_whole tiles (the
// last round, when it would keep few SMs busy; or ALL tiles, when there is one row of them and they are
// fewer than SMs) are cut over K into PIECES.  For all tiles cut, "stream-K" fashion: their R * nkb
// slices of K (64 wide) form one sequence that is dealt out to the G blocks in equal contiguous shares, so
// a block gets at most two pieces (the end of one tile and the start of the next), and a tile is covered
// by the pieces of a few consecutive blocks.  For a last round: equal pieces per tile (see tc_piece).
struct TcPlan {
  int n_whole, R, nkb, G;
  int sp;                      // > 0: every cut tile has exactly sp pieces of equal length and no block has two (see tc_piece)
  long long U;                 // R * nkb
  __host__ __device__ long long share_begin(int c) const { return U * c / G; }
  // the block whose share holds unit u
  __host__ __device__ int block_of(long long u) const { return (int)(((u + 1) * G - 1) / U); }
};
struct TcPiece {
  int tile;                    // tile number (n_whole + index among the cut tiles)
  int kb_lo, kb_hi;            // its slices of K
  int z, nz;                   // which of the tile's pieces this is, and how many there are
};
// piece i (0 or 1) of block c; false if the block has no such piece.
// With whole tiles after the pieces (p.sp > 0) the shares are NOT dealt out stream-K fashion: a block with two
// pieces stores two partial tiles and adds up twice, which took longer than the whole tile's MMAs it should hide
// behind (measured 51 against 38 us for 2,048 x 2,560 x 4,096).  Tile t then simply has the sp = G / R pieces of
// blocks t sp .. t sp + sp - 1, and G - R sp blocks have none.
__host__ __device__ inline bool tc_piece(const TcPlan& p, int c, int i, TcPiece& out) {
  if (p.R <= 0) return false;
  if (p.sp > 0) {
    if (i != 0 || c >= p.R * p.sp) return false;
    const int t = c / p.sp, z = c % p.sp;
    const int kper = (p.nkb + p.sp - 1) / p.sp;
    out.tile = p.n_whole + t;
    out.kb_lo = z * kper;
    out.kb_hi = out.kb_lo + kper < p.nkb ? out.kb_lo + kper : p.nkb;
    out.z = z;
    out.nz = (p.nkb + kper - 1) / kper;              // pieces that are not empty
    return out.kb_lo < out.kb_hi;
  }
  long long u0 = p.share_begin(c);
  const long long u1 = p.share_begin(c + 1);
  if (u0 >= u1) return false;
  long long t = u0 / p.nkb;
  if (i == 1) {
    u0 = (t + 1) * p.nkb;
    if (u0 >= u1) return false;
    ++t;
  }
  out.tile = p.n_whole + (int)t;
  out.kb_lo = (int)(u0 - t * p.nkb);
  out.kb_hi = (int)((u1 < (t + 1) * p.nkb ? u1 : (t + 1) * p.nkb) - t * p.nkb);
  const int c_lo = p.block_of(t * p.nkb), c_hi = p.block_of((t + 1) * p.nkb - 1);
  out.z = c - c_lo;
  out.nz = c_hi - c_lo + 1;
  return true;
}

template <int EPI, int BN>
__global__ void __launch_bounds__(TcThreads<EPI>::N, 1) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                           const __grid_constant__ CUtensorMap map_w,
                                                                           void* __restrict__ out, int M, int N, int K,
                                                                           int n_whole, int zmax, int sp,
                                                                           float* __restrict__ piece_ws,
                                                                           int* __restrict__ piece_count,
                                                                           int* __restrict__ status, const TcQkv qk) {
  constexpr int STAGES = TcShape<BN>::STAGES, B_BYTES = TcShape<BN>::B_BYTES, STAGE_BYTES = TcShape<BN>::STAGE_BYTES;
  extern __shared__ unsigned char tc_smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);   // full[S], empty[S], acc_full[2], acc_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* piece_ok = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + STAGES);
  const uint32_t acc_full0 = tc_smem(bars + 2 * STAGES), acc_empty0 = tc_smem(bars + 2 * STAGES + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_out = (EPI == TC_EPI_SILU_MUL) ? N / 2 : N;
  const int tile_n = (EPI == TC_EPI_SILU_MUL) ? BN / 2 : BN;
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (n_out + tile_n - 1) / tile_n;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  TcPlan plan;
  plan.n_whole = n_whole; plan.R = tiles_m * tiles_n - n_whole; plan.nkb = nkb; plan.G = (int)gridDim.x;
  plan.sp = sp;
  plan.U = (long long)plan.R * nkb;
  const bool coop = sp > 0;            // the blocks of a cut tile add up in this kernel (else a second kernel does)
  // This block's work in order: its pieces of the cut tiles FIRST (short, so that adding the partial tiles up
  // hides behind the MMAs of the whole tiles), then whole tiles blockIdx.x, blockIdx.x + G, ...
  TcPiece pc[2];
  int n_pc = 0;
  if (tc_piece(plan, blockIdx.x, 0, pc[0])) { n_pc = 1; if (tc_piece(plan, blockIdx.x, 1, pc[1])) n_pc = 2; }
  const int n_mine = n_whole > (int)blockIdx.x ? (n_whole - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int n_work = n_pc + n_mine;
  auto work_of = [&](int w, int& tile, int& kb_lo, int& kb_hi) {
    if (w < n_pc) { tile = pc[w].tile; kb_lo = pc[w].kb_lo; kb_hi = pc[w].kb_hi; }
    else { tile = blockIdx.x + (w - n_pc) * gridDim.x; kb_lo = 0; kb_hi = nkb; }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc_mbar_init(full0 + 8 * s, 1);
      tc_mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc_mbar_init(acc_full0 + 8 * b, 1);
      tc_mbar_init(acc_empty0 + 8 * b, (TcThreads<EPI>::N - 64) / 32);          // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();          // barriers and tensor memory are set up; the operands may come from the kernel before
  pdl_trigger();

  // Producer and MMA warp: the WHOLE warp walks the work (so that addresses and descriptors are computed in uniform
  // control flow and stay in uniform registers; with one lane branching off alone each tcgen05.mma cost tens of
  // nanoseconds to issue), and one elected lane issues.
  if (warp == 0) {
    const bool leader = tc_elect_one();
    const uint32_t tiles_addr = tc_smem(tiles);
    uint32_t it = 0;
    bool ok = true;
    for (int w = 0; w < n_work && ok; ++w) {
      int tile, kb_lo, kb_hi;
      work_of(w, tile, kb_lo, kb_hi);
      const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * tile_n;
      for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
        const uint32_t s = it % STAGES;
        ok = __all_sync(0xffffffffu, tc_mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1));
        if (!ok) {
          if (leader) sx_set_status(status, 1);
          break;
        }
        const uint32_t a_dst = tiles_addr + s * STAGE_BYTES, b_dst = a_dst + TC_A_BYTES, bar = full0 + 8 * s;
        if (leader) {
          tc_mbar_expect_tx(bar, STAGE_BYTES);
          tc_tma_load_2d(a_dst, &map_a, kb * TC_BK, m0, bar);
          tc_tma_load_2d(b_dst, &map_w, kb * TC_BK, n0, bar);
          if (BN == 256)
            tc_tma_load_2d(b_dst + B_BYTES / 2, &map_w, kb * TC_BK, (EPI == TC_EPI_SILU_MUL) ? N / 2 + n0 : n0 + BN / 2, bar);
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    constexpr uint32_t idesc = tc_instr_desc(TC_BM, BN);
    const bool leader = tc_elect_one();
    const uint32_t tiles_addr = tc_smem(tiles);
    uint32_t it = 0;
    bool ok = true;
    for (int w = 0; w < n_work && ok; ++w) {
      int tile, kb_lo, kb_hi;
      work_of(w, tile, kb_lo, kb_hi);
      const uint32_t buf = w & 1, use = w >> 1;
      ok = __all_sync(0xffffffffu, tc_mbar_wait(acc_empty0 + 8 * buf, (use & 1) ^ 1));
      if (!ok) {
        if (leader) sx_set_status(status, 4);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
        const uint32_t s = it % STAGES;
        ok = __all_sync(0xffffffffu, tc_mbar_wait(full0 + 8 * s, (it / STAGES) & 1));
        if (!ok) {
          if (leader) sx_set_status(status, 2);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t a_addr = tiles_addr + s * STAGE_BYTES;
        const uint64_t da = tc_smem_desc(a_addr), db = tc_smem_desc(a_addr + TC_A_BYTES);
        const uint32_t acc = kb != kb_lo;
        if (leader) {
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)          // 32 bytes further along K: 2 in the descriptor's 16-byte units
            tc_mma(d_tmem, da + 2 * k, db + 2 * k, idesc, acc | (k != 0));
          tc_commit(empty0 + 8 * s);
        }
        __syncwarp();
      }
      if (leader) tc_commit(acc_full0 + 8 * buf);
      __syncwarp();
    }
  } else {
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;                                    // 0..127 among the epilogue threads
    // a partial tile in the workspace: [tile among the cut ones][piece][128 rows][BN columns] float32
    auto ws_of = [&](int tile, int z) { return piece_ws + ((size_t)(tile - n_whole) * zmax + z) * (TC_BM * BN); };
    // a finished accumulator -> out, with the epilogue
    auto finish_tile = [&](int w, int tile) -> bool {
      const uint32_t buf = w & 1, use = w >> 1;
      const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * tile_n;
      const int row = m0 + quarter * 32 + lane;
      // (head preparation: where this thread's token goes is looked up while the tile's MMAs still run)
      const bool live = row < M;
      int pos = 0, page = -1;
      if (EPI == TC_EPI_QKV && live) {
        pos = qk.positions[row];
        page = qk.block_table[(size_t)qk.seq_of_token[row] * qk.maxp + (pos >> 6)];
      }
      if (!tc_mbar_wait(acc_full0 + 8 * buf, use & 1)) {
        if (lane == 0) sx_set_status(status, 3);
        return false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t t_row = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      if (EPI == TC_EPI_QKV) {
        // head preparation: this thread's token, the tile's two heads one after the other
        const bool page_ok = page >= 0 && page < qk.n_pages;
        {
          const int hh = (warp - 2) >> 2;                 // warps 2-5 take the tile's first head, warps 6-9 its second
          const int head = n0 / 128 + hh;
          float x[128];
#pragma unroll
          for (int c = 0; c < 4; ++c) tc_ld32(t_row + hh * 128 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&x[c * 32]));
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int i = 0; i < 128; ++i) x[i] = __bfloat162float(__float2bfloat16_rn(x[i]));
          // this warp's part of the accumulator is in registers: hand it back
          asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
          __syncwarp();
          if (lane == 0) tc_mbar_arrive(acc_empty0 + 8 * buf);
          const bool is_q = head < qk.nh, is_k = !is_q && head < qk.nh + qk.nkv, is_v = !is_q && !is_k && head < qk.nh + 2 * qk.nkv;
          bf16* dst = nullptr;
          if (live) {
            if (is_q) {
              dst = qk.q_out + ((size_t)row * qk.nh + head) * 128;
            } else if (is_k || is_v) {
              bf16* base = is_k ? qk.k_pages : qk.v_pages;
              const int kvh = is_k ? head - qk.nh : head - qk.nh - qk.nkv;
              if (base && page_ok) dst = base + (((size_t)page * qk.nkv + kvh) * SX_PAGE + (pos & 63)) * 128;
            }
          }
          if (!dst) return true;
          if (is_q || is_k) {
            // (four sums side by side: this thread has no other warp to hide behind; every index a constant, so that
            //  the head stays in registers)
            const float* w = is_q ? qk.wq : qk.wk;
            float inv = 1.f;
            if (w) {
              float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
              for (int i = 0; i < 128; i += 4) {
                s0 += x[i] * x[i]; s1 += x[i + 1] * x[i + 1]; s2 += x[i + 2] * x[i + 2]; s3 += x[i + 3] * x[i + 3];
              }
              inv = rsqrtf(((s0 + s1) + (s2 + s3)) / 128.f + qk.eps);
            }
            const float4* cs4 = qk.cs ? reinterpret_cast<const float4*>(qk.cs + (size_t)row * 64) : nullptr;
            const float4* sn4 = qk.cs ? reinterpret_cast<const float4*>(qk.sn + (size_t)row * 64) : nullptr;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float4 glo = make_float4(1.f, 1.f, 1.f, 1.f), ghi = glo, c4 = glo, s4 = make_float4(0.f, 0.f, 0.f, 0.f);
              if (w) {
                glo = *reinterpret_cast<const float4*>(w + 4 * i);
                ghi = *reinterpret_cast<const float4*>(w + 64 + 4 * i);
              }
              if (cs4) { c4 = cs4[i]; s4 = sn4[i]; }
              const float gl[4] = {glo.x, glo.y, glo.z, glo.w}, gh[4] = {ghi.x, ghi.y, ghi.z, ghi.w};
              const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float a = x[4 * i + j] * inv * gl[j], bb = x[64 + 4 * i + j] * inv * gh[j];
                x[4 * i + j] = a * cc[j] - bb * sv[j];
                x[64 + 4 * i + j] = a * sv[j] + bb * cc[j];
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            uint4 pk;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(x[8 * i], x[8 * i + 1]), t1 = __floats2bfloat162_rn(x[8 * i + 2], x[8 * i + 3]);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(x[8 * i + 4], x[8 * i + 5]), t3 = __floats2bfloat162_rn(x[8 * i + 6], x[8 * i + 7]);
            pk.x = *reinterpret_cast<uint32_t*>(&t0); pk.y = *reinterpret_cast<uint32_t*>(&t1);
            pk.z = *reinterpret_cast<uint32_t*>(&t2); pk.w = *reinterpret_cast<uint32_t*>(&t3);
            reinterpret_cast<uint4*>(dst)[i] = pk;
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < tile_n; c0 += 32) {
          uint32_t v[32], u[32];
          tc_ld32(t_row + c0, v);
          if (EPI == TC_EPI_SILU_MUL) tc_ld32(t_row + BN / 2 + c0, u);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (c0 + 32 >= tile_n) {
            // everything of this accumulator is in registers: hand it back before the last stores
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(acc_empty0 + 8 * buf);
          }
          if (row < M && n0 + c0 < n_out) tc_store_chunk<EPI>(v, u, out, row, n0 + c0, n_out);
        }
      }
      return true;
    };
    bool alive = true;
    // 1: this block's pieces.  A piece that is a whole tile is finished at once; the others leave their raw
    // accumulators (all BN columns) in the workspace and are counted.  Nobody waits yet: a block stores ALL its
    // pieces first, so that no block's second piece waits behind its neighbour's first.
    for (int w = 0; w < n_pc && alive; ++w) {
      const int tile = pc[w].tile;
      if (pc[w].nz == 1) { alive = finish_tile(w, tile); continue; }
      const uint32_t buf = w & 1, use = w >> 1;
      const int m0 = (tile % tiles_m) * TC_BM;
      const int row = m0 + quarter * 32 + lane;
      if (!tc_mbar_wait(acc_full0 + 8 * buf, use & 1)) {
        if (lane == 0) sx_set_status(status, 3);
        alive = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t t_row = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      float* dst = ws_of(tile, pc[w].z) + (size_t)(quarter * 32 + lane) * BN;
      // (four tcgen05.ld on the way per wait)
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 128) {
        uint32_t v[4][32];
#pragma unroll
        for (int j = 0; j < 4; ++j) tc_ld32(t_row + c0 + 32 * j, v[j]);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (c0 + 128 >= BN) {
          asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
          __syncwarp();
          if (lane == 0) tc_mbar_arrive(acc_empty0 + 8 * buf);
        }
        if (row < M) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(dst + c0 + 32 * j)[i] = make_float4(__uint_as_float(v[j][4 * i]), __uint_as_float(v[j][4 * i + 1]),
                                                                            __uint_as_float(v[j][4 * i + 2]), __uint_as_float(v[j][4 * i + 3]));
        }
      }
      if (coop) {
        __threadfence();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");                 // the four epilogue warps
        if (threadIdx.x == 64) atomicAdd(piece_count + 2 * (tile - n_whole), 1);
      }
    }
    // 2: the blocks that hold the pieces of one tile add its partial tiles up together: each waits (bounded)
    // until all of them have stored theirs, then takes a share of the tile's rows and adds the partial tiles
    // in piece order, with the epilogue.  All pieces are computed first thing by blocks that are resident
    // together, so the wait is short, and the MMAs of this block's first whole tile run meanwhile.
    // piece_count[2 t], [2 t + 1] count arrivals and departures at tile t; the last block to leave zeroes both.
    // (Without whole tiles to hide behind, coop == 0, a second kernel adds up instead: tc_pieces_reduce_kernel.)
    for (int w = 0; w < n_pc && alive && coop; ++w) {
      if (pc[w].nz == 1) continue;
      const int tile = pc[w].tile, nz = pc[w].nz, z = pc[w].z;
      int* cnt = piece_count + 2 * (tile - n_whole);
      if (threadIdx.x == 64) {
        bool all = false;
        for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
          int v;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(cnt) : "memory");
          if (v >= nz) { all = true; break; }
        }
        if (!all) sx_set_status(status, 5);
        *piece_ok = all;
      }
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      if (*piece_ok) {
        __threadfence();
        const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * tile_n;
        const int rows_here = min(TC_BM, M - m0);
        const int per = (rows_here + nz - 1) / nz;
        const int r_lo = m0 + z * per, r_hi = min(m0 + rows_here, r_lo + per);
        const int cols = min(tile_n, n_out - n0);                        // output columns of this tile
        constexpr int TPR = EPI == TC_EPI_SILU_MUL ? 32 : 64;            // threads a row (four columns a thread)
        constexpr int RPI = 128 / TPR;                                   // rows at a time
        const int c4 = (et % TPR) * 4;
        const float* base = ws_of(tile, 0);
        const size_t plane = (size_t)TC_BM * BN;
        // TC_RED_ROWS of a thread's rows at a time and four pieces unrolled, so that dozens of loads are in flight:
        // this adding-up runs on 128 threads a block, and with 8 loads in flight it took 40 us for a tile cut
        // into 13 pieces (longer than the 26 us of MMAs it is meant to hide behind)
        for (int rb = r_lo + et / TPR; rb < r_hi && c4 < cols; rb += TC_RED_ROWS * RPI) {
          float4 a[TC_RED_ROWS], b[TC_RED_ROWS];
#pragma unroll
          for (int i = 0; i < TC_RED_ROWS; ++i) a[i] = b[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
          for (int zz = 0; zz < nz; ++zz) {
#pragma unroll
            for (int i = 0; i < TC_RED_ROWS; ++i) {
              const int r = rb + i * RPI;
              if (r < r_hi) {
                const float* p = base + zz * plane + (size_t)(r - m0) * BN + c4;
                const float4 f = __ldcg(reinterpret_cast<const float4*>(p));
                a[i].x += f.x; a[i].y += f.y; a[i].z += f.z; a[i].w += f.w;
                if (EPI == TC_EPI_SILU_MUL) {
                  const float4 h = __ldcg(reinterpret_cast<const float4*>(p + BN / 2));
                  b[i].x += h.x; b[i].y += h.y; b[i].z += h.z; b[i].w += h.w;
                }
              }
            }
          }
#pragma unroll
          for (int i = 0; i < TC_RED_ROWS; ++i) {
            const int r = rb + i * RPI;
            if (r >= r_hi) continue;
            float o[4] = {a[i].x, a[i].y, a[i].z, a[i].w};
            if (EPI == TC_EPI_SILU_MUL) {
              const float u[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
#pragma unroll
              for (int j = 0; j < 4; ++j) o[j] = o[j] / (1.f + __expf(-o[j])) * u[j];
            }
            const size_t at = (size_t)r * n_out + n0 + c4;
            const bool vec = c4 + 3 < cols && (n_out & 3) == 0;
            if (EPI == TC_EPI_F32) {
              float* dst = reinterpret_cast<float*>(out) + at;
              if (vec) *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
              else
#pragma unroll
                for (int j = 0; j < 4; ++j) if (c4 + j < cols) dst[j] = o[j];
            } else {
              bf16* dst = reinterpret_cast<bf16*>(out) + at;
              if (vec) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
                uint2 pkd;
                pkd.x = *reinterpret_cast<uint32_t*>(&lo); pkd.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst) = pkd;
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) if (c4 + j < cols) dst[j] = __float2bfloat16_rn(o[j]);
              }
            }
          }
        }
      }
      asm volatile("bar.sync 1, 128;\n" ::: "memory");                   // everyone has read; piece_ok is free again
      if (threadIdx.x == 64 && *piece_ok) {
        if (atomicAdd(cnt + 1, 1) == nz - 1) { cnt[1] = 0; __threadfence(); cnt[0] = 0; }
      }
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
    }
    // 3: the whole tiles
    for (int w = n_pc; w < n_work && alive; ++w) {
      alive = finish_tile(w, blockIdx.x + (w - n_pc) * gridDim.x);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
// a [rows, K] row-major bfloat16 matrix as a 2-D tensor map with 128-row x 64-column boxes
static int tc_make_map(CUtensorMap* map, const void* base, int rows, int K) { return tc_make_map_rows(map, base, rows, K, 128); }

static int* tc_status_word() {
  static int* p = nullptr;
  if (!p) p = sx_status_word_alloc();
  return p;
}


template <int EPI, int BN>
static int tc_launch(const CUtensorMap& ma, const CUtensorMap& mw, void* out, int M, int N, int K, int splits,
                     cudaStream_t stream) {
  int* status = tc_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  const int tile_n = (EPI == TC_EPI_SILU_MUL) ? BN / 2 : BN;
  const int n_out = (EPI == TC_EPI_SILU_MUL) ? N / 2 : N;
  dim3 grid((n_out + tile_n - 1) / tile_n, (M + TC_BM - 1) / TC_BM, splits);
  if (grid.y > 65535 || grid.z > 65535) return SX_ERR_SIZE;
  const size_t smem = 1024 + TcShape<BN>::STAGES * TcShape<BN>::STAGE_BYTES + (2 * TcShape<BN>::STAGES + 1) * sizeof(uint64_t) + 16;
  auto kern = gemm_tc_kernel<EPI, BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return sx_launch(kern, grid, dim3(TC_THREADS), smem, stream, ma, mw, out, M, N, K, status);
}

static int tc_sm_count() {
  static int n[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!n[dev]) {
    if (cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n[dev] <= 0) n[dev] = 148;
  }
  return n[dev];
}

// The partial tiles of the cut tiles, added up in piece order, with the epilogue: one thread per (cut tile, row,
// four columns).  Used when the persistent kernel had no whole tiles to hide its own adding-up behind.
template <int EPI, int BN>
__global__ void tc_pieces_reduce_kernel(const float* __restrict__ ws, void* __restrict__ out, int M, int N, int n_whole,
                                        int R, int nkb, int G, int zmax, int sp) {
  pdl_wait();
  pdl_trigger();
  const int n_out = (EPI == TC_EPI_SILU_MUL) ? N / 2 : N;
  const int tile_n = (EPI == TC_EPI_SILU_MUL) ? BN / 2 : BN;
  const int tiles_m = (M + TC_BM - 1) / TC_BM;
  const int per_row = tile_n / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)R * TC_BM * per_row;
  if (idx >= total) return;
  const int t = (int)(idx / (TC_BM * per_row));
  const int rem = (int)(idx - (long long)t * TC_BM * per_row);
  const int rr = rem / per_row, c4 = (rem % per_row) * 4;
  const int tile = n_whole + t;
  const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * tile_n;
  const int r = m0 + rr, cols = min(tile_n, n_out - n0);
  if (r >= M || c4 >= cols) return;
  TcPlan p;
  p.n_whole = n_whole; p.R = R; p.nkb = nkb; p.G = G; p.sp = sp; p.U = (long long)R * nkb;
  const int nz = p.block_of((long long)(t + 1) * nkb - 1) - p.block_of((long long)t * nkb) + 1;      // (stream-K shares: sp == 0 here)
  if (nz == 1) return;                               // that tile was one block's and is finished
  const float* src = ws + ((size_t)t * zmax) * (TC_BM * BN) + (size_t)rr * BN + c4;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
  for (int z = 0; z < nz; ++z) {
    const float4 f = *reinterpret_cast<const float4*>(src + (size_t)z * (TC_BM * BN));
    a.x += f.x; a.y += f.y; a.z += f.z; a.w += f.w;
    if (EPI == TC_EPI_SILU_MUL) {
      const float4 h = *reinterpret_cast<const float4*>(src + (size_t)z * (TC_BM * BN) + BN / 2);
      b.x += h.x; b.y += h.y; b.z += h.z; b.w += h.w;
    }
  }
  float o[4] = {a.x, a.y, a.z, a.w};
  if (EPI == TC_EPI_SILU_MUL) {
    const float u[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = o[j] / (1.f + __expf(-o[j])) * u[j];
  }
  const size_t at = (size_t)r * n_out + n0 + c4;
  const bool vec = c4 + 3 < cols && (n_out & 3) == 0;
  if (EPI == TC_EPI_F32) {
    float* dst = reinterpret_cast<float*>(out) + at;
    if (vec) *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
    else
      for (int j = 0; j < 4; ++j) if (c4 + j < cols) dst[j] = o[j];
  } else {
    bf16* dst = reinterpret_cast<bf16*>(out) + at;
    if (vec) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
      uint2 pkd;
      pkd.x = *reinterpret_cast<uint32_t*>(&lo); pkd.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst) = pkd;
    } else {
      for (int j = 0; j < 4; ++j) if (c4 + j < cols) dst[j] = __float2bfloat16_rn(o[j]);
    }
  }
}

// What the persistent kernel does for a product: how many tiles are computed whole, how many are cut, the most
// pieces a cut tile has, and the grid.
struct TcHostPlan { int n_whole, R, zmax, G, sp; };
// Several rows of tiles that are fewer than the SMs (a prompt step of a few hundred rows: 512 x 2,560 has 40
// tiles) can be cut over K as well.  Whole tiles leave most SMs idle and take 5 + 0.352 us x slices whatever their
// number (a 128 x 256 tile with K = 4,096: 27.5 us, K = 9,728: 58.5 us), and the uniform split over K in 128-wide
// tiles (sx_gemm_tc with splits > 1) took 40 us for 512 x 2,560 x 4,096 and 69 us for K = 9,728.  Cut into G
// shares the same products take about 6.5 + 0.352 x slices / G + 0.07 G us (the last term: G partial tiles written
// and read again by the second kernel): 23.5 and 37 us for the two products above.
// The figures are measured on a B200 with the weights coming from HBM; a product is cut only when the estimate is
// a tenth below the whole tiles'.  Not for a handful of tiles (the uniform split is faster up to a dozen).  The
// pieces of the row tiles over one block of W run at different times, so W is read once per row of tiles, from HBM
// when L2 cannot keep it (5,120 x 25,600 at 512 rows: 196 us cut, 153 us whole): for a matrix larger than half
// of L2 the estimate is at least that traffic's time.
static int g_tc_cut_few = 1;
extern "C" void sx_gemm_tc_cut_few(int on) { g_tc_cut_few = on ? 1 : 0; }
static bool tc_cut_few(int tiles_m, int n_tiles, int nkb, long long U, long long w_bytes, int sms, int* G) {
  if (!g_tc_cut_few || tiles_m <= 1 || n_tiles >= sms || n_tiles <= 12) return false;
  // a matrix larger than half of L2 comes from HBM once per row of tiles
  const double t_hbm = w_bytes > (64LL << 20) ? (double)tiles_m * (double)w_bytes / 6.0e6 : 0.0;
  // every tile into the same number of pieces, so that no block's share begins in one tile and ends in the next
  // (a block with two pieces stores two partial tiles: 30 tiles in 97 shares took 24.4 us, in 120 shares 18.4 us)
  const double t_whole = 5.0 + 0.352 * nkb;
  double best = 0.9 * t_whole;
  int pieces = 0;
  for (int z = 2; z * n_tiles <= sms && z <= nkb; ++z) {
    double t_cut = 6.5 + 0.352 * (double)nkb / z + 0.07 * z * n_tiles;
    if (t_cut < t_hbm + 6.5) t_cut = t_hbm + 6.5;
    if (t_cut < best) { best = t_cut; pieces = z; }
  }
  if (!pieces) return false;
  *G = pieces * n_tiles;
  return true;
}

static TcHostPlan tc_plan_stream(int M, int N, int K, int epi, bool allow_cut) {
  const int tile_n = epi == TC_EPI_SILU_MUL ? 128 : 256;
  const int n_out = epi == TC_EPI_SILU_MUL ? N / 2 : N;
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (n_out + tile_n - 1) / tile_n;
  const long long n_tiles_ll = (long long)tiles_m * tiles_n;
  const int sms = tc_sm_count();
  const int nkb = (K + TC_BK - 1) / TC_BK;
  TcHostPlan h;
  h.sp = 0;
  if (n_tiles_ll > 0x3fffffffLL) { h.n_whole = -1; h.R = h.zmax = h.G = 0; return h; }
  const int n_tiles = (int)n_tiles_ll;
  const int R0 = n_tiles >= sms ? n_tiles % sms : n_tiles;
  // cut when the round would be at most half full, or for a single row of tiles (few rows: the partial tiles are small)
  const long long U = (long long)R0 * nkb;
  // (every block must get at least one slice, so that the blocks of a tile are consecutive: with whole tiles
  //  before them the grid is all SMs and there must be that many slices; alone, the grid shrinks to the slices)
  // Fewer tiles than SMs are cut only when they are at least half as many (each then falls into two or three
  // pieces); a handful of tiles would fall into a dozen pieces each, and the older uniform split (sx_gemm_tc with
  // splits > 1: 128-wide tiles, fewer and larger partial tiles) measured faster there.
  // Behind three or more rounds of whole tiles a short last round costs little, and cutting it did not pay
  // (gate/up at 2,048 rows: 1,216 tiles, 164 us cut against 155 us whole).
  int G_few = 0;
  const bool few = tc_cut_few(tiles_m, n_tiles, nkb, U, (long long)N * K * 2, sms, &G_few);
  // Behind whole tiles a piece costs its share of a tile's slices and about 8.6 us for the partial tiles' trip and the
  // adding up (by the four epilogue warps, before their whole tile's epilogue); that has to stay well under the
  // round of whole tiles it saves (1,024 x 6,144 x 2,560, 44 tiles in three pieces each: 40.1 us cut, 34.7 whole;
  // the same rows x 6,144 x 4,096: 48.2 cut, 52.3 whole).
  bool last_round_pays = false;
  if (n_tiles >= sms && R0 > 0) {
    int sp = sms / R0;
    if (sp > nkb) sp = nkb;
    last_round_pays = 5.0 + 0.352 * nkb / sp + 8.6 < 0.8 * (5.0 + 0.352 * nkb);
  }
  const bool cut = allow_cut && R0 > 0 && nkb >= 2 && R0 < sms &&
                   (n_tiles >= sms ? (2 * R0 <= sms && U >= sms && n_tiles < 3 * sms && last_round_pays)
                                   : ((tiles_m == 1 && 2 * R0 >= sms) || few));
  if (!cut) { h.n_whole = n_tiles; h.R = 0; h.zmax = 0; h.G = n_tiles < sms ? n_tiles : sms; return h; }
  h.n_whole = n_tiles - R0; h.R = R0; h.G = U < sms ? (int)U : sms;
  if (few && n_tiles < sms && tiles_m > 1 && G_few < h.G) h.G = G_few;
  // (a second kernel adds these up: the blocks of a tile adding up among themselves, as behind whole tiles, took 7 to
  //  10 us longer here, 512 x 2,560 x 4,096: 30.4 against 20.5 us, with nothing to hide behind and 128 threads a block)
  if (h.n_whole > 0) {                               // equal pieces per tile, one piece a block
    h.sp = sms / R0;
    if (h.sp > nkb) h.sp = nkb;
    h.zmax = h.sp;
    return h;
  }
  TcPlan p;
  p.n_whole = h.n_whole; p.R = R0; p.nkb = nkb; p.G = h.G; p.sp = 0; p.U = U;
  h.zmax = 1;
  for (int t = 0; t < R0; ++t) {
    const int nz = p.block_of((long long)(t + 1) * nkb - 1) - p.block_of((long long)t * nkb) + 1;
    if (nz > h.zmax) h.zmax = nz;
  }
  return h;
}

// n_whole, cut tiles, most pieces a tile, grid: what sx_gemm_tc will do with a workspace (out4[1] * out4[2] * 128 * 256 floats)
extern "C" int sx_gemm_tc_plan(int M, int N, int K, int epi, int* out4) {
  if (M <= 0 || N <= 0 || K <= 0) return SX_ERR_SIZE;
  const TcHostPlan h = tc_plan_stream(M, N, K, epi, true);
  if (h.n_whole < 0) return SX_ERR_SIZE;
  out4[0] = h.n_whole; out4[1] = h.R; out4[2] = h.zmax; out4[3] = h.G;
  return 0;
}

template <int EPI, int BN>
static int tc_launch_persistent(const CUtensorMap& ma, const CUtensorMap& mw, void* out, int M, int N, int K,
                                const TcHostPlan& h, float* ws, int* counts, cudaStream_t stream, const TcQkv& qk = TcQkv()) {
  int* status = tc_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  if (h.n_whole < 0 || h.G <= 0) return SX_ERR_SIZE;
  const size_t smem = 1024 + TcShape<BN>::STAGES * TcShape<BN>::STAGE_BYTES + (2 * TcShape<BN>::STAGES + 4) * sizeof(uint64_t) + 32;
  auto kern = gemm_tc_persistent_kernel<EPI, BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  // with whole tiles after them, the blocks of a cut tile add up inside the kernel; without, a second kernel does
  int rc = sx_launch(kern, h.G, dim3(TcThreads<EPI>::N), smem, stream, ma, mw, out, M, N, K, h.n_whole, h.zmax, h.sp, ws, counts, status, qk);
  if (rc || h.R == 0 || h.sp > 0 || EPI == TC_EPI_QKV) return rc;
  const int tile_n = (EPI == TC_EPI_SILU_MUL) ? BN / 2 : BN;
  const long long total = (long long)h.R * TC_BM * (tile_n / 4);
  return sx_launch(tc_pieces_reduce_kernel<EPI, BN>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const float*)ws, out,
                   M, N, h.n_whole, h.R, (K + TC_BK - 1) / TC_BK, h.G, h.zmax, 0);
}

// sum of the split-K partial tiles ws[splits][M][N] in split order, then the epilogue
template <int EPI>
// (out has rows of ldo values: a block of a larger matrix when ldo > the block's width)
__global__ void tc_splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ out, int splits, int M, int N,
                                        long long ldo) {
  pdl_wait();
  pdl_trigger();
  const int n_out = (EPI == TC_EPI_SILU_MUL) ? N / 2 : N;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)M * n_out) return;
  const size_t m = idx / n_out;
  const int n = (int)(idx - m * n_out);
  const size_t plane = (size_t)M * N;
  float a = 0.f, b = 0.f;
  for (int z = 0; z < splits; ++z) {
    a += ws[z * plane + m * N + n];
    if (EPI == TC_EPI_SILU_MUL) b += ws[z * plane + m * N + n_out + n];
  }
  const size_t o = m * (size_t)ldo + n;
  if (EPI == TC_EPI_SILU_MUL) reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(a / (1.f + expf(-a)) * b);
  else if (EPI == TC_EPI_F32) reinterpret_cast<float*>(out)[o] = a;
  else reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(a);
}

// K split over `splits` blocks per 128 x 128 tile, float32 partial tiles in `workspace` [splits, M, N], then the sum
// in split order with the epilogue into out (rows of ldo values)
static int tc_split_product(const void* A, const void* W, void* out, int M, int N, int K, int epi, int splits,
                            float* workspace, long long ldo, cudaStream_t stream) {
  CUtensorMap ma, mw;
  int rc = tc_make_map(&ma, A, M, K);
  if (rc) return rc;
  if ((rc = tc_make_map(&mw, W, N, K))) return rc;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  if (splits > nkb) splits = nkb;
  const int kper = (nkb + splits - 1) / splits;
  splits = (nkb + kper - 1) / kper;                 // no empty range
  rc = tc_launch<TC_EPI_PARTIAL, 128>(ma, mw, workspace, M, N, K, splits, stream);
  if (rc) return rc;
  const size_t n_elems = (size_t)M * (epi == TC_EPI_SILU_MUL ? N / 2 : N);
  const unsigned grid = (unsigned)((n_elems + 255) / 256);
  switch (epi) {
    case TC_EPI_BF16: return sx_launch(tc_splitk_reduce_kernel<TC_EPI_BF16>, dim3(grid), dim3(256), 0, stream, (const float*)workspace, out, splits, M, N, ldo);
    case TC_EPI_F32: return sx_launch(tc_splitk_reduce_kernel<TC_EPI_F32>, dim3(grid), dim3(256), 0, stream, (const float*)workspace, out, splits, M, N, ldo);
    case TC_EPI_SILU_MUL: return sx_launch(tc_splitk_reduce_kernel<TC_EPI_SILU_MUL>, dim3(grid), dim3(256), 0, stream, (const float*)workspace, out, splits, M, N, ldo);
    default: return SX_ERR_DTYPE;
  }
}

// A [M, K], W [N, K] bfloat16 row-major, 16-byte aligned, K % 8 == 0.
// epi 0: out bf16 [M, N]; 1: out f32 [M, N]; 2: W = [gate; up] stacked, out bf16 [M, N/2].
// splits == 1: the persistent kernel over 128 x 256 tiles, epilogue in the kernel.  With a workspace it cuts the
//   tiles that would not fill a round of all SMs over K (sx_gemm_tc_plan says how): `workspace` holds
//   ws_floats >= cut tiles * most pieces a tile * 128 * 256 floats, `counts` 2 * cut tiles ints that are zero
//   (the kernel leaves them zero).  Without a workspace every tile is computed whole.
// splits > 1: 128 x 128 tiles, K split over `splits` blocks whose float32 partial tiles go to `workspace`
//   [splits, M, N] and are added, in split order, by a second kernel that applies the epilogue.  Every split
//   gets a non-empty range of K.
extern "C" int sx_gemm_tc(const void* A, const void* W, void* out, int M, int N, int K, int epi, int splits,
                          float* workspace, unsigned long long ws_floats, int* counts, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || splits < 1) return SX_ERR_SIZE;
  if (epi == TC_EPI_SILU_MUL && (N & 1)) return SX_ERR_SIZE;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return SX_ERR_ALIGN;
  if (splits > 1) {
    if (!workspace || ws_floats < (unsigned long long)splits * M * N) return SX_ERR_SIZE;
    return tc_split_product(A, W, out, M, N, K, epi, splits, workspace, epi == TC_EPI_SILU_MUL ? N / 2 : N, stream);
  }
  CUtensorMap ma, mw;
  int rc = tc_make_map(&ma, A, M, K);
  if (rc) return rc;
  rc = tc_make_map(&mw, W, N, K);
  if (rc) return rc;
  TcHostPlan h = tc_plan_stream(M, N, K, epi, workspace != nullptr && counts != nullptr);
  if (h.R > 0 && (ws_floats < (unsigned long long)h.R * h.zmax * TC_BM * 256 || ((uintptr_t)workspace & 15))) return SX_ERR_SIZE;
  switch (epi) {
    // (128-wide tiles were tried for shapes whose last wave is nearly empty: the MMA then waits on
    //  shared-memory reads of A and the product got slower, 607 against 828 TFLOP/s)
    case TC_EPI_BF16: return tc_launch_persistent<TC_EPI_BF16, 256>(ma, mw, out, M, N, K, h, workspace, counts, stream);
    case TC_EPI_F32: return tc_launch_persistent<TC_EPI_F32, 256>(ma, mw, out, M, N, K, h, workspace, counts, stream);
    case TC_EPI_SILU_MUL: return tc_launch_persistent<TC_EPI_SILU_MUL, 256>(ma, mw, out, M, N, K, h, workspace, counts, stream);
    default: return SX_ERR_DTYPE;
  }
}

// The fused q/k/v projection of a prompt step with its head preparation as the epilogue (see TcQkv): A [M, K], W [N, K] with
// N = (nh + 2 nkv) * 128 a multiple of 256; q_out [M, nh * 128]; k_pages / v_pages [n_pages, nkv, 64, 128] (null: nothing is
// written to the cache); wq / wk [128] (null: no norm); cs / sn [M, 64] (null: no rotation).  All tiles are computed whole.
extern "C" int sx_gemm_tc_qkv(const void* A, const void* W, int M, int N, int K, void* q_out, void* k_pages, void* v_pages,
                              const float* wq, const float* wk, const float* cs, const float* sn, const int* positions,
                              const int* seq_of_token, const int* block_table, int maxp, int nh, int nkv, int n_pages,
                              float eps, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K <= 0 || (K & 7) || nh <= 0 || nkv <= 0 || N != (nh + 2 * nkv) * 128 || (N & 255) || !q_out || (!cs) != (!sn)) return SX_ERR_SIZE;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)q_out & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) ||
      ((uintptr_t)wq & 15) || ((uintptr_t)wk & 15) || ((uintptr_t)cs & 15) || ((uintptr_t)sn & 15))
    return SX_ERR_ALIGN;
  CUtensorMap ma, mw;
  int rc = tc_make_map(&ma, A, M, K);
  if (rc) return rc;
  if ((rc = tc_make_map(&mw, W, N, K))) return rc;
  const TcHostPlan h = tc_plan_stream(M, N, K, TC_EPI_BF16, false);
  TcQkv qk;
  qk.q_out = (bf16*)q_out; qk.k_pages = (bf16*)k_pages; qk.v_pages = (bf16*)v_pages; qk.wq = wq; qk.wk = wk; qk.cs = cs; qk.sn = sn;
  qk.positions = positions; qk.seq_of_token = seq_of_token; qk.block_table = block_table;
  qk.maxp = maxp; qk.nh = nh; qk.nkv = nkv; qk.n_pages = n_pages; qk.eps = eps;
  return tc_launch_persistent<TC_EPI_QKV, 256>(ma, mw, nullptr, M, N, K, h, nullptr, nullptr, stream, qk);
}

// 0, or which bounded wait ran out (1 producer, 2 and 4 MMA issuer, 3 epilogue, 5 the blocks of a cut tile waiting for one another)
// Reads the word in host memory: no device call.  It tells of kernels the host has already waited for.
// With reset != 0 the word goes back to 0.
extern "C" int sx_gemm_tc_status(int* host_value, int reset) {
  int* p = tc_status_word();
  if (!p) return (int)cudaErrorMemoryAllocation;
  *host_value = *(volatile int*)p;
  if (reset) *(volatile int*)p = 0;
  return 0;
}
