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
#include <cuda.h>
#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_A_BYTES (TC_BM * TC_BK * 2)            // 16 KB
#define TC_THREADS 192
#define TC_SPIN_LIMIT (1u << 26)

enum { TC_EPI_BF16 = 0, TC_EPI_F32 = 1, TC_EPI_SILU_MUL = 2, TC_EPI_PARTIAL = 3 };

// BN: columns of W per block (256, or 128 for the split-K form); stages fill the shared memory
template <int BN> struct TcShape {
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
};

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tc_tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);          // start address, 16-byte units
  d |= (uint64_t)1 << 16;                         // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                         // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
  return d;
}
// instruction descriptor: D f32, A and B bf16, both K-major, N and M of the instruction
__host__ __device__ constexpr uint32_t tc_instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

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
        if (!tc_mbar_wait(empty0 + 8 * s, ((kb / TC_STAGES) & 1) ^ 1)) { atomicExch(status, 1); break; }
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
        if (!tc_mbar_wait(full0 + 8 * s, (kb / TC_STAGES) & 1)) { atomicExch(status, 2); ok = false; break; }
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
      if (lane == 0) atomicExch(status, 3);
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
// acc_full/acc_empty per accumulator.
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

template <int EPI, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                           const __grid_constant__ CUtensorMap map_w,
                                                                           void* __restrict__ out, int M, int N, int K,
                                                                           int tail_tiles, int tail_splits,
                                                                           float* __restrict__ tail_ws,
                                                                           int* __restrict__ tail_count,
                                                                           int* __restrict__ status) {
  constexpr int STAGES = TcShape<BN>::STAGES, B_BYTES = TcShape<BN>::B_BYTES, STAGE_BYTES = TcShape<BN>::STAGE_BYTES;
  extern __shared__ unsigned char tc_smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);   // full[S], empty[S], acc_full[2], acc_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* tail_last = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + STAGES);
  const uint32_t acc_full0 = tc_smem(bars + 2 * STAGES), acc_empty0 = tc_smem(bars + 2 * STAGES + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_out = (EPI == TC_EPI_SILU_MUL) ? N / 2 : N;
  const int tile_n = (EPI == TC_EPI_SILU_MUL) ? BN / 2 : BN;
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (n_out + tile_n - 1) / tile_n;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  // Work items.  Each of the last tail_tiles tiles (the bottom of the last column of tiles) is cut into
  // tail_splits items that take a range of K each and leave a float32 partial tile in tail_ws [split][rows
  // of the tail][columns of the last column of tiles]; the blocks of a tile's items then add the partial
  // tiles up together, in split order.  These short items come FIRST (one round, padded to the grid), the
  // whole tiles after them, so that the adding-up hides behind the next tile's MMAs.
  const int n_full = tiles_m * tiles_n - tail_tiles;
  const int n_tail_items = tail_tiles * tail_splits;
  const int tail_round = n_tail_items > 0 ? ((n_tail_items + (int)gridDim.x - 1) / (int)gridDim.x) * (int)gridDim.x : 0;
  const int n_items = tail_round + n_full;
  const int tail_kper = tail_splits > 0 ? (nkb + tail_splits - 1) / tail_splits : nkb;
  // false: a padding item, nothing to do
  auto item_of = [&](int item, int& tile, int& kb_lo, int& kb_hi, int& z) -> bool {
    if (item >= tail_round) { tile = item - tail_round; kb_lo = 0; kb_hi = nkb; z = -1; return true; }
    if (item >= n_tail_items) return false;
    tile = n_full + item / tail_splits;
    z = item % tail_splits;
    kb_lo = z * tail_kper;
    kb_hi = min(nkb, kb_lo + tail_kper);
    return true;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc_mbar_init(full0 + 8 * s, 1);
      tc_mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc_mbar_init(acc_full0 + 8 * b, 1);
      tc_mbar_init(acc_empty0 + 8 * b, 4);          // one arrival per epilogue warp
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

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        int tile, kb_lo, kb_hi, z;
        if (!item_of(item, tile, kb_lo, kb_hi, z)) continue;
        const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * tile_n;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          if (!tc_mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1)) { atomicExch(status, 1); ok = false; break; }
          tc_mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
          const uint32_t a_dst = tc_smem(tiles + s * STAGE_BYTES), b_dst = a_dst + TC_A_BYTES;
          tc_tma_load_2d(a_dst, &map_a, kb * TC_BK, m0, full0 + 8 * s);
          tc_tma_load_2d(b_dst, &map_w, kb * TC_BK, n0, full0 + 8 * s);
          if (BN == 256)
            tc_tma_load_2d(b_dst + B_BYTES / 2, &map_w, kb * TC_BK, (EPI == TC_EPI_SILU_MUL) ? N / 2 + n0 : n0 + BN / 2, full0 + 8 * s);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc_instr_desc(TC_BM, BN);
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        int tile, kb_lo, kb_hi, z;
        if (!item_of(item, tile, kb_lo, kb_hi, z)) continue;
        const uint32_t buf = t & 1, use = t >> 1;
        ++t;
        if (!tc_mbar_wait(acc_empty0 + 8 * buf, (use & 1) ^ 1)) { atomicExch(status, 4); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          if (!tc_mbar_wait(full0 + 8 * s, (it / STAGES) & 1)) { atomicExch(status, 2); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_addr = tc_smem(tiles + s * STAGE_BYTES), b_addr = a_addr + TC_A_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)
            tc_mma(d_tmem, tc_smem_desc(a_addr + k * 32), tc_smem_desc(b_addr + k * 32), idesc, kb != kb_lo || k != 0);
          tc_commit(empty0 + 8 * s);
        }
        tc_commit(acc_full0 + 8 * buf);
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    uint32_t t = 0;
    // the tail's block of the output: rows from tail_m0 on, the last column of tiles
    const int tail_m0 = (tiles_m - tail_tiles) * TC_BM, tail_n0 = (tiles_n - 1) * tile_n;
    const int tail_rows = M - tail_m0, tail_cols = n_out - tail_n0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      int tile, kb_lo, kb_hi, z;
      if (!item_of(item, tile, kb_lo, kb_hi, z)) continue;
      const uint32_t buf = t & 1, use = t >> 1;
      ++t;
      const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * tile_n;
      const int row = m0 + quarter * 32 + lane;
      if (!tc_mbar_wait(acc_full0 + 8 * buf, use & 1)) {
        if (lane == 0) atomicExch(status, 3);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t t_row = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
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
        if (row < M && n0 + c0 < n_out) {
          if (z < 0) tc_store_chunk<EPI>(v, u, out, row, n0 + c0, n_out);
          else tc_store_chunk<TC_EPI_F32>(v, u, tail_ws + (size_t)z * tail_rows * tail_cols, row - tail_m0, c0, tail_cols);
        }
      }
      if (z >= 0) {
        // The blocks that hold the items of one tile add its partial tiles up together: each waits (bounded)
        // until all of them have stored theirs, then takes a share of the tile's rows and adds the partial
        // tiles in split order.  All items of the tail run in the same first round on blocks that are
        // resident together, so the wait is short.  tail_count[2 tile], [2 tile + 1] count arrivals and
        // departures; the last block to leave sets both back to zero.
        int* cnt = tail_count + 2 * (tile - n_full);
        __threadfence();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");                 // the four epilogue warps
        if (threadIdx.x == 64) {
          atomicAdd(cnt, 1);
          bool all = false;
          for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(cnt) : "memory");
            if (v >= tail_splits) { all = true; break; }
          }
          if (!all) atomicExch(status, 5);
          *tail_last = all;
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (*tail_last) {
          __threadfence();
          const int et = threadIdx.x - 64;                                // 0..127 among the epilogue threads
          const int per = (TC_BM + tail_splits - 1) / tail_splits;
          const int r_lo = m0 + z * per, r_hi = min(min(m0 + TC_BM, M), r_lo + per);
          const size_t plane = (size_t)tail_rows * tail_cols;
          if ((tail_cols & 3) == 0) {
            // two rows at a time: 64 threads a row, four columns a thread
            const int c4 = (et & 63) * 4;
            // six of a thread's rows at a time, so that 24 loads are in flight (a row at a time took one
            // round trip to L2 per four loads: 18 us for this step, now 3)
            for (int rb = r_lo + (et >> 6); rb < r_hi && c4 < tail_cols; rb += 12) {
              float4 acc[6];
#pragma unroll
              for (int i = 0; i < 6; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
              for (int zz = 0; zz < tail_splits; ++zz) {
#pragma unroll
                for (int i = 0; i < 6; ++i) {
                  const int r = rb + 2 * i;
                  if (r < r_hi) {
                    const float4 f = __ldcg(reinterpret_cast<const float4*>(tail_ws + zz * plane + (size_t)(r - tail_m0) * tail_cols + c4));
                    acc[i].x += f.x; acc[i].y += f.y; acc[i].z += f.z; acc[i].w += f.w;
                  }
                }
              }
#pragma unroll
              for (int i = 0; i < 6; ++i) {
                const int r = rb + 2 * i;
                if (r >= r_hi) continue;
                if (EPI == TC_EPI_F32) {
                  *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)r * n_out + tail_n0 + c4) = acc[i];
                } else {
                  bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)r * n_out + tail_n0 + c4;
                  __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x, acc[i].y), hi = __floats2bfloat162_rn(acc[i].z, acc[i].w);
                  if ((n_out & 3) == 0) {
                    uint2 pkd;
                    pkd.x = *reinterpret_cast<uint32_t*>(&lo); pkd.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst) = pkd;
                  } else {
                    dst[0] = __low2bfloat16(lo); dst[1] = __high2bfloat16(lo); dst[2] = __low2bfloat16(hi); dst[3] = __high2bfloat16(hi);
                  }
                }
              }
            }
          } else {
            for (int r = r_lo; r < r_hi; ++r)
              for (int c = et; c < tail_cols; c += 128) {
                const float* src = tail_ws + (size_t)(r - tail_m0) * tail_cols + c;
                float acc = 0.f;
                for (int zz = 0; zz < tail_splits; ++zz) acc += __ldcg(src + zz * plane);
                if (EPI == TC_EPI_F32) reinterpret_cast<float*>(out)[(size_t)r * n_out + tail_n0 + c] = acc;
                else reinterpret_cast<bf16*>(out)[(size_t)r * n_out + tail_n0 + c] = __float2bfloat16_rn(acc);
              }
          }
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");                 // everyone has read; tail_last is free again
        if (threadIdx.x == 64 && *tail_last) {
          if (atomicAdd(cnt + 1, 1) == tail_splits - 1) { cnt[1] = 0; __threadfence(); cnt[0] = 0; }
        }
      }
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
typedef CUresult (*tc_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static tc_encode_fn tc_get_encode() {
  static tc_encode_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = (tc_encode_fn)p;
  }
  return fn;
}

// a [rows, K] row-major bfloat16 matrix as a 2-D tensor map with 128-row x 64-column boxes
static int tc_make_map(CUtensorMap* map, const void* base, int rows, int K) {
  tc_encode_fn enc = tc_get_encode();
  if (!enc) return SX_ERR_SIZE;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {TC_BK, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

static int* tc_status_word() {
  static int* p = nullptr;
  if (!p) {
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
  }
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

template <int EPI, int BN>
static int tc_launch_persistent(const CUtensorMap& ma, const CUtensorMap& mw, void* out, int M, int N, int K,
                                int tail_tiles, int tail_splits, float* tail_ws, int* tail_count, cudaStream_t stream) {
  int* status = tc_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  const int tile_n = (EPI == TC_EPI_SILU_MUL) ? BN / 2 : BN;
  const int n_out = (EPI == TC_EPI_SILU_MUL) ? N / 2 : N;
  const long long n_tiles = (long long)((n_out + tile_n - 1) / tile_n) * ((M + TC_BM - 1) / TC_BM) - tail_tiles;
  if (n_tiles <= 0 || n_tiles > 0x3fffffffLL) return SX_ERR_SIZE;
  const int sms = tc_sm_count();
  const int grid = (int)(n_tiles < sms ? n_tiles : sms);
  const size_t smem = 1024 + TcShape<BN>::STAGES * TcShape<BN>::STAGE_BYTES + (2 * TcShape<BN>::STAGES + 4) * sizeof(uint64_t) + 32;
  auto kern = gemm_tc_persistent_kernel<EPI, BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return sx_launch(kern, grid, dim3(TC_THREADS), smem, stream, ma, mw, out, M, N, K, tail_tiles, tail_splits, tail_ws, tail_count, status);
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
// splits == 1: the persistent kernel over 128 x 256 tiles, epilogue in the kernel.  With tail_tiles > 0 (epi 0 and 1)
//   each of the LAST tail_tiles tiles (the bottom rows of the last column of tiles; tail_tiles <= row tiles) is
//   computed as tail_splits work items that split K and leave float32 partial tiles in the workspace; the blocks
//   of a tile's items then add them up together, in split order: when the last round of tiles would keep only a
//   few SMs busy, the whole product otherwise takes a full tile's time longer.
// splits > 1 (for few rows, where whole tiles would leave most SMs idle): 128 x 128 tiles, K split over
//   `splits` blocks whose float32 partial tiles go to `workspace` [splits, M, N] and are added, in split
//   order, by a second kernel that applies the epilogue.  Every split gets a non-empty range of K.
// workspace: splits * M * N floats, or tail_splits * (rows of the tail) * (columns of the last column of tiles) floats.
// tail_count: 2 * tail_tiles ints that are zero (the kernel leaves them zero).
extern "C" int sx_gemm_tc(const void* A, const void* W, void* out, int M, int N, int K, int epi, int splits,
                          float* workspace, int tail_tiles, int tail_splits, int* tail_count, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || splits < 1 || tail_tiles < 0) return SX_ERR_SIZE;
  if (epi == TC_EPI_SILU_MUL && (N & 1)) return SX_ERR_SIZE;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return SX_ERR_ALIGN;
  if (splits > 1) {
    if (!workspace || tail_tiles) return SX_ERR_SIZE;
    return tc_split_product(A, W, out, M, N, K, epi, splits, workspace, epi == TC_EPI_SILU_MUL ? N / 2 : N, stream);
  }
  CUtensorMap ma, mw;
  int rc = tc_make_map(&ma, A, M, K);
  if (rc) return rc;
  rc = tc_make_map(&mw, W, N, K);
  if (rc) return rc;
  if (tail_tiles > 0) {
    const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + 255) / 256;
    const int nkb = (K + TC_BK - 1) / TC_BK;
    if (epi == TC_EPI_SILU_MUL || tail_tiles > tiles_m || tail_tiles >= tiles_m * tiles_n || tail_splits < 1 || !workspace || !tail_count)
      return SX_ERR_SIZE;
    if (tail_splits > nkb) tail_splits = nkb;
    const int kper = (nkb + tail_splits - 1) / tail_splits;
    tail_splits = (nkb + kper - 1) / kper;          // no empty range
    return epi == TC_EPI_F32
               ? tc_launch_persistent<TC_EPI_F32, 256>(ma, mw, out, M, N, K, tail_tiles, tail_splits, workspace, tail_count, stream)
               : tc_launch_persistent<TC_EPI_BF16, 256>(ma, mw, out, M, N, K, tail_tiles, tail_splits, workspace, tail_count, stream);
  }
  switch (epi) {
    // (128-wide tiles were tried for shapes whose last wave is nearly empty: the MMA then waits on
    //  shared-memory reads of A and the product got slower, 607 against 828 TFLOP/s)
    case TC_EPI_BF16: return tc_launch_persistent<TC_EPI_BF16, 256>(ma, mw, out, M, N, K, 0, 0, nullptr, nullptr, stream);
    case TC_EPI_F32: return tc_launch_persistent<TC_EPI_F32, 256>(ma, mw, out, M, N, K, 0, 0, nullptr, nullptr, stream);
    case TC_EPI_SILU_MUL: return tc_launch_persistent<TC_EPI_SILU_MUL, 256>(ma, mw, out, M, N, K, 0, 0, nullptr, nullptr, stream);
    default: return SX_ERR_DTYPE;
  }
}

// 0, or which bounded wait ran out (1 producer, 2 and 4 MMA issuer, 3 epilogue, 5 the tail's blocks waiting for one another)
extern "C" int sx_gemm_tc_status(int* host_value) {
  int* p = tc_status_word();
  if (!p) return (int)cudaErrorMemoryAllocation;
  return (int)cudaMemcpy(host_value, p, sizeof(int), cudaMemcpyDeviceToHost);
}
